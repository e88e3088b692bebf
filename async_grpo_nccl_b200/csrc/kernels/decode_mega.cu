// All decoder layers of one decode step in ONE persistent launch (one CTA per SM, cooperative launch).
//
// A decode step at small batch is bound by streaming the weights once; as ~140 separate launches each GEMM pays a
// cold start (first TMA round trip, barrier set-up, TMEM allocation) and a tail that are as long as its streaming time.
// Here the weight stream never stops: a dedicated warp issues the TMA loads of every weight tile of every phase of every
// layer in order, limited only by the depth of its shared-memory ring, so the loads of the next phase are in flight
// while the current phase's results are still being reduced. Only the (small) activation loads wait for the phase before.
//
// The GEMMs run "swapped": the weight tile supplies the 128 MMA rows (output features), the batch rows are the MMA N
// dimension (BT = 32 .. 256), so a small batch costs a small MMA and no padding traffic.
//
//   per layer:  qkv = rs(x) * (x . Wqkv'^T) + b, RoPE, KV-cache write      (phase 0, split K)
//               attention over the paged cache, split-KV                     (compute warps)
//               x1  = x + attn . Wo^T, row sums of squares                    (phase 1, split K)
//               act = silu(rs * x1 . Wg'^T) * (rs * x1 . Wu'^T)               (phase 2)
//               x   = x1 + act . Wd^T, row sums of squares                    (phase 3, split K)
//   (W' = weight with the RMSNorm weight folded into its columns, rs = 1 / rms of the row.)
//
// Work item of a GEMM phase = (128-feature tile, K split). Every item writes its fp32 partial tile to a scratch slot
// (L2-resident), bumps the tile's arrival counter, waits (bounded) until all S splits of the tile have arrived, then
// reduces ITS share of the batch rows over the S partials in a fixed order and applies the epilogue: the reduction is
// spread over all CTAs and its result does not depend on arrival order. A global counter `done` counts finished shares;
// the activation producer of the next phase waits for the count that says the whole phase is complete.
//
// Every wait is bounded; a wait that runs out records a status code, makes the CTA leave through its normal exit (TMEM
// freed) and the other CTAs follow as soon as they see the status word.
#include <cuda_bf16.h>

#include "../common/ptx.cuh"
#include "../common/tensormap.h"
#include "../launchers.h"
#include "decode_attn.cuh"
#include "decode_sync.cuh"

namespace agrpo {

namespace {

constexpr int kMegaThreads = 256;
constexpr int kFT = 128;                    // features per item (MMA M)
constexpr int kMBK = 64;                    // K per stage
constexpr int kWStage = kFT * kMBK * 2;     // 16 KB
constexpr int kMaxGroups = 512;             // arrival counters per GEMM phase

struct MegaPhase {
  int n_groups;  // feature tiles
  int S;         // K splits per tile
  int num_kb;    // K / 64
};

struct MegaParams {
  int L, B, H, Q, QD, F, Hq, Hkv, grid;
  MegaPhase ph[4];
  int att_groups, splits;
  unsigned int per_layer;  // `done` increments per layer
  __nv_bfloat16 *x, *x1, *qkv, *attn, *act;
  const __nv_bfloat16* bqkv;
  long long bqkv_stride;
  sumsq_t* ss;
  int ss_stride;
  float eps, inv_h;
  const float *cos_t, *sin_t;
  int max_pos;
  const int* block_tables;
  int max_blocks;
  const int* seq_lens;
  __nv_bfloat16* cache;
  long long cache_layer_stride, cache_v_off;
  int num_cache_blocks;
  float scale_log2;
  float *part_o, *part_ml;
  int* att_tickets;
  float* partials;
  unsigned int* arrive;  // [4][kMaxGroups] monotonic arrival counters
  unsigned int* done;
  int* status;
  long long* trace;  // optional: clock64 stamps of CTA 0 in layer trace_layer (32 slots), nullptr = off
  int trace_layer;
  int prefetch_tiles;  // weight tiles (16 KB) per CTA requested into L2 ahead of the shared-memory ring (0 = off)
  int trace_all;     // also record 4 global-timer stamps per CTA (trace must hold 32 + 4 * grid words)
};

__device__ __forceinline__ long long global_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// per-CTA stamps (global nanosecond timer) behind the 32 slots of CTA 0: trace[32 + 4 * cta + k]
#define MEGA_STAMP_ALL(k)                                                                       \
  do {                                                                                          \
    if (p.trace != nullptr && p.trace_all && l == p.trace_layer) p.trace[32 + 4 * cta + (k)] = global_ns(); \
  } while (0)

#define MEGA_STAMP(slot)                                                                        \
  do {                                                                                          \
    if (p.trace != nullptr && cta == 0 && l == p.trace_layer) p.trace[slot] = clock64();        \
  } while (0)

__device__ __forceinline__ float4 shfl_xor4(float4 v, int m) {
  return make_float4(__shfl_xor_sync(0xffffffffu, v.x, m), __shfl_xor_sync(0xffffffffu, v.y, m),
                     __shfl_xor_sync(0xffffffffu, v.z, m), __shfl_xor_sync(0xffffffffu, v.w, m));
}
template <int BT>
struct MegaCfg {
  static constexpr int kXStage = BT * kMBK * 2;
  static constexpr int kNSW = 7;
  static constexpr int kXA = 98304;  // activation ring; the attention phase stages K/V tiles here (3 blocks per warp)
  static constexpr int kAttStages = 3;
  static constexpr int kNSX = (kXA / kXStage) > 8 ? 8 : (kXA / kXStage);
  static constexpr int kAcc = 2;
  static constexpr uint32_t kTmemCols = (kAcc * BT) < 32 ? 32 : (kAcc * BT);
  static constexpr int kSmem = kNSW * kWStage + kXA + 1024 /* barriers */ + 1024 /* alignment */;
};

// What the roles of one CTA share.
struct MegaShared {
  uint64_t full_w[8], empty_w[8], full_x[8], empty_x[8], tmem_full[2], tmem_empty[2], xa_bar;
  uint32_t tmem_slot;
  int s_last;
  int abort;
};

template <int BT>
__global__ void __launch_bounds__(kMegaThreads, 1)
decode_layers_kernel(const __grid_constant__ CUtensorMap tmWqkv, const __grid_constant__ CUtensorMap tmWo,
                     const __grid_constant__ CUtensorMap tmWgu, const __grid_constant__ CUtensorMap tmWd,
                     const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmAttn,
                     const __grid_constant__ CUtensorMap tmX1, const __grid_constant__ CUtensorMap tmAct, const MegaParams p) {
  using Cfg = MegaCfg<BT>;
  constexpr int NSW = Cfg::kNSW, NSX = Cfg::kNSX;
  constexpr uint32_t kIdesc = umma_idesc_bf16(kFT, BT, 0, 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* w_ring = smem;
  uint8_t* xa = smem + NSW * kWStage;
  MegaShared* sh = reinterpret_cast<MegaShared*>(xa + Cfg::kXA);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, G = p.grid;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 8; ++s) {
      mbar_init(&sh->full_w[s], 1);
      mbar_init(&sh->empty_w[s], 1);
      mbar_init(&sh->full_x[s], 1);
      mbar_init(&sh->empty_x[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sh->tmem_full[a], 1);
      mbar_init(&sh->tmem_empty[a], 1);
    }
    mbar_init(&sh->xa_bar, 128);
    sh->s_last = 0;
    sh->abort = 0;
    fence_mbar_init();
  }
  if (warp == 3) {
    tmem_alloc(&sh->tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_slot;

  // done-counter value at which the inputs of GEMM phase ph of layer l are complete
  auto target = [&](int l, int ph) -> unsigned int {
    unsigned int t = (unsigned int)l * p.per_layer;
    if (ph >= 1) t += (unsigned int)(p.ph[0].n_groups * p.ph[0].S) + (unsigned int)p.att_groups;
    if (ph >= 2) t += (unsigned int)(p.ph[1].n_groups * p.ph[1].S);
    if (ph >= 3) t += (unsigned int)(p.ph[2].n_groups * p.ph[2].S);
    return t;
  };

  if (warp == 0) {
    // ================= weight producer: never waits for another CTA =================
    // Two cursors walk the same sequence of weight tiles (layer, phase, item, K block): `ld` issues the TMA loads into
    // the shared-memory ring, `pf` runs prefetch_tiles ahead of it and only asks for the tiles to be brought into L2.
    // The ring alone covers a few microseconds of streaming; the L2 window keeps HBM busy through the attention phase
    // and the hand-offs between phases, when the ring is full and nobody consumes it.
    if (elect_one()) {
      struct Cur {
        int l, ph, item, kb, kb1, ft;
      };
      auto seek = [&](Cur& c) -> bool {  // first K block of the item at (l, ph, item), or of the next one that exists
        while (c.l < p.L) {
          const int S = p.ph[c.ph].S, nkb = p.ph[c.ph].num_kb;
          if (c.item < p.ph[c.ph].n_groups * S) {
            c.ft = c.item / S;
            const int ks = c.item - c.ft * S;
            c.kb = (int)((long long)nkb * ks / S);
            c.kb1 = (int)((long long)nkb * (ks + 1) / S);
            if (c.kb < c.kb1) return true;
            c.item += G;
            continue;
          }
          c.item = cta;
          if (++c.ph == 4) {
            c.ph = 0;
            ++c.l;
          }
        }
        return false;
      };
      auto step = [&](Cur& c) -> bool {
        if (++c.kb < c.kb1) return true;
        c.item += G;
        return seek(c);
      };
      auto tmap = [&](int ph) { return ph == 0 ? &tmWqkv : ph == 1 ? &tmWo : ph == 2 ? &tmWgu : &tmWd; };
      Cur ld{0, 0, cta, 0, 0, 0}, pf{0, 0, cta, 0, 0, 0};
      bool ld_on = seek(ld), pf_on = seek(pf);
      int ahead = 0;
      int st = 0;
      uint32_t par = 0;
      bool ok = true;
      while (ld_on) {
        while (pf_on && ahead < p.prefetch_tiles) {
          if (pf.ph == 2) {
            tma_prefetch_l2_3d(tmap(2), pf.kb * kMBK, pf.ft * 64, pf.l);
            tma_prefetch_l2_3d(tmap(2), pf.kb * kMBK, p.F + pf.ft * 64, pf.l);
          } else {
            tma_prefetch_l2_3d(tmap(pf.ph), pf.kb * kMBK, pf.ft * kFT, pf.l);
          }
          pf_on = step(pf);
          ++ahead;
        }
        if (!mbar_wait_s(&sh->empty_w[st], par ^ 1, p.status)) {
          report_status(p.status, kStatusWaitEmptyTimeout);
          ok = false;
          break;
        }
        uint8_t* dst = w_ring + st * kWStage;
        mbar_expect_tx(&sh->full_w[st], kWStage);
        if (ld.ph == 2) {  // 64 gate features on MMA rows 0..63, the matching 64 up features on rows 64..127
          tma_load_3d(dst, tmap(2), &sh->full_w[st], ld.kb * kMBK, ld.ft * 64, ld.l);
          tma_load_3d(dst + 64 * kMBK * 2, tmap(2), &sh->full_w[st], ld.kb * kMBK, p.F + ld.ft * 64, ld.l);
        } else {
          tma_load_3d(dst, tmap(ld.ph), &sh->full_w[st], ld.kb * kMBK, ld.ft * kFT, ld.l);
        }
        if (++st == NSW) {
          st = 0;
          par ^= 1;
        }
        ld_on = step(ld);
        --ahead;
      }
      if (!ok) sh->abort = 1;
    }
  } else if (warp == 1) {
    // ================= activation producer: waits for the phase that writes its operand =================
    if (elect_one()) {
      int st = 0;
      uint32_t par = 0;
      bool ok = true;
      for (int l = 0; l < p.L && ok; ++l) {
        for (int ph = 0; ph < 4 && ok; ++ph) {
          const CUtensorMap* tm = ph == 0 ? &tmX : ph == 1 ? &tmAttn : ph == 2 ? &tmX1 : &tmAct;
          const int S = p.ph[ph].S, nkb = p.ph[ph].num_kb, n_items = p.ph[ph].n_groups * S;
          if (ph == 1) {
            // the attention phase used this ring's memory through the generic proxy: its threads fenced and arrived
            if (!mbar_wait_s(&sh->xa_bar, (uint32_t)(l & 1), p.status)) {
              report_status(p.status, kStatusBarrierTimeout);
              ok = false;
              break;
            }
          }
          bool waited = (l == 0 && ph == 0);
          for (int item = cta; item < n_items && ok; item += G) {
            if (!waited) {
              if (!wait_counter(p.done, target(l, ph), p.status)) {
                report_status(p.status, kStatusPeerFlagTimeout);
                ok = false;
                break;
              }
              fence_proxy_async_all();  // other SMs wrote the operand with ordinary stores; TMA reads it
              waited = true;
            }
            const int ft = item / S, ks = item - ft * S;
            const int kb0 = (int)((long long)nkb * ks / S), kb1 = (int)((long long)nkb * (ks + 1) / S);
            for (int kb = kb0; kb < kb1; ++kb) {
              if (!mbar_wait_s(&sh->empty_x[st], par ^ 1, p.status)) {
                report_status(p.status, kStatusWaitEmptyTimeout);
                ok = false;
                break;
              }
              mbar_expect_tx(&sh->full_x[st], Cfg::kXStage);
              tma_load_2d(xa + st * Cfg::kXStage, tm, &sh->full_x[st], kb * kMBK, 0);
              if (++st == NSX) {
                st = 0;
                par ^= 1;
              }
            }
          }
        }
      }
      if (!ok) sh->abort = 1;
    }
  } else if (warp == 2) {
    // ================= MMA issuer =================
    if (elect_one()) {
      int sw = 0, sx = 0, acc = 0;
      uint32_t pw = 0, px = 0, pa = 0;
      bool ok = true;
      for (int l = 0; l < p.L && ok; ++l) {
        for (int ph = 0; ph < 4 && ok; ++ph) {
          const int S = p.ph[ph].S, nkb = p.ph[ph].num_kb, n_items = p.ph[ph].n_groups * S;
          for (int item = cta; item < n_items && ok; item += G) {
            const int ft = item / S, ks = item - ft * S;
            const int kb0 = (int)((long long)nkb * ks / S), kb1 = (int)((long long)nkb * (ks + 1) / S);
            if (!mbar_wait_s(&sh->tmem_empty[acc], pa ^ 1, p.status)) {
              report_status(p.status, kStatusWaitTmemEmptyTimeout);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t d_addr = tmem_base + (uint32_t)(acc * BT);
            for (int kb = kb0; kb < kb1; ++kb) {
              if (!mbar_wait_s(&sh->full_w[sw], pw, p.status) || !mbar_wait_s(&sh->full_x[sx], px, p.status)) {
                report_status(p.status, kStatusWaitFullTimeout);
                ok = false;
                break;
              }
              tc_fence_after();
              if (kb == kb0) MEGA_STAMP(ph * 6 + 0);
              if (kb == kb0 && ph == 1) MEGA_STAMP_ALL(2);
              if (kb == kb0 && ph == 0) MEGA_STAMP_ALL(3);
              const uint32_t sa = smem_u32(w_ring + sw * kWStage);
              const uint32_t sb = smem_u32(xa + sx * Cfg::kXStage);
#pragma unroll
              for (int k = 0; k < kMBK / 16; ++k)
                tc_mma_f16(d_addr, umma_smem_desc(sa + k * 32, 16, 1024), umma_smem_desc(sb + k * 32, 16, 1024), kIdesc,
                           (kb > kb0 || k > 0) ? 1u : 0u);
              tc_commit(&sh->empty_w[sw]);
              tc_commit(&sh->empty_x[sx]);
              if (++sw == NSW) {
                sw = 0;
                pw ^= 1;
              }
              if (++sx == NSX) {
                sx = 0;
                px ^= 1;
              }
            }
            if (!ok) break;
            tc_commit(&sh->tmem_full[acc]);
            MEGA_STAMP(ph * 6 + 1);
            if (++acc == Cfg::kAcc) {
              acc = 0;
              pa ^= 1;
            }
          }
        }
      }
      if (!ok) sh->abort = 1;
    }
  } else if (warp >= 4) {
    // ================= compute warps: GEMM reductions + epilogues, attention =================
    const int cw = warp - 4;             // TMEM lane quarter (warp % 4)
    const int tid = threadIdx.x - 128;   // 0..127
    const uint32_t lane_off = static_cast<uint32_t>(cw * 32) << 16;
    int acc = 0;
    uint32_t pa = 0;
    bool ok = true;
    const int B = p.B;

    DecodeParams dp;
    dp.q = p.qkv;
    dp.ldq = p.Q;
    dp.q_col0 = 0;
    dp.block_tables = p.block_tables;
    dp.seq_lens = p.seq_lens;
    dp.max_blocks = p.max_blocks;
    dp.Hq = p.Hq;
    dp.Hkv = p.Hkv;
    dp.G = p.Hq / p.Hkv;
    dp.scale_log2 = p.scale_log2;
    dp.splits = p.splits;
    dp.out = p.attn;
    dp.ldo = p.QD;
    dp.part_o = p.part_o;
    dp.part_ml = p.part_ml;
    dp.num_cache_blocks = p.num_cache_blocks;
    dp.status = p.status;
    dp.tickets = p.att_tickets;

    for (int l = 0; l < p.L && ok; ++l) {
      __nv_bfloat16* k_cache = p.cache + (long long)l * p.cache_layer_stride;
      __nv_bfloat16* v_cache = k_cache + p.cache_v_off;
      if (tid == 0) MEGA_STAMP(26);
      for (int ph = 0; ph < 4 && ok; ++ph) {
        if (ph == 1) {
          // ---------------- attention over the paged cache ----------------
          if (tid == 0) {
            if (!wait_counter(p.done, (unsigned int)l * p.per_layer + (unsigned int)(p.ph[0].n_groups * p.ph[0].S), p.status)) {
              report_status(p.status, kStatusPeerFlagTimeout);
              sh->abort = 1;
            }
          }
          dec_bar_sync();
          if (sh->abort) {
            ok = false;
            break;
          }
          if (tid == 0) MEGA_STAMP(24);
          if (tid == 0) MEGA_STAMP_ALL(0);
          dp.k_cache = k_cache;
          dp.v_cache = v_cache;
          const int n_att = p.att_groups * p.splits;
          for (int it = cta; it < n_att; it += G) {
            const int split = it % p.splits;
            const int rest = it / p.splits;
            const int kvh = rest % p.Hkv, b = rest / p.Hkv;
            if (p.seq_lens[b] <= 0) {
              // an idle row (a free slot inside the batch): nothing to attend to, its output is never used
              if (split == 0 && tid == 0) red_release_gpu_add(p.done, 1u);
              continue;
            }
            const bool fin = paged_decode_attend<Cfg::kAttStages>(dp, split, kvh, b, xa, cw, tid, &sh->s_last);
            if (fin) {
              dec_bar_sync();  // every thread's output stores are issued
              if (tid == 0) {
                __threadfence();
                red_release_gpu_add(p.done, 1u);
              }
            }
          }
          fence_proxy_async_smem();   // the activation ring is handed back to TMA
          mbar_arrive(&sh->xa_bar);
          if (tid == 0) MEGA_STAMP(25);
          if (tid == 0) MEGA_STAMP_ALL(1);
        }
        // ---------------- GEMM items of this phase ----------------
        const int S = p.ph[ph].S, n_items = p.ph[ph].n_groups * S;
        for (int item = cta; item < n_items && ok; item += G) {
          const int grp = item / S, ks = item - grp * S;
          bool have_acc = true;
          if (!mbar_wait_s(&sh->tmem_full[acc], pa, p.status)) {
            report_status(p.status, kStatusWaitTmemFullTimeout);
            sh->abort = 1;  // read by every compute thread after the barriers below: they all leave together
            have_acc = false;
          }
          tc_fence_after();
          if (tid == 0) MEGA_STAMP(ph * 6 + 2);
          float* slot = p.partials + (size_t)item * (BT * kFT);
          if (have_acc) {
#pragma unroll 1
            for (int c = 0; c < BT / 32; ++c) {
              if (c * 32 >= B) break;  // padding rows
              uint32_t r[32];
              tmem_ld_32x32(tmem_base + lane_off + (uint32_t)(acc * BT + c * 32), r);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (c * 32 + i < B) __stcg(slot + (size_t)(c * 32 + i) * kFT + cw * 32 + lane, __uint_as_float(r[i]));
            }
          }
          tc_fence_before();
          // Row statistics, lengths and the residual of my first rows do not depend on the other splits: request them now,
          // they arrive while this CTA waits for the tile's other splits.
          const int r0 = (int)((long long)B * ks / S), r1 = (int)((long long)B * (ks + 1) / S);
          constexpr int RU = 4;
          const int b_first = r0 + cw * RU;
          sumsq_t m_ss[RU];
          int m_len[RU];
          float4 m_rr[RU], m_cs[RU], m_sn[RU];
          int m_blk[RU];
          auto load_meta = [&](int b0) {
#pragma unroll
            for (int j = 0; j < RU; ++j) {
              const int b = (b0 + j < r1) ? b0 + j : r0;
              m_ss[j] = 0;
              m_len[j] = 0;
              m_rr[j] = make_float4(0.f, 0.f, 0.f, 0.f);
              if (b0 < r1) {
                if (ph == 0) {
                  m_ss[j] = ld_sumsq_l2(p.ss + (size_t)(2 * l) * p.ss_stride + b);
                  m_len[j] = p.seq_lens[b];
                } else if (ph == 2) {
                  m_ss[j] = ld_sumsq_l2(p.ss + (size_t)(2 * l + 1) * p.ss_stride + b);
                } else {
                  m_rr[j] = ld_bf16x4((ph == 1 ? p.x : p.x1) + (size_t)b * p.H + grp * kFT + 4 * lane);
                }
              }
            }
            if (ph == 0 && b0 < r1) {  // rotary table entries and the cache block of each row's position
              const bool not_q = grp >= p.Hq;
              const int jr = (4 * lane) & 63;
#pragma unroll
              for (int j = 0; j < RU; ++j) {
                const int b = (b0 + j < r1) ? b0 + j : r0;
                const int pos = m_len[j] > 0 ? m_len[j] - 1 : 0;
                const int pp = pos >= p.max_pos ? p.max_pos - 1 : pos;
                m_cs[j] = *reinterpret_cast<const float4*>(p.cos_t + (size_t)pp * 64 + jr);
                m_sn[j] = *reinterpret_cast<const float4*>(p.sin_t + (size_t)pp * 64 + jr);
                m_blk[j] = (not_q && m_len[j] > 0) ? p.block_tables[(long long)b * p.max_blocks + pos / kDecBlock] : 0;
              }
            }
          };
          load_meta(b_first);
          // the CTA barrier orders every thread's partial stores before the release below (cumulative at GPU scope)
          dec_bar_sync();
          if (tid == 0) {
            mbar_arrive(&sh->tmem_empty[acc]);
            unsigned int* ctr = p.arrive + ph * kMaxGroups + grp;
            red_release_gpu_add(ctr, 1u);
            MEGA_STAMP(ph * 6 + 3);
            if (!wait_counter(ctr, (unsigned int)S * (unsigned int)(l + 1), p.status)) {
              report_status(p.status, kStatusBarrierTimeout);
              sh->abort = 1;
            }
          }
          if (++acc == Cfg::kAcc) {
            acc = 0;
            pa ^= 1;
          }
          dec_bar_sync();
          if (sh->abort) {
            ok = false;
            break;
          }
          if (tid == 0) MEGA_STAMP(ph * 6 + 4);
          // ---- my share of the rows: reduce over the S partials, epilogue ----
          const float* gbase = p.partials + (size_t)(grp * S) * (BT * kFT);
          // Four rows per warp pass. Everything a row needs from memory (its S partials, statistics, residual, rotary
          // table entries, cache slot) is requested before the first use, so that the L2 round trips of the four rows
          // and of the splits overlap instead of adding up.
          for (int b0 = b_first; b0 < r1; b0 += 4 * RU) {
            if (b0 != b_first) load_meta(b0);
            float4 v[RU];
            bool on[RU];
#pragma unroll
            for (int j = 0; j < RU; ++j) {
              on[j] = b0 + j < r1;
              v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            for (int s = 0; s < S; s += 2) {
              float4 t0[RU], t1[RU];
              const bool two = s + 1 < S;
#pragma unroll
              for (int j = 0; j < RU; ++j) {
                const float4* src = reinterpret_cast<const float4*>(gbase + ((size_t)s * BT + (on[j] ? b0 + j : r0)) * kFT) + lane;
                t0[j] = __ldcg(src);
                t1[j] = two ? __ldcg(src + (size_t)BT * kFT / 4) : make_float4(0.f, 0.f, 0.f, 0.f);
              }
#pragma unroll
              for (int j = 0; j < RU; ++j) {  // fixed order: split s, then split s + 1
                v[j].x += t0[j].x; v[j].y += t0[j].y; v[j].z += t0[j].z; v[j].w += t0[j].w;
                v[j].x += t1[j].x; v[j].y += t1[j].y; v[j].z += t1[j].z; v[j].w += t1[j].w;
              }
            }
            if (ph == 0) {
              const bool is_q = grp < p.Hq, is_k = !is_q && grp < p.Hq + p.Hkv;
              float4 bb = make_float4(0.f, 0.f, 0.f, 0.f);
              if (p.bqkv != nullptr) bb = ld_bf16x4(p.bqkv + (long long)l * p.bqkv_stride + grp * kFT + 4 * lane);
              const int* len = m_len;
              const int* blk = m_blk;
              const float4* cs = m_cs;
              const float4* sn = m_sn;
#pragma unroll
              for (int j = 0; j < RU; ++j) {
                if (!on[j]) continue;  // warp-uniform
                const int b = b0 + j;
                const float rs = rsqrtf(sumsq_from_fixed(m_ss[j]) * p.inv_h + p.eps);
                float4 w = make_float4(v[j].x * rs + bb.x, v[j].y * rs + bb.y, v[j].z * rs + bb.z, v[j].w * rs + bb.w);
                if (is_q || is_k) {
                  const float4 o = shfl_xor4(w, 16);
                  const float sg = lane < 16 ? -1.f : 1.f;  // lanes < 16 hold x1 (x1 c - x2 s), the others x2 (x2 c + x1 s)
                  w = make_float4(w.x * cs[j].x + sg * o.x * sn[j].x, w.y * cs[j].y + sg * o.y * sn[j].y,
                                  w.z * cs[j].z + sg * o.z * sn[j].z, w.w * cs[j].w + sg * o.w * sn[j].w);
                }
                st_bf16x4(p.qkv + (size_t)b * p.Q + grp * kFT + 4 * lane, w);
                if (!is_q && len[j] > 0) {
                  if (blk[j] < 0 || blk[j] >= p.num_cache_blocks) {
                    report_status(p.status, kStatusBadIndex);
                  } else {
                    const int pos = len[j] - 1;
                    const int h = grp - p.Hq - (is_k ? 0 : p.Hkv);
                    __nv_bfloat16* row = (is_k ? k_cache : v_cache) +
                                         (((long long)blk[j] * p.Hkv + h) * kDecBlock + pos % kDecBlock) * kDecD;
                    st_bf16x4(row + 4 * lane, w);
                  }
                }
              }
            } else if (ph == 2) {
#pragma unroll
              for (int j = 0; j < RU; ++j) {
                if (!on[j]) continue;
                const float rs = rsqrtf(sumsq_from_fixed(m_ss[j]) * p.inv_h + p.eps);
                const float4 u = shfl_xor4(v[j], 16);  // lanes < 16 hold gate features, lanes >= 16 the matching up features
                if (lane < 16) {
                  float4 o;
                  const float g0 = v[j].x * rs, g1 = v[j].y * rs, g2 = v[j].z * rs, g3 = v[j].w * rs;
                  o.x = g0 / (1.f + __expf(-g0)) * (u.x * rs);
                  o.y = g1 / (1.f + __expf(-g1)) * (u.y * rs);
                  o.z = g2 / (1.f + __expf(-g2)) * (u.z * rs);
                  o.w = g3 / (1.f + __expf(-g3)) * (u.w * rs);
                  st_bf16x4(p.act + (size_t)(b0 + j) * p.F + grp * 64 + 4 * lane, o);
                }
              }
            } else {
              __nv_bfloat16* obase = ph == 1 ? p.x1 : p.x;
#pragma unroll
              for (int j = 0; j < RU; ++j) {
                if (!on[j]) continue;
                const float4 w = make_float4(v[j].x + m_rr[j].x, v[j].y + m_rr[j].y, v[j].z + m_rr[j].z, v[j].w + m_rr[j].w);
                st_bf16x4(obase + (size_t)(b0 + j) * p.H + grp * kFT + 4 * lane, w);
                float sq = w.x * w.x + w.y * w.y + w.z * w.z + w.w * w.w;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                if (lane == 0) sumsq_atomic_add(p.ss + (size_t)(2 * l + (ph == 1 ? 1 : 2)) * p.ss_stride + b0 + j, sq);
              }
            }
          }
          dec_bar_sync();
          if (tid == 0) {
            red_release_gpu_add(p.done, 1u);
            MEGA_STAMP(ph * 6 + 5);
          }
        }
      }
    }
    if (!ok && tid == 0) sh->abort = 1;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 3) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// 3-D map over per-layer weight matrices that sit at a constant stride in one flat buffer:
// (K inner, rows, layer); box = 64 x box_rows x 1, 128-byte swizzle.
CUtensorMap make_tmap_w3d(const void* base, uint64_t K, uint64_t rows, uint64_t layers, uint64_t layer_stride_elems,
                          uint32_t box_rows) {
  if ((reinterpret_cast<uint64_t>(base) & 15) != 0 || (K * 2) % 16 != 0 || (layer_stride_elems * 2) % 16 != 0)
    throw std::runtime_error("decode_layers: weight tensor map alignment");
  CUtensorMap m;
  cuuint64_t dims[3] = {K, rows, layers};
  cuuint64_t strides[2] = {K * 2, layer_stride_elems * 2};
  cuuint32_t box[3] = {kMBK, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = get_encode_tiled()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("decode_layers: cuTensorMapEncodeTiled failed: " + std::to_string((int)r));
  return m;
}

template <int BT>
void launch_mega(const CUtensorMap* tm, const MegaParams& p, cudaStream_t stream) {
  using Cfg = MegaCfg<BT>;
  auto kernel = decode_layers_kernel<BT>;
  AGRPO_SET_MAX_DYN_SMEM(kernel, Cfg::kSmem, "decode_layers smem attr");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.grid, 1, 1);
  cfg.blockDim = dim3(kMegaThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident together: they wait on one another
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  check_cuda(cudaLaunchKernelEx(&cfg, kernel, tm[0], tm[1], tm[2], tm[3], tm[4], tm[5], tm[6], tm[7], p), "decode_layers launch");
}

int split_for(int n_groups, int num_kb, int grid) {
  int S = grid / n_groups;
  if (S < 1) S = 1;
  if (S > num_kb) S = num_kb;
  if (S > 16) S = 16;
  return S;
}

}  // namespace

// Bytes of fp32 scratch the kernel needs for `rows` batch rows (partial tiles of the phase with the most work items).
long long decode_layers_scratch_bytes(int rows, int H, int Q, int QD, int F, int num_sms) {
  const int BT = rows <= 32 ? 32 : rows <= 64 ? 64 : rows <= 128 ? 128 : 256;
  const int groups[4] = {Q / kFT, H / kFT, F / 64, H / kFT};
  const int kbs[4] = {H / kMBK, QD / kMBK, H / kMBK, F / kMBK};
  long long items = 0;
  for (int i = 0; i < 4; ++i) {
    const long long n = (long long)groups[i] * split_for(groups[i], kbs[i], num_sms);
    if (n > items) items = n;
  }
  return items * BT * kFT * 4;
}

bool decode_layers_supported(int rows, int H, int Q, int QD, int F, int Hq, int Hkv, int head_dim) {
  return rows >= 1 && rows <= 256 && head_dim == 128 && H % 128 == 0 && Q % 128 == 0 && QD % 64 == 0 && F % 64 == 0 &&
         Q == (Hq + 2 * Hkv) * 128 && QD == Hq * 128 && Hkv > 0 && Hq % Hkv == 0 && Hq / Hkv <= 8 && Q / 128 <= kMaxGroups &&
         F / 64 <= kMaxGroups && H / 128 <= kMaxGroups;
}

void launch_decode_layers(const DecodeLayersArgs& a, cudaStream_t stream) {
  if (!decode_layers_supported(a.B, a.H, a.Q, a.QD, a.F, a.Hq, a.Hkv, 128)) throw std::runtime_error("decode_layers: shape not served");
  MegaParams p;
  p.L = a.L; p.B = a.B; p.H = a.H; p.Q = a.Q; p.QD = a.QD; p.F = a.F; p.Hq = a.Hq; p.Hkv = a.Hkv;
  p.grid = a.num_sms;
  const int groups[4] = {a.Q / kFT, a.H / kFT, a.F / 64, a.H / kFT};
  const int kbs[4] = {a.H / kMBK, a.QD / kMBK, a.H / kMBK, a.F / kMBK};
  unsigned int per_layer = 0;
  long long max_items = 0;
  for (int i = 0; i < 4; ++i) {
    p.ph[i].n_groups = groups[i];
    p.ph[i].num_kb = kbs[i];
    p.ph[i].S = split_for(groups[i], kbs[i], p.grid);
    per_layer += (unsigned int)(groups[i] * p.ph[i].S);
    if ((long long)groups[i] * p.ph[i].S > max_items) max_items = (long long)groups[i] * p.ph[i].S;
  }
  p.att_groups = a.B * a.Hkv;
  p.splits = a.splits < 1 ? 1 : a.splits;
  p.per_layer = per_layer + (unsigned int)p.att_groups;
  const int BT = a.B <= 32 ? 32 : a.B <= 64 ? 64 : a.B <= 128 ? 128 : 256;
  if (max_items * BT * kFT * 4 > a.partials_bytes) throw std::runtime_error("decode_layers: scratch buffer too small");
  p.x = (__nv_bfloat16*)a.x; p.x1 = (__nv_bfloat16*)a.x1; p.qkv = (__nv_bfloat16*)a.qkv; p.attn = (__nv_bfloat16*)a.attn;
  p.act = (__nv_bfloat16*)a.act;
  p.bqkv = (const __nv_bfloat16*)a.bqkv; p.bqkv_stride = a.bqkv_stride;
  p.ss = a.ss; p.ss_stride = a.ss_stride;
  p.eps = a.eps; p.inv_h = 1.f / (float)a.H;
  p.cos_t = a.cos_t; p.sin_t = a.sin_t; p.max_pos = a.max_pos;
  p.block_tables = a.block_tables; p.max_blocks = a.max_blocks; p.seq_lens = a.seq_lens;
  p.cache = (__nv_bfloat16*)a.cache; p.cache_layer_stride = a.cache_layer_stride; p.cache_v_off = a.cache_v_off;
  p.num_cache_blocks = a.num_cache_blocks;
  p.scale_log2 = a.softmax_scale * 1.4426950408889634f;
  p.part_o = a.part_o; p.part_ml = a.part_ml; p.att_tickets = a.att_tickets;
  p.partials = a.partials;
  p.arrive = a.counters;
  p.done = a.counters + 4 * kMaxGroups;
  p.status = a.status;
  p.trace = a.trace;
  p.trace_layer = a.trace_layer;
  p.prefetch_tiles = a.prefetch_tiles;
  p.trace_all = a.trace_words >= 32 + 4 * a.num_sms ? 1 : 0;
  // counters start from zero in every launch (stream-ordered, also inside a captured graph)
  check_cuda(cudaMemsetAsync(a.counters, 0, (4 * kMaxGroups + 4) * sizeof(unsigned int), stream), "decode_layers counters");
  CUtensorMap tm[8];
  tm[0] = make_tmap_w3d(a.wqkv, a.H, a.Q, a.L, a.wqkv_stride, kFT);
  tm[1] = make_tmap_w3d(a.wo, a.QD, a.H, a.L, a.wo_stride, kFT);
  tm[2] = make_tmap_w3d(a.wgu, a.H, 2 * (uint64_t)a.F, a.L, a.wgu_stride, 64);
  tm[3] = make_tmap_w3d(a.wd, a.F, a.H, a.L, a.wd_stride, kFT);
  tm[4] = make_tmap_2d(a.x, a.H, a.rows_alloc, a.H, kMBK, BT);
  tm[5] = make_tmap_2d(a.attn, a.QD, a.rows_alloc, a.QD, kMBK, BT);
  tm[6] = make_tmap_2d(a.x1, a.H, a.rows_alloc, a.H, kMBK, BT);
  tm[7] = make_tmap_2d(a.act, a.F, a.rows_alloc, a.F, kMBK, BT);
  switch (BT) {
    case 32: launch_mega<32>(tm, p, stream); break;
    case 64: launch_mega<64>(tm, p, stream); break;
    case 128: launch_mega<128>(tm, p, stream); break;
    default: launch_mega<256>(tm, p, stream); break;
  }
}

int decode_layers_counter_words() { return 4 * kMaxGroups + 4; }

}  // namespace agrpo
