// Skinny bf16 GEMM for decode-time shapes (M <= 256 rows, weights streamed once): split-K across a thread-block
// cluster with the reduction done through distributed shared memory.
//
//   D[M, N] = rs[m] * (A[M, K] . B[N, K]^T) (+ bias) (+ residual), bf16 in / bf16 out, fp32 accumulation
//
// rs[m] = rsqrt(ss_in[m] / K + eps) is optional: with the RMSNorm weight folded into B's columns it makes the GEMM
// consume the un-normalised residual stream directly (the norm kernel disappears from the decode step). ss_out,
// also optional, receives the row sums of squares of the result, i.e. the statistic the NEXT folded GEMM needs.
//
// With a handful of rows the GEMM is bound by streaming B (the weights) from HBM, and a 128 x BN output tile
// per CTA leaves most SMs idle when N is small (N = 1536 gives 12 tiles on 148 SMs). Here the S CTAs of a
// cluster share one output tile and split K between them: each runs the usual TMA -> tcgen05.mma pipeline over
// its K slice into TMEM and then PUSHES its fp32 partial tile, column slice by column slice, into the shared memory of
// the CTA that owns the slice (st.async through distributed shared memory, completing on the owner's mbarrier).
// CTA r owns columns [r * BN / S, (r + 1) * BN / S): once the bytes of all S contributions have landed in its inbox it
// sums them from its own shared memory, applies the epilogue and stores bf16. No partial ever goes to global memory,
// nobody reads a peer's memory (so no CTA has to outlive its peers' reads), and no TMA load targets more than one
// CTA. The only cross-CTA waits are the start-up cluster barrier and the bounded wait on the inbox barrier.
#include <cuda_bf16.h>

#include "../common/ptx.cuh"
#include "../common/tensormap.h"
#include "../launchers.h"

namespace agrpo {

namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kThreads = 192;

// Optional decode-step epilogue for the fused qkv projection (BN = head_dim = 128, one head per column tile): rotary
// embedding of the q and k heads at position seq_lens[row] - 1 and the write of the rotated k and of v into the paged
// KV cache, both on the fp32 sums before they are rounded. Column ownership is then paired: an owner sums columns
// [j, j + wh) and [64 + j, 64 + j + wh) of the tile so that both elements of every rotation pair meet in one thread.
struct SkRope {
  int enabled;
  const float* cos_t;        // [max_pos, 64]
  const float* sin_t;
  int max_pos;
  const int* block_tables;   // [rows, max_blocks]
  int max_blocks;
  const int* seq_lens;       // [rows] tokens in the cache including the current one
  __nv_bfloat16* k_cache;    // [num_cache_blocks, Hkv, block_size, 128]
  __nv_bfloat16* v_cache;
  int Hq, Hkv, block_size, num_cache_blocks;
};

struct SkParams {
  int M, N, K;
  SkRope rope;
  __nv_bfloat16* D;
  long long ldd;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  long long ldr;
  const sumsq_t* ss_in;  // [M] sum of squares of each row of A (fixed point), or nullptr
  sumsq_t* ss_out;       // [M] += sum of squares of each row of D (integer atomic), or nullptr
  float inv_k;          // 1 / K
  float eps;
  int* status;
  long long* trace;  // optional: clock64 stamps of the phases of cluster 0 / CTA 0 (16 slots), nullptr = off
};

#define SK_STAMP(slot)                                                         \
  do {                                                                         \
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0) p.trace[slot] = clock64(); \
  } while (0)

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t remote_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait_cluster(bar, parity)) {
    if (clock64() - t0 > kWaitBudgetTicks) return false;
  }
  return true;
}
__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr) {
  float v;
  // no memory clobber: the loads of one reduction step are independent and must be allowed to overlap; ordering
  // against the hand-off is given by the acquire wait (a volatile asm with a memory clobber) that precedes them
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float4 ld_dsmem_f32x4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
// 16 bytes into a peer's shared memory; the peer's mbarrier counts them (complete_tx) when they land.
__device__ __forceinline__ void st_async_f32x4(uint32_t remote_addr, float a, float b, float c, float d, uint32_t remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(remote_addr),
               "f"(a), "f"(b), "f"(c), "f"(d), "r"(remote_bar)
               : "memory");
}
__device__ __forceinline__ void fence_cluster_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  // only used once at start-up (barrier initialisation must be visible before any remote arrive); the hardware
  // cluster barrier cannot stall here because every CTA of a cluster is resident and reaches it unconditionally
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// MT row-tiles of 128 per CTA (M <= 128 * MT), BN columns per cluster, S = cluster size = K splits.
template <int BN, int MT, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_splitk_cluster_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const SkParams p,
                           const int S) {
  constexpr int kABytes = MT * kBM * kBK * 2;
  constexpr int kBBytes = BN * kBK * 2;
  constexpr int kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = (MT * BN) < 32 ? 32 : (MT * BN);
  constexpr uint32_t kIdesc = umma_idesc_bf16(kBM, BN, 0, 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // inbox: the S contributions to my column slice, as float4 groups of 4 consecutive columns:
  // part[(peer * (w / 4) + group) * rows + row] with w = BN / S columns per owner (16-byte, conflict-free accesses)
  float4* part = reinterpret_cast<float4*>(smem + STAGES * kStageBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(part) + (size_t)BN * MT * kBM * 4);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_bar = empty_bar + STAGES;
  uint64_t* inbox_bar = acc_bar + 1;   // completes when all BN * MT * 128 * 4 bytes of my inbox have landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(inbox_bar + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();
  if (threadIdx.x == 0) SK_STAMP(0);
  const int n0 = blockIdx.y * BN;
  const int num_kb = (p.K + kBK - 1) / kBK;
  const int kb0 = (int)((long long)num_kb * crank / S);
  const int kb1 = (int)((long long)num_kb * (crank + 1) / S);
  const int n_pre = (kb1 - kb0) < STAGES ? (kb1 - kb0) : STAGES;  // loads issued during the prologue

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_bar, 1);
    mbar_init(inbox_bar, 1);
    fence_cluster_barrier_init();
    // only warps that hold rows below M push (32 rows each): the inbox expects exactly their bytes
    const int rows_pushed = (((p.M < MT * kBM ? p.M : MT * kBM) + 31) / 32) * 32;
    mbar_expect_tx(inbox_bar, (uint32_t)(BN * 4 * rows_pushed));
    // The first weight (B) loads depend on nothing that another thread, CTA or the preceding kernel produces: issue
    // them before any synchronisation so that their ~2 us cold latency overlaps the prologue and, under programmatic
    // dependent launch, the tail of the previous kernel. The activation (A) loads follow once that kernel is complete.
    for (int i = 0; i < n_pre; ++i) {
      mbar_expect_tx(&full_bar[i], kStageBytes);
      tma_load_2d(smem + i * kStageBytes + kABytes, &tmB, &full_bar[i], (kb0 + i) * kBK, n0);
    }
    pdl_wait();
    for (int i = 0; i < n_pre; ++i) {
      uint8_t* sa = smem + i * kStageBytes;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) tma_load_2d(sa + mt * (kBM * kBK * 2), &tmA, &full_bar[i], (kb0 + i) * kBK, mt * kBM);
    }
    SK_STAMP(3);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) SK_STAMP(1);
  cluster_sync_all();
  tc_fence_after();
  pdl_wait();
  pdl_launch();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) SK_STAMP(2);

  if (warp == 0) {
    if (elect_one()) {
      int stage = n_pre == STAGES ? 0 : n_pre;
      uint32_t phase = n_pre == STAGES ? 1 : 0;
      for (int kb = kb0 + n_pre; kb < kb1; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
          report_status(p.status, kStatusWaitEmptyTimeout);
          break;
        }
        uint8_t* sa = smem + stage * kStageBytes;
        uint8_t* sb = sa + kABytes;
        mbar_expect_tx(&full_bar[stage], kStageBytes);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) tma_load_2d(sa + mt * (kBM * kBK * 2), &tmA, &full_bar[stage], kb * kBK, mt * kBM);
        tma_load_2d(sb, &tmB, &full_bar[stage], kb * kBK, n0);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase)) {
          report_status(p.status, kStatusWaitFullTimeout);
          ok = false;
          break;
        }
        tc_fence_after();
        if (kb == kb0) SK_STAMP(4);
        const uint32_t sa = smem_u32(smem + stage * kStageBytes);
        const uint32_t sb = sa + kABytes;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)
            tc_mma_f16(tmem_base + mt * BN, umma_smem_desc(sa + mt * (kBM * kBK * 2) + k * 32, 16, 1024),
                       umma_smem_desc(sb + k * 32, 16, 1024), kIdesc, (kb > kb0 || k > 0) ? 1u : 0u);
        }
        tc_commit(&empty_bar[stage]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) tc_commit(acc_bar);
      SK_STAMP(5);
    }
  } else {
    // ---- epilogue warps: TMEM -> owners' inboxes (push), wait for my inbox, sum my slice, store ----
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const int w = BN / S;              // columns per owner (a power of two, at least 8)
    const int w_shift = __ffs(w) - 1;
    const int gpo = w / 4;             // float4 groups per owner
    const bool paired = p.rope.enabled != 0;
    constexpr int kRows = MT * kBM;
    bool ok = true;
    if (kb1 > kb0) {
      if (!mbar_wait(acc_bar, 0)) {
        report_status(p.status, kStatusWaitTmemFullTimeout);
        ok = false;
      }
    }
    tc_fence_after();
    if (threadIdx.x == 64) SK_STAMP(6);
    {
      const uint32_t part_local = smem_u32(part);
      const uint32_t bar_local = smem_u32(inbox_bar);
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        if (mt * kBM + quarter * 32 >= p.M) continue;  // this warp's 32 rows are all padding
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          if (kb1 > kb0 && ok) {
            tmem_ld_32x32(tmem_base + lane_off + mt * BN + c * 32, r);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const int col = c * 32 + i;
            uint32_t owner;
            int g;
            if (paired) {  // owner of columns j and 64 + j alike; local order: first-half columns, then second-half
              owner = (uint32_t)((col & 63) >> (w_shift - 1));
              g = (((col >> 6) << (w_shift - 1)) + (col & ((w >> 1) - 1))) >> 2;
            } else {
              owner = (uint32_t)(col >> w_shift);
              g = (col - (int)owner * w) >> 2;
            }
            const uint32_t off = (uint32_t)((((int)crank * gpo + g) * kRows + mt * kBM + row_in_tile) * 16);
            st_async_f32x4(mapa_shared(part_local + off, owner), __uint_as_float(r[i]), __uint_as_float(r[i + 1]),
                           __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]), mapa_shared(bar_local, owner));
          }
        }
      }
    }
    if (threadIdx.x == 64) SK_STAMP(7);
    // every contribution to my slice (my own included) is counted in bytes by my inbox barrier
    if (!mbar_wait_cluster(inbox_bar, 0)) {
      report_status(p.status, kStatusBarrierTimeout);
      ok = false;
    }
    if (threadIdx.x == 64) SK_STAMP(8);
    // sum my column slice over the S contributions (local shared memory)
    const int c0 = (int)crank * w;
    if (ok && paired) {
      const SkRope& rp = p.rope;
      const int wh = w >> 1;                 // columns per half
      const int tile = blockIdx.y;           // one head per tile: q heads, then k heads, then v heads
      const int row = row_in_tile;           // MT == 1 in this mode
      if (quarter * 32 < p.M && row < p.M) {
        const float rs = p.ss_in != nullptr ? rsqrtf(sumsq_from_fixed(p.ss_in[row]) * p.inv_k + p.eps) : 1.f;
        const int len = rp.seq_lens[row];
        const int pos = len > 0 ? len - 1 : 0;
        const int pp = pos >= rp.max_pos ? rp.max_pos - 1 : pos;
        const bool is_q = tile < rp.Hq, is_k = !is_q && tile < rp.Hq + rp.Hkv;
        __nv_bfloat16* cache_row = nullptr;
        if (!is_q && len > 0) {
          const int blk = rp.block_tables[(long long)row * rp.max_blocks + pos / rp.block_size];
          if (blk < 0 || blk >= rp.num_cache_blocks) {
            report_status(p.status, kStatusBadIndex);
          } else {
            const int h = tile - rp.Hq - (is_k ? 0 : rp.Hkv);
            cache_row = (is_k ? rp.k_cache : rp.v_cache) +
                        (((long long)blk * rp.Hkv + h) * rp.block_size + pos % rp.block_size) * 128;
          }
        }
#pragma unroll 1
        for (int cb = 0; cb < wh; cb += 8) {
          float a1[8], a2[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) a1[i] = a2[i] = 0.f;
#pragma unroll
          for (int peer = 0; peer < 8; ++peer) {
            if (peer < S) {
              const float4* base = part + (size_t)(peer * gpo) * kRows + row;
              const float4 u0 = base[(size_t)(cb / 4) * kRows], u1 = base[(size_t)(cb / 4 + 1) * kRows];
              const float4 v0 = base[(size_t)((wh + cb) / 4) * kRows], v1 = base[(size_t)((wh + cb) / 4 + 1) * kRows];
              a1[0] += u0.x; a1[1] += u0.y; a1[2] += u0.z; a1[3] += u0.w;
              a1[4] += u1.x; a1[5] += u1.y; a1[6] += u1.z; a1[7] += u1.w;
              a2[0] += v0.x; a2[1] += v0.y; a2[2] += v0.z; a2[3] += v0.w;
              a2[4] += v1.x; a2[5] += v1.y; a2[6] += v1.z; a2[7] += v1.w;
            }
          }
          const int j = (int)crank * wh + cb;   // column inside the head, first half; the partner is j + 64
          const int col1 = n0 + j, col2 = col1 + 64;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            a1[i] *= rs;
            a2[i] *= rs;
          }
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              a1[i] += __bfloat162float(p.bias[col1 + i]);
              a2[i] += __bfloat162float(p.bias[col2 + i]);
            }
          }
          if (is_q || is_k) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float cs = rp.cos_t[(size_t)pp * 64 + j + i], sn = rp.sin_t[(size_t)pp * 64 + j + i];
              const float x1 = a1[i], x2 = a2[i];
              a1[i] = x1 * cs - x2 * sn;
              a2[i] = x2 * cs + x1 * sn;
            }
          }
          uint4 o1, o2;
          o1.x = pack_bf16x2(a1[0], a1[1]); o1.y = pack_bf16x2(a1[2], a1[3]);
          o1.z = pack_bf16x2(a1[4], a1[5]); o1.w = pack_bf16x2(a1[6], a1[7]);
          o2.x = pack_bf16x2(a2[0], a2[1]); o2.y = pack_bf16x2(a2[2], a2[3]);
          o2.z = pack_bf16x2(a2[4], a2[5]); o2.w = pack_bf16x2(a2[6], a2[7]);
          __nv_bfloat16* dst = p.D + (long long)row * p.ldd;
          *reinterpret_cast<uint4*>(dst + col1) = o1;
          *reinterpret_cast<uint4*>(dst + col2) = o2;
          if (cache_row != nullptr) {
            *reinterpret_cast<uint4*>(cache_row + j) = o1;
            *reinterpret_cast<uint4*>(cache_row + j + 64) = o2;
          }
        }
      }
    } else if (ok) {
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        if (mt * kBM + quarter * 32 >= p.M) continue;
        const int row = mt * kBM + row_in_tile;
        const float rs = (p.ss_in != nullptr && row < p.M) ? rsqrtf(sumsq_from_fixed(p.ss_in[row]) * p.inv_k + p.eps) : 1.f;
        float sq = 0.f;
#pragma unroll 1
        for (int cb = 0; cb < w; cb += 8) {
          float acc[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
          for (int peer = 0; peer < 8; ++peer) {
            if (peer < S) {
              const float4 v0 = part[(size_t)(peer * gpo + cb / 4) * kRows + row];
              const float4 v1 = part[(size_t)(peer * gpo + cb / 4 + 1) * kRows + row];
              acc[0] += v0.x; acc[1] += v0.y; acc[2] += v0.z; acc[3] += v0.w;
              acc[4] += v1.x; acc[5] += v1.y; acc[6] += v1.z; acc[7] += v1.w;
            }
          }
          const int col = n0 + c0 + cb;
          if (row < p.M && col < p.N) {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] *= rs;
            if (p.bias != nullptr) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (col + i < p.N) acc[i] += __bfloat162float(p.bias[col + i]);
            }
            if (p.residual != nullptr) {
              const __nv_bfloat16* rp = p.residual + (long long)row * p.ldr + col;
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (col + i < p.N) acc[i] += __bfloat162float(rp[i]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (col + i < p.N) sq += acc[i] * acc[i];
            __nv_bfloat16* dst = p.D + (long long)row * p.ldd + col;
            if (col + 8 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
              uint4 o;
              o.x = pack_bf16x2(acc[0], acc[1]);
              o.y = pack_bf16x2(acc[2], acc[3]);
              o.z = pack_bf16x2(acc[4], acc[5]);
              o.w = pack_bf16x2(acc[6], acc[7]);
              *reinterpret_cast<uint4*>(dst) = o;
            } else {
              for (int i = 0; i < 8; ++i)
                if (col + i < p.N) dst[i] = __float2bfloat16(acc[i]);
            }
          }
        }
        if (p.ss_out != nullptr && row < p.M) sumsq_atomic_add(p.ss_out + row, sq);
      }
    }
    if (threadIdx.x == 64) SK_STAMP(9);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) SK_STAMP(11);
}

template <int BN, int MT, int STAGES>
void launch_sk(const CUtensorMap& ta, const CUtensorMap& tb, const SkParams& p, int S, int n_tiles, cudaStream_t stream) {
  constexpr int smem = STAGES * (MT * kBM * kBK * 2 + BN * kBK * 2) + BN * MT * kBM * 4 + 256 + 1024;
  auto kernel = gemm_splitk_cluster_kernel<BN, MT, STAGES>;
  AGRPO_SET_MAX_DYN_SMEM(kernel, smem, "gemm_splitk smem attr");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(S, n_tiles, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_flag() ? 2 : 1;
  check_cuda(cudaLaunchKernelEx(&cfg, kernel, ta, tb, p, S), "gemm_splitk launch");
}

}  // namespace

// Number of K splits (= cluster size) the skinny kernel would use, 0 when it does not serve the shape.
int gemm_skinny_splits(int M, int N, int K, int num_sms) {
  if (M > 256 || K < 512 || N < 64) return 0;
  const int BN = M <= 128 ? 128 : 64;
  const int n_tiles = (N + BN - 1) / BN;
  const int num_kb = (K + kBK - 1) / kBK;
  int S = 8;
  while (S > 1 && (n_tiles * S > (num_sms * 3) / 2 || num_kb / S < 2)) S >>= 1;
  return S == 1 ? 0 : S;
}

// Returns false when the shape is not one this kernel serves (the caller then uses the general GEMM).
bool launch_gemm_skinny(const void* a, long long lda, const void* b, long long ldb, void* d, long long ldd, int M, int N, int K,
                        const void* bias, const void* residual, long long ldr, int* status, int num_sms, cudaStream_t stream,
                        long long* trace, const long long* ss_in, long long* ss_out, float eps, const DecodeRopeArgs* rope) {
  const int S = gemm_skinny_splits(M, N, K, num_sms);
  if (S == 0) return false;
  if (rope != nullptr) {
    // one 128-wide head per column tile, one 128-row tile, D and the output 16-byte aligned, no residual
    if (M > 128 || N != (rope->Hq + 2 * rope->Hkv) * 128 || residual != nullptr || ss_out != nullptr || ldd % 8 != 0 ||
        (reinterpret_cast<uintptr_t>(d) & 15) != 0 || S > 8)
      return false;
  }
  const int MT = M <= 128 ? 1 : 2;
  const int BN = MT == 1 ? 128 : 64;
  const int n_tiles = (N + BN - 1) / BN;
  const CUtensorMap ta = make_tmap_2d(a, K, M, lda, 64, kBM);
  const CUtensorMap tb = make_tmap_2d(b, K, N, ldb, 64, BN);
  SkParams p;
  p.M = M; p.N = N; p.K = K;
  p.D = reinterpret_cast<__nv_bfloat16*>(d);
  p.ldd = ldd;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.rope = SkRope{};
  if (rope != nullptr) {
    p.rope.enabled = 1;
    p.rope.cos_t = rope->cos_t; p.rope.sin_t = rope->sin_t; p.rope.max_pos = rope->max_pos;
    p.rope.block_tables = rope->block_tables; p.rope.max_blocks = rope->max_blocks; p.rope.seq_lens = rope->seq_lens;
    p.rope.k_cache = reinterpret_cast<__nv_bfloat16*>(rope->k_cache);
    p.rope.v_cache = reinterpret_cast<__nv_bfloat16*>(rope->v_cache);
    p.rope.Hq = rope->Hq; p.rope.Hkv = rope->Hkv; p.rope.block_size = rope->block_size;
    p.rope.num_cache_blocks = rope->num_cache_blocks;
  }
  p.ss_in = ss_in;
  p.ss_out = ss_out;
  p.inv_k = 1.f / (float)K;
  p.eps = eps;
  p.status = status;
  p.trace = trace;
  if (MT == 1) launch_sk<128, 1, 4>(ta, tb, p, S, n_tiles, stream);
  else         launch_sk<64, 2, 3>(ta, tb, p, S, n_tiles, stream);
  return true;
}

}  // namespace agrpo
