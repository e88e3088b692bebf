// Paged-KV decode attention (one query token per sequence) as a device function, shared by the stand-alone
// kernel of the rollout engine and by the persistent decode-layers kernel.
#pragma once
#include <cuda_bf16.h>

#include "../common/ptx.cuh"

namespace agrpo {

namespace {

// ------------------------------------------------------------------------------------------------
// Paged decode attention (one query token per sequence), D = 128, block_size = 16, G = Hq/Hkv <= 8.
// CTA = (split, kv head, sequence), 4 warps; a warp owns whole 16-token blocks: cp.async double
// buffering into swizzled shared memory, QK^T and PV on mma.sync m16n8k16 with the query heads of the
// group as the (zero-padded) M rows, online softmax in registers. Warps and splits are merged with
// the usual (max, sum, O) rule.
// ------------------------------------------------------------------------------------------------
constexpr int kDecD = 128;
constexpr int kDecBlock = 16;
constexpr int kDecWarps = 4;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct DecodeParams {
  const __nv_bfloat16* q;   // [B, row pitch ldq], head h at column q_col0 + h*D
  long long ldq;
  int q_col0;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_tables;  // [B, max_blocks]
  const int* seq_lens;      // [B] tokens in the cache including the current one
  int max_blocks;
  int Hq, Hkv, G;
  float scale_log2;
  int splits;
  __nv_bfloat16* out;       // [B, ldo]
  long long ldo;
  float* part_o;            // [B, Hkv, splits, 8, D]
  float* part_ml;           // [B, Hkv, splits, 8, 2]
  int num_cache_blocks;
  int* status;
  int* tickets;             // [B, Hkv] zero-initialised arrival counters, or nullptr: the last split CTA to finish merges
};

// Shared-memory tile of one 16-token block: 16 rows x 256 bytes, 16-byte chunk c of row r stored at c ^ (r & 7).
__device__ __forceinline__ uint8_t* tile_chunk(uint8_t* tile, int row, int chunk) {
  return tile + row * 256 + ((chunk ^ (row & 7)) << 4);
}

// 128 threads (4 warps) work on one (split, kv head, sequence) item; `dsm` is 64 KB of shared memory that they own for
// the duration of the call, `warp` in [0, 4) and `tid` in [0, 128) index the caller's threads, `s_last` is one shared
// int. Threads synchronise on named barrier 1 (128 threads), so the function may be called by a subset of a larger CTA.
// Returns true in every thread of the CTA that produced the final output row group (splits == 1, or the last split).
__device__ __forceinline__ void dec_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// STAGES = K/V blocks a warp keeps in shared memory (one being consumed, STAGES - 1 in flight): dsm must hold
// 4 * STAGES * 8 KB. A decode item is a chain of block loads, so its time is (blocks per warp) x (load latency) /
// (loads in flight).
template <int STAGES>
__device__ __forceinline__ bool paged_decode_attend(const DecodeParams& p, int split, int kvh, int b, uint8_t* dsm, int warp,
                                                    int tid, int* s_last) {
  const int lane = tid & 31;
  dec_bar_sync();  // a caller that loops over items: the previous item's merge has finished reading the staging area
  const int seq_len = p.seq_lens[b];
  const int n_blocks = (seq_len + kDecBlock - 1) / kDecBlock;
  const int blk_begin = (int)((long long)n_blocks * split / p.splits);
  const int blk_end = (int)((long long)n_blocks * (split + 1) / p.splits);
  // per-warp staging: STAGES x (K tile 4 KB + V tile 4 KB)
  uint8_t* wbuf = dsm + warp * (STAGES * 8192);
  const int* table = p.block_tables + (long long)b * p.max_blocks;

  // Q fragments (A operand, rows = query heads of this kv head, zero above G), pre-scaled later in fp32.
  uint32_t qa[kDecD / 16][2];
  {
    const int g = lane >> 2;
    const __nv_bfloat16* qrow = p.q + (long long)b * p.ldq + p.q_col0 + (long long)(kvh * p.G + g) * kDecD;
#pragma unroll
    for (int kk = 0; kk < kDecD / 16; ++kk) {
      const int c = kk * 16 + (lane & 3) * 2;
      // L2 loads: inside a persistent kernel the query row was written by another SM during this launch, and this SM
      // may still hold the previous layer's row at the same address in its L1
      qa[kk][0] = (g < p.G) ? __ldcg(reinterpret_cast<const uint32_t*>(qrow + c)) : 0u;
      qa[kk][1] = (g < p.G) ? __ldcg(reinterpret_cast<const uint32_t*>(qrow + c + 8)) : 0u;
    }
  }
  float o[kDecD / 8][2];
#pragma unroll
  for (int n = 0; n < kDecD / 8; ++n) o[n][0] = o[n][1] = 0.f;
  float m = -INFINITY, l = 0.f;

  auto issue_load = [&](int blk_idx, int stage) {
    int phys = table[blk_idx];
    if (phys < 0 || phys >= p.num_cache_blocks) {
      report_status(p.status, kStatusBadIndex);
      phys = 0;
    }
    const __nv_bfloat16* ksrc = p.k_cache + ((long long)phys * p.Hkv + kvh) * kDecBlock * kDecD;
    const __nv_bfloat16* vsrc = p.v_cache + ((long long)phys * p.Hkv + kvh) * kDecBlock * kDecD;
    uint8_t* kt = wbuf + stage * 8192;
    uint8_t* vt = kt + 4096;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = i * 32 + lane;  // 256 chunks of 16 bytes per tile
      const int row = idx >> 4, chunk = idx & 15;
      cp_async16(tile_chunk(kt, row, chunk), ksrc + row * kDecD + chunk * 8);
      cp_async16(tile_chunk(vt, row, chunk), vsrc + row * kDecD + chunk * 8);
    }
  };

  // One commit group per loop iteration (empty when there is nothing left to load), so that "at most STAGES - 1 groups
  // pending" always means: the block about to be consumed has landed.
  int my = blk_begin + warp;
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {
    if (my + i * kDecWarps < blk_end) issue_load(my + i * kDecWarps, i);
    cp_async_commit();
  }
  int stage = 0;
  for (; my < blk_end; my += kDecWarps, stage = (stage + 1 == STAGES ? 0 : stage + 1)) {
    const int nxt = my + (STAGES - 1) * kDecWarps;
    if (nxt < blk_end) issue_load(nxt, stage == 0 ? STAGES - 1 : stage - 1);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncwarp();
    uint8_t* kt = wbuf + stage * 8192;
    uint8_t* vt = kt + 4096;
    // S = Q K^T for 16 tokens: two n-tiles of 8 tokens.
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int kk = 0; kk < kDecD / 16; ++kk) {
      uint32_t kb[4];
      const int row = (lane & 7) + ((lane >> 4) << 3);
      const int chunk = kk * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(kb, tile_chunk(kt, row, chunk));
      mma_16816(s0, qa[kk][0], 0u, qa[kk][1], 0u, kb[0], kb[1]);
      mma_16816(s1, qa[kk][0], 0u, qa[kk][1], 0u, kb[2], kb[3]);
    }
    // scores of head lane/4 for tokens {2i, 2i+1, 8+2i, 9+2i}, i = lane%4
    const int tok0 = my * kDecBlock + (lane & 3) * 2;
    float sc[4] = {s0[0] * p.scale_log2, s0[1] * p.scale_log2, s1[0] * p.scale_log2, s1[1] * p.scale_log2};
    if (tok0 >= seq_len) sc[0] = -INFINITY;
    if (tok0 + 1 >= seq_len) sc[1] = -INFINITY;
    if (tok0 + 8 >= seq_len) sc[2] = -INFINITY;
    if (tok0 + 9 >= seq_len) sc[3] = -INFINITY;
    float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m, mx);
    const float alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
    const float base = (m_new == -INFINITY) ? 0.f : m_new;
    float pr[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) pr[i] = exp2f(sc[i] - base);
    float ps = pr[0] + pr[1] + pr[2] + pr[3];
    ps += __shfl_xor_sync(0xffffffffu, ps, 1);
    ps += __shfl_xor_sync(0xffffffffu, ps, 2);
    l = l * alpha + ps;
    m = m_new;
    const uint32_t pa0 = pack_bf16x2(pr[0], pr[1]);
    const uint32_t pa2 = pack_bf16x2(pr[2], pr[3]);
#pragma unroll
    for (int n = 0; n < kDecD / 8; ++n) {
      o[n][0] *= alpha;
      o[n][1] *= alpha;
    }
    // O += P V : V^T fragments through transposing ldmatrix, two n-tiles (16 dims) per instruction.
#pragma unroll
    for (int n2 = 0; n2 < kDecD / 16; ++n2) {
      uint32_t vb[4];
      const int row = (lane & 7) + (((lane >> 3) & 1) << 3);
      const int chunk = n2 * 2 + (lane >> 4);
      ldmatrix_x4_trans(vb, tile_chunk(vt, row, chunk));
      float c0[4] = {o[n2 * 2][0], o[n2 * 2][1], 0.f, 0.f};
      float c1[4] = {o[n2 * 2 + 1][0], o[n2 * 2 + 1][1], 0.f, 0.f};
      mma_16816(c0, pa0, 0u, pa2, 0u, vb[0], vb[1]);
      mma_16816(c1, pa0, 0u, pa2, 0u, vb[2], vb[3]);
      o[n2 * 2][0] = c0[0];
      o[n2 * 2][1] = c0[1];
      o[n2 * 2 + 1][0] = c1[0];
      o[n2 * 2 + 1][1] = c1[1];
    }
    __syncwarp();
  }

  // Merge the four warps through shared memory (reusing the staging area after everyone is done).
  dec_bar_sync();
  float* mo = reinterpret_cast<float*>(dsm);           // [warps][8][D]
  float* mml = mo + kDecWarps * 8 * kDecD;             // [warps][8][2]
  {
    const int g = lane >> 2;
#pragma unroll
    for (int n = 0; n < kDecD / 8; ++n) {
      const int d = n * 8 + (lane & 3) * 2;
      mo[(warp * 8 + g) * kDecD + d] = o[n][0];
      mo[(warp * 8 + g) * kDecD + d + 1] = o[n][1];
    }
    if ((lane & 3) == 0) {
      mml[(warp * 8 + g) * 2] = m;
      mml[(warp * 8 + g) * 2 + 1] = l;
    }
  }
  dec_bar_sync();
  for (int idx = tid; idx < p.G * kDecD; idx += kDecWarps * 32) {
    const int g = idx / kDecD, d = idx % kDecD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, mml[(w * 8 + g) * 2]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float mw = mml[(w * 8 + g) * 2];
      const float wgt = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      L += mml[(w * 8 + g) * 2 + 1] * wgt;
      acc += mo[(w * 8 + g) * kDecD + d] * wgt;
    }
    if (p.splits == 1) {
      p.out[(long long)b * p.ldo + (long long)(kvh * p.G + g) * kDecD + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
    } else {
      const long long base = (((long long)b * p.Hkv + kvh) * p.splits + split) * 8 + g;
      p.part_o[base * kDecD + d] = acc;
      if (d == 0) {
        p.part_ml[base * 2] = M;
        p.part_ml[base * 2 + 1] = L;
      }
    }
  }
  // Split-KV merge without a second kernel: every split CTA of a (sequence, kv head) takes a ticket after its
  // partials are visible device-wide; the one that draws the last ticket merges all of them and re-arms the counter.
  bool final_writer = p.splits == 1;
  if (p.splits > 1 && p.tickets != nullptr) {
    __threadfence();
    dec_bar_sync();
    if (tid == 0) {
      int* t = p.tickets + (long long)b * p.Hkv + kvh;
      const int ticket = atomicAdd(t, 1);
      *s_last = (ticket == p.splits - 1) ? 1 : 0;
      if (*s_last) *t = 0;
    }
    dec_bar_sync();
    if (*s_last) {
      final_writer = true;
      __threadfence();
      // four output dims per thread (16-byte loads of the partial outputs), eight splits at a time with all their loads
      // issued before the first use: they are L2 round trips, and the merging CTA is on the step's critical path
      for (int idx = tid; idx < p.G * (kDecD / 4); idx += kDecWarps * 32) {
        const int g = idx / (kDecD / 4), d = (idx % (kDecD / 4)) * 4;
        const long long base0 = (((long long)b * p.Hkv + kvh) * p.splits) * 8 + g;
        float M = -INFINITY, L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < p.splits; s0 += 8) {
          float ms[8], ls[8];
          float4 os[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const bool on = s0 + j < p.splits;
            const long long bs = base0 + (long long)(on ? s0 + j : s0) * 8;
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + bs * 2));
            ms[j] = on ? ml.x : -INFINITY;
            ls[j] = on ? ml.y : 0.f;
            os[j] = __ldcg(reinterpret_cast<const float4*>(p.part_o + bs * kDecD + d));
          }
          float Mn = M;
#pragma unroll
          for (int j = 0; j < 8; ++j) Mn = fmaxf(Mn, ms[j]);
          const float keep = (M == -INFINITY) ? 0.f : exp2f(M - Mn);
          L *= keep;
          acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float w = (ms[j] == -INFINITY) ? 0.f : exp2f(ms[j] - Mn);
            L += ls[j] * w;
            acc.x += os[j].x * w; acc.y += os[j].y * w; acc.z += os[j].z * w; acc.w += os[j].w * w;
          }
          M = Mn;
        }
        uint2 o;  // same expression as the stand-alone combine kernel: both paths give the same bits
        o.x = pack_bf16x2(L > 0.f ? acc.x / L : 0.f, L > 0.f ? acc.y / L : 0.f);
        o.y = pack_bf16x2(L > 0.f ? acc.z / L : 0.f, L > 0.f ? acc.w / L : 0.f);
        *reinterpret_cast<uint2*>(p.out + (long long)b * p.ldo + (long long)(kvh * p.G + g) * kDecD + d) = o;
      }
    }
  }
  return final_writer;
}

}  // namespace

}  // namespace agrpo
