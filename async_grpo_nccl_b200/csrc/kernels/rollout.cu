// Rollout-engine kernels: paged KV-cache write, paged-KV decode attention with native GQA and split-KV,
// and the fused lm_head + sampling epilogue (Gumbel-max over logits that never leave tensor memory).
// Together with the prefill path (the varlen attention kernel) they stand in for the vLLM engine the
// reference drives (vllm_worker.py:203-284, 709-737).
#include <cuda_bf16.h>

#include "../common/tensormap.h"
#include "../launchers.h"
#include "gemm_tcgen05.cuh"

namespace agrpo {

namespace {

// ------------------------------------------------------------------------------------------------
// KV-cache write. Cache layout per layer: [num_blocks, Hkv, block_size, D] for K and for V.
// slot[t] = block * block_size + offset, negative = skip the token.
// ------------------------------------------------------------------------------------------------
__global__ void kv_cache_write_kernel(const __nv_bfloat16* __restrict__ qkv, long long row_pitch, int k_col0, int v_col0,
                                      const int* __restrict__ slots, __nv_bfloat16* __restrict__ k_cache,
                                      __nv_bfloat16* __restrict__ v_cache, int T, int Hkv, int D, int block_size) {
  const int t = blockIdx.x;
  if (t >= T) return;
  const int slot = slots[t];
  if (slot < 0) return;
  const int blk = slot / block_size, off = slot % block_size;
  const int per_row = Hkv * D / 8;  // 16-byte chunks per token per tensor
  for (int i = threadIdx.x; i < 2 * per_row; i += blockDim.x) {
    const bool is_v = i >= per_row;
    const int j = is_v ? i - per_row : i;
    const int h = j / (D / 8), c = j % (D / 8);
    const uint4 val = *reinterpret_cast<const uint4*>(qkv + (long long)t * row_pitch + (is_v ? v_col0 : k_col0) + h * D + c * 8);
    __nv_bfloat16* dst = (is_v ? v_cache : k_cache) + (((long long)blk * Hkv + h) * block_size + off) * D + c * 8;
    *reinterpret_cast<uint4*>(dst) = val;
  }
}

// Decode-time variant: row b is the newest token of batch row b, written at position seq_lens[b] - 1 of the
// sequence whose block table is row b. Rows with seq_lens[b] <= 0 are idle.
__global__ void kv_cache_write_decode_kernel(const __nv_bfloat16* __restrict__ qkv, long long row_pitch, int k_col0,
                                             int v_col0, const int* __restrict__ block_tables, int max_blocks,
                                             const int* __restrict__ seq_lens, __nv_bfloat16* __restrict__ k_cache,
                                             __nv_bfloat16* __restrict__ v_cache, int B, int Hkv, int D, int block_size,
                                             int num_cache_blocks, int* status) {
  const int b = blockIdx.x;
  if (b >= B) return;
  const int len = seq_lens[b];
  if (len <= 0) return;
  const int pos = len - 1;
  const int blk = block_tables[(long long)b * max_blocks + pos / block_size];
  if (blk < 0 || blk >= num_cache_blocks) {
    if (threadIdx.x == 0) report_status(status, kStatusBadIndex);
    return;
  }
  const int off = pos % block_size;
  const int per_row = Hkv * D / 8;
  for (int i = threadIdx.x; i < 2 * per_row; i += blockDim.x) {
    const bool is_v = i >= per_row;
    const int j = is_v ? i - per_row : i;
    const int h = j / (D / 8), c = j % (D / 8);
    const uint4 val = *reinterpret_cast<const uint4*>(qkv + (long long)b * row_pitch + (is_v ? v_col0 : k_col0) + h * D + c * 8);
    __nv_bfloat16* dst = (is_v ? v_cache : k_cache) + (((long long)blk * Hkv + h) * block_size + off) * D + c * 8;
    *reinterpret_cast<uint4*>(dst) = val;
  }
}

// Per-step inputs of the decode graph from ONE staged host buffer (one copy + one launch per step instead of a copy and
// half a dozen small tensor ops). Staging layout, int32 words, S = max sequences:
//   [0, S) sequence lengths | [S] number of block-table updates n | [S + 1] seed increment of this step | [S + 2, S + 4) unused
//   [S + 4, S + 4 + S) flat block-table index of update i | [S + 4 + S, S + 4 + 2 S) block id of update i
__global__ void decode_step_inputs_kernel(const int* __restrict__ stage, int S, int* __restrict__ seq_lens,
                                          int* __restrict__ positions, int* __restrict__ block_tables, long long table_elems,
                                          const long long* __restrict__ base_seeds, long long* __restrict__ step_seeds,
                                          int* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= S) return;
  const int len = stage[i];
  seq_lens[i] = len;
  positions[i] = len > 0 ? len - 1 : 0;
  step_seeds[i] = base_seeds[i] + static_cast<long long>(stage[S + 1]);
  if (i < stage[S]) {
    const int idx = stage[S + 4 + i];
    if (idx < 0 || idx >= table_elems) report_status(status, kStatusBadIndex);
    else block_tables[idx] = stage[S + 4 + S + i];
  }
}

// Decode-time RoPE + KV write in one pass: rotates the q and k heads of row b in place (position seq_lens[b] - 1)
// and stores the rotated k and the v of that token into the sequence's cache page.
__global__ void rope_kv_write_decode_kernel(__nv_bfloat16* __restrict__ qkv, long long row_pitch, const float* __restrict__ cos_t,
                                            const float* __restrict__ sin_t, int max_pos, const int* __restrict__ block_tables,
                                            int max_blocks, const int* __restrict__ seq_lens, __nv_bfloat16* __restrict__ k_cache,
                                            __nv_bfloat16* __restrict__ v_cache, int B, int Hq, int Hkv, int D, int block_size,
                                            int num_cache_blocks, int* status) {
  pdl_wait();
  pdl_launch();
  const int b = blockIdx.x;
  if (b >= B) return;
  const int len = seq_lens[b];
  const int pos = len > 0 ? len - 1 : 0;
  const int p = pos >= max_pos ? max_pos - 1 : pos;
  const int half = D / 2;
  __nv_bfloat16* row = qkv + (long long)b * row_pitch;
  // rotate q and k heads (pairs (i, i + D/2))
  for (int idx = threadIdx.x; idx < (Hq + Hkv) * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    const float c = cos_t[(size_t)p * half + i], s = sin_t[(size_t)p * half + i];
    __nv_bfloat16* base = row + (size_t)h * D;
    const float x1 = __bfloat162float(base[i]), x2 = __bfloat162float(base[i + half]);
    base[i] = __float2bfloat16(x1 * c - x2 * s);
    base[i + half] = __float2bfloat16(x2 * c + x1 * s);
  }
  if (len <= 0) return;
  __syncthreads();
  const int blk = block_tables[(long long)b * max_blocks + pos / block_size];
  if (blk < 0 || blk >= num_cache_blocks) {
    if (threadIdx.x == 0) report_status(status, kStatusBadIndex);
    return;
  }
  const int off = pos % block_size;
  const int per_row = Hkv * D / 8;
  for (int i = threadIdx.x; i < 2 * per_row; i += blockDim.x) {
    const bool is_v = i >= per_row;
    const int j = is_v ? i - per_row : i;
    const int h = j / (D / 8), c = j % (D / 8);
    const uint4 val = *reinterpret_cast<const uint4*>(row + (size_t)(Hq + (is_v ? Hkv : 0)) * D + (size_t)h * D + c * 8);
    __nv_bfloat16* dst = (is_v ? v_cache : k_cache) + (((long long)blk * Hkv + h) * block_size + off) * D + c * 8;
    *reinterpret_cast<uint4*>(dst) = val;
  }
}

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

__global__ void __launch_bounds__(kDecWarps * 32)
paged_decode_attn_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t dsm[];
  pdl_wait();
  pdl_launch();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq_len = p.seq_lens[b];
  const int n_blocks = (seq_len + kDecBlock - 1) / kDecBlock;
  const int blk_begin = (int)((long long)n_blocks * split / p.splits);
  const int blk_end = (int)((long long)n_blocks * (split + 1) / p.splits);
  // per-warp staging: 2 stages x (K tile 4 KB + V tile 4 KB)
  uint8_t* wbuf = dsm + warp * (2 * 2 * 4096);
  const int* table = p.block_tables + (long long)b * p.max_blocks;

  // Q fragments (A operand, rows = query heads of this kv head, zero above G), pre-scaled later in fp32.
  uint32_t qa[kDecD / 16][2];
  {
    const int g = lane >> 2;
    const __nv_bfloat16* qrow = p.q + (long long)b * p.ldq + p.q_col0 + (long long)(kvh * p.G + g) * kDecD;
#pragma unroll
    for (int kk = 0; kk < kDecD / 16; ++kk) {
      const int c = kk * 16 + (lane & 3) * 2;
      qa[kk][0] = (g < p.G) ? *reinterpret_cast<const uint32_t*>(qrow + c) : 0u;
      qa[kk][1] = (g < p.G) ? *reinterpret_cast<const uint32_t*>(qrow + c + 8) : 0u;
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
    cp_async_commit();
  };

  int my = blk_begin + warp;
  if (my < blk_end) issue_load(my, 0);
  int stage = 0;
  for (; my < blk_end; my += kDecWarps, stage ^= 1) {
    const int nxt = my + kDecWarps;
    if (nxt < blk_end) {
      issue_load(nxt, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
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
  __syncthreads();
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
  __syncthreads();
  for (int idx = threadIdx.x; idx < p.G * kDecD; idx += blockDim.x) {
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
  if (p.splits > 1 && p.tickets != nullptr) {
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      int* t = p.tickets + (long long)b * p.Hkv + kvh;
      const int ticket = atomicAdd(t, 1);
      s_last = (ticket == p.splits - 1) ? 1 : 0;
      if (s_last) *t = 0;
    }
    __syncthreads();
    if (s_last) {
      __threadfence();
      for (int idx = threadIdx.x; idx < p.G * kDecD; idx += blockDim.x) {
        const int g = idx / kDecD, d = idx % kDecD;
        const long long base0 = (((long long)b * p.Hkv + kvh) * p.splits) * 8 + g;
        float M = -INFINITY;
        for (int s = 0; s < p.splits; ++s) M = fmaxf(M, __ldcg(p.part_ml + (base0 + (long long)s * 8) * 2));
        float L = 0.f, acc = 0.f;
        for (int s = 0; s < p.splits; ++s) {
          const long long bs = base0 + (long long)s * 8;
          const float ms = __ldcg(p.part_ml + bs * 2);
          const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
          L += __ldcg(p.part_ml + bs * 2 + 1) * w;
          acc += __ldcg(p.part_o + bs * kDecD + d) * w;
        }
        p.out[(long long)b * p.ldo + (long long)(kvh * p.G + g) * kDecD + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
      }
    }
  }
}

__global__ void paged_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits,
                                            int Hkv, int G, __nv_bfloat16* __restrict__ out, long long ldo) {
  pdl_wait();
  pdl_launch();
  const int b = blockIdx.y, kvh = blockIdx.x;
  for (int idx = threadIdx.x; idx < G * kDecD; idx += blockDim.x) {
    const int g = idx / kDecD, d = idx % kDecD;
    const long long base0 = (((long long)b * Hkv + kvh) * splits) * 8 + g;
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[(base0 + (long long)s * 8) * 2]);
    float L = 0.f, acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      const long long bs = base0 + (long long)s * 8;
      const float ms = part_ml[bs * 2];
      const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
      L += part_ml[bs * 2 + 1] * w;
      acc += part_o[bs * kDecD + d] * w;
    }
    out[(long long)b * ldo + (long long)(kvh * G + g) * kDecD + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
  }
}

// ------------------------------------------------------------------------------------------------
// lm_head + sampling. The epilogue keeps, per row, the running argmax of z/temperature + Gumbel noise
// (exact sampling from softmax(z/temperature)) and online-softmax statistics for the chosen token's
// logprob. Noise comes from a counter-based hash of (row seed, vocabulary column).
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t hash_u32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352dU;
  x ^= x >> 15;
  x *= 0x846ca68bU;
  x ^= x >> 16;
  return x;
}

struct LmSampleEpilogue {
  const unsigned long long* seeds;  // [rows] per-row stream id (request seed mixed with the step)
  float inv_temp;                   // 1/temperature (1 when greedy)
  int greedy;
  float* part_best;                 // [groups, rows] best perturbed value
  int* part_idx;                    // [groups, rows]
  float* part_z;                    // [groups, rows] unperturbed scaled logit at the best index
  float* part_m;                    // [groups, rows] online softmax
  float* part_s;
  // per-thread state
  float best, best_z, m, s;
  int best_idx;
  uint32_t seed_lo, seed_hi;

  __device__ __forceinline__ void item_begin(int row, int M, int) {
    best = -INFINITY;
    best_z = 0.f;
    best_idx = 0;
    m = -INFINITY;
    s = 0.f;
    const unsigned long long sd = row < M ? seeds[row] : 0ull;
    seed_lo = (uint32_t)sd;
    seed_hi = (uint32_t)(sd >> 32);
  }
  __device__ __forceinline__ void chunk(int row, int col0, const uint32_t (&r)[32], int M, int N) {
    if (row >= M || col0 >= N) return;
    float cm = -INFINITY;
    float z[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      z[i] = (col0 + i < N) ? __uint_as_float(r[i]) * inv_temp : -INFINITY;
      cm = fmaxf(cm, z[i]);
    }
    if (cm > m) {
      s *= (m == -INFINITY) ? 0.f : __expf(m - cm);
      m = cm;
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      s += __expf(z[i] - m);
      float v = z[i];
      if (!greedy) {
        const uint32_t h = hash_u32(hash_u32((uint32_t)(col0 + i) ^ seed_lo) + seed_hi);
        const float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
        v += -__logf(-__logf(u));
      }
      if (v > best) {
        best = v;
        best_z = z[i];
        best_idx = col0 + i;
      }
    }
  }
  __device__ __forceinline__ void item_end(int row, int M, int, int group) {
    if (row >= M) return;
    const long long o = (long long)group * M + row;
    part_best[o] = best;
    part_idx[o] = best_idx;
    part_z[o] = best_z;
    part_m[o] = m;
    part_s[o] = s;
  }
};

// One warp per row: lanes stride over the column groups, then a warp reduction (argmax of the perturbed value, and
// the usual (max, sum) merge for the log-sum-exp).
__global__ void lm_sample_combine_kernel(const float* __restrict__ part_best, const int* __restrict__ part_idx,
                                         const float* __restrict__ part_z, const float* __restrict__ part_m,
                                         const float* __restrict__ part_s, int groups, int rows, int* __restrict__ tokens,
                                         float* __restrict__ logprobs) {
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  float best = -INFINITY, bz = 0.f, M = -INFINITY, S = 0.f;
  int bi = 0x7fffffff;
  for (int g = lane; g < groups; g += 32) {
    const long long o = (long long)g * rows + r;
    const float v = part_best[o];
    const int idx = part_idx[o];
    if (v > best || (v == best && idx < bi)) {
      best = v;
      bi = idx;
      bz = part_z[o];
    }
    const float m = part_m[o];
    if (m > M) {
      S = S * ((M == -INFINITY) ? 0.f : __expf(M - m)) + part_s[o];
      M = m;
    } else if (m != -INFINITY) {
      S += part_s[o] * __expf(m - M);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, off);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
    const float oz = __shfl_xor_sync(0xffffffffu, bz, off);
    if (ob > best || (ob == best && oi < bi)) {
      best = ob;
      bi = oi;
      bz = oz;
    }
    const float om = __shfl_xor_sync(0xffffffffu, M, off);
    const float os = __shfl_xor_sync(0xffffffffu, S, off);
    const float nm = fmaxf(M, om);
    const float sa = (M == -INFINITY) ? 0.f : S * __expf(M - nm);
    const float sb = (om == -INFINITY) ? 0.f : os * __expf(om - nm);
    S = sa + sb;
    M = nm;
  }
  if (lane == 0) {
    tokens[r] = bi == 0x7fffffff ? 0 : bi;
    if (logprobs != nullptr) logprobs[r] = bz - (M + logf(S));
  }
}

}  // namespace

void launch_kv_cache_write(const void* qkv, long long row_pitch, int k_col0, int v_col0, const int* slots, void* k_cache,
                           void* v_cache, int T, int Hkv, int D, int block_size, cudaStream_t s) {
  if (T == 0) return;
  AGRPO_PREFER_SMEM(kv_cache_write_kernel);
  kv_cache_write_kernel<<<T, 64, 0, s>>>((const __nv_bfloat16*)qkv, row_pitch, k_col0, v_col0, slots, (__nv_bfloat16*)k_cache,
                                         (__nv_bfloat16*)v_cache, T, Hkv, D, block_size);
  check_cuda(cudaGetLastError(), "kv_cache_write");
}

void launch_kv_cache_write_decode(const void* qkv, long long row_pitch, int k_col0, int v_col0, const int* block_tables,
                                  int max_blocks, const int* seq_lens, void* k_cache, void* v_cache, int B, int Hkv, int D,
                                  int block_size, int num_cache_blocks, int* status, cudaStream_t s) {
  if (B == 0) return;
  AGRPO_PREFER_SMEM(kv_cache_write_decode_kernel);
  kv_cache_write_decode_kernel<<<B, 64, 0, s>>>((const __nv_bfloat16*)qkv, row_pitch, k_col0, v_col0, block_tables, max_blocks,
                                                seq_lens, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, B, Hkv, D,
                                                block_size, num_cache_blocks, status);
  check_cuda(cudaGetLastError(), "kv_cache_write_decode");
}

void launch_rope_kv_write_decode(void* qkv, long long row_pitch, const float* cos_t, const float* sin_t, int max_pos,
                                 const int* block_tables, int max_blocks, const int* seq_lens, void* k_cache, void* v_cache, int B,
                                 int Hq, int Hkv, int D, int block_size, int num_cache_blocks, int* status, cudaStream_t s) {
  if (B == 0) return;
  AGRPO_PREFER_SMEM(rope_kv_write_decode_kernel);
  launch_kernel(rope_kv_write_decode_kernel, dim3(B), dim3(128), 0, s, "rope_kv_write_decode", (__nv_bfloat16*)qkv, row_pitch, cos_t,
                sin_t, max_pos, block_tables, max_blocks, seq_lens, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, B, Hq, Hkv, D,
                block_size, num_cache_blocks, status);
}

void launch_decode_step_inputs(const int* stage, int S, int* seq_lens, int* positions, int* block_tables, long long table_elems,
                               const long long* base_seeds, long long* step_seeds, int* status, cudaStream_t s) {
  if (S == 0) return;
  AGRPO_PREFER_SMEM(decode_step_inputs_kernel);
  decode_step_inputs_kernel<<<(S + 255) / 256, 256, 0, s>>>(stage, S, seq_lens, positions, block_tables, table_elems, base_seeds,
                                                            step_seeds, status);
  check_cuda(cudaGetLastError(), "decode_step_inputs");
}

void launch_paged_decode_attn(const void* q, long long ldq, int q_col0, const void* k_cache, const void* v_cache,
                              const int* block_tables, const int* seq_lens, int B, int max_blocks, int num_cache_blocks,
                              int Hq, int Hkv, int D, int block_size, float softmax_scale, int splits, void* out,
                              long long ldo, float* part_o, float* part_ml, int* status, cudaStream_t s, int* tickets) {
  if (B == 0) return;
  if (D != kDecD || block_size != kDecBlock) throw std::runtime_error("paged_decode_attn: head_dim 128 and block_size 16 only");
  const int G = Hq / Hkv;
  if (G > 8 || G * Hkv != Hq) throw std::runtime_error("paged_decode_attn: query heads per kv head must be <= 8");
  if (splits < 1) splits = 1;
  DecodeParams p;
  p.q = (const __nv_bfloat16*)q;
  p.ldq = ldq;
  p.q_col0 = q_col0;
  p.k_cache = (const __nv_bfloat16*)k_cache;
  p.v_cache = (const __nv_bfloat16*)v_cache;
  p.block_tables = block_tables;
  p.seq_lens = seq_lens;
  p.max_blocks = max_blocks;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.G = G;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.splits = splits;
  p.out = (__nv_bfloat16*)out;
  p.ldo = ldo;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.num_cache_blocks = num_cache_blocks;
  p.status = status;
  p.tickets = tickets;
  constexpr int smem = kDecWarps * 2 * 2 * 4096;  // 64 KB staging (>= merge area of 16.6 KB)
  static bool configured = false;
  if (!configured) {
    check_cuda(cudaFuncSetAttribute(paged_decode_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
               "paged_decode smem attr");
    configured = true;
  }
  dim3 grid(splits, Hkv, B);
  AGRPO_PREFER_SMEM(paged_decode_attn_kernel);
  launch_kernel(paged_decode_attn_kernel, grid, dim3(kDecWarps * 32), smem, s, "paged_decode_attn", p);
  if (splits > 1 && tickets == nullptr) {
    dim3 g2(Hkv, B);
    AGRPO_PREFER_SMEM(paged_decode_combine_kernel);
    launch_kernel(paged_decode_combine_kernel, g2, dim3(128), 0, s, "paged_decode_combine", (const float*)part_o,
                  (const float*)part_ml, splits, Hkv, G, (__nv_bfloat16*)out, ldo);
  }
}

int lm_sample_num_groups(int V, int rows) { return lmhead_num_groups(V, rows); }

void launch_lm_sample(const void* hidden, long long ldh, const void* weight, long long ldw, int rows, int H, int V,
                      float temperature, const unsigned long long* seeds, float* part_f, int* part_i, int* tokens,
                      float* logprobs, int* status, int num_sms, cudaStream_t stream) {
  if (rows == 0) return;
  const int groups = lmhead_num_groups(V, rows);
  const int tiles_n = (V + 255) / 256;
  const int group_n = (tiles_n + groups - 1) / groups;
  const CUtensorMap ta = make_tmap_2d(hidden, H, rows, ldh, 64, kGemmBM);
  const CUtensorMap tb = make_tmap_2d(weight, H, V, ldw, 64, 256);
  GemmShape p;
  p.M = rows; p.N = V; p.K = H;
  p.group_n = group_n;
  p.status = status;
  LmSampleEpilogue e;
  e.seeds = seeds;
  e.greedy = temperature <= 0.f ? 1 : 0;
  e.inv_temp = e.greedy ? 1.f : 1.f / temperature;
  const size_t n = (size_t)groups * rows;
  e.part_best = part_f;
  e.part_z = part_f + n;
  e.part_m = part_f + 2 * n;
  e.part_s = part_f + 3 * n;
  e.part_idx = part_i;
  e.best = 0.f; e.best_z = 0.f; e.m = 0.f; e.s = 0.f; e.best_idx = 0; e.seed_lo = 0; e.seed_hi = 0;
  gemm_launch<256, false, false>(ta, tb, p, e, num_sms, stream);
  AGRPO_PREFER_SMEM(lm_sample_combine_kernel);
  launch_kernel(lm_sample_combine_kernel, dim3((rows + 3) / 4), dim3(128), 0, stream, "lm_sample_combine", (const float*)e.part_best,
                (const int*)e.part_idx, (const float*)e.part_z, (const float*)e.part_m, (const float*)e.part_s, groups, rows, tokens,
                logprobs);
}

}  // namespace agrpo
