// Rollout-engine kernels: paged KV-cache write, paged-KV decode attention with native GQA and split-KV,
// and the fused lm_head + sampling epilogue (Gumbel-max over logits that never leave tensor memory).
// Together with the prefill path (the varlen attention kernel) they stand in for the vLLM engine the
// reference drives (vllm_worker.py:203-284, 709-737).
#include <cuda_bf16.h>

#include "../common/tensormap.h"
#include "../launchers.h"
#include "decode_attn.cuh"
#include "gemm_tcgen05.cuh"

namespace agrpo {

namespace {

// ------------------------------------------------------------------------------------------------
// KV-cache write. Cache layout per layer: [num_blocks, Hkv, block_size, D] for K and for V.
// slot[t] = block * block_size + offset, negative = skip the token.
// ------------------------------------------------------------------------------------------------
__global__ void kv_cache_write_kernel(const __nv_bfloat16* __restrict__ qkv, long long row_pitch, int k_col0, int v_col0,
                                      const int* __restrict__ slots, __nv_bfloat16* __restrict__ k_cache,
                                      __nv_bfloat16* __restrict__ v_cache, int T, int Hkv, int D, int block_size,
                                      long long num_slots, int* status) {
  const int t = blockIdx.x;
  if (t >= T) return;
  const int slot = slots[t];
  if (slot < 0) return;
  if (slot >= num_slots) {  // beyond the cache: record it and skip the write
    if (threadIdx.x == 0) report_status(status, kStatusBadIndex);
    return;
  }
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

__global__ void __launch_bounds__(kDecWarps * 32)
paged_decode_attn_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t dsm[];
  __shared__ int s_last;
  pdl_wait();
  pdl_launch();
  paged_decode_attend<2>(p, blockIdx.x, blockIdx.y, blockIdx.z, dsm, threadIdx.x >> 5, threadIdx.x, &s_last);
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

// One CTA (4 warps) per row: threads stride over the column groups (a handful of iterations even for a 150k vocabulary,
// every load of an iteration in flight before the first use), then a warp reduction and a 4-way merge through shared
// memory (argmax of the perturbed value with ties to the lower index, and the usual (max, sum) merge for the
// log-sum-exp). This kernel sits on the critical path of every decode step.
__global__ void __launch_bounds__(128)
lm_sample_combine_kernel(const float* __restrict__ part_best, const int* __restrict__ part_idx,
                         const float* __restrict__ part_z, const float* __restrict__ part_m,
                         const float* __restrict__ part_s, int groups, int rows, int* __restrict__ tokens,
                         float* __restrict__ logprobs) {
  pdl_wait();
  pdl_launch();
  __shared__ float s_best[4], s_bz[4], s_m[4], s_s[4];
  __shared__ int s_bi[4];
  const int r = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float best = -INFINITY, bz = 0.f, M = -INFINITY, S = 0.f;
  int bi = 0x7fffffff;
  for (int g = threadIdx.x; g < groups; g += 128) {
    const long long o = (long long)g * rows + r;
    const float v = part_best[o];
    const int idx = part_idx[o];
    const float z = part_z[o];
    const float m = part_m[o];
    const float sv = part_s[o];
    if (v > best || (v == best && idx < bi)) {
      best = v;
      bi = idx;
      bz = z;
    }
    if (m > M) {
      S = S * ((M == -INFINITY) ? 0.f : __expf(M - m)) + sv;
      M = m;
    } else if (m != -INFINITY) {
      S += sv * __expf(m - M);
    }
  }
  auto merge = [&](float ob, int oi, float oz, float om, float os) {
    if (ob > best || (ob == best && oi < bi)) {
      best = ob;
      bi = oi;
      bz = oz;
    }
    const float nm = fmaxf(M, om);
    const float sa = (M == -INFINITY) ? 0.f : S * __expf(M - nm);
    const float sb = (om == -INFINITY) ? 0.f : os * __expf(om - nm);
    S = sa + sb;
    M = nm;
  };
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, off);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
    const float oz = __shfl_xor_sync(0xffffffffu, bz, off);
    const float om = __shfl_xor_sync(0xffffffffu, M, off);
    const float os = __shfl_xor_sync(0xffffffffu, S, off);
    merge(ob, oi, oz, om, os);
  }
  if (lane == 0) {
    s_best[warp] = best;
    s_bi[warp] = bi;
    s_bz[warp] = bz;
    s_m[warp] = M;
    s_s[warp] = S;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 4; ++w) merge(s_best[w], s_bi[w], s_bz[w], s_m[w], s_s[w]);
    tokens[r] = bi == 0x7fffffff ? 0 : bi;
    if (logprobs != nullptr) logprobs[r] = bz - (M + logf(S));
  }
}

}  // namespace

void launch_kv_cache_write(const void* qkv, long long row_pitch, int k_col0, int v_col0, const int* slots, void* k_cache,
                           void* v_cache, int T, int Hkv, int D, int block_size, int num_cache_blocks, int* status,
                           cudaStream_t s) {
  if (T == 0) return;
  AGRPO_PREFER_SMEM(kv_cache_write_kernel);
  kv_cache_write_kernel<<<T, 64, 0, s>>>((const __nv_bfloat16*)qkv, row_pitch, k_col0, v_col0, slots, (__nv_bfloat16*)k_cache,
                                         (__nv_bfloat16*)v_cache, T, Hkv, D, block_size,
                                         (long long)num_cache_blocks * block_size, status);
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
  AGRPO_SET_MAX_DYN_SMEM(paged_decode_attn_kernel, smem, "paged_decode smem attr");
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
  launch_kernel(lm_sample_combine_kernel, dim3(rows), dim3(128), 0, stream, "lm_sample_combine", (const float*)e.part_best,
                (const int*)e.part_idx, (const float*)e.part_z, (const float*)e.part_m, (const float*)e.part_s, groups, rows, tokens,
                logprobs);
}

}  // namespace agrpo
