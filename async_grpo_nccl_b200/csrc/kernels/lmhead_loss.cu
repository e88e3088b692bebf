// Fused lm_head + log-softmax + entropy + GRPO dual-clip / KL objective.
//
// The reference materialises [T, V] logits per time-chunk (grpo_loss.py:286-313), runs gather -
// logsumexp and a separate entropy pass over them (grpo_loss.py:146-208), and forms the clipped-ratio
// objective with ATen elementwise ops and about fifteen host syncs for diagnostics
// (grpo_loss.py:323-346, 410-483). Here:
//   forward : one tcgen05 GEMM whose epilogue keeps online-softmax statistics per row (max, sum exp,
//             sum exp*z, label logit); logits never leave tensor memory. A combine kernel turns the
//             per-column-group partials into logprob / entropy / lse per token.
//   loss    : one elementwise kernel computes the per-token objective, d loss / d logprob and a small
//             statistics vector (read by the host once per microbatch).
//   backward: per vocabulary chunk, the GEMM is recomputed with an epilogue that writes
//             dlogits = g * (onehot - softmax) / temperature as bf16 into a chunk buffer, which feeds the
//             dH and dW tcgen05 GEMMs.
#include <cuda_bf16.h>

#include "../common/tensormap.h"
#include "../launchers.h"
#include "gemm_tcgen05.cuh"

namespace agrpo {

namespace {

constexpr int kLmBN = 256;

struct LmStatsEpilogue {
  const int* labels;   // [T] target token per row, < 0 = masked
  float inv_temp;
  float* part_m;       // [groups, T]
  float* part_s;
  float* part_sz;
  float* label_logit;  // [T]
  // per-thread running state
  float m, s, sz;
  int label;

  __device__ __forceinline__ void item_begin(int row, int M, int) {
    m = -INFINITY;
    s = 0.f;
    sz = 0.f;
    label = row < M ? labels[row] : -1;
  }
  __device__ __forceinline__ void chunk(int row, int col0, const uint32_t (&r)[32], int M, int N) {
    if (row >= M || col0 >= N) return;
    float z[32];
    float cm = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      z[i] = (col0 + i < N) ? __uint_as_float(r[i]) * inv_temp : -INFINITY;
      cm = fmaxf(cm, z[i]);
    }
    if (cm > m) {
      const float sc = (m == -INFINITY) ? 0.f : __expf(m - cm);
      s *= sc;
      sz *= sc;
      m = cm;
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float e = __expf(z[i] - m);
      s += e;
      sz += (z[i] == -INFINITY) ? 0.f : e * z[i];
    }
    if (label >= col0 && label < col0 + 32) {
      float zl = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i == label) zl = z[i];
      label_logit[row] = zl;
    }
  }
  __device__ __forceinline__ void item_end(int row, int M, int, int group) {
    if (row >= M) return;
    const long long o = (long long)group * M + row;
    part_m[o] = m;
    part_s[o] = s;
    part_sz[o] = sz;
  }
};

struct LmDlogitsEpilogue {
  const int* labels;
  const float* lse;    // [T]
  const float* g;      // [T] d loss / d logprob
  float inv_temp;
  int v0;              // first vocabulary column of this chunk
  __nv_bfloat16* dz;   // [T, ld]
  long long ld;
  float lse_r, g_r;
  int label;

  __device__ __forceinline__ void item_begin(int row, int M, int) {
    const bool ok = row < M;
    lse_r = ok ? lse[row] : 0.f;
    g_r = ok ? g[row] : 0.f;
    label = ok ? labels[row] - v0 : -1;
  }
  __device__ __forceinline__ void item_end(int, int, int, int) {}
  __device__ __forceinline__ void chunk(int row, int col0, const uint32_t (&r)[32], int M, int N) {
    if (row >= M || col0 >= N) return;
    float d[32];
    const float gs = g_r * inv_temp;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float p = __expf(__uint_as_float(r[i]) * inv_temp - lse_r);
      d[i] = gs * (((col0 + i == label) ? 1.f : 0.f) - p);
    }
    __nv_bfloat16* dst = dz + (long long)row * ld + col0;
    if (col0 + 32 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 o;
        o.x = pack_bf16x2(d[i], d[i + 1]);
        o.y = pack_bf16x2(d[i + 2], d[i + 3]);
        o.z = pack_bf16x2(d[i + 4], d[i + 5]);
        o.w = pack_bf16x2(d[i + 6], d[i + 7]);
        *reinterpret_cast<uint4*>(dst + i) = o;
      }
    } else {
      for (int i = 0; i < 32; ++i)
        if (col0 + i < N) dst[i] = __float2bfloat16(d[i]);
    }
  }
};

__global__ void lmhead_combine_kernel(const float* __restrict__ part_m, const float* __restrict__ part_s,
                                      const float* __restrict__ part_sz, const float* __restrict__ label_logit,
                                      const int* __restrict__ labels, int groups, int T, float* __restrict__ logp,
                                      float* __restrict__ entropy, float* __restrict__ lse_out) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float M = -INFINITY;
  for (int g = 0; g < groups; ++g) M = fmaxf(M, part_m[(long long)g * T + t]);
  float S = 0.f, SZ = 0.f;
  for (int g = 0; g < groups; ++g) {
    const float w = __expf(part_m[(long long)g * T + t] - M);
    S += part_s[(long long)g * T + t] * w;
    SZ += part_sz[(long long)g * T + t] * w;
  }
  const float lse = M + logf(S);
  if (lse_out != nullptr) lse_out[t] = lse;
  const bool valid = labels[t] >= 0;
  if (logp != nullptr) logp[t] = valid ? label_logit[t] - lse : 0.f;
  if (entropy != nullptr) entropy[t] = lse - SZ / S;
}

// Slots of the statistics vector (sums over valid tokens; the host divides).
enum LossStat : int {
  kStatCount = 0, kStatLossSum, kStatAbsLogRatio, kStatApproxKl, kStatClipUpper, kStatClipLower, kStatLogRatio,
  kStatLogRatioSq, kStatEntropy, kStatAdv, kStatAdvSq, kStatAdvPos, kStatAdvZero, kStatPgClip, kStatOldEntropy,
  kStatKlRef, kStatLogp, kStatDualClip, kNumLossStats
};

__global__ void grpo_token_loss_kernel(const float* __restrict__ logp, const float* __restrict__ old_logp,
                                       const float* __restrict__ ref_logp, const float* __restrict__ adv,
                                       const int* __restrict__ labels, const float* __restrict__ entropy,
                                       const float* __restrict__ old_entropy, int T, float clip_low, float clip_high,
                                       float clip_c, float kl_beta, float grad_weight, float* __restrict__ dlogp,
                                       float* __restrict__ stats) {
  float acc[kNumLossStats];
#pragma unroll
  for (int i = 0; i < kNumLossStats; ++i) acc[i] = 0.f;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < T; t += gridDim.x * blockDim.x) {
    float g = 0.f;
    if (labels[t] >= 0) {
      const float lp = logp[t];
      const float lo = old_logp != nullptr ? old_logp[t] : lp;
      const float a = adv[t];
      const float lr = lp - lo;
      const float ratio = __expf(lr);
      const float lower = 1.f - clip_low, upper = 1.f + clip_high;
      const float unclipped = -a * ratio;
      const float clamped = fminf(fmaxf(ratio, lower), upper);
      const float clipped = -a * clamped;
      const bool use_unclipped = unclipped >= clipped;
      const float clip1 = use_unclipped ? unclipped : clipped;
      const float dual = -a * clip_c;
      float loss = clip1;
      bool dual_active = false;
      if (a < 0.f && dual < clip1) {
        loss = dual;
        dual_active = true;
      }
      // d loss / d logprob: -a * ratio where the ratio term is live, 0 where a clamp is active.
      if (!dual_active) {
        if (use_unclipped) g = -a * ratio;
        else g = (ratio > lower && ratio < upper) ? -a * ratio : 0.f;
      }
      float klr = 0.f;
      if (kl_beta > 0.f && ref_logp != nullptr) {
        const float d = ref_logp[t] - lp;
        const float e = __expf(d);
        klr = e - d - 1.f;
        loss += kl_beta * klr;
        g += kl_beta * (1.f - e);
      }
      g *= grad_weight;
      acc[kStatCount] += 1.f;
      acc[kStatLossSum] += loss;
      acc[kStatAbsLogRatio] += fabsf(lr);
      acc[kStatApproxKl] += ratio - 1.f - lr;
      acc[kStatClipUpper] += ratio > upper ? 1.f : 0.f;
      acc[kStatClipLower] += ratio < lower ? 1.f : 0.f;
      acc[kStatLogRatio] += lr;
      acc[kStatLogRatioSq] += lr * lr;
      acc[kStatEntropy] += entropy != nullptr ? entropy[t] : 0.f;
      acc[kStatAdv] += a;
      acc[kStatAdvSq] += a * a;
      acc[kStatAdvPos] += a > 0.f ? 1.f : 0.f;
      acc[kStatAdvZero] += a == 0.f ? 1.f : 0.f;
      acc[kStatPgClip] += clipped > unclipped ? 1.f : 0.f;
      acc[kStatOldEntropy] += old_entropy != nullptr ? old_entropy[t] : 0.f;
      acc[kStatKlRef] += klr;
      acc[kStatLogp] += lp;
      acc[kStatDualClip] += dual_active ? 1.f : 0.f;
    }
    if (dlogp != nullptr) dlogp[t] = g;
  }
  __shared__ float sm[kNumLossStats][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < kNumLossStats; ++i) {
    float v = acc[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) sm[i][warp] = v;
  }
  __syncthreads();
  if (threadIdx.x < kNumLossStats) {
    float v = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) v += sm[threadIdx.x][w];
    if (v != 0.f) atomicAdd(stats + threadIdx.x, v);
  }
}

}  // namespace

int lmhead_num_groups(int V, int T) {
  const int tiles_n = (V + kLmBN - 1) / kLmBN;
  const int tiles_m = (T + kGemmBM - 1) / kGemmBM;
  // Aim for at least ~4 work items per SM; at most 16 column-tiles share one set of partials.
  int group_n = 16;
  while (group_n > 1 && (long long)tiles_m * ((tiles_n + group_n - 1) / group_n) < 148 * 4) group_n >>= 1;
  return (tiles_n + group_n - 1) / group_n;
}
static int lmhead_group_n(int V, int T) {
  const int tiles_n = (V + kLmBN - 1) / kLmBN;
  const int groups = lmhead_num_groups(V, T);
  return (tiles_n + groups - 1) / groups;
}

void launch_lmhead_logprob(const void* hidden, long long ldh, const void* weight, long long ldw, const int* labels, int T,
                           int H, int V, float temperature, float* partials, float* label_logit, float* logp,
                           float* entropy, float* lse, int* status, int num_sms, cudaStream_t stream) {
  if (T == 0) return;
  const int group_n = lmhead_group_n(V, T);
  const int tiles_n = (V + kLmBN - 1) / kLmBN;
  const int groups = (tiles_n + group_n - 1) / group_n;
  const CUtensorMap ta = make_tmap_2d(hidden, H, T, ldh, 64, kGemmBM);
  const CUtensorMap tb = make_tmap_2d(weight, H, V, ldw, 64, kLmBN);
  GemmShape p;
  p.M = T; p.N = V; p.K = H;
  p.group_n = group_n;
  p.status = status;
  LmStatsEpilogue e;
  e.labels = labels;
  e.inv_temp = 1.f / temperature;
  e.part_m = partials;
  e.part_s = partials + (size_t)groups * T;
  e.part_sz = partials + 2 * (size_t)groups * T;
  e.label_logit = label_logit;
  e.m = 0.f; e.s = 0.f; e.sz = 0.f; e.label = -1;
  gemm_launch<kLmBN, false, false>(ta, tb, p, e, num_sms, stream);
  lmhead_combine_kernel<<<(T + 255) / 256, 256, 0, stream>>>(e.part_m, e.part_s, e.part_sz, label_logit, labels, groups, T,
                                                            logp, entropy, lse);
  check_cuda(cudaGetLastError(), "lmhead_combine");
}

void launch_grpo_token_loss(const float* logp, const float* old_logp, const float* ref_logp, const float* adv,
                            const int* labels, const float* entropy, const float* old_entropy, int T, float clip_low,
                            float clip_high, float clip_c, float kl_beta, float grad_weight, float* dlogp, float* stats,
                            cudaStream_t stream) {
  if (T == 0) return;
  int blocks = (T + 255) / 256;
  if (blocks > 148 * 2) blocks = 148 * 2;
  grpo_token_loss_kernel<<<blocks, 256, 0, stream>>>(logp, old_logp, ref_logp, adv, labels, entropy, old_entropy, T, clip_low,
                                                     clip_high, clip_c, kl_beta, grad_weight, dlogp, stats);
  check_cuda(cudaGetLastError(), "grpo_token_loss");
}

int grpo_num_loss_stats() { return kNumLossStats; }

void launch_lmhead_backward(const void* hidden, long long ldh, const void* weight, long long ldw, const int* labels,
                            const float* lse, const float* dlogp, int T, int H, int V, float temperature, void* dz_chunk,
                            int chunk_cols, float* dh_acc, float* dweight, long long ld_dw, int* status, int num_sms,
                            cudaStream_t stream) {
  if (T == 0) return;
  const CUtensorMap ta = make_tmap_2d(hidden, H, T, ldh, 64, kGemmBM);
  for (int v0 = 0, ci = 0; v0 < V; v0 += chunk_cols, ++ci) {
    const int vc = (V - v0) < chunk_cols ? (V - v0) : chunk_cols;
    const __nv_bfloat16* wc = reinterpret_cast<const __nv_bfloat16*>(weight) + (long long)v0 * ldw;
    // 1. dlogits chunk [T, vc] (recompute logits tile on tcgen05, transform in the epilogue)
    {
      const CUtensorMap tb = make_tmap_2d(wc, H, vc, ldw, 64, kLmBN);
      GemmShape p;
      p.M = T; p.N = vc; p.K = H;
      p.group_n = 1;
      p.status = status;
      LmDlogitsEpilogue e;
      e.labels = labels;
      e.lse = lse;
      e.g = dlogp;
      e.inv_temp = 1.f / temperature;
      e.v0 = v0;
      e.dz = reinterpret_cast<__nv_bfloat16*>(dz_chunk);
      e.ld = chunk_cols;
      e.lse_r = 0.f; e.g_r = 0.f; e.label = -1;
      gemm_launch<kLmBN, false, false>(ta, tb, p, e, num_sms, stream);
    }
    // 2. dH += dZ . W_chunk        (A = dZ [T, vc] K-major, B = W_chunk as [N = H, K = vc], MN-major)
    launch_gemm_bf16(dz_chunk, chunk_cols, wc, ldw, dh_acc, H, T, H, vc, false, true, nullptr, 1.f, true, ci > 0, status,
                     num_sms, stream);
    // 3. dW_chunk += dZ^T . hidden (A = dZ as [M = vc, K = T] MN-major, B = hidden as [N = H, K = T], MN-major)
    if (dweight != nullptr)
      launch_gemm_bf16(dz_chunk, chunk_cols, hidden, ldh, dweight + (long long)v0 * ld_dw, ld_dw, vc, H, T, true, true,
                       nullptr, 1.f, true, true, status, num_sms, stream);
  }
}

}  // namespace agrpo
