// Flat-buffer optimizer kernels: sum of squares of the fp32 gradient shard, and AdamW on fp32 master
// weights that also writes the bf16 compute copy. The clip coefficient is derived on the device from
// the squared-norm word, so the step needs no host synchronisation. This is the single-rank case of
// the reference's clip_grad_norm_ + AdamW step (gpu_process_worker.py:1052-1079).
#include <cuda_bf16.h>

#include "../launchers.h"

namespace agrpo {

namespace {

__global__ void sumsq_kernel(const float* __restrict__ g, long long n, float scale, float* __restrict__ out) {
  float acc = 0.f;
  const long long n4 = n / 4;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = g4[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  for (long long i = n4 * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    acc += g[i] * g[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float sm[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sm[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    acc = lane < (blockDim.x >> 5) ? sm[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) atomicAdd(out, acc * scale * scale);
  }
}

// norm_sq points at the squared global gradient norm (already scaled by grad_scale^2).
// clip coefficient = min(1, max_norm / (sqrt(norm_sq) + 1e-6)); max_norm <= 0 disables clipping.
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             float* __restrict__ g, __nv_bfloat16* __restrict__ p16, long long n, float lr, float beta1,
                             float beta2, float eps, float wd, float bc1, float bc2, float grad_scale,
                             const float* __restrict__ norm_sq, float max_norm, int zero_grad) {
  float coef = grad_scale;
  if (max_norm > 0.f && norm_sq != nullptr) {
    const float nrm = sqrtf(*norm_sq);
    coef *= fminf(1.f, max_norm / (nrm + 1e-6f));
  }
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gi = g[i] * coef;
    float pi = p[i];
    float mi = m[i], vi = v[i];
    pi *= (1.f - lr * wd);
    mi = beta1 * mi + (1.f - beta1) * gi;
    vi = beta2 * vi + (1.f - beta2) * gi * gi;
    const float denom = sqrtf(vi) * inv_sqrt_bc2 + eps;
    pi -= lr * inv_bc1 * mi / denom;
    p[i] = pi;
    m[i] = mi;
    v[i] = vi;
    if (p16 != nullptr) p16[i] = __float2bfloat16(pi);
    if (zero_grad) g[i] = 0.f;
  }
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16(in[i]);
}

}  // namespace

void launch_sumsq(const float* g, long long n, float scale, float* out, cudaStream_t s) {
  if (n == 0) return;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  sumsq_kernel<<<(int)blocks, 256, 0, s>>>(g, n, scale, out);
  check_cuda(cudaGetLastError(), "sumsq");
}

void launch_adamw(float* p, float* m, float* v, float* g, void* p16, long long n, float lr, float beta1, float beta2,
                  float eps, float wd, int step, float grad_scale, const float* norm_sq, float max_norm, bool zero_grad,
                  cudaStream_t s) {
  if (n == 0) return;
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2 = 1.f - powf(beta2, (float)step);
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  adamw_kernel<<<(int)blocks, 256, 0, s>>>(p, m, v, g, (__nv_bfloat16*)p16, n, lr, beta1, beta2, eps, wd, bc1, bc2,
                                           grad_scale, norm_sq, max_norm, zero_grad ? 1 : 0);
  check_cuda(cudaGetLastError(), "adamw");
}

void launch_cast_f32_bf16(const float* in, void* out, long long n, cudaStream_t s) {
  if (n == 0) return;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cast_f32_bf16_kernel<<<(int)blocks, 256, 0, s>>>(in, (__nv_bfloat16*)out, n);
  check_cuda(cudaGetLastError(), "cast_f32_bf16");
}

}  // namespace agrpo
