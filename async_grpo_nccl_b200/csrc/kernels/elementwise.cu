// Bandwidth-bound decoder ops: embedding gather / scatter-add, RMSNorm fwd / bwd, RoPE (in place on the
// fused qkv buffer), SwiGLU fwd / bwd, column sums (bias and norm-weight gradients).
// They replace the HF Qwen2 modules the reference runs through transformers (grpo_loss.py:77-89).
// All activations are bf16 with fp32 math; 16-byte vector accesses; rows are processed by one warp.
#include <cuda_bf16.h>

#include "../common/ptx.cuh"
#include "../launchers.h"

namespace agrpo {

namespace {

struct alignas(16) Bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------------------------------------
// Embedding
// ------------------------------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, int T, int H, int V) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T) return;
  const int lane = threadIdx.x & 31;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const Bf16x8* src = reinterpret_cast<const Bf16x8*>(table + (size_t)id * H);
  Bf16x8* dst = reinterpret_cast<Bf16x8*>(out + (size_t)row * H);
  for (int i = lane; i < H / 8; i += 32) dst[i] = src[i];
}

// Decode-step variant: besides the lookup it writes the row's sum of squares to ss[0][row] and clears ss[1..n_ss)[row],
// the per-layer statistics that the folded-norm GEMMs of the step accumulate into (ss is [n_ss, ss_stride] fp32).
__global__ void embedding_sumsq_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                       __nv_bfloat16* __restrict__ out, sumsq_t* __restrict__ ss, int n_ss, int ss_stride, int T,
                                       int H, int V) {
  pdl_wait();
  pdl_launch();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T) return;
  const int lane = threadIdx.x & 31;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const Bf16x8* src = reinterpret_cast<const Bf16x8*>(table + (size_t)id * H);
  Bf16x8* dst = reinterpret_cast<Bf16x8*>(out + (size_t)row * H);
  float acc = 0.f;
  for (int i = lane; i < H / 8; i += 32) {
    const Bf16x8 v = src[i];
    dst[i] = v;
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      acc += f.x * f.x + f.y * f.y;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) ss[row] = sumsq_to_fixed(acc);
  for (int k = 1 + lane; k < n_ss; k += 32) ss[(size_t)k * ss_stride + row] = 0;
}

// out[n, k] = w[n, k] * g[k]: an RMSNorm weight folded into the columns of the matrix that consumes the normalised rows.
__global__ void fold_norm_weight_kernel(const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ g,
                                        __nv_bfloat16* __restrict__ out, long long n_rows, int K) {
  const long long total = n_rows * (long long)(K / 8);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int kc = (int)(i % (K / 8));
    const Bf16x8 a = reinterpret_cast<const Bf16x8*>(w)[i];
    const Bf16x8 b = reinterpret_cast<const Bf16x8*>(g)[kc];
    const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
    Bf16x8 o;
    __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 fa = __bfloat1622float2(ha[j]), fb = __bfloat1622float2(hb[j]);
      ho[j] = __floats2bfloat162_rn(fa.x * fb.x, fa.y * fb.y);
    }
    reinterpret_cast<Bf16x8*>(out)[i] = o;
  }
}

__global__ void embedding_bwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dtable, int T, int H, int V) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T) return;
  const int lane = threadIdx.x & 31;
  int id = ids[row];
  if (id < 0 || id >= V) return;
  const __nv_bfloat162* src = reinterpret_cast<const __nv_bfloat162*>(dout + (size_t)row * H);
  float* dst = dtable + (size_t)id * H;
  for (int i = lane; i < H / 2; i += 32) {
    const float2 f = __bfloat1622float2(src[i]);
    atomicAdd(dst + 2 * i, f.x);
    atomicAdd(dst + 2 * i + 1, f.y);
  }
}

// ------------------------------------------------------------------------------------------------
// RMSNorm: y = x * rstd * w, rstd = rsqrt(mean(x^2) + eps)
// ------------------------------------------------------------------------------------------------
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int T, int H,
                                   float eps) {
  pdl_wait();
  pdl_launch();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T) return;
  const int lane = threadIdx.x & 31;
  const Bf16x8* xr = reinterpret_cast<const Bf16x8*>(x + (size_t)row * H);
  const Bf16x8* wr = reinterpret_cast<const Bf16x8*>(w);
  Bf16x8* yr = reinterpret_cast<Bf16x8*>(y + (size_t)row * H);
  float ss = 0.f;
  for (int i = lane; i < H / 8; i += 32) {
    const Bf16x8 a = xr[i];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(a.v[j]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)H + eps);
  if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
  for (int i = lane; i < H / 8; i += 32) {
    const Bf16x8 a = xr[i];
    const Bf16x8 g = wr[i];
    Bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(a.v[j]);
      const float2 gw = __bfloat1622float2(g.v[j]);
      o.v[j] = __floats2bfloat162_rn(f.x * rstd * gw.x, f.y * rstd * gw.y);
    }
    yr[i] = o;
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)), xhat = x*rstd. If accumulate != 0, dx += result.
__global__ void rmsnorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                      const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                                      __nv_bfloat16* __restrict__ dx, int T, int H, int accumulate) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T) return;
  const int lane = threadIdx.x & 31;
  const Bf16x8* xr = reinterpret_cast<const Bf16x8*>(x + (size_t)row * H);
  const Bf16x8* dyr = reinterpret_cast<const Bf16x8*>(dy + (size_t)row * H);
  const Bf16x8* wr = reinterpret_cast<const Bf16x8*>(w);
  Bf16x8* dxr = reinterpret_cast<Bf16x8*>(dx + (size_t)row * H);
  const float rstd = rstd_in[row];
  float dot = 0.f;
  for (int i = lane; i < H / 8; i += 32) {
    const Bf16x8 a = xr[i], d = dyr[i], g = wr[i];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(a.v[j]);
      const float2 df = __bfloat1622float2(d.v[j]);
      const float2 gw = __bfloat1622float2(g.v[j]);
      dot += df.x * gw.x * f.x + df.y * gw.y * f.y;
    }
  }
  dot = warp_sum(dot) * rstd / (float)H;  // mean(dy*w*xhat)
  for (int i = lane; i < H / 8; i += 32) {
    const Bf16x8 a = xr[i], d = dyr[i], g = wr[i];
    Bf16x8 o;
    Bf16x8 old;
    if (accumulate) old = dxr[i];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(a.v[j]);
      const float2 df = __bfloat1622float2(d.v[j]);
      const float2 gw = __bfloat1622float2(g.v[j]);
      float rx = rstd * (df.x * gw.x - f.x * rstd * dot);
      float ry = rstd * (df.y * gw.y - f.y * rstd * dot);
      if (accumulate) {
        const float2 of = __bfloat1622float2(old.v[j]);
        rx += of.x;
        ry += of.y;
      }
      o.v[j] = __floats2bfloat162_rn(rx, ry);
    }
    dxr[i] = o;
  }
}

// out[c] += sum_r a[r,c] * (b ? b[r,c] : 1) * (rscale ? rscale[r] : 1); out is fp32 (atomic adds).
// Block = 32 x 8 threads: a lane owns two adjacent columns, warps stride over the block's rows.
__global__ void colsum_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                              const float* __restrict__ rscale, float* __restrict__ out, int T, int C, long long lda,
                              int rows_per_block) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 64 + lane * 2;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(T, r0 + rows_per_block);
  float s0 = 0.f, s1 = 0.f;
  if (c < C) {
    for (int r = r0 + warp; r < r1; r += 8) {
      float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a + (size_t)r * lda + c));
      if (b != nullptr) {
        const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(b + (size_t)r * lda + c));
        f.x *= g.x;
        f.y *= g.y;
      }
      if (rscale != nullptr) {
        const float s = rscale[r];
        f.x *= s;
        f.y *= s;
      }
      s0 += f.x;
      s1 += f.y;
    }
  }
  __shared__ float sm[8][64];
  sm[warp][lane * 2] = s0;
  sm[warp][lane * 2 + 1] = s1;
  __syncthreads();
  if (warp == 0) {
    float t0 = 0.f, t1 = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      t0 += sm[k][lane * 2];
      t1 += sm[k][lane * 2 + 1];
    }
    if (c < C) atomicAdd(out + c, t0);
    if (c + 1 < C) atomicAdd(out + c + 1, t1);
  }
}

// ------------------------------------------------------------------------------------------------
// RoPE (rotate-half convention) applied in place to the q and k heads of a fused qkv row.
// cos/sin tables are fp32 [max_pos, D/2]. sign = +1 forward, -1 backward (transpose rotation).
// ------------------------------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t, int T, int n_rot_heads,
                            int D, long long row_pitch, int max_pos, float sign) {
  const int half = D / 2;
  const long long total = (long long)T * n_rot_heads * half;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int i = (int)(idx % half);
    const long long th = idx / half;
    const int h = (int)(th % n_rot_heads);
    const int t = (int)(th / n_rot_heads);
    int p = pos[t];
    p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
    const float c = cos_t[(size_t)p * half + i];
    const float s = sin_t[(size_t)p * half + i] * sign;
    __nv_bfloat16* base = qkv + (size_t)t * row_pitch + (size_t)h * D;
    const float x1 = __bfloat162float(base[i]);
    const float x2 = __bfloat162float(base[i + half]);
    base[i] = __float2bfloat16(x1 * c - x2 * s);
    base[i + half] = __float2bfloat16(x2 * c + x1 * s);
  }
}

// ------------------------------------------------------------------------------------------------
// SwiGLU on a fused [T, 2F] gate|up buffer.
// ------------------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int T, int F) {
  const long long total = (long long)T * (F / 8);
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / (F / 8);
    const int c = (int)(idx % (F / 8));
    const Bf16x8 g = reinterpret_cast<const Bf16x8*>(gu + (size_t)t * 2 * F)[c];
    const Bf16x8 u = reinterpret_cast<const Bf16x8*>(gu + (size_t)t * 2 * F + F)[c];
    Bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 gf = __bfloat1622float2(g.v[j]);
      const float2 uf = __bfloat1622float2(u.v[j]);
      const float a0 = gf.x / (1.f + __expf(-gf.x));
      const float a1 = gf.y / (1.f + __expf(-gf.y));
      o.v[j] = __floats2bfloat162_rn(a0 * uf.x, a1 * uf.y);
    }
    reinterpret_cast<Bf16x8*>(out + (size_t)t * F)[c] = o;
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ dgu, int T, int F) {
  const long long total = (long long)T * (F / 8);
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / (F / 8);
    const int c = (int)(idx % (F / 8));
    const Bf16x8 g = reinterpret_cast<const Bf16x8*>(gu + (size_t)t * 2 * F)[c];
    const Bf16x8 u = reinterpret_cast<const Bf16x8*>(gu + (size_t)t * 2 * F + F)[c];
    const Bf16x8 d = reinterpret_cast<const Bf16x8*>(dout + (size_t)t * F)[c];
    Bf16x8 dg, du;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 gf = __bfloat1622float2(g.v[j]);
      const float2 uf = __bfloat1622float2(u.v[j]);
      const float2 df = __bfloat1622float2(d.v[j]);
      const float s0 = 1.f / (1.f + __expf(-gf.x));
      const float s1 = 1.f / (1.f + __expf(-gf.y));
      const float dg0 = df.x * uf.x * s0 * (1.f + gf.x * (1.f - s0));
      const float dg1 = df.y * uf.y * s1 * (1.f + gf.y * (1.f - s1));
      dg.v[j] = __floats2bfloat162_rn(dg0, dg1);
      du.v[j] = __floats2bfloat162_rn(df.x * gf.x * s0, df.y * gf.y * s1);
    }
    reinterpret_cast<Bf16x8*>(dgu + (size_t)t * 2 * F)[c] = dg;
    reinterpret_cast<Bf16x8*>(dgu + (size_t)t * 2 * F + F)[c] = du;
  }
}

// out = a + b (bf16), used for residual joins that are not folded into a GEMM epilogue.
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ out, long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const Bf16x8 x = reinterpret_cast<const Bf16x8*>(a)[i];
    const Bf16x8 y = reinterpret_cast<const Bf16x8*>(b)[i];
    Bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 xf = __bfloat1622float2(x.v[j]);
      const float2 yf = __bfloat1622float2(y.v[j]);
      o.v[j] = __floats2bfloat162_rn(xf.x + yf.x, xf.y + yf.y);
    }
    reinterpret_cast<Bf16x8*>(out)[i] = o;
  }
}

inline int grid_for(long long work, int block, int cap = 148 * 16) {
  long long g = (work + block - 1) / block;
  if (g < 1) g = 1;
  return (int)(g > cap ? cap : g);
}

}  // namespace

void launch_embedding_fwd(const int* ids, const void* table, void* out, int T, int H, int V, cudaStream_t s) {
  if (T == 0) return;
  AGRPO_PREFER_SMEM(embedding_fwd_kernel);
  embedding_fwd_kernel<<<(T + 7) / 8, 256, 0, s>>>(ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, T, H, V);
  check_cuda(cudaGetLastError(), "embedding_fwd");
}
void launch_embedding_sumsq(const int* ids, const void* table, void* out, long long* ss, int n_ss, int ss_stride, int T, int H,
                            int V, cudaStream_t s) {
  if (T == 0) return;
  AGRPO_PREFER_SMEM(embedding_sumsq_kernel);
  launch_kernel(embedding_sumsq_kernel, dim3((T + 7) / 8), dim3(256), 0, s, "embedding_sumsq", ids, (const __nv_bfloat16*)table,
                (__nv_bfloat16*)out, ss, n_ss, ss_stride, T, H, V);
}
void launch_fold_norm_weight(const void* w, const void* g, void* out, long long n_rows, int K, cudaStream_t s) {
  if (n_rows == 0) return;
  const long long total = n_rows * (K / 8);
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  fold_norm_weight_kernel<<<blocks, 256, 0, s>>>((const __nv_bfloat16*)w, (const __nv_bfloat16*)g, (__nv_bfloat16*)out, n_rows, K);
  check_cuda(cudaGetLastError(), "fold_norm_weight");
}
void launch_embedding_bwd(const int* ids, const void* dout, float* dtable, int T, int H, int V, cudaStream_t s) {
  if (T == 0) return;
  embedding_bwd_kernel<<<(T + 7) / 8, 256, 0, s>>>(ids, (const __nv_bfloat16*)dout, dtable, T, H, V);
  check_cuda(cudaGetLastError(), "embedding_bwd");
}
void launch_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int T, int H, float eps, cudaStream_t s) {
  if (T == 0) return;
  AGRPO_PREFER_SMEM(rmsnorm_fwd_kernel);
  launch_kernel(rmsnorm_fwd_kernel, dim3((T + 7) / 8), dim3(256), 0, s, "rmsnorm_fwd", (const __nv_bfloat16*)x,
                (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rstd, T, H, eps);
}
void launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw, int T,
                        int H, bool accumulate_dx, cudaStream_t s) {
  if (T == 0) return;
  rmsnorm_bwd_dx_kernel<<<(T + 7) / 8, 256, 0, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                    (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx, T, H,
                                                    accumulate_dx ? 1 : 0);
  check_cuda(cudaGetLastError(), "rmsnorm_bwd_dx");
  if (dw != nullptr) {
    const int rows_per_block = 256;
    dim3 grid((H + 63) / 64, (T + rows_per_block - 1) / rows_per_block);
    colsum_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, rstd, dw, T, H, H,
                                       rows_per_block);
    check_cuda(cudaGetLastError(), "rmsnorm_bwd_dw");
  }
}
void launch_colsum(const void* a, float* out, int T, int C, long long lda, cudaStream_t s) {
  if (T == 0) return;
  const int rows_per_block = 256;
  dim3 grid((C + 63) / 64, (T + rows_per_block - 1) / rows_per_block);
  colsum_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)a, nullptr, nullptr, out, T, C, lda, rows_per_block);
  check_cuda(cudaGetLastError(), "colsum");
}
void launch_rope(void* qkv, const int* pos, const float* cos_t, const float* sin_t, int T, int n_rot_heads, int D,
                 long long row_pitch, int max_pos, bool backward, cudaStream_t s) {
  if (T == 0) return;
  const long long work = (long long)T * n_rot_heads * (D / 2);
  AGRPO_PREFER_SMEM(rope_kernel);
  rope_kernel<<<grid_for(work, 256), 256, 0, s>>>((__nv_bfloat16*)qkv, pos, cos_t, sin_t, T, n_rot_heads, D, row_pitch,
                                                  max_pos, backward ? -1.f : 1.f);
  check_cuda(cudaGetLastError(), "rope");
}
void launch_swiglu_fwd(const void* gu, void* out, int T, int F, cudaStream_t s) {
  if (T == 0) return;
  AGRPO_PREFER_SMEM(swiglu_fwd_kernel);
  swiglu_fwd_kernel<<<grid_for((long long)T * (F / 8), 256), 256, 0, s>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out,
                                                                           T, F);
  check_cuda(cudaGetLastError(), "swiglu_fwd");
}
void launch_swiglu_bwd(const void* gu, const void* dout, void* dgu, int T, int F, cudaStream_t s) {
  if (T == 0) return;
  swiglu_bwd_kernel<<<grid_for((long long)T * (F / 8), 256), 256, 0, s>>>(
      (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dgu, T, F);
  check_cuda(cudaGetLastError(), "swiglu_bwd");
}
void launch_add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t s) {
  if (n == 0) return;
  add_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, s>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                       (__nv_bfloat16*)out, n / 8);
  check_cuda(cudaGetLastError(), "add_bf16");
}

}  // namespace agrpo
