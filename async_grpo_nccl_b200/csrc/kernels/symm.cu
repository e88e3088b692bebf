// Peer-memory kernels over NVLink 5 / NVSwitch. Every rank maps every peer's symmetric buffer, so a kernel
// on one GPU can load from and store to the others directly; the collectives below are fused into the
// compute that surrounds them instead of being separate NCCL calls:
//
//  * weight_push       trainer -> rollout / logprob / trainer peers: read the local fp32 (or bf16) shard, cast
//                      to bf16, write it straight into every destination's flat parameter buffer. Replaces
//                      the reference's per-tensor full_tensor() all-gather + broadcast + load_weights
//                      (gpu_process_worker.py:1609-1637, 1716-1753, 1888-1915).
//  * rs_pull_sumsq     gradient reduce-scatter: the owner of a shard sums that slice out of every peer's fp32
//                      gradient buffer (peer loads) and accumulates the squared norm of the result. Replaces
//                      FSDP2's reduce-scatter + the norm pass of clip_grad_norm_ (gpu_process_worker.py:1056-1065).
//  * adamw_push        AdamW on the local shard with the clip coefficient taken from the summed per-rank norm
//                      partials, the bf16 result written to every destination (all-gather + weight sync in
//                      the same pass as the optimizer).
//  * flag_barrier      epoch flags in the symmetric buffers, release-stores to peers, bounded acquire-spin.
//
// All waits are bounded (see ptx.cuh); a wait that runs out records kStatusPeerFlagTimeout / kStatusBarrierTimeout
// in the status word and the kernel returns.
#include <cuda_bf16.h>

#include "../common/ptx.cuh"
#include "../launchers.h"

namespace agrpo {

namespace {

constexpr int kMaxPeers = 16;

struct PeerPtrs {
  void* p[kMaxPeers];
  int n;
};

// Status word of the peer group whose barrier precedes the kernels below on this thread's stream (nullptr = none).
// A barrier that ran out of time has written an error code there; every kernel that would then read buffers peers may
// still be writing, or overwrite parameters, optimizer state or inference weights, returns at entry instead, so a late
// rank costs one raised error on the host and not the state of every rank.
thread_local const int* t_guard = nullptr;

__device__ __forceinline__ bool guard_tripped(const int* guard) {
  return guard != nullptr && *reinterpret_cast<const volatile int*>(guard) != 0;
}

__global__ void wait_flag_probe_kernel(const uint64_t* flag, uint64_t want, long long budget, int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    if (!wait_flag_ge(flag, want, budget)) report_status(status, kStatusPeerFlagTimeout);
  }
}

// Each rank: flags[my_rank] of every peer <- epoch (release), then wait until all of my flags[r] >= epoch.
__global__ void flag_barrier_kernel(PeerPtrs flags, int my_rank, uint64_t epoch, long long budget, int* status) {
  const int r = threadIdx.x;
  if (r < flags.n) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint64_t*>(flags.p[r]) + my_rank, epoch);
  }
  __syncthreads();
  if (r < flags.n) {
    const uint64_t* mine = reinterpret_cast<const uint64_t*>(flags.p[my_rank]) + r;
    if (!wait_flag_ge(mine, epoch, budget)) report_status(status, kStatusBarrierTimeout);
  }
}

// Tensor-parallel all-reduce of a row-parallel projection, fused with the arrival barrier before it and with what follows
// it in a decoder layer:
//   out[b, :] = residual[b, :] + sum_r partial_r[b, :]     (fp32 sum in rank order: every rank gets the same bits)
//   ss[b]    += sum_h out[b, h]^2                          (row statistic of the next folded RMSNorm, fixed point)
// partial_r is rank r's bf16 [rows, H] product in ITS symmetric buffer, read here with plain peer loads (one-shot
// all-reduce: every rank reads every partial; [rows, H] is a few hundred KB, far below the point where a ring pays).
//
// One CTA per row, one 16-byte vector per thread (two when H > 8192): every peer load of a row is in flight at the same
// time, so the kernel costs about one NVLink round trip instead of one per loop iteration.
//
// Arrival: the GEMM that wrote this rank's partial precedes this kernel in the stream. CTA 0 tells every member "my
// partial number `epoch` is complete" (release store into the member's flag row), and every CTA waits until all members
// have said so for this epoch (bounded acquire polls of LOCAL memory). The epoch lives on the device (*epoch_counter,
// advanced by the last CTA of each launch), so the launch has no per-call argument and replays from a CUDA graph; every
// member replays the same number of all-reduces. The arrival of the NEXT all-reduce (which uses the other partial
// buffer) also says that everybody has finished reading this buffer before its owner overwrites it.
template <int NR>  // upper bound on the number of members (2, 4 or 8): sizes the register tile of loads in flight
__global__ void __launch_bounds__(1024)
tp_allreduce_residual_kernel(PeerPtrs partials, PeerPtrs flags, int my_rank, unsigned long long* epoch_counter,
                             unsigned int* arrive, const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out,
                             sumsq_t* __restrict__ ss, int rows, int H, long long budget, int* status) {
  __shared__ unsigned long long s_epoch;
  __shared__ int s_ok;
  __shared__ float s_red[32];
  const int tid = threadIdx.x, n = partials.n;
  pdl_wait();    // this rank's partial (and the residual) are complete
  pdl_launch();  // the next GEMM may start fetching its weights
  if (tid == 0) {
    s_epoch = *reinterpret_cast<volatile unsigned long long*>(epoch_counter) + 1ull;
    s_ok = 1;
  }
  __syncthreads();
  const uint64_t epoch = s_epoch;
  if (blockIdx.x == 0 && tid < n) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint64_t*>(flags.p[tid]) + my_rank, epoch);
  }
  if (tid < n) {
    if (!wait_flag_ge(reinterpret_cast<const uint64_t*>(flags.p[my_rank]) + tid, epoch, budget)) {
      report_status(status, kStatusBarrierTimeout);
      s_ok = 0;
    }
  }
  __syncthreads();
  if (tid == 0) {
    // every CTA has read the epoch by now; the last one to pass here publishes it for the next launch
    if (atomicAdd(arrive, 1u) == gridDim.x - 1) {
      *arrive = 0u;
      *reinterpret_cast<volatile unsigned long long*>(epoch_counter) = epoch;
    }
  }
  if (!s_ok) return;
  const int b = blockIdx.x;
  const int nv = H >> 3;
  float sq = 0.f;
  uint4 res[2], part[2][NR];
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int v = tid + it * (int)blockDim.x;
    if (v < nv) {
      res[it] = *reinterpret_cast<const uint4*>(residual + (size_t)b * H + v * 8);
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        if (r < n) {
          const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(partials.p[r]) + (size_t)b * H + v * 8);
          asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(part[it][r].x), "=r"(part[it][r].y), "=r"(part[it][r].z), "=r"(part[it][r].w)
                       : "l"(src)
                       : "memory");
        }
      }
    }
  }
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int v = tid + it * (int)blockDim.x;
    if (v < nv) {
      float acc[8];
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&res[it]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h2[i]);
        acc[2 * i] = f.x;
        acc[2 * i + 1] = f.y;
      }
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        if (r < n) {
          const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&part[it][r]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(p2[i]);
            acc[2 * i] += f.x;
            acc[2 * i + 1] += f.y;
          }
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(out + (size_t)b * H + v * 8) = o;
      // the statistic is taken from the rounded values, as the GEMM epilogues of the unsharded path take it
      const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(o2[i]);
        sq += f.x * f.x + f.y * f.y;
      }
    }
  }
  if (ss == nullptr) return;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  if ((tid & 31) == 0) s_red[tid >> 5] = sq;
  __syncthreads();
  if (tid < 32) {
    float t = tid < (int)(blockDim.x >> 5) ? s_red[tid] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (tid == 0) sumsq_atomic_add(ss + b, t);
  }
}

// dst[d][global_off + i] = bf16(src[local_off + i]) for every destination d. SrcT = float or bf16.
template <typename SrcT>
__global__ void weight_push_kernel(const SrcT* __restrict__ src, long long local_off, long long global_off, long long n,
                                   PeerPtrs dst, const int* guard) {
  if (guard_tripped(guard)) return;
  const long long n8 = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    uint4 w;
    if constexpr (sizeof(SrcT) == 4) {
      const float4 a = reinterpret_cast<const float4*>(src + local_off)[2 * i];
      const float4 b = reinterpret_cast<const float4*>(src + local_off)[2 * i + 1];
      w.x = pack_bf16x2(a.x, a.y);
      w.y = pack_bf16x2(a.z, a.w);
      w.z = pack_bf16x2(b.x, b.y);
      w.w = pack_bf16x2(b.z, b.w);
    } else {
      w = reinterpret_cast<const uint4*>(src + local_off)[i];
    }
#pragma unroll 1
    for (int d = 0; d < dst.n; ++d) reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.p[d]) + global_off)[i] = w;
  }
  // tail (n is a multiple of 8 for every layout unit, kept for safety)
  for (long long i = n8 * 8 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const __nv_bfloat16 v = __float2bfloat16(static_cast<float>(src[local_off + i]));
    for (int d = 0; d < dst.n; ++d) reinterpret_cast<__nv_bfloat16*>(dst.p[d])[global_off + i] = v;
  }
}

// dst[owner(i)][...] += src[i] for a local fp32 vector that sits unit_rel elements into an evenly sharded unit; the
// source is zeroed afterwards when asked. Serves the gradients that no GEMM epilogue produces (norm weights, biases,
// the embedding group).
__global__ void scatter_add_f32_kernel(float* __restrict__ src, long long n, long long unit_rel, PeerPtrs dst,
                                       long long n_per_owner, int zero_src, const int* guard) {
  if (guard_tripped(guard)) return;
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(src)[i];
    if (zero_src) reinterpret_cast<float4*>(src)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (v.x == 0.f && v.y == 0.f && v.z == 0.f && v.w == 0.f) continue;  // untouched embedding rows
    const long long flat = unit_rel + 4 * i;
    const int owner = (int)(flat / n_per_owner);
    float* d = reinterpret_cast<float*>(dst.p[owner]) + (flat - (long long)owner * n_per_owner);
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
  }
  for (long long i = n4 * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = src[i];
    if (zero_src) src[i] = 0.f;
    const long long flat = unit_rel + i;
    const int owner = (int)(flat / n_per_owner);
    atomicAdd(reinterpret_cast<float*>(dst.p[owner]) + (flat - (long long)owner * n_per_owner), v);
  }
}

// out[local_off + i] = sum_r grads[r][global_off + i]; *norm_sq += sum(out^2). Peers are visited starting with
// (my_rank + 1) so that ranks do not all read the same source at the same time.
__global__ void rs_pull_sumsq_kernel(PeerPtrs grads, int my_rank, long long global_off, long long local_off, long long n,
                                     float* __restrict__ out, float* __restrict__ norm_sq, const int* guard) {
  if (guard_tripped(guard)) return;
  float acc2 = 0.f;
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
    for (int k = 0; k < grads.n; ++k) {
      const int r = (my_rank + 1 + k) % grads.n;
      const float4 v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + global_off)[i];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    reinterpret_cast<float4*>(out + local_off)[i] = s;
    acc2 += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc2 += __shfl_xor_sync(0xffffffffu, acc2, o);
  __shared__ float sm[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sm[warp] = acc2;
  __syncthreads();
  if (warp == 0) {
    acc2 = lane < (int)(blockDim.x >> 5) ? sm[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc2 += __shfl_xor_sync(0xffffffffu, acc2, o);
    if (lane == 0 && acc2 != 0.f) atomicAdd(norm_sq, acc2);
  }
}

// NVSwitch multicast (NVLS) variants. `mc` is the multicast address of a symmetric buffer: one store to it lands in
// every rank's copy, one ld_reduce from it returns the sum over every rank's copy, both done inside the switch.
//
// Weight push: each 16-byte group is written once and replicated by the switch, so the source's egress does not grow
// with the number of receivers.
template <typename SrcT>
__global__ void weight_push_mc_kernel(const SrcT* __restrict__ src, long long local_off, long long global_off, long long n,
                                      __nv_bfloat16* mc, const int* guard) {
  if (guard_tripped(guard)) return;
  const long long n8 = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    uint4 w;
    if constexpr (sizeof(SrcT) == 4) {
      const float4 a = reinterpret_cast<const float4*>(src + local_off)[2 * i];
      const float4 b = reinterpret_cast<const float4*>(src + local_off)[2 * i + 1];
      w.x = pack_bf16x2(a.x, a.y);
      w.y = pack_bf16x2(a.z, a.w);
      w.z = pack_bf16x2(b.x, b.y);
      w.w = pack_bf16x2(b.z, b.w);
    } else {
      w = reinterpret_cast<const uint4*>(src + local_off)[i];
    }
    uint4* d = reinterpret_cast<uint4*>(mc + global_off) + i;
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d), "f"(__uint_as_float(w.x)),
                 "f"(__uint_as_float(w.y)), "f"(__uint_as_float(w.z)), "f"(__uint_as_float(w.w))
                 : "memory");
  }
  __threadfence_system();
}

// Gradient reduce-scatter with the addition done in the switch: out[local_off + i] = sum over ALL ranks of the
// multicast group of grads[global_off + i] (ranks that are not trainers hold zeros); *norm_sq += sum(out^2).
__global__ void rs_pull_sumsq_mc_kernel(const float* mc, long long global_off, long long local_off, long long n,
                                        float* __restrict__ out, float* __restrict__ norm_sq, const int* guard) {
  if (guard_tripped(guard)) return;
  float acc2 = 0.f;
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 s;
    const float4* a = reinterpret_cast<const float4*>(mc + global_off) + i;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(s.x), "=f"(s.y), "=f"(s.z), "=f"(s.w)
                 : "l"(a)
                 : "memory");
    reinterpret_cast<float4*>(out + local_off)[i] = s;
    acc2 += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc2 += __shfl_xor_sync(0xffffffffu, acc2, o);
  __shared__ float sm[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sm[warp] = acc2;
  __syncthreads();
  if (warp == 0) {
    acc2 = lane < (int)(blockDim.x >> 5) ? sm[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc2 += __shfl_xor_sync(0xffffffffu, acc2, o);
    if (lane == 0 && acc2 != 0.f) atomicAdd(norm_sq, acc2);
  }
}

// Publishes this rank's squared-norm partial into slot my_rank of every peer's partial table.
__global__ void publish_norm_kernel(const float* norm_sq, PeerPtrs tables, int my_rank, const int* guard) {
  if (guard_tripped(guard)) return;
  const int r = threadIdx.x;
  if (r < tables.n) reinterpret_cast<float*>(tables.p[r])[my_rank] = *norm_sq;
}

// AdamW on [local_off, local_off + n) of the shard; bf16 result to dst[d][global_off + i] for every destination.
__global__ void adamw_push_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, float* __restrict__ g,
                                  long long local_off, long long global_off, long long n, float lr, float beta1, float beta2,
                                  float eps, float wd, float bc1, float bc2, float grad_scale, const float* __restrict__ partials,
                                  int n_partials, float max_norm, PeerPtrs dst, const int* guard) {
  if (guard_tripped(guard)) return;
  float coef = grad_scale;
  if (max_norm > 0.f && partials != nullptr) {
    float tot = 0.f;
    for (int r = 0; r < n_partials; ++r) tot += partials[r];
    coef *= fminf(1.f, max_norm / (sqrtf(tot) + 1e-6f));
  }
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
  const long long n2 = n / 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n2; i += (long long)gridDim.x * blockDim.x) {
    float r2[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const long long k = local_off + 2 * i + j;
      const float gi = g[k] * coef;
      float pi = p[k] * (1.f - lr * wd);
      const float mi = beta1 * m[k] + (1.f - beta1) * gi;
      const float vi = beta2 * v[k] + (1.f - beta2) * gi * gi;
      pi -= lr * inv_bc1 * mi / (sqrtf(vi) * inv_sqrt_bc2 + eps);
      p[k] = pi;
      m[k] = mi;
      v[k] = vi;
      g[k] = 0.f;
      r2[j] = pi;
    }
    const uint32_t w = pack_bf16x2(r2[0], r2[1]);
#pragma unroll 1
    for (int d = 0; d < dst.n; ++d) reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(dst.p[d]) + global_off)[i] = w;
  }
}

inline PeerPtrs make_peers(const long long* ptrs, int n) {
  if (n > kMaxPeers) throw std::runtime_error("too many peers");
  PeerPtrs pp;
  pp.n = n;
  for (int i = 0; i < kMaxPeers; ++i) pp.p[i] = i < n ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return pp;
}

inline int blocks_for(long long work, int cap = 148 * 8) {
  long long b = (work + 255) / 256;
  if (b < 1) b = 1;
  return (int)(b > cap ? cap : b);
}

inline long long ticks_for(double seconds) { return (long long)(seconds * 1.9e9); }

}  // namespace

void set_comm_guard(const int* status) { t_guard = status; }

void launch_wait_flag_probe(const void* flag, unsigned long long want, double budget_s, int* status, cudaStream_t s) {
  wait_flag_probe_kernel<<<1, 32, 0, s>>>(reinterpret_cast<const uint64_t*>(flag), want, ticks_for(budget_s), status);
  check_cuda(cudaGetLastError(), "wait_flag_probe");
}

void launch_flag_barrier(const long long* flag_ptrs, int world, int my_rank, unsigned long long epoch, double budget_s,
                         int* status, cudaStream_t s) {
  flag_barrier_kernel<<<1, 32, 0, s>>>(make_peers(flag_ptrs, world), my_rank, epoch, ticks_for(budget_s), status);
  check_cuda(cudaGetLastError(), "flag_barrier");
}

void launch_tp_allreduce_residual(const long long* partial_ptrs, const long long* flag_ptrs, int world, int my_rank,
                                  unsigned long long* epoch_counter, unsigned int* arrive, const void* residual, void* out,
                                  long long* ss, int rows, int H, double budget_s, int* status, cudaStream_t s) {
  if (rows == 0) return;
  if (world > 8 || H % 8 != 0 || H > 16384) throw std::runtime_error("tp_allreduce_residual: at most 8 ranks, H a multiple of 8 up to 16384");
  int threads = ((H / 8 + 31) / 32) * 32;
  if (threads > 1024) threads = ((H / 16 + 31) / 32) * 32;
  auto kernel = world <= 2 ? tp_allreduce_residual_kernel<2> : world <= 4 ? tp_allreduce_residual_kernel<4> : tp_allreduce_residual_kernel<8>;
  launch_kernel(kernel, dim3(rows), dim3(threads), 0, s, "tp_allreduce_residual",
                make_peers(partial_ptrs, world), make_peers(flag_ptrs, world), my_rank, epoch_counter, arrive,
                (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, ss, rows, H, ticks_for(budget_s), status);
}

void launch_weight_push(const void* src, bool src_fp32, long long local_off, long long global_off, long long n,
                        const long long* dst_ptrs, int n_dst, cudaStream_t s) {
  if (n == 0 || n_dst == 0) return;
  const PeerPtrs d = make_peers(dst_ptrs, n_dst);
  if (src_fp32) weight_push_kernel<float><<<blocks_for(n / 8), 256, 0, s>>>((const float*)src, local_off, global_off, n, d, t_guard);
  else weight_push_kernel<__nv_bfloat16><<<blocks_for(n / 8), 256, 0, s>>>((const __nv_bfloat16*)src, local_off, global_off, n, d, t_guard);
  check_cuda(cudaGetLastError(), "weight_push");
}

void launch_scatter_add_f32(float* src, long long n, long long unit_rel, const ScatterArgs& sc, bool zero_src,
                            cudaStream_t s) {
  if (n == 0) return;
  PeerPtrs d;
  d.n = sc.world;
  for (int r = 0; r < sc.world; ++r) d.p[r] = sc.dst[r];
  scatter_add_f32_kernel<<<blocks_for(n / 4 + 1), 256, 0, s>>>(src, n, unit_rel, d, sc.n_per_owner, zero_src ? 1 : 0, t_guard);
  check_cuda(cudaGetLastError(), "scatter_add_f32");
}

void launch_weight_push_mc(const void* src, bool src_fp32, long long local_off, long long global_off, long long n, void* mc,
                           cudaStream_t s) {
  if (n == 0) return;
  if (src_fp32) weight_push_mc_kernel<float><<<blocks_for(n / 8), 256, 0, s>>>((const float*)src, local_off, global_off, n, (__nv_bfloat16*)mc, t_guard);
  else weight_push_mc_kernel<__nv_bfloat16><<<blocks_for(n / 8), 256, 0, s>>>((const __nv_bfloat16*)src, local_off, global_off, n, (__nv_bfloat16*)mc, t_guard);
  check_cuda(cudaGetLastError(), "weight_push_mc");
}

void launch_rs_pull_sumsq_mc(const void* mc, long long global_off, long long local_off, long long n, float* out, float* norm_sq,
                             cudaStream_t s) {
  if (n == 0) return;
  rs_pull_sumsq_mc_kernel<<<blocks_for(n / 4), 256, 0, s>>>((const float*)mc, global_off, local_off, n, out, norm_sq, t_guard);
  check_cuda(cudaGetLastError(), "rs_pull_sumsq_mc");
}

void launch_rs_pull_sumsq(const long long* grad_ptrs, int world, int my_rank, long long global_off, long long local_off,
                          long long n, float* out, float* norm_sq, cudaStream_t s) {
  if (n == 0) return;
  rs_pull_sumsq_kernel<<<blocks_for(n / 4), 256, 0, s>>>(make_peers(grad_ptrs, world), my_rank, global_off, local_off, n, out,
                                                         norm_sq, t_guard);
  check_cuda(cudaGetLastError(), "rs_pull_sumsq");
}

void launch_publish_norm(const float* norm_sq, const long long* table_ptrs, int world, int my_rank, cudaStream_t s) {
  publish_norm_kernel<<<1, 32, 0, s>>>(norm_sq, make_peers(table_ptrs, world), my_rank, t_guard);
  check_cuda(cudaGetLastError(), "publish_norm");
}

void launch_adamw_push(float* p, float* m, float* v, float* g, long long local_off, long long global_off, long long n, float lr,
                       float beta1, float beta2, float eps, float wd, int step, float grad_scale, const float* partials,
                       int n_partials, float max_norm, const long long* dst_ptrs, int n_dst, cudaStream_t s) {
  if (n == 0) return;
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2 = 1.f - powf(beta2, (float)step);
  adamw_push_kernel<<<blocks_for(n / 2, 148 * 16), 256, 0, s>>>(p, m, v, g, local_off, global_off, n, lr, beta1, beta2, eps, wd,
                                                               bc1, bc2, grad_scale, partials, n_partials, max_norm,
                                                               make_peers(dst_ptrs, n_dst), t_guard);
  check_cuda(cudaGetLastError(), "adamw_push");
}

}  // namespace agrpo
