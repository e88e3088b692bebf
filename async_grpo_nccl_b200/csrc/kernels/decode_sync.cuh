// Small helpers of the persistent decode kernel: GPU-scope counters with bounded waits, status-aware mbarrier
// waits, 4-element bf16 loads / stores.
#pragma once
#include <cuda_bf16.h>

#include "../common/ptx.cuh"

namespace agrpo {

namespace {

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool status_set(const int* status) {
  return status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0;
}
// Bounded wait until *ctr >= want. Gives up early when another CTA has already reported a failure.
__device__ __forceinline__ bool wait_counter(const unsigned int* ctr, unsigned int want, const int* status) {
  if (ld_acquire_gpu(ctr) >= want) return true;
  const long long t0 = clock64();
  int it = 0;
  while (ld_acquire_gpu(ctr) < want) {
    if ((++it & 31) == 0) {
      if (status_set(status)) return false;
      if (clock64() - t0 > kWaitBudgetTicks) return false;
    }
  }
  return true;
}
// mbarrier wait that also gives up when the status word is set.
__device__ __forceinline__ bool mbar_wait_s(uint64_t* bar, uint32_t parity, const int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int it = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++it & 63) == 0) {
      if (status_set(status)) return false;
      if (clock64() - t0 > kWaitBudgetTicks) return false;
    }
  }
  return true;
}

// Loads served by L2: what the persistent kernels read here may have been written by another SM during the same launch,
// and an L1 line of this SM could still hold the value of an earlier layer.
__device__ __forceinline__ sumsq_t ld_sumsq_l2(const sumsq_t* p) { return __ldcg(p); }
__device__ __forceinline__ float4 ld_bf16x4(const __nv_bfloat16* p) {
  const uint2 u = __ldcg(reinterpret_cast<const uint2*>(p));
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st_bf16x4(__nv_bfloat16* p, float4 v) {
  uint2 u;
  u.x = pack_bf16x2(v.x, v.y);
  u.y = pack_bf16x2(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = u;
}

}  // namespace

}  // namespace agrpo
