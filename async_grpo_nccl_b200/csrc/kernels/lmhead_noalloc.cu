// Allocation-free variant of the lm_head log-probability entry point: same kernels, scratch in a file-scope device
// array instead of caller-allocated memory. See include/agrpo_noalloc.h for the contract.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "../include/agrpo_noalloc.h"
#include "../launchers.h"

namespace {

constexpr size_t kScratchFloats = AGRPO_NOALLOC_SCRATCH_BYTES / sizeof(float);
constexpr int kMaxDevices = 64;

// Part of the library image: one copy per GPU that loads the library.
static __device__ __align__(256) float g_lmhead_scratch[kScratchFloats];
// Status word of the kernels behind this entry point (0 = fine; non-zero: a bounded wait inside the GEMM ran out and the
// outputs of that call are not to be trusted). Cleared by every call, read back by agrpo_lmhead_noalloc_status().
static __device__ int g_lmhead_status;

// In host code the name above is only a handle for the runtime, not a device address; the address is looked up once
// per device (with that device current) and cached here.
float* g_scratch_addr[kMaxDevices] = {nullptr};
int* g_status_addr[kMaxDevices] = {nullptr};
int g_num_sms[kMaxDevices] = {0};
std::mutex g_setup_mutex;

void set_msg(char* dst, int cap, const char* msg) {
  if (dst == nullptr || cap <= 0) return;
  std::strncpy(dst, msg, (size_t)cap - 1);
  dst[cap - 1] = '\0';
}

}  // namespace

extern "C" int agrpo_lmhead_logprob_noalloc(const void* hidden_bf16, long long hidden_pitch, const void* weight_bf16,
                                            long long weight_pitch, const int* labels, int T, int H, int V,
                                            float temperature, float* logp, float* entropy, float* lse, void* stream,
                                            char* err_msg, int err_cap) {
  set_msg(err_msg, err_cap, "");
  if (hidden_bf16 == nullptr || weight_bf16 == nullptr || labels == nullptr || logp == nullptr) {
    set_msg(err_msg, err_cap, "hidden, weight, labels and logp must not be NULL");
    return AGRPO_NOALLOC_E_BAD_ARGUMENT;
  }
  if (T < 0 || H <= 0 || V <= 0 || H % 8 != 0 || hidden_pitch % 8 != 0 || weight_pitch % 8 != 0 || hidden_pitch < H ||
      weight_pitch < H || !(temperature > 0.f)) {
    set_msg(err_msg, err_cap, "need T >= 0, H > 0 and a multiple of 8, V > 0, pitches >= H and multiples of 8, temperature > 0");
    return AGRPO_NOALLOC_E_BAD_ARGUMENT;
  }
  if ((reinterpret_cast<uintptr_t>(hidden_bf16) & 15) != 0 || (reinterpret_cast<uintptr_t>(weight_bf16) & 15) != 0) {
    set_msg(err_msg, err_cap, "hidden and weight must be 16-byte aligned");
    return AGRPO_NOALLOC_E_BAD_ARGUMENT;
  }
  if (T == 0) return AGRPO_NOALLOC_OK;
  const long long groups = agrpo::lmhead_num_groups(V, T);
  const long long need = (3 * groups + 1) * (long long)T;
  if (need > (long long)kScratchFloats) {
    char buf[256];
    std::snprintf(buf, sizeof(buf),
                  "problem too large for the built-in scratch: T=%d V=%d needs %lld bytes, the library holds %u bytes", T, V,
                  need * 4, (unsigned)AGRPO_NOALLOC_SCRATCH_BYTES);
    set_msg(err_msg, err_cap, buf);
    return AGRPO_NOALLOC_E_TOO_LARGE;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_msg(err_msg, err_cap, e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range");
    return AGRPO_NOALLOC_E_CUDA;
  }
  {
    // first call on this device: resolve the scratch array's device address
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_addr[dev] == nullptr) {
      float* ptr = nullptr;
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_lmhead_scratch);
      if (e != cudaSuccess || ptr == nullptr) {
        set_msg(err_msg, err_cap, e != cudaSuccess ? cudaGetErrorString(e) : "cudaGetSymbolAddress returned NULL");
        return AGRPO_NOALLOC_E_CUDA;
      }
      int sms = 0;
      e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess || sms <= 0) {
        set_msg(err_msg, err_cap, e != cudaSuccess ? cudaGetErrorString(e) : "could not read the SM count");
        return AGRPO_NOALLOC_E_CUDA;
      }
      int* sptr = nullptr;
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&sptr), g_lmhead_status);
      if (e != cudaSuccess || sptr == nullptr) {
        set_msg(err_msg, err_cap, e != cudaSuccess ? cudaGetErrorString(e) : "cudaGetSymbolAddress returned NULL");
        return AGRPO_NOALLOC_E_CUDA;
      }
      g_num_sms[dev] = sms;
      g_status_addr[dev] = sptr;
      g_scratch_addr[dev] = ptr;
    }
  }
  float* scratch = g_scratch_addr[dev];
  float* partials = scratch;                       // [3 * groups * T], fully overwritten by the kernel
  float* label_logit = scratch + 3 * groups * T;   // [T], rows without a valid label are never written: clear it
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  e = cudaMemsetAsync(label_logit, 0, sizeof(float) * (size_t)T, s);
  if (e == cudaSuccess) e = cudaMemsetAsync(g_status_addr[dev], 0, sizeof(int), s);
  if (e != cudaSuccess) {
    set_msg(err_msg, err_cap, cudaGetErrorString(e));
    return AGRPO_NOALLOC_E_CUDA;
  }
  try {
    agrpo::launch_lmhead_logprob(hidden_bf16, hidden_pitch, weight_bf16, weight_pitch, labels, T, H, V, temperature, partials,
                                 label_logit, logp, entropy, lse, g_status_addr[dev], g_num_sms[dev], s);
  } catch (const std::exception& ex) {
    set_msg(err_msg, err_cap, ex.what());
    return AGRPO_NOALLOC_E_CUDA;
  }
  return AGRPO_NOALLOC_OK;
}

extern "C" int agrpo_lmhead_noalloc_status(void* stream) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return AGRPO_NOALLOC_E_CUDA;
  int* addr = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    addr = g_status_addr[dev];
  }
  if (addr == nullptr) return 0;  // no call was made on this device yet
  int word = 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(&word, addr, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess) return AGRPO_NOALLOC_E_CUDA;
  if (cudaStreamSynchronize(s) != cudaSuccess) return AGRPO_NOALLOC_E_CUDA;
  return word;
}
