// Host-side helper that builds (and caches) 2-D bf16 TMA tensor maps with 128-byte swizzle.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>

namespace agrpo {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || p == nullptr) throw std::runtime_error("cuTensorMapEncodeTiled entry point not found");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct TmapKey {
  uint64_t ptr, d0, d1, ld;
  uint32_t b0, b1, esize, swz;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && ld == o.ld && b0 == o.b0 && b1 == o.b1 && esize == o.esize &&
           swz == o.swz;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = k.ptr * 0x9E3779B97F4A7C15ull;
    h ^= (k.d0 + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= (k.d1 + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= (k.ld + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= ((uint64_t(k.b0) << 32 | k.b1) + (h << 6) + (h >> 2));
    h ^= ((uint64_t(k.esize) << 8 | k.swz) + (h << 6) + (h >> 2));
    return static_cast<size_t>(h);
  }
};

// 2-D map over a row-major matrix: `inner` contiguous elements per row, `outer` rows, row pitch
// `ld` elements. Box = box_inner x box_outer elements. elem_size 2 (bf16) or 4 (fp32).
// swizzle128: box_inner * elem_size must equal 128 bytes.
inline CUtensorMap make_tmap_2d(const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                                uint32_t box_outer, int elem_size = 2, bool swizzle128 = true) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  static std::mutex mu;
  TmapKey key{reinterpret_cast<uint64_t>(base), inner, outer, ld, box_inner, box_outer, (uint32_t)elem_size,
              swizzle128 ? 1u : 0u};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
  }
  if ((reinterpret_cast<uint64_t>(base) & 15) != 0) throw std::runtime_error("TMA base address must be 16-byte aligned");
  if ((ld * elem_size) % 16 != 0) throw std::runtime_error("TMA row pitch must be a multiple of 16 bytes");
  CUtensorMap m;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * (uint64_t)elem_size};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = get_encode_tiled()(&m, elem_size == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                                  2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed: " + std::to_string((int)r));
  {
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, m);
  }
  return m;
}

}  // namespace agrpo
