// Persistent warp-specialised bf16 GEMM for sm_100a: TMA -> shared-memory ring -> tcgen05.mma with the
// accumulator in tensor memory -> tcgen05.ld epilogue.
//
//   D[M, N] = alpha * (A . B^T) (+ bias[N]) (+ D)          A is M x K, B is N x K (logical)
//
// Either operand may be stored K-major (row-major [rows, K]) or MN-major (row-major [K, rows]); the
// three combinations a transformer needs are forward y = x W^T (K,K), input gradient dx = dy W
// (K,MN) and weight gradient dW = dy^T x (MN,MN). This replaces the cuBLAS calls behind the
// reference's HF linear layers (gpu_process_worker.py:988-1041 runs them under bf16 autocast).
//
// CTA = 6 warps: warp 0 issues TMA loads, warp 1 issues MMAs (and owns the TMEM allocation), warps
// 2-5 run the epilogue, one TMEM lane quarter each. Two accumulator buffers of BN columns let the
// epilogue of tile i overlap the main loop of tile i+1.
#pragma once
#include <stdexcept>
#include <string>

#include "../common/ptx.cuh"

namespace agrpo {

// Problem shape and scheduling. A work item is one row-tile crossed with `group_n` consecutive
// column-tiles; the epilogue functor sees item_begin / chunk... / item_end so that it can carry
// per-row state (e.g. online-softmax statistics) across the column-tiles of an item.
struct GemmShape {
  int M, N, K;
  int group_n;        // column-tiles per work item (1 for a plain GEMM)
  int* status;        // error word, may be nullptr
};

// Default epilogue: D = alpha * acc (+ bias) (+ D), bf16 or fp32 output.
struct StoreEpilogue {
  void* D;            // bf16 or fp32, row-major
  long long ldd;      // elements
  const __nv_bfloat16* bias;  // [N] or nullptr
  const __nv_bfloat16* residual;  // [M, ldr] added to the result, or nullptr
  long long ldr;
  float alpha;
  int out_fp32;       // 1: D is fp32
  int accumulate;     // 1: D += result (read-modify-write)

  __device__ __forceinline__ void item_begin(int, int, int) {}
  __device__ __forceinline__ void item_end(int, int, int, int) {}
  __device__ __forceinline__ void chunk(int row, int col0, const uint32_t (&r)[32], int M, int N) {
    if (row >= M || col0 >= N) return;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * alpha;
    if (bias != nullptr) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < N) v[i] += __bfloat162float(bias[col0 + i]);
    }
    const bool full = (col0 + 32 <= N);
    if (residual != nullptr) {
      const __nv_bfloat16* rp = residual + static_cast<long long>(row) * ldr + col0;
      if (full && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0)) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          const uint4 w = *reinterpret_cast<const uint4*>(rp + i);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            v[i + 2 * j] += f.x;
            v[i + 2 * j + 1] += f.y;
          }
        }
      } else {
        for (int i = 0; i < 32; ++i)
          if (col0 + i < N) v[i] += __bfloat162float(rp[i]);
      }
    }
    if (out_fp32) {
      float* d = reinterpret_cast<float*>(D) + static_cast<long long>(row) * ldd + col0;
      if (full && ((reinterpret_cast<uintptr_t>(d) & 15) == 0)) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
          if (accumulate) {
            const float4 old = *reinterpret_cast<const float4*>(d + i);
            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
          }
          *reinterpret_cast<float4*>(d + i) = o;
        }
      } else {
        for (int i = 0; i < 32; ++i)
          if (col0 + i < N) d[i] = accumulate ? d[i] + v[i] : v[i];
      }
    } else {
      __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(D) + static_cast<long long>(row) * ldd + col0;
      if (full && !accumulate && ((reinterpret_cast<uintptr_t>(d) & 15) == 0)) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 o;
          o.x = pack_bf16x2(v[i], v[i + 1]);
          o.y = pack_bf16x2(v[i + 2], v[i + 3]);
          o.z = pack_bf16x2(v[i + 4], v[i + 5]);
          o.w = pack_bf16x2(v[i + 6], v[i + 7]);
          *reinterpret_cast<uint4*>(d + i) = o;
        }
      } else {
        for (int i = 0; i < 32; ++i)
          if (col0 + i < N) {
            const float o = accumulate ? __bfloat162float(d[i]) + v[i] : v[i];
            d[i] = __float2bfloat16(o);
          }
      }
    }
  }
};

static constexpr int kGemmBM = 128;
static constexpr int kGemmBK = 64;
static constexpr int kGemmThreads = 192;

template <int BN>
struct GemmSmem {
  static constexpr int kABytes = kGemmBM * kGemmBK * 2;
  static constexpr int kBBytes = BN * kGemmBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + 1024;  // + alignment slack
};

// Work-item order.
//  group_n == 1: bands of 16 row-tiles, column-tile fastest across a band, so that the CTAs running at
//                the same time share A and B tiles through L2.
//  group_n  > 1: row-tile fastest; the CTAs of a wave walk the same column-tiles of B in step.
__device__ __forceinline__ void gemm_item_coords(int idx, int tiles_m, int tiles_n, int group_n, int& tm, int& tn0,
                                                 int& count) {
  if (group_n <= 1) {
    constexpr int kBand = 16;
    const int per_band = kBand * tiles_n;
    const int band = idx / per_band;
    const int rem = idx - band * per_band;
    const int band_rows = min(kBand, tiles_m - band * kBand);
    tm = band * kBand + rem % band_rows;
    tn0 = rem / band_rows;
    count = 1;
  } else {
    tm = idx % tiles_m;
    tn0 = (idx / tiles_m) * group_n;
    count = min(group_n, tiles_n - tn0);
  }
}
__host__ __device__ inline int gemm_num_items(int M, int N, int BN, int group_n) {
  const int tiles_m = (M + kGemmBM - 1) / kGemmBM;
  const int tiles_n = (N + BN - 1) / BN;
  const int g = group_n <= 1 ? 1 : group_n;
  return tiles_m * ((tiles_n + g - 1) / g);
}

template <int BN, bool A_MN, bool B_MN, class Epi>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmShape p, Epi epi) {
  using S = GemmSmem<BN>;
  constexpr int kStages = S::kStages;
  constexpr uint32_t kTmemCols = 2 * BN;
  constexpr uint32_t kIdesc = umma_idesc_bf16(kGemmBM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * S::kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (p.M + kGemmBM - 1) / kGemmBM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_items = gemm_num_items(p.M, p.N, BN, p.group_n);
  const int num_kb = (p.K + kGemmBK - 1) / kGemmBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        int tm, tn0, count;
        gemm_item_coords(item, tiles_m, tiles_n, p.group_n, tm, tn0, count);
        const int m0 = tm * kGemmBM;
        for (int t = 0; t < count && ok; ++t) {
          const int n0 = (tn0 + t) * BN;
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
              report_status(p.status, kStatusWaitEmptyTimeout);
              ok = false;
              break;
            }
            uint8_t* sa = smem + stage * S::kStageBytes;
            uint8_t* sb = sa + S::kABytes;
            mbar_expect_tx(&full_bar[stage], S::kStageBytes);
            const int k0 = kb * kGemmBK;
            if constexpr (!A_MN) {
              tma_load_2d(sa, &tmA, &full_bar[stage], k0, m0);
            } else {
#pragma unroll
              for (int j = 0; j < kGemmBM / 64; ++j) tma_load_2d(sa + j * 8192, &tmA, &full_bar[stage], m0 + j * 64, k0);
            }
            if constexpr (!B_MN) {
              tma_load_2d(sb, &tmB, &full_bar[stage], k0, n0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tmB, &full_bar[stage], n0 + j * 64, k0);
            }
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        int tm, tn0, count;
        gemm_item_coords(item, tiles_m, tiles_n, p.group_n, tm, tn0, count);
        for (int t = 0; t < count && ok; ++t, ++local) {
          const int buf = local & 1;
          const uint32_t acc_phase = (local >> 1) & 1;
          if (!mbar_wait(&tempty_bar[buf], acc_phase ^ 1)) {
            report_status(p.status, kStatusWaitTmemEmptyTimeout);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + buf * BN;
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(&full_bar[stage], phase)) {
              report_status(p.status, kStatusWaitFullTimeout);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
            const uint32_t sb = sa + S::kABytes;
#pragma unroll
            for (int k = 0; k < kGemmBK / 16; ++k) {
              const uint64_t da = A_MN ? umma_smem_desc(sa + k * 2048, 8192, 1024) : umma_smem_desc(sa + k * 32, 16, 1024);
              const uint64_t db = B_MN ? umma_smem_desc(sb + k * 2048, 8192, 1024) : umma_smem_desc(sb + k * 32, 16, 1024);
              tc_mma_f16(tmem_d, da, db, kIdesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            tc_commit(&empty_bar[stage]);
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (ok) tc_commit(&tfull_bar[buf]);
        }
      }
    }
  } else {
    // ------------------------------ Epilogue ------------------------------
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter + 32)
    int local = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      int tm, tn0, count;
      gemm_item_coords(item, tiles_m, tiles_n, p.group_n, tm, tn0, count);
      const int row = tm * kGemmBM + quarter * 32 + lane;
      epi.item_begin(row, p.M, p.N);
      for (int t = 0; t < count; ++t, ++local) {
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&tfull_bar[buf], acc_phase)) {
          report_status(p.status, kStatusWaitTmemFullTimeout);
          ok = false;
          break;
        }
        tc_fence_after();
        const int n0 = (tn0 + t) * BN;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tc_wait_ld();
          epi.chunk(row, n0 + c * 32, r, p.M, p.N);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      }
      if (ok) epi.item_end(row, p.M, p.N, p.group_n <= 1 ? tn0 : tn0 / p.group_n);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Host-side launch of the generic kernel with any epilogue functor.
template <int BN, bool A_MN, bool B_MN, class Epi>
inline void gemm_launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmShape& p, const Epi& epi, int num_sms,
                        cudaStream_t stream) {
  using S = GemmSmem<BN>;
  auto kernel = gemm_tcgen05_kernel<BN, A_MN, B_MN, Epi>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) throw std::runtime_error(std::string("gemm smem attr: ") + cudaGetErrorString(e));
    configured = true;
  }
  const int items = gemm_num_items(p.M, p.N, BN, p.group_n);
  const int grid = items < num_sms ? items : num_sms;
  kernel<<<grid, kGemmThreads, S::kTotal, stream>>>(ta, tb, p, epi);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("gemm_tcgen05 launch: ") + cudaGetErrorString(e));
}

}  // namespace agrpo
