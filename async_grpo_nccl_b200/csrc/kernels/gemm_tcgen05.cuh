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
#include "../launchers.h"

namespace agrpo {

// Problem shape and scheduling. A work item is one row-tile crossed with `group_n` consecutive
// column-tiles; the epilogue functor sees item_begin / chunk... / item_end so that it can carry
// per-row state (e.g. online-softmax statistics) across the column-tiles of an item.
struct GemmShape {
  int M, N, K;
  int group_n;        // column-tiles per work item (1 for a plain GEMM)
  int* status;        // error word, may be nullptr
  // > 0 (K-major B only): a column tile is made of two half tiles of B rows, [t * BN/2, ...) and
  // [dual_b + t * BN/2, ...): accumulator columns [0, BN/2) and [BN/2, BN) of tile t then hold the two projections of
  // the same output columns (gate and up of a SwiGLU MLP). N counts both halves (2 * dual_b).
  int dual_b = 0;
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

// SwiGLU epilogue for a dual-B GEMM (GemmShape::dual_b): out[m, j] = silu(rs * g) * (rs * u) where g and u are the two
// halves of the accumulator tile and rs[m] = rsqrt(ss_in[m] / K + eps) is the optional folded-RMSNorm row scale (see
// gemm_splitk.cu). Replaces the gate/up GEMM + separate SwiGLU kernel (and the norm kernel before them) in the
// decode step; bn is the kernel's column tile (64 or 128).
struct SwigluEpilogue {
  __nv_bfloat16* D;     // [M, F]
  long long ldd;
  int F;
  int bn;
  const sumsq_t* ss_in; // [M] fixed-point row sums of squares, or nullptr
  float inv_k;
  float eps;
  float g0[32], g1[32];
  float rs;

  __device__ __forceinline__ void item_begin(int row, int M, int) {
    rs = (ss_in != nullptr && row < M) ? rsqrtf(sumsq_from_fixed(ss_in[row]) * inv_k + eps) : 1.f;
  }
  __device__ __forceinline__ void item_end(int, int, int, int) {}
  __device__ __forceinline__ void chunk(int row, int col0, const uint32_t (&r)[32], int M, int) {
    const int half = bn >> 1;
    const int j = col0 % bn;
    if (j < half) {
      if (j == 0) {
#pragma unroll
        for (int i = 0; i < 32; ++i) g0[i] = __uint_as_float(r[i]) * rs;
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) g1[i] = __uint_as_float(r[i]) * rs;
      }
      return;
    }
    const int jj = j - half;
    const int col = (col0 / bn) * half + jj;
    if (row >= M || col >= F) return;
    float o[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float g = jj == 0 ? g0[i] : g1[i];
      const float u = __uint_as_float(r[i]) * rs;
      o[i] = g / (1.f + __expf(-g)) * u;
    }
    __nv_bfloat16* d = D + static_cast<long long>(row) * ldd + col;
    if (col + 32 <= F && ((reinterpret_cast<uintptr_t>(d) & 15) == 0)) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 w;
        w.x = pack_bf16x2(o[i], o[i + 1]);
        w.y = pack_bf16x2(o[i + 2], o[i + 3]);
        w.z = pack_bf16x2(o[i + 4], o[i + 5]);
        w.w = pack_bf16x2(o[i + 6], o[i + 7]);
        *reinterpret_cast<uint4*>(d + i) = w;
      }
    } else {
      for (int i = 0; i < 32; ++i)
        if (col + i < F) d[i] = __float2bfloat16(o[i]);
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

// GEMM -> reduce-scatter in one kernel (FSDP / ZeRO-3 gradient path; replaces the per-block reduce-scatter that
// FSDP2 issues after each block's backward, gpu_process_worker.py:415-418, 696-713). The fp32 result tile is not
// stored locally: every element is added, with a vector `red` over NVLink, straight into the slice of the gradient
// shard that its OWNER rank holds. The unit is sharded evenly in flat order, owner r holding elements
// [r * n_per_owner, (r + 1) * n_per_owner) of the unit; `unit_rel` is where the weight matrix starts inside its unit.
// Reductions from all ranks and all microbatches meet in the owner's shard; the only synchronisation is one barrier
// before the optimizer reads it. Offsets and pitches are multiples of 4 elements and n_per_owner a multiple of 128,
// so a 16-byte group never straddles two owners.
struct ScatterReduceEpilogue {
  static constexpr int kMaxOwners = 8;
  float* dst[kMaxOwners];   // owner r's gradient shard, already offset to the unit's slice (peer addresses)
  long long n_per_owner;
  long long unit_rel;       // element offset of D[0, 0] inside the unit
  long long ldd;            // row pitch of the weight matrix in elements
  float alpha;

  // selects instead of a dynamic index, which would copy the pointer table to local memory
  __device__ __forceinline__ float* owner_base(int owner) const {
    float* b = dst[0];
#pragma unroll
    for (int r = 1; r < kMaxOwners; ++r)
      if (owner == r) b = dst[r];
    return b;
  }
  __device__ __forceinline__ void item_begin(int, int, int) {}
  __device__ __forceinline__ void item_end(int, int, int, int) {}
  __device__ __forceinline__ void chunk(int row, int col0, const uint32_t (&r)[32], int M, int N) {
    if (row >= M || col0 >= N) return;
    const long long flat = unit_rel + static_cast<long long>(row) * ldd + col0;
    int owner = static_cast<int>(flat / n_per_owner);
    long long off = flat - static_cast<long long>(owner) * n_per_owner;
    float* base = owner_base(owner);
    if (col0 + 32 <= N) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        if (off >= n_per_owner) { off -= n_per_owner; base = owner_base(++owner); }
        float* d = base + off;
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d), "f"(__uint_as_float(r[i]) * alpha),
                     "f"(__uint_as_float(r[i + 1]) * alpha), "f"(__uint_as_float(r[i + 2]) * alpha),
                     "f"(__uint_as_float(r[i + 3]) * alpha)
                     : "memory");
        off += 4;
      }
    } else {
      for (int i = 0; i < 32 && col0 + i < N; ++i) {
        if (off >= n_per_owner) { off -= n_per_owner; base = owner_base(++owner); }
        atomicAdd(base + off, __uint_as_float(r[i]) * alpha);
        off += 1;
      }
    }
  }
};

// Optional all-gather job fused into a GEMM launch (FSDP / ZeRO-3 parameter gather, the reference's FSDP2
// all-gather before each block, gpu_process_worker.py:415-418). The first `n_copy` CTAs of the grid do not compute:
// they pull the unit's shards out of every owner's memory over NVLink (plain peer loads) into a local staging
// buffer, chunk by chunk in flat order, and publish a ready flag per chunk. The GEMM CTAs of the SAME launch wait
// (bounded) for the chunks that cover the B rows of their tile before the first TMA load of that tile, so the
// transfer overlaps the math tile by tile. A launch may also gather a unit that a later GEMM consumes (prefetch).
struct NoGather {
  static constexpr bool kEnabled = false;
  int n_copy;
};

struct GatherJob {
  static constexpr bool kEnabled = true;
  static constexpr int kMaxOwners = 8;
  int n_copy;                              // copier CTAs at the front of the grid (0: wait-only launch)
  const __nv_bfloat16* src[kMaxOwners];    // owner r's slice of the unit (n_per_owner elements), peer addresses
  __nv_bfloat16* dst;                      // local staging buffer of the whole unit
  long long unit_elems;                    // world * n_per_owner
  long long n_per_owner;
  int world;
  int my_rank;
  unsigned long long* flags;               // [ceil(unit_elems / chunk_elems)] ready flags of dst
  unsigned long long epoch;                // value that marks "ready" for this gather
  int chunk_elems;                         // elements per flag (multiple of 8)
  long long b_unit_offset;                 // element offset of the GEMM's B matrix inside the unit; < 0: B is not in the unit
  long long b_row_elems;                   // row pitch of B in elements
  long long b_total_elems;                 // > 0: every tile waits for [b_unit_offset, b_unit_offset + b_total_elems)

  __device__ __forceinline__ const __nv_bfloat16* src_of(int owner) const {
    const __nv_bfloat16* b = src[0];
#pragma unroll
    for (int r = 1; r < kMaxOwners; ++r)
      if (owner == r) b = src[r];
    return b;
  }
  // Copier CTA: one thread streams pieces of the owners' slices into a shared-memory ring with bulk loads (the source
  // is peer memory for the other owners), a second thread drains the ring into the local staging buffer with bulk
  // stores and publishes the ready flag of each finished chunk. `full` / `empty` are mbarriers initialised to one
  // arrival each; every wait is bounded.
  __device__ __forceinline__ void copy_role(int cta, uint8_t* ring, uint32_t piece_bytes, int n_slots, uint64_t* full,
                                            uint64_t* empty, int* status) const {
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) != 0 || warp > 1) return;
    const long long piece_elems = piece_bytes / 2;
    const long long n_chunks = (unit_elems + chunk_elems - 1) / chunk_elems;
    int slot = 0;
    uint32_t phase = 0;
    int held = -1;  // storer: slot whose bulk store may still be reading shared memory
    for (long long c = cta; c < n_chunks; c += n_copy) {
      const long long a = c * chunk_elems;
      const long long b = (a + chunk_elems < unit_elems) ? a + chunk_elems : unit_elems;
      long long i = a;
      while (i < b) {
        const int owner = (int)(i / n_per_owner);
        const long long off = i - (long long)owner * n_per_owner;
        long long n = n_per_owner - off;  // a piece stays inside one owner's slice and one chunk
        if (n > b - i) n = b - i;
        if (n > piece_elems) n = piece_elems;
        const uint32_t bytes = (uint32_t)(n * 2);
        uint8_t* buf = ring + (size_t)slot * piece_bytes;
        if (warp == 0) {
          if (!mbar_wait(&empty[slot], phase ^ 1)) {
            report_status(status, kStatusPeerFlagTimeout);
            return;
          }
          mbar_expect_tx(&full[slot], bytes);
          bulk_load_g2s(buf, src_of(owner) + off, bytes, &full[slot]);
        } else {
          if (!mbar_wait(&full[slot], phase)) {
            report_status(status, kStatusPeerFlagTimeout);
            bulk_wait_all<0>();
            return;
          }
          bulk_store_s2g(dst + i, buf, bytes);
          bulk_commit();
          bulk_wait_read<1>();  // every store but the newest has finished reading its slot
          if (held >= 0) mbar_arrive(&empty[held]);
          held = slot;
        }
        i += n;
        if (++slot == n_slots) {
          slot = 0;
          phase ^= 1;
        }
      }
      if (warp == 1) {
        bulk_wait_all<0>();  // the chunk's stores are complete
        if (held >= 0) mbar_arrive(&empty[held]);
        held = -1;
        __threadfence();
        asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(flags + c), "l"(epoch) : "memory");
      }
    }
  }
  // Called by the TMA-issuing thread before it loads B rows [n0, n0 + rows).
  __device__ __forceinline__ bool wait_rows(int n0, int rows, int n_total) const {
    if (b_unit_offset < 0) return true;
    const int last_row = (n0 + rows < n_total ? n0 + rows : n_total);
    const long long a = b_unit_offset + (b_total_elems > 0 ? 0 : (long long)n0 * b_row_elems);
    const long long b = b_unit_offset + (b_total_elems > 0 ? b_total_elems : (long long)last_row * b_row_elems) - 1;
    const long long c0 = a / chunk_elems, c1 = b / chunk_elems;
    for (long long c = c0; c <= c1; ++c) {
      unsigned long long v;
      asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(flags + c) : "memory");
      if (v >= epoch) continue;
      const long long t0 = clock64();
      while (true) {
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(flags + c) : "memory");
        if (v >= epoch) break;
        if (clock64() - t0 > kWaitBudgetTicks) return false;
        __nanosleep(100);
      }
    }
    fence_proxy_async_all();  // staged by generic-proxy stores, read next by TMA (async proxy)
    return true;
  }
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

template <int BN, bool A_MN, bool B_MN, class Epi, class Gather = NoGather>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmShape p, Epi epi, const Gather gj) {
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
  // everything above (barriers, tensor-map prefetch, TMEM allocation) overlapped the previous kernel's tail
  pdl_wait();
  pdl_launch();
  const uint32_t tmem_base = *tmem_slot;
  // with a gather job the first n_copy CTAs are copiers and the work items are spread over the others
  const int first_cta = Gather::kEnabled ? gj.n_copy : 0;
  const int my_cta = (int)blockIdx.x - first_cta;
  const int cta_stride = (int)gridDim.x - first_cta;

  if constexpr (Gather::kEnabled) {
    // the ring reuses the operand stages; one stage-sized piece may be as large as 32 KB
    constexpr uint32_t kPiece = S::kStageBytes >= 32768 ? 32768u : 16384u;
    if (my_cta < 0) gj.copy_role((int)blockIdx.x, smem, kPiece, kStages, full_bar, empty_bar, p.status);
  }
  if (my_cta < 0) {
    // copier CTA: nothing else to do
  } else if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = my_cta; item < num_items && ok; item += cta_stride) {
        int tm, tn0, count;
        gemm_item_coords(item, tiles_m, tiles_n, p.group_n, tm, tn0, count);
        const int m0 = tm * kGemmBM;
        for (int t = 0; t < count && ok; ++t) {
          const int n0 = (tn0 + t) * BN;
          if constexpr (Gather::kEnabled) {
            if (!gj.wait_rows(n0, BN, p.N)) {
              report_status(p.status, kStatusPeerFlagTimeout);
              ok = false;
              break;
            }
          }
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
              if (p.dual_b > 0) {  // the tensor map's box is BN/2 rows high in this mode
                tma_load_2d(sb, &tmB, &full_bar[stage], k0, n0 / 2);
                tma_load_2d(sb + (BN / 2) * (kGemmBK * 2), &tmB, &full_bar[stage], k0, p.dual_b + n0 / 2);
              } else {
                tma_load_2d(sb, &tmB, &full_bar[stage], k0, n0);
              }
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
      for (int item = my_cta; item < num_items && ok; item += cta_stride) {
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
    for (int item = my_cta; item < num_items && ok; item += cta_stride) {
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
template <int BN, bool A_MN, bool B_MN, class Epi, class Gather = NoGather>
inline void gemm_launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmShape& p, const Epi& epi, int num_sms,
                        cudaStream_t stream, const Gather& gj = Gather{0}) {
  using S = GemmSmem<BN>;
  auto kernel = gemm_tcgen05_kernel<BN, A_MN, B_MN, Epi, Gather>;
  AGRPO_SET_MAX_DYN_SMEM(kernel, S::kTotal, "gemm smem attr");
  const int items = gemm_num_items(p.M, p.N, BN, p.group_n);
  // every CTA of the grid must be resident at once when CTAs wait on one another (copiers + workers <= SMs)
  const int n_copy = Gather::kEnabled ? gj.n_copy : 0;
  const int workers = items < num_sms - n_copy ? items : num_sms - n_copy;
  const int grid = workers + n_copy;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = S::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_flag() ? 1 : 0;
  check_cuda(cudaLaunchKernelEx(&cfg, kernel, ta, tb, p, epi, gj), "gemm_tcgen05 launch");
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("gemm_tcgen05 launch: ") + cudaGetErrorString(e));
}

}  // namespace agrpo
