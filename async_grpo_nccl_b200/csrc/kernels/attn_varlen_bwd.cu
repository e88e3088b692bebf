// Causal varlen flash-attention backward with native GQA on tcgen05.
//
// The reference gets this pass from flash-attn's autograd function behind flash_attn_varlen_func
// (gpu_process_worker.py:265-276), on K/V that were first repeated to the query head count.
//
// One CTA owns one 128-key tile of one kv head and walks over the query heads of its group and the
// query tiles at or below the diagonal. Per step five tcgen05 GEMMs run with every accumulator in
// tensor memory (512 columns: S^T/P^T/dQ, dP^T/dS^T, dV, dK):
//   S^T  = K Q^T          dP^T = V dO^T                 (operands from shared memory, TMA-fed)
//   dV  += P^T dO         dK  += dS^T Q                 (A operand read back from tensor memory)
//   dQ   = dS K                                         (dS^T staged in shared memory, MN-major)
// dK / dV leave as bf16 once per CTA; dQ partial tiles are added to an fp32 accumulator with vector
// reductions and converted by attn_bwd_finalize_dq.
#include <cuda_bf16.h>

#include "../common/ptx.cuh"
#include "../common/tensormap.h"
#include "../launchers.h"

namespace agrpo {

namespace {

constexpr int kT = 128;  // tile edge (keys per CTA, queries per step)
constexpr int kBwdThreads = 192;

struct AttnBwdParams {
  const int4* tiles;  // {seq_start, seq_len, k0, unused}
  const float* lse;   // [Hq, T]
  const float* delta; // [Hq, T]
  float* dq_acc;      // [T, Hq*D] fp32, zeroed by the caller
  __nv_bfloat16* dk;  // row pitch ldk, head h at column dk_col0 + h*D
  __nv_bfloat16* dv;
  long long ld_dk, ld_dv;
  int dk_col0, dv_col0;
  int T, Hq, group;
  int q_col0, k_col0, v_col0;
  float scale, scale_log2;
  int* status;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                const AttnBwdParams p) {
  constexpr int kChunks = D / 64;
  constexpr int kTileBytes = kT * D * 2;
  constexpr int kChunkBytes = kT * 128;     // one 64-column swizzle chunk of a 128-row tile
  constexpr int kDsBytes = kT * kT * 2;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kIdescST = umma_idesc_bf16(kT, kT, 0, 0);  // S^T, dP^T: both operands K-major
  constexpr uint32_t kIdescKV = umma_idesc_bf16(kT, D, 0, 1);   // dV, dK: A from TMEM, B MN-major
  constexpr uint32_t kIdescDQ = umma_idesc_bf16(kT, D, 1, 1);   // dQ: A (dS^T in smem) MN-major, B MN-major

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + kTileBytes;
  uint8_t* sQ = sV + kTileBytes;           // two stages
  uint8_t* sDO = sQ + 2 * kTileBytes;
  uint8_t* sDS = sDO + kTileBytes;
  float* sLse = reinterpret_cast<float*>(sDS + kDsBytes);  // [2][128]
  float* sDelta = sLse + 2 * kT;                           // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDelta + 2 * kT);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;   // [2]
  uint64_t* q_empty = bars + 3;  // [2]
  uint64_t* do_full = bars + 5;
  uint64_t* sdp_full = bars + 6;
  uint64_t* pds_ready = bars + 7;
  uint64_t* dv_done = bars + 8;
  uint64_t* dq_full = bars + 9;
  uint64_t* dq_read = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_head = blockIdx.x;
  // The table is sorted for the forward pass (heaviest query tile first); the heaviest key tile is the last.
  const int4 tile = p.tiles[gridDim.y - 1 - blockIdx.y];
  const int seq_start = tile.x, seq_len = tile.y, k0 = tile.z;
  const int n_q = (seq_len - k0 + kT - 1) / kT;
  const int n_it = n_q * p.group;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(&q_full[0], 1);
    mbar_init(&q_full[1], 1);
    mbar_init(&q_empty[0], 1);
    mbar_init(&q_empty[1], 1);
    mbar_init(do_full, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_ready, 4);
    mbar_init(dv_done, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_read, 4);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_R1 = tmem_base;        // S^T -> P^T (bf16) -> dQ
  const uint32_t tmem_R2 = tmem_base + 128;  // dP^T -> dS^T (bf16)
  const uint32_t tmem_dV = tmem_base + 256;
  const uint32_t tmem_dK = tmem_base + 256 + D;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(kv_full, 2 * kTileBytes);
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        tma_load_2d(sK + c * kChunkBytes, &tmK, kv_full, p.k_col0 + kv_head * D + c * 64, seq_start + k0);
        tma_load_2d(sV + c * kChunkBytes, &tmV, kv_full, p.v_col0 + kv_head * D + c * 64, seq_start + k0);
      }
      for (int it = 0; it < n_it; ++it) {
        const int hg = it / n_q, qt = it - hg * n_q;
        const int head = kv_head * p.group + hg;
        const int row = seq_start + k0 + qt * kT;
        const int s = it & 1;
        if (it >= 2 && !mbar_wait(&q_empty[s], ((it >> 1) - 1) & 1)) {
          report_status(p.status, kStatusWaitEmptyTimeout);
          break;
        }
        mbar_expect_tx(&q_full[s], kTileBytes);
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          tma_load_2d(sQ + s * kTileBytes + c * kChunkBytes, &tmQ, &q_full[s], p.q_col0 + head * D + c * 64, row);
        if (it >= 1 && !mbar_wait(dv_done, (it - 1) & 1)) {
          report_status(p.status, kStatusWaitEmptyTimeout);
          break;
        }
        mbar_expect_tx(do_full, kTileBytes);
#pragma unroll
        for (int c = 0; c < kChunks; ++c) tma_load_2d(sDO + c * kChunkBytes, &tmDO, do_full, head * D + c * 64, row);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      bool ok = mbar_wait(kv_full, 0);
      if (!ok) report_status(p.status, kStatusWaitFullTimeout);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aDO = smem_u32(sDO), aDS = smem_u32(sDS);
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1;
        const uint32_t aQ = smem_u32(sQ + s * kTileBytes);
        if (!mbar_wait(&q_full[s], (it >> 1) & 1) || !mbar_wait(do_full, it & 1)) {
          report_status(p.status, kStatusWaitFullTimeout);
          break;
        }
        if (it >= 1 && !mbar_wait(dq_read, (it - 1) & 1)) {
          report_status(p.status, kStatusWaitTmemEmptyTimeout);
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * kChunkBytes + (k % 4) * 32;
          tc_mma_f16(tmem_R1, umma_smem_desc(aK + off, 16, 1024), umma_smem_desc(aQ + off, 16, 1024), kIdescST,
                     k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * kChunkBytes + (k % 4) * 32;
          tc_mma_f16(tmem_R2, umma_smem_desc(aV + off, 16, 1024), umma_smem_desc(aDO + off, 16, 1024), kIdescST,
                     k > 0 ? 1u : 0u);
        }
        tc_commit(sdp_full);
        if (!mbar_wait(pds_ready, it & 1)) {
          report_status(p.status, kStatusWaitTmemFullTimeout);
          break;
        }
        tc_fence_after();
        // dV += P^T dO   (A: P^T packed bf16 in R1, B: dO as [N = D, K = queries], MN-major)
#pragma unroll
        for (int k = 0; k < kT / 16; ++k)
          tc_mma_f16_ts(tmem_dV, tmem_R1 + k * 8, umma_smem_desc(aDO + k * 2048, kChunkBytes, 1024), kIdescKV,
                        (it > 0 || k > 0) ? 1u : 0u);
        tc_commit(dv_done);
        // dK += dS^T Q
#pragma unroll
        for (int k = 0; k < kT / 16; ++k)
          tc_mma_f16_ts(tmem_dK, tmem_R2 + k * 8, umma_smem_desc(aQ + k * 2048, kChunkBytes, 1024), kIdescKV,
                        (it > 0 || k > 0) ? 1u : 0u);
        tc_commit(&q_empty[s]);
        // dQ = dS K      (A: dS^T tile in shared memory read MN-major, B: K as [N = D, K = keys], MN-major)
#pragma unroll
        for (int k = 0; k < kT / 16; ++k)
          tc_mma_f16(tmem_R1, umma_smem_desc(aDS + k * 2048, kChunkBytes, 1024),
                     umma_smem_desc(aK + k * 2048, kChunkBytes, 1024), kIdescDQ, k > 0 ? 1u : 0u);
        tc_commit(dq_full);
      }
    }
  } else {
    // Compute warps: thread = one key row (P^T / dS^T) and, for the dQ read-out, one query row.
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int kj = k0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int hg = it / n_q, qt = it - hg * n_q;
      const int head = kv_head * p.group + hg;
      const int q0 = k0 + qt * kT;
      const int b = it & 1;
      {
        const int qi = q0 + r;
        const bool valid = qi < seq_len;
        const long long idx = (long long)head * p.T + seq_start + qi;
        sLse[b * kT + r] = valid ? p.lse[idx] * 1.4426950408889634f : INFINITY;
        sDelta[b * kT + r] = valid ? p.delta[idx] : 0.f;
      }
      named_bar_sync(1, 128);
      if (!mbar_wait(sdp_full, it & 1)) {
        report_status(p.status, kStatusWaitTmemFullTimeout);
        ok = false;
        break;
      }
      tc_fence_after();
      const bool diag = (qt == 0);
#pragma unroll 1
      for (int c = 0; c < kT / 32; ++c) {
        uint32_t sv[32], dp[32];
        tmem_ld_32x32(tmem_R1 + lane_off + c * 32, sv);
        tmem_ld_32x32(tmem_R2 + lane_off + c * 32, dp);
        tc_wait_ld();
        uint32_t pk[16], dsk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const int qa = c * 32 + i;
          float p0 = exp2f(__uint_as_float(sv[i]) * p.scale_log2 - sLse[b * kT + qa]);
          float p1 = exp2f(__uint_as_float(sv[i + 1]) * p.scale_log2 - sLse[b * kT + qa + 1]);
          if (diag) {
            if (kj > q0 + qa) p0 = 0.f;
            if (kj > q0 + qa + 1) p1 = 0.f;
          }
          float d0 = p0 * (__uint_as_float(dp[i]) - sDelta[b * kT + qa]) * p.scale;
          float d1 = p1 * (__uint_as_float(dp[i + 1]) - sDelta[b * kT + qa + 1]) * p.scale;
          if (p0 == 0.f) d0 = 0.f;
          if (p1 == 0.f) d1 = 0.f;
          pk[i / 2] = pack_bf16x2(p0, p1);
          dsk[i / 2] = pack_bf16x2(d0, d1);
        }
        tmem_st_32x16(tmem_R1 + lane_off + c * 16, pk);
        tmem_st_32x16(tmem_R2 + lane_off + c * 16, dsk);
        // dS^T row r, queries [32c, 32c+32) into the 128-byte-swizzled [keys x queries] tile.
        uint8_t* rowp = sDS + (c >> 1) * kChunkBytes + r * 128;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int unit = ((c & 1) * 4 + u) ^ (r & 7);
          *reinterpret_cast<uint4*>(rowp + unit * 16) = make_uint4(dsk[u * 4], dsk[u * 4 + 1], dsk[u * 4 + 2], dsk[u * 4 + 3]);
        }
      }
      tc_wait_st();
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_ready);

      if (!mbar_wait(dq_full, it & 1)) {
        report_status(p.status, kStatusWaitTmemFullTimeout);
        ok = false;
        break;
      }
      tc_fence_after();
      {
        const int qi = q0 + r;
        const bool valid = qi < seq_len;
        float* dst = p.dq_acc + ((long long)seq_start + qi) * ((long long)p.Hq * D) + (long long)head * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_R1 + lane_off + c * 32, o);
          tc_wait_ld();
          if (valid) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              red_add_v4(dst + c * 32 + i, __uint_as_float(o[i]), __uint_as_float(o[i + 1]), __uint_as_float(o[i + 2]),
                         __uint_as_float(o[i + 3]));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_read);
    }
    if (ok && n_it > 0) {
      // The last dq_full wait also covered the final dV / dK MMAs (commits are cumulative).
      const bool valid = kj < seq_len;
      const long long t = (long long)seq_start + kj;
      __nv_bfloat16* dvp = p.dv + t * p.ld_dv + p.dv_col0 + (long long)kv_head * D;
      __nv_bfloat16* dkp = p.dk + t * p.ld_dk + p.dk_col0 + (long long)kv_head * D;
#pragma unroll 1
      for (int c = 0; c < 2 * D / 32; ++c) {
        const bool is_k = c >= D / 32;
        const int cc = is_k ? c - D / 32 : c;
        uint32_t o[32];
        tmem_ld_32x32((is_k ? tmem_dK : tmem_dV) + lane_off + cc * 32, o);
        tc_wait_ld();
        if (valid) {
          __nv_bfloat16* dst = (is_k ? dkp : dvp) + cc * 32;
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[i]), __uint_as_float(o[i + 1]));
            w.y = pack_bf16x2(__uint_as_float(o[i + 2]), __uint_as_float(o[i + 3]));
            w.z = pack_bf16x2(__uint_as_float(o[i + 4]), __uint_as_float(o[i + 5]));
            w.w = pack_bf16x2(__uint_as_float(o[i + 6]), __uint_as_float(o[i + 7]));
            *reinterpret_cast<uint4*>(dst + i) = w;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (t, h).
__global__ void attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                      float* __restrict__ delta, int T, int Hq, int D, long long ldo, long long lddo) {
  const long long w = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)T * Hq) return;
  const int lane = threadIdx.x & 31;
  const int t = (int)(w / Hq), h = (int)(w % Hq);
  const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(o + (long long)t * ldo + (long long)h * D);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(d_o + (long long)t * lddo + (long long)h * D);
  float acc = 0.f;
  for (int i = lane; i < D / 2; i += 32) {
    const float2 x = __bfloat1622float2(a[i]);
    const float2 y = __bfloat1622float2(b[i]);
    acc += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[(long long)h * T + t] = acc;
}

// dq (bf16, pitch ld, first `cols` columns of each row) = dq_acc (fp32 [T, cols]).
__global__ void attn_bwd_finalize_dq_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long T,
                                            int cols, long long ld) {
  const long long total = T * (cols / 4);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / (cols / 4);
    const int c = (int)(i % (cols / 4)) * 4;
    const float4 v = *reinterpret_cast<const float4*>(acc + t * cols + c);
    uint2 w;
    w.x = pack_bf16x2(v.x, v.y);
    w.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(dq + t * ld + c) = w;
  }
}

template <int D>
void launch_bwd_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                  const AttnBwdParams& p, int n_tiles, int Hkv, cudaStream_t s) {
  constexpr int smem = 5 * kT * D * 2 + kT * kT * 2 + 4 * kT * 4 + 128 + 1024;
  auto kernel = attn_bwd_kernel<D>;
  AGRPO_SET_MAX_DYN_SMEM(kernel, smem, "attn_bwd smem attr");
  dim3 grid(Hkv, n_tiles);
  kernel<<<grid, kBwdThreads, smem, s>>>(tq, tk, tv, tdo, p);
  check_cuda(cudaGetLastError(), "attn_bwd launch");
}

}  // namespace

void launch_attn_varlen_bwd(const void* q, long long ldq, int q_cols, const void* k, long long ldk, int k_cols,
                            const void* v, long long ldv, int v_cols, int q_col0, int k_col0, int v_col0, const void* out,
                            long long ldo, const void* dout, long long lddo, const float* lse, float* delta, float* dq_acc,
                            void* dq, long long ld_dq, void* dk, long long ld_dk, int dk_col0, void* dv, long long ld_dv,
                            int dv_col0, const int* tiles, int n_tiles, int T, int Hq, int Hkv, int D, float softmax_scale,
                            int* status, cudaStream_t s) {
  if (n_tiles == 0 || T == 0) return;
  if (D != 64 && D != 128) throw std::runtime_error("attn_varlen_bwd: head_dim must be 64 or 128");
  {
    const long long warps = (long long)T * Hq;
    attn_bwd_delta_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, s>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)dout,
                                                                     delta, T, Hq, D, ldo, lddo);
    check_cuda(cudaGetLastError(), "attn_bwd_delta");
  }
  check_cuda(cudaMemsetAsync(dq_acc, 0, (size_t)T * Hq * D * sizeof(float), s), "attn_bwd dq memset");
  const CUtensorMap tq = make_tmap_2d(q, q_cols, T, ldq, 64, kT);
  const CUtensorMap tk = make_tmap_2d(k, k_cols, T, ldk, 64, kT);
  const CUtensorMap tv = make_tmap_2d(v, v_cols, T, ldv, 64, kT);
  const CUtensorMap tdo = make_tmap_2d(dout, (uint64_t)Hq * D, T, lddo, 64, kT);
  AttnBwdParams p;
  p.tiles = reinterpret_cast<const int4*>(tiles);
  p.lse = lse;
  p.delta = delta;
  p.dq_acc = dq_acc;
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.ld_dk = ld_dk;
  p.ld_dv = ld_dv;
  p.dk_col0 = dk_col0;
  p.dv_col0 = dv_col0;
  p.T = T;
  p.Hq = Hq;
  p.group = Hq / Hkv;
  p.q_col0 = q_col0;
  p.k_col0 = k_col0;
  p.v_col0 = v_col0;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  if (D == 128) launch_bwd_t<128>(tq, tk, tv, tdo, p, n_tiles, Hkv, s);
  else          launch_bwd_t<64>(tq, tk, tv, tdo, p, n_tiles, Hkv, s);
  {
    const long long work = (long long)T * (Hq * D / 4);
    long long blocks = (work + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    attn_bwd_finalize_dq_kernel<<<(unsigned)blocks, 256, 0, s>>>(dq_acc, (__nv_bfloat16*)dq, T, Hq * D, ld_dq);
    check_cuda(cudaGetLastError(), "attn_bwd_finalize_dq");
  }
}

}  // namespace agrpo
