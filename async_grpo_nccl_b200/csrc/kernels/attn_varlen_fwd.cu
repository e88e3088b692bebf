// Causal varlen (packed, padding-free) flash-attention forward with native GQA on tcgen05.
//
// Replaces the flash_attn_varlen_func call the reference reaches through its FA2 monkey-patch
// (gpu_process_worker.py:164-305), without repeating K/V heads for GQA (gpu_process_worker.py:156-162)
// and without the host sync that computes max_seqlen (gpu_process_worker.py:252): the host packer
// supplies the query-tile table.
//
// One CTA = one 128-row query tile of one head. S = Q K^T and O += P V run on tcgen05 with S/P and O
// in tensor memory: the softmax warps read S with tcgen05.ld (one thread per query row), write P back
// as packed bf16 over the same columns with tcgen05.st, and the P V MMA takes P straight from TMEM.
// K and V tiles arrive by TMA. Two CTAs fit per SM (96 KB shared memory, 256 TMEM columns each) so
// one CTA's softmax overlaps the other's MMAs.
#include <cuda_bf16.h>

#include "../common/ptx.cuh"
#include "../common/tensormap.h"
#include "../launchers.h"

namespace agrpo {

namespace {

constexpr int kBM = 128;  // query rows per CTA
constexpr int kBN = 128;  // keys per inner tile
constexpr int kAttnThreads = 192;

struct AttnFwdParams {
  const int4* tiles;  // {seq_start, seq_len, q0, unused}
  __nv_bfloat16* out;  // [T, Hq*D]
  float* lse;          // [Hq, T]
  long long ldo;
  int T;
  int q_col0, k_col0, v_col0;  // column of head 0 of q / k / v inside the TMA-mapped matrices
  int group;                   // query heads per kv head
  float scale_log2;            // softmax scale * log2(e)
  int* status;
};

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
  constexpr int kChunks = D / 64;                // 128-byte swizzle atoms along the head dim
  constexpr int kTileBytes = kBM * D * 2;        // one Q / K / V tile
  constexpr uint32_t kTmemCols = 256;            // S/P: [0,128), O: [128, 128+D)
  constexpr uint32_t kIdescS = umma_idesc_bf16(kBM, kBN, 0, 0);
  constexpr uint32_t kIdescO = umma_idesc_bf16(kBM, D, 0, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTileBytes;
  uint8_t* sV = smem + 2 * kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * kTileBytes);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;
  uint64_t* v_full = bars + 2;
  uint64_t* s_full = bars + 3;
  uint64_t* p_ready = bars + 4;
  uint64_t* o_done = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x;
  const int kv_head = head / p.group;
  const int4 tile = p.tiles[blockIdx.y];
  const int seq_start = tile.x, seq_len = tile.y, q0 = tile.z;
  const int n_kv = q0 / kBN + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 4);
    mbar_init(o_done, 1);
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
  const uint32_t tmem_S = tmem_base;
  const uint32_t tmem_O = tmem_base + 128;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(q_full, kTileBytes);
#pragma unroll
      for (int c = 0; c < kChunks; ++c)
        tma_load_2d(sQ + c * (kBM * 128), &tmQ, q_full, p.q_col0 + head * D + c * 64, seq_start + q0);
      for (int j = 0; j < n_kv; ++j) {
        const int row = seq_start + j * kBN;
        if (j > 0 && !mbar_wait(s_full, (j - 1) & 1)) {
          report_status(p.status, kStatusWaitEmptyTimeout);
          break;
        }
        mbar_expect_tx(k_full, kTileBytes);
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          tma_load_2d(sK + c * (kBN * 128), &tmK, k_full, p.k_col0 + kv_head * D + c * 64, row);
        if (j > 0 && !mbar_wait(o_done, (j - 1) & 1)) {
          report_status(p.status, kStatusWaitEmptyTimeout);
          break;
        }
        mbar_expect_tx(v_full, kTileBytes);
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          tma_load_2d(sV + c * (kBN * 128), &tmV, v_full, p.v_col0 + kv_head * D + c * 64, row);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      bool ok = mbar_wait(q_full, 0);
      if (!ok) report_status(p.status, kStatusWaitFullTimeout);
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (!mbar_wait(k_full, j & 1)) {
          report_status(p.status, kStatusWaitFullTimeout);
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (kBM * 128) + (k % 4) * 32;
          tc_mma_f16(tmem_S, umma_smem_desc(aQ + off, 16, 1024), umma_smem_desc(aK + off, 16, 1024), kIdescS,
                     k > 0 ? 1u : 0u);
        }
        tc_commit(s_full);
        if (!mbar_wait(p_ready, j & 1)) {
          report_status(p.status, kStatusWaitTmemFullTimeout);
          break;
        }
        if (!mbar_wait(v_full, j & 1)) {
          report_status(p.status, kStatusWaitFullTimeout);
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kBN / 16; ++k) {
          tc_mma_f16_ts(tmem_O, tmem_S + k * 8, umma_smem_desc(aV + k * 2048, kBN * 128, 1024), kIdescO,
                        (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(o_done);
      }
    }
  } else {
    // Softmax / correction / epilogue: thread = one query row.
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int qi = q0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    float m = -INFINITY;  // running (possibly stale) max, log2 domain
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(s_full, j & 1)) {
        report_status(p.status, kStatusWaitTmemFullTimeout);
        ok = false;
        break;
      }
      tc_fence_after();
      const bool diag = (j == n_kv - 1);
      const int key0 = j * kBN;
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t s[32];
        tmem_ld_32x32(tmem_S + lane_off + c * 32, s);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(s[i]);
          if (diag && (key0 + c * 32 + i > qi)) v = -INFINITY;
          mx = fmaxf(mx, v);
        }
      }
      mx *= p.scale_log2;
      float m_new = m;
      float alpha = 1.f;
      // Keep a stale maximum unless it grew by more than 2^8: P stays bounded and O rarely needs rescaling.
      if (mx > m + 8.f) {
        m_new = mx;
        alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
      }
      if (m_new == -INFINITY) m_new = 0.f;  // fully masked row so far
      const bool need = (j > 0) && (alpha != 1.f);
      if (j > 0) {
        // O of the previous tile must be complete before it is rescaled or before P is overwritten.
        if (!mbar_wait(o_done, (j - 1) & 1)) {
          report_status(p.status, kStatusWaitTmemFullTimeout);
          ok = false;
          break;
        }
        tc_fence_after();
      }
      if (__any_sync(0xffffffffu, need)) {
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_O + lane_off + c * 32, o);
          tc_wait_ld();
          uint32_t lo[16], hi[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            lo[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            hi[i] = __float_as_uint(__uint_as_float(o[16 + i]) * alpha);
          }
          tmem_st_32x16(tmem_O + lane_off + c * 32, lo);
          tmem_st_32x16(tmem_O + lane_off + c * 32 + 16, hi);
        }
      }
      l *= alpha;
      m = m_new;
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t s[32];
        tmem_ld_32x32(tmem_S + lane_off + c * 32, s);
        tc_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = exp2f(__uint_as_float(s[i]) * p.scale_log2 - m);
          float p1 = exp2f(__uint_as_float(s[i + 1]) * p.scale_log2 - m);
          if (diag) {
            if (key0 + c * 32 + i > qi) p0 = 0.f;
            if (key0 + c * 32 + i + 1 > qi) p1 = 0.f;
          }
          l += p0 + p1;
          pk[i / 2] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x16(tmem_S + lane_off + c * 16, pk);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    if (ok && mbar_wait(o_done, (n_kv - 1) & 1)) {
      tc_fence_after();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const bool valid = qi < seq_len;
      const long long t = (long long)seq_start + qi;
      __nv_bfloat16* dst = p.out + t * p.ldo + (long long)head * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_O + lane_off + c * 32, o);
        tc_wait_ld();
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[i]) * inv_l, __uint_as_float(o[i + 1]) * inv_l);
            w.y = pack_bf16x2(__uint_as_float(o[i + 2]) * inv_l, __uint_as_float(o[i + 3]) * inv_l);
            w.z = pack_bf16x2(__uint_as_float(o[i + 4]) * inv_l, __uint_as_float(o[i + 5]) * inv_l);
            w.w = pack_bf16x2(__uint_as_float(o[i + 6]) * inv_l, __uint_as_float(o[i + 7]) * inv_l);
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = w;
          }
        }
      }
      if (valid && p.lse != nullptr)
        p.lse[(long long)head * p.T + t] = (l > 0.f) ? (m * 0.6931471805599453f + logf(l)) : -INFINITY;
    } else if (ok) {
      report_status(p.status, kStatusWaitTmemFullTimeout);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int D>
void launch_fwd_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnFwdParams& p, int n_tiles,
                  int Hq, cudaStream_t s) {
  constexpr int smem = 3 * kBM * D * 2 + 128 + 1024;
  auto kernel = attn_fwd_kernel<D>;
  AGRPO_SET_MAX_DYN_SMEM(kernel, smem, "attn_fwd smem attr");
  dim3 grid(Hq, n_tiles);
  kernel<<<grid, kAttnThreads, smem, s>>>(tq, tk, tv, p);
  check_cuda(cudaGetLastError(), "attn_fwd launch");
}

}  // namespace

void launch_attn_varlen_fwd(const void* q, long long ldq, int q_cols, const void* k, long long ldk, int k_cols,
                            const void* v, long long ldv, int v_cols, int q_col0, int k_col0, int v_col0, void* out,
                            long long ldo, float* lse, const int* tiles, int n_tiles, int T, int Hq, int Hkv, int D,
                            float softmax_scale, int* status, cudaStream_t s) {
  if (n_tiles == 0 || T == 0) return;
  if (D != 64 && D != 128) throw std::runtime_error("attn_varlen_fwd: head_dim must be 64 or 128");
  const CUtensorMap tq = make_tmap_2d(q, q_cols, T, ldq, 64, kBM);
  const CUtensorMap tk = make_tmap_2d(k, k_cols, T, ldk, 64, kBN);
  const CUtensorMap tv = make_tmap_2d(v, v_cols, T, ldv, 64, kBN);
  AttnFwdParams p;
  p.tiles = reinterpret_cast<const int4*>(tiles);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.ldo = ldo;
  p.T = T;
  p.q_col0 = q_col0;
  p.k_col0 = k_col0;
  p.v_col0 = v_col0;
  p.group = Hq / Hkv;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  if (D == 128) launch_fwd_t<128>(tq, tk, tv, p, n_tiles, Hq, s);
  else          launch_fwd_t<64>(tq, tk, tv, p, n_tiles, Hq, s);
}

}  // namespace agrpo
