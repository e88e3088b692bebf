// Host launcher for the tcgen05 GEMM (kernel in gemm_tcgen05.cuh).
#include "../common/tensormap.h"
#include "../launchers.h"
#include "gemm_tcgen05.cuh"

namespace agrpo {

namespace {

template <int BN, class Epi, class Gather>
void dispatch_major(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmShape& p,
                    const Epi& e, int sms, cudaStream_t s, const Gather& gj) {
  if (!a_mn && !b_mn) return gemm_launch<BN, false, false>(ta, tb, p, e, sms, s, gj);
  if (!a_mn && b_mn) return gemm_launch<BN, false, true>(ta, tb, p, e, sms, s, gj);
  if (a_mn && b_mn) return gemm_launch<BN, true, true>(ta, tb, p, e, sms, s, gj);
  return gemm_launch<BN, true, false>(ta, tb, p, e, sms, s, gj);
}

template <class Gather>
void launch_gemm_impl(const void* a, long long lda, const void* b, long long ldb, void* d, long long ldd, int M, int N,
                      int K, bool a_mn, bool b_mn, const void* bias, float alpha, bool out_fp32, bool accumulate,
                      int* status, int num_sms, cudaStream_t stream, const void* residual, long long ldr,
                      const Gather& gj) {
  // Widest column tile that still yields about one work item per SM; the 64 / 32 wide tiles serve
  // skinny decode-time GEMMs (K-major operands only) where the weight stream must be spread over all SMs.
  const int tiles_m = (M + kGemmBM - 1) / kGemmBM;
  const bool plain = !a_mn && !b_mn;
  const int cands[4] = {256, 128, 64, 32};
  int BN = plain ? 32 : 128;
  for (int i = 0; i < (plain ? 4 : 2); ++i) {
    const int bn = cands[i];
    if ((long long)tiles_m * ((N + bn - 1) / bn) >= 120) {
      BN = bn;
      break;
    }
  }
  CUtensorMap ta, tb;
  if (!a_mn) ta = make_tmap_2d(a, K, M, lda, 64, kGemmBM);
  else       ta = make_tmap_2d(a, M, K, lda, 64, 64);
  if (!b_mn) tb = make_tmap_2d(b, K, N, ldb, 64, BN);
  else       tb = make_tmap_2d(b, N, K, ldb, 64, 64);
  GemmShape p;
  p.M = M; p.N = N; p.K = K;
  p.group_n = 1;
  p.status = status;
  StoreEpilogue e;
  e.D = d;
  e.ldd = ldd;
  e.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  e.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  e.ldr = ldr;
  e.alpha = alpha;
  e.out_fp32 = out_fp32 ? 1 : 0;
  e.accumulate = accumulate ? 1 : 0;
  if (BN == 256) dispatch_major<256>(a_mn, b_mn, ta, tb, p, e, num_sms, stream, gj);
  else if (BN == 128) dispatch_major<128>(a_mn, b_mn, ta, tb, p, e, num_sms, stream, gj);
  else if (BN == 64) gemm_launch<64, false, false>(ta, tb, p, e, num_sms, stream, gj);
  else gemm_launch<32, false, false>(ta, tb, p, e, num_sms, stream, gj);
}

// Copies one sharded unit out of its owners' memory with no GEMM to ride on (the first unit of a pass).
constexpr int kGatherSlots = 8;
constexpr uint32_t kGatherPiece = 16384;
constexpr int kGatherSmem = kGatherSlots * kGatherPiece + 1024 + 256;

__global__ void __launch_bounds__(64) unit_gather_kernel(const GatherJob gj, int* status) {
  extern __shared__ uint8_t gather_smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gather_smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + kGatherSlots * kGatherPiece);
  uint64_t* empty = full + kGatherSlots;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kGatherSlots; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    fence_mbar_init();
  }
  __syncthreads();
  gj.copy_role((int)blockIdx.x, ring, kGatherPiece, kGatherSlots, full, empty, status);
}

}  // namespace

// d[M,N] = alpha * op(a) . op(b)^T (+ bias) (+ d); see launchers.h for the operand conventions.
void launch_gemm_bf16(const void* a, long long lda, const void* b, long long ldb, void* d, long long ldd, int M, int N,
                      int K, bool a_mn, bool b_mn, const void* bias, float alpha, bool out_fp32, bool accumulate,
                      int* status, int num_sms, cudaStream_t stream, const void* residual, long long ldr) {
  if (!a_mn && !b_mn && !out_fp32 && !accumulate && alpha == 1.f && M <= 256 &&
      launch_gemm_skinny(a, lda, b, ldb, d, ldd, M, N, K, bias, residual, ldr, status, num_sms, stream))
    return;
  launch_gemm_impl(a, lda, b, ldb, d, ldd, M, N, K, a_mn, b_mn, bias, alpha, out_fp32, accumulate, status, num_sms,
                   stream, residual, ldr, NoGather{0});
}

namespace {
GatherJob make_gather_job(const GatherArgs& g, int n_copy) {
  GatherJob gj{};
  gj.n_copy = n_copy;
  for (int r = 0; r < g.world && r < GatherJob::kMaxOwners; ++r)
    gj.src[r] = reinterpret_cast<const __nv_bfloat16*>(g.src[r]);
  gj.dst = reinterpret_cast<__nv_bfloat16*>(g.dst);
  gj.unit_elems = g.n_per_owner * g.world;
  gj.n_per_owner = g.n_per_owner;
  gj.world = g.world;
  gj.my_rank = g.my_rank;
  gj.flags = reinterpret_cast<unsigned long long*>(g.flags);
  gj.epoch = g.epoch;
  gj.chunk_elems = g.chunk_elems;
  gj.b_unit_offset = -1;
  gj.b_row_elems = 0;
  gj.b_total_elems = 0;
  return gj;
}
bool gather_args_ok(const GatherArgs& g) {
  return g.world >= 1 && g.world <= GatherJob::kMaxOwners && g.n_per_owner > 0 && g.n_per_owner % 8 == 0 &&
         g.chunk_elems > 0 && g.chunk_elems % 8 == 0 && g.dst && g.flags;
}
}  // namespace

// GEMM with an all-gather job in the same launch (see GatherJob in gemm_tcgen05.cuh). `b_unit_offset` >= 0 says that
// B lives inside the unit being gathered, at that element offset of the staging buffer: the producer warp then waits
// for the chunks under each tile before it loads them. With b_unit_offset < 0 the job is a prefetch for later GEMMs.
bool launch_ag_gemm_bf16(const void* a, long long lda, const void* b, long long ldb, void* d, long long ldd, int M,
                         int N, int K, bool a_mn, bool b_mn, const void* bias, float alpha, bool out_fp32,
                         bool accumulate, int* status, int num_sms, cudaStream_t stream, const void* residual,
                         long long ldr, const GatherArgs& g, int n_copy, long long b_unit_offset) {
  if (!gather_args_ok(g) || n_copy < 1 || n_copy > num_sms / 2) return false;
  GatherJob gj = make_gather_job(g, n_copy);
  if (b_unit_offset >= 0) {
    gj.b_unit_offset = b_unit_offset;
    gj.b_row_elems = ldb;
    // an MN-major B is read across all of its rows by every tile: wait for the whole matrix
    gj.b_total_elems = b_mn ? (long long)(K - 1) * ldb + N : 0;
  }
  launch_gemm_impl(a, lda, b, ldb, d, ldd, M, N, K, a_mn, b_mn, bias, alpha, out_fp32, accumulate, status, num_sms,
                   stream, residual, ldr, gj);
  return true;
}

// d_owner[flat] += alpha * op(a) . op(b)^T, every element added into the gradient shard of the rank that owns it.
bool launch_gemm_rs_bf16(const void* a, long long lda, const void* b, long long ldb, int M, int N, int K, bool a_mn, bool b_mn,
                         float alpha, const ScatterArgs& sc, long long unit_rel, long long ldd, int* status, int num_sms,
                         cudaStream_t stream) {
  if (sc.world < 1 || sc.world > ScatterReduceEpilogue::kMaxOwners || sc.n_per_owner <= 0 || sc.n_per_owner % 128 != 0 ||
      unit_rel % 4 != 0 || ldd % 4 != 0 || unit_rel < 0 ||
      unit_rel + (long long)(M - 1) * ldd + N > sc.n_per_owner * sc.world)
    return false;
  const int tiles_m = (M + kGemmBM - 1) / kGemmBM;
  const int BN = ((long long)tiles_m * ((N + 255) / 256) >= 120) ? 256 : 128;
  CUtensorMap ta, tb;
  if (!a_mn) ta = make_tmap_2d(a, K, M, lda, 64, kGemmBM);
  else       ta = make_tmap_2d(a, M, K, lda, 64, 64);
  if (!b_mn) tb = make_tmap_2d(b, K, N, ldb, 64, BN);
  else       tb = make_tmap_2d(b, N, K, ldb, 64, 64);
  GemmShape p;
  p.M = M; p.N = N; p.K = K;
  p.group_n = 1;
  p.status = status;
  ScatterReduceEpilogue e;
  for (int r = 0; r < ScatterReduceEpilogue::kMaxOwners; ++r)
    e.dst[r] = r < sc.world ? reinterpret_cast<float*>(sc.dst[r]) : nullptr;
  e.n_per_owner = sc.n_per_owner;
  e.unit_rel = unit_rel;
  e.ldd = ldd;
  e.alpha = alpha;
  if (BN == 256) dispatch_major<256>(a_mn, b_mn, ta, tb, p, e, num_sms, stream, NoGather{0});
  else dispatch_major<128>(a_mn, b_mn, ta, tb, p, e, num_sms, stream, NoGather{0});
  return true;
}

// act[M, F] = silu(rs * (a . Wg^T)) * (rs * (a . Wu^T)) with b = [Wg; Wu] stacked ([2F, K], the fused gate/up weight).
bool launch_gemm_swiglu_bf16(const void* a, long long lda, const void* b, long long ldb, void* d, long long ldd, int M, int F,
                             int K, const long long* ss_in, float eps, int* status, int num_sms, cudaStream_t stream) {
  if (F % 8 != 0 || M <= 0 || F <= 0) return false;
  const int tiles_m = (M + kGemmBM - 1) / kGemmBM;
  const int BN = ((long long)tiles_m * ((2 * F + 127) / 128) >= 120) ? 128 : 64;
  const CUtensorMap ta = make_tmap_2d(a, K, M, lda, 64, kGemmBM);
  const CUtensorMap tb = make_tmap_2d(b, K, 2 * F, ldb, 64, BN / 2);
  GemmShape p;
  p.M = M; p.N = 2 * ((F + BN / 2 - 1) / (BN / 2)) * (BN / 2); p.K = K;
  p.group_n = 1;
  p.status = status;
  p.dual_b = F;
  SwigluEpilogue e;
  e.D = reinterpret_cast<__nv_bfloat16*>(d);
  e.ldd = ldd;
  e.F = F;
  e.bn = BN;
  e.ss_in = ss_in;
  e.inv_k = 1.f / (float)K;
  e.eps = eps;
  if (BN == 128) gemm_launch<128, false, false>(ta, tb, p, e, num_sms, stream);
  else gemm_launch<64, false, false>(ta, tb, p, e, num_sms, stream);
  return true;
}

bool launch_unit_gather(const GatherArgs& g, int n_ctas, int* status, cudaStream_t stream) {
  if (!gather_args_ok(g) || n_ctas < 1) return false;
  GatherJob gj = make_gather_job(g, n_ctas);
  AGRPO_SET_MAX_DYN_SMEM(unit_gather_kernel, kGatherSmem, "unit_gather attr");
  unit_gather_kernel<<<n_ctas, 64, kGatherSmem, stream>>>(gj, status);
  check_cuda(cudaGetLastError(), "unit_gather_kernel");
  return true;
}

}  // namespace agrpo
