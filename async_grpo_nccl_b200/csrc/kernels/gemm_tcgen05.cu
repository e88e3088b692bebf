// Host launcher for the tcgen05 GEMM (kernel in gemm_tcgen05.cuh).
#include "../common/tensormap.h"
#include "../launchers.h"
#include "gemm_tcgen05.cuh"

namespace agrpo {

namespace {

template <int BN>
void dispatch_major(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmShape& p,
                    const StoreEpilogue& e, int sms, cudaStream_t s) {
  if (!a_mn && !b_mn) return gemm_launch<BN, false, false>(ta, tb, p, e, sms, s);
  if (!a_mn && b_mn) return gemm_launch<BN, false, true>(ta, tb, p, e, sms, s);
  if (a_mn && b_mn) return gemm_launch<BN, true, true>(ta, tb, p, e, sms, s);
  return gemm_launch<BN, true, false>(ta, tb, p, e, sms, s);
}

}  // namespace

// d[M,N] = alpha * op(a) . op(b)^T (+ bias) (+ d); see launchers.h for the operand conventions.
void launch_gemm_bf16(const void* a, long long lda, const void* b, long long ldb, void* d, long long ldd, int M, int N,
                      int K, bool a_mn, bool b_mn, const void* bias, float alpha, bool out_fp32, bool accumulate,
                      int* status, int num_sms, cudaStream_t stream, const void* residual, long long ldr) {
  if (!a_mn && !b_mn && !out_fp32 && !accumulate && alpha == 1.f && M <= 256 &&
      launch_gemm_skinny(a, lda, b, ldb, d, ldd, M, N, K, bias, residual, ldr, status, num_sms, stream))
    return;
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
  if (BN == 256) dispatch_major<256>(a_mn, b_mn, ta, tb, p, e, num_sms, stream);
  else if (BN == 128) dispatch_major<128>(a_mn, b_mn, ta, tb, p, e, num_sms, stream);
  else if (BN == 64) gemm_launch<64, false, false>(ta, tb, p, e, num_sms, stream);
  else gemm_launch<32, false, false>(ta, tb, p, e, num_sms, stream);
}

}  // namespace agrpo
