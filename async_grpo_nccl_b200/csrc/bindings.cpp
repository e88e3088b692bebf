// Python bindings: tensor checks here, raw-pointer launchers in the .cu files.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <cstdlib>

#include <pybind11/numpy.h>
#include <pybind11/stl.h>

#include "host/kv_allocator.h"
#include "host/packer.h"
#include "launchers.h"

namespace {

using torch::Tensor;
using OptTensor = c10::optional<torch::Tensor>;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream(); }
// Per-thread cap on the SMs that persistent kernels (GEMMs, lm_head) launched from this thread may fill. A trainer or
// logprob thread that shares its GPU with a rollout engine can leave a few SMs to the latency-bound decode kernels.
inline int& sm_limit() {
  static thread_local int v = 0;
  return v;
}
inline int num_sms() {
  const int n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int lim = sm_limit();
  return (lim > 0 && lim < n) ? lim : n;
}

inline void check_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, ": CUDA tensor required");
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16, name, ": bf16 required");
}
inline void check_f32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, ": CUDA tensor required");
  TORCH_CHECK(t.scalar_type() == torch::kFloat32, name, ": fp32 required");
}
inline void check_i64(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, ": CUDA tensor required");
  TORCH_CHECK(t.scalar_type() == torch::kInt64, name, ": int64 required (row sums of squares are fixed point, value * 2^30)");
}
inline long long* opt_i64(const OptTensor& t) {
  return (t.has_value() && t->defined()) ? reinterpret_cast<long long*>(t->data_ptr<int64_t>()) : nullptr;
}
inline void check_i32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, ": CUDA tensor required");
  TORCH_CHECK(t.scalar_type() == torch::kInt32, name, ": int32 required");
}
template <typename T>
inline T* opt_ptr(const OptTensor& t) {
  return (t.has_value() && t->defined()) ? reinterpret_cast<T*>(t->data_ptr()) : nullptr;
}

void gemm_bf16(const Tensor& a, const Tensor& b, Tensor& d, bool a_mn, bool b_mn, const OptTensor& bias, double alpha,
               bool accumulate, const OptTensor& status, const OptTensor& residual) {
  check_bf16(a, "gemm a");
  check_bf16(b, "gemm b");
  TORCH_CHECK(d.is_cuda() && (d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat32), "gemm d");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && d.dim() == 2, "gemm: 2-D tensors");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && d.stride(1) == 1, "gemm: inner stride must be 1");
  const c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  const int64_t Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm: K mismatch ", K, " vs ", Kb);
  TORCH_CHECK(d.size(0) == M && d.size(1) == N, "gemm: output shape mismatch");
  if (M == 0 || N == 0) return;
  TORCH_CHECK(K > 0, "gemm: K must be positive");
  TORCH_CHECK(a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0, "gemm: row pitch must be a multiple of 8 elements");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(a.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(b.data_ptr()) & 15) == 0,
              "gemm: operands must be 16-byte aligned");
  if (bias.has_value() && bias->defined()) {
    check_bf16(*bias, "gemm bias");
    TORCH_CHECK(bias->numel() == N && bias->is_contiguous(), "gemm: bias must be contiguous [N]");
  }
  if (status.has_value() && status->defined()) check_i32(*status, "gemm status");
  long long ldr = 0;
  if (residual.has_value() && residual->defined()) {
    check_bf16(*residual, "gemm residual");
    TORCH_CHECK(residual->dim() == 2 && residual->size(0) == M && residual->size(1) == N && residual->stride(1) == 1, "gemm: residual [M, N]");
    ldr = residual->stride(0);
  }
  agrpo::launch_gemm_bf16(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), d.data_ptr(), d.stride(0), (int)M, (int)N,
                          (int)K, a_mn, b_mn, opt_ptr<void>(bias), (float)alpha, d.scalar_type() == torch::kFloat32,
                          accumulate, opt_ptr<int>(status), num_sms(), cur_stream(), opt_ptr<void>(residual), ldr);
}

// Runs the skinny split-K GEMM with its phase tracer on; returns false when the shape is not served by that kernel.
bool gemm_skinny_trace(const Tensor& a, const Tensor& b, Tensor& d, Tensor& trace) {
  check_bf16(a, "a"); check_bf16(b, "b"); check_bf16(d, "d");
  TORCH_CHECK(trace.is_cuda() && trace.scalar_type() == torch::kInt64 && trace.numel() >= 16, "trace: int64[16] cuda");
  const c10::cuda::CUDAGuard guard(a.device());
  return agrpo::launch_gemm_skinny(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), d.data_ptr(), d.stride(0), (int)a.size(0),
                                   (int)b.size(0), (int)a.size(1), nullptr, nullptr, 0, nullptr, num_sms(), cur_stream(),
                                   reinterpret_cast<long long*>(trace.data_ptr<int64_t>()));
}

void embedding_fwd(const Tensor& ids, const Tensor& table, Tensor& out) {
  check_i32(ids, "ids"); check_bf16(table, "table"); check_bf16(out, "out");
  TORCH_CHECK(table.is_contiguous() && out.is_contiguous() && table.size(1) % 8 == 0, "embedding_fwd layout");
  const c10::cuda::CUDAGuard guard(table.device());
  agrpo::launch_embedding_fwd(ids.data_ptr<int>(), table.data_ptr(), out.data_ptr(), (int)ids.numel(), (int)table.size(1),
                              (int)table.size(0), cur_stream());
}
void embedding_sumsq(const Tensor& ids, const Tensor& table, Tensor& out, Tensor& ss) {
  check_i32(ids, "ids"); check_bf16(table, "table"); check_bf16(out, "out"); check_i64(ss, "ss");
  TORCH_CHECK(table.is_contiguous() && out.is_contiguous() && table.size(1) % 8 == 0, "embedding_sumsq layout");
  TORCH_CHECK(ss.dim() == 2 && ss.stride(1) == 1 && ss.size(1) >= ids.numel(), "embedding_sumsq: ss [n, >= rows]");
  const c10::cuda::CUDAGuard guard(table.device());
  agrpo::launch_embedding_sumsq(ids.data_ptr<int>(), table.data_ptr(), out.data_ptr(), reinterpret_cast<long long*>(ss.data_ptr<int64_t>()), (int)ss.size(0),
                                (int)ss.stride(0), (int)ids.numel(), (int)table.size(1), (int)table.size(0), cur_stream());
}
void fold_norm_weight(const Tensor& w, const Tensor& g, Tensor& out) {
  check_bf16(w, "w"); check_bf16(g, "g"); check_bf16(out, "out");
  TORCH_CHECK(w.dim() == 2 && w.is_contiguous() && out.is_contiguous() && out.numel() == w.numel() && g.is_contiguous() &&
              g.numel() == w.size(1) && w.size(1) % 8 == 0, "fold_norm_weight layout");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(w.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(out.data_ptr()) & 15) == 0 &&
              (reinterpret_cast<uintptr_t>(g.data_ptr()) & 15) == 0, "fold_norm_weight: 16-byte alignment");
  const c10::cuda::CUDAGuard guard(w.device());
  agrpo::launch_fold_norm_weight(w.data_ptr(), g.data_ptr(), out.data_ptr(), w.size(0), (int)w.size(1), cur_stream());
}
// Decode-step GEMMs (M <= 256, K-major operands). gemm_decode runs the cluster split-K kernel with the optional folded
// RMSNorm row scale (ss_in) and row sum-of-squares output (ss_out); it returns false, having launched nothing, when
// that kernel does not serve the shape. gemm_swiglu fuses the gate/up projection with SwiGLU.
bool gemm_decode(const Tensor& a, const Tensor& b, Tensor& d, const OptTensor& bias, const OptTensor& residual, const OptTensor& ss_in,
                 const OptTensor& ss_out, double eps, const OptTensor& status) {
  check_bf16(a, "gemm_decode a"); check_bf16(b, "gemm_decode b"); check_bf16(d, "gemm_decode d");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && d.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && d.stride(1) == 1, "gemm_decode: 2-D");
  const int64_t M = a.size(0), K = a.size(1), N = b.size(0);
  TORCH_CHECK(b.size(1) == K && d.size(0) == M && d.size(1) == N, "gemm_decode: shape mismatch");
  TORCH_CHECK(a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0, "gemm_decode: row pitch must be a multiple of 8 elements");
  if (ss_in.has_value() && ss_in->defined()) { check_i64(*ss_in, "ss_in"); TORCH_CHECK(ss_in->numel() >= M && ss_in->is_contiguous(), "ss_in [M]"); }
  if (ss_out.has_value() && ss_out->defined()) { check_i64(*ss_out, "ss_out"); TORCH_CHECK(ss_out->numel() >= M && ss_out->is_contiguous(), "ss_out [M]"); }
  if (status.has_value() && status->defined()) check_i32(*status, "gemm_decode status");
  long long ldr = 0;
  if (residual.has_value() && residual->defined()) { check_bf16(*residual, "residual"); ldr = residual->stride(0); }
  if (bias.has_value() && bias->defined()) check_bf16(*bias, "bias");
  const c10::cuda::CUDAGuard guard(a.device());
  return agrpo::launch_gemm_skinny(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), d.data_ptr(), d.stride(0), (int)M, (int)N,
                                   (int)K, opt_ptr<void>(bias), opt_ptr<void>(residual), ldr, opt_ptr<int>(status), num_sms(),
                                   cur_stream(), nullptr, opt_i64(ss_in), opt_i64(ss_out), (float)eps);
}
int64_t gemm_skinny_splits(int64_t M, int64_t N, int64_t K) { return agrpo::gemm_skinny_splits((int)M, (int)N, (int)K, num_sms()); }
void gemm_swiglu(const Tensor& a, const Tensor& b, Tensor& d, const OptTensor& ss_in, double eps, const OptTensor& status) {
  check_bf16(a, "gemm_swiglu a"); check_bf16(b, "gemm_swiglu b"); check_bf16(d, "gemm_swiglu d");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && d.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && d.stride(1) == 1, "gemm_swiglu: 2-D");
  const int64_t M = a.size(0), K = a.size(1), F = d.size(1);
  TORCH_CHECK(b.size(0) == 2 * F && b.size(1) == K && d.size(0) == M, "gemm_swiglu: b must be the stacked [2F, K] gate/up weight");
  TORCH_CHECK(a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0 && F % 8 == 0, "gemm_swiglu: pitches and F must be multiples of 8");
  if (ss_in.has_value() && ss_in->defined()) { check_i64(*ss_in, "ss_in"); TORCH_CHECK(ss_in->numel() >= M && ss_in->is_contiguous(), "ss_in [M]"); }
  if (status.has_value() && status->defined()) check_i32(*status, "gemm_swiglu status");
  const c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(agrpo::launch_gemm_swiglu_bf16(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), d.data_ptr(), d.stride(0), (int)M,
                                             (int)F, (int)K, opt_i64(ss_in), (float)eps, opt_ptr<int>(status), num_sms(),
                                             cur_stream()),
              "gemm_swiglu: arguments not served");
}
void embedding_bwd(const Tensor& ids, const Tensor& dout, Tensor& dtable) {
  check_i32(ids, "ids"); check_bf16(dout, "dout"); check_f32(dtable, "dtable");
  TORCH_CHECK(dtable.is_contiguous() && dout.is_contiguous(), "embedding_bwd layout");
  const c10::cuda::CUDAGuard guard(dout.device());
  agrpo::launch_embedding_bwd(ids.data_ptr<int>(), dout.data_ptr(), dtable.data_ptr<float>(), (int)ids.numel(),
                              (int)dtable.size(1), (int)dtable.size(0), cur_stream());
}
void rmsnorm_fwd(const Tensor& x, const Tensor& w, Tensor& y, const OptTensor& rstd, double eps) {
  check_bf16(x, "x"); check_bf16(w, "w"); check_bf16(y, "y");
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && w.is_contiguous() && x.size(-1) % 8 == 0, "rmsnorm_fwd layout");
  const int H = (int)x.size(-1);
  const int T = (int)(x.numel() / H);
  const c10::cuda::CUDAGuard guard(x.device());
  agrpo::launch_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), opt_ptr<float>(rstd), T, H, (float)eps, cur_stream());
}
void rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd, Tensor& dx, const OptTensor& dw,
                 bool accumulate_dx) {
  check_bf16(dy, "dy"); check_bf16(x, "x"); check_bf16(w, "w"); check_f32(rstd, "rstd"); check_bf16(dx, "dx");
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous() && dx.is_contiguous(), "rmsnorm_bwd layout");
  const int H = (int)x.size(-1);
  const int T = (int)(x.numel() / H);
  const c10::cuda::CUDAGuard guard(x.device());
  agrpo::launch_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(),
                            opt_ptr<float>(dw), T, H, accumulate_dx, cur_stream());
}
void colsum(const Tensor& a, Tensor& out) {
  check_bf16(a, "a"); check_f32(out, "out");
  TORCH_CHECK(a.dim() == 2 && a.stride(1) == 1 && a.stride(0) % 2 == 0 && out.numel() == a.size(1), "colsum layout");
  const c10::cuda::CUDAGuard guard(a.device());
  agrpo::launch_colsum(a.data_ptr(), out.data_ptr<float>(), (int)a.size(0), (int)a.size(1), a.stride(0), cur_stream());
}
void rope_inplace(Tensor& qkv, const Tensor& pos, const Tensor& cos_t, const Tensor& sin_t, int64_t n_rot_heads,
                  int64_t head_dim, bool backward) {
  check_bf16(qkv, "qkv"); check_i32(pos, "pos"); check_f32(cos_t, "cos"); check_f32(sin_t, "sin");
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1, "rope: qkv [T, C]");
  TORCH_CHECK(cos_t.is_contiguous() && sin_t.is_contiguous() && cos_t.size(1) == head_dim / 2, "rope tables");
  TORCH_CHECK(n_rot_heads * head_dim <= qkv.size(1), "rope: heads exceed row");
  const c10::cuda::CUDAGuard guard(qkv.device());
  agrpo::launch_rope(qkv.data_ptr(), pos.data_ptr<int>(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(),
                     (int)qkv.size(0), (int)n_rot_heads, (int)head_dim, qkv.stride(0), (int)cos_t.size(0), backward,
                     cur_stream());
}
void swiglu_fwd(const Tensor& gu, Tensor& out) {
  check_bf16(gu, "gu"); check_bf16(out, "out");
  TORCH_CHECK(gu.is_contiguous() && out.is_contiguous() && gu.size(-1) == 2 * out.size(-1) && out.size(-1) % 8 == 0, "swiglu layout");
  const int F = (int)out.size(-1);
  const c10::cuda::CUDAGuard guard(gu.device());
  agrpo::launch_swiglu_fwd(gu.data_ptr(), out.data_ptr(), (int)(out.numel() / F), F, cur_stream());
}
void swiglu_bwd(const Tensor& gu, const Tensor& dout, Tensor& dgu) {
  check_bf16(gu, "gu"); check_bf16(dout, "dout"); check_bf16(dgu, "dgu");
  TORCH_CHECK(gu.is_contiguous() && dout.is_contiguous() && dgu.is_contiguous(), "swiglu_bwd layout");
  const int F = (int)dout.size(-1);
  const c10::cuda::CUDAGuard guard(gu.device());
  agrpo::launch_swiglu_bwd(gu.data_ptr(), dout.data_ptr(), dgu.data_ptr(), (int)(dout.numel() / F), F, cur_stream());
}
void add_bf16(const Tensor& a, const Tensor& b, Tensor& out) {
  check_bf16(a, "a"); check_bf16(b, "b"); check_bf16(out, "out");
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && out.is_contiguous() && a.numel() == b.numel() && a.numel() % 8 == 0, "add layout");
  const c10::cuda::CUDAGuard guard(a.device());
  agrpo::launch_add_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), cur_stream());
}
void sumsq(const Tensor& g, double scale, Tensor& out) {
  check_f32(g, "g"); check_f32(out, "out");
  TORCH_CHECK(g.is_contiguous(), "sumsq layout");
  const c10::cuda::CUDAGuard guard(g.device());
  agrpo::launch_sumsq(g.data_ptr<float>(), g.numel(), (float)scale, out.data_ptr<float>(), cur_stream());
}
void adamw_step(Tensor& p, Tensor& m, Tensor& v, Tensor& g, const OptTensor& p16, double lr, double beta1, double beta2,
                double eps, double wd, int64_t step, double grad_scale, const OptTensor& norm_sq, double max_norm,
                bool zero_grad) {
  check_f32(p, "p"); check_f32(m, "m"); check_f32(v, "v"); check_f32(g, "g");
  TORCH_CHECK(p.is_contiguous() && m.is_contiguous() && v.is_contiguous() && g.is_contiguous(), "adamw layout");
  TORCH_CHECK(p.numel() == m.numel() && p.numel() == v.numel() && p.numel() == g.numel(), "adamw sizes");
  if (p16.has_value() && p16->defined()) { check_bf16(*p16, "p16"); TORCH_CHECK(p16->numel() == p.numel() && p16->is_contiguous(), "p16"); }
  const c10::cuda::CUDAGuard guard(p.device());
  agrpo::launch_adamw(p.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), g.data_ptr<float>(), opt_ptr<void>(p16),
                      p.numel(), (float)lr, (float)beta1, (float)beta2, (float)eps, (float)wd, (int)step, (float)grad_scale,
                      opt_ptr<float>(norm_sq), (float)max_norm, zero_grad, cur_stream());
}
void cast_f32_bf16(const Tensor& in, Tensor& out) {
  check_f32(in, "in"); check_bf16(out, "out");
  TORCH_CHECK(in.is_contiguous() && out.is_contiguous() && in.numel() == out.numel(), "cast layout");
  const c10::cuda::CUDAGuard guard(in.device());
  agrpo::launch_cast_f32_bf16(in.data_ptr<float>(), out.data_ptr(), in.numel(), cur_stream());
}

// qkv: [T, (Hq + 2*Hkv) * D] fused projection output (q heads, then k heads, then v heads).
void attn_varlen_fwd(const Tensor& qkv, Tensor& out, const OptTensor& lse, const Tensor& tiles, int64_t Hq, int64_t Hkv,
                     int64_t D, double softmax_scale, const OptTensor& status) {
  check_bf16(qkv, "qkv"); check_bf16(out, "out"); check_i32(tiles, "tiles");
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.size(1) == (Hq + 2 * Hkv) * D, "attn: qkv shape");
  TORCH_CHECK(out.dim() == 2 && out.stride(1) == 1 && out.size(1) == Hq * D && out.size(0) == qkv.size(0), "attn: out shape");
  TORCH_CHECK(tiles.is_contiguous() && tiles.dim() == 2 && tiles.size(1) == 4, "attn: tiles [n,4]");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(tiles.data_ptr()) & 15) == 0, "attn: tile table must be 16-byte aligned");
  TORCH_CHECK(qkv.stride(0) % 8 == 0 && out.stride(0) % 8 == 0, "attn: pitches must be multiples of 8");
  if (lse.has_value() && lse->defined()) { check_f32(*lse, "lse"); TORCH_CHECK(lse->is_contiguous() && lse->numel() == Hq * qkv.size(0), "attn: lse [Hq,T]"); }
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int T = (int)qkv.size(0);
  const int C = (int)qkv.size(1);
  agrpo::launch_attn_varlen_fwd(qkv.data_ptr(), qkv.stride(0), C, qkv.data_ptr(), qkv.stride(0), C, qkv.data_ptr(),
                                qkv.stride(0), C, 0, (int)(Hq * D), (int)((Hq + Hkv) * D), out.data_ptr(), out.stride(0),
                                opt_ptr<float>(lse), tiles.data_ptr<int>(), (int)tiles.size(0), T, (int)Hq, (int)Hkv, (int)D,
                                (float)softmax_scale, opt_ptr<int>(status), cur_stream());
}

// dqkv: [T, (Hq + 2*Hkv) * D] receives dq | dk | dv. delta [Hq, T] and dq_acc [T, Hq*D] are fp32 scratch.
void attn_varlen_bwd(const Tensor& qkv, const Tensor& out, const Tensor& dout, const Tensor& lse, Tensor& delta,
                     Tensor& dq_acc, Tensor& dqkv, const Tensor& tiles, int64_t Hq, int64_t Hkv, int64_t D,
                     double softmax_scale, const OptTensor& status) {
  check_bf16(qkv, "qkv"); check_bf16(out, "out"); check_bf16(dout, "dout"); check_bf16(dqkv, "dqkv");
  check_f32(lse, "lse"); check_f32(delta, "delta"); check_f32(dq_acc, "dq_acc"); check_i32(tiles, "tiles");
  const int64_t T = qkv.size(0), C = (Hq + 2 * Hkv) * D;
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.size(1) == C, "attn_bwd: qkv shape");
  TORCH_CHECK(dqkv.dim() == 2 && dqkv.stride(1) == 1 && dqkv.size(1) == C && dqkv.size(0) == T, "attn_bwd: dqkv shape");
  TORCH_CHECK(out.size(0) == T && out.size(1) == Hq * D && out.stride(1) == 1, "attn_bwd: out shape");
  TORCH_CHECK(dout.size(0) == T && dout.size(1) == Hq * D && dout.stride(1) == 1, "attn_bwd: dout shape");
  TORCH_CHECK(lse.is_contiguous() && lse.numel() == Hq * T && delta.is_contiguous() && delta.numel() == Hq * T, "attn_bwd: lse/delta");
  TORCH_CHECK(dq_acc.is_contiguous() && dq_acc.numel() == T * Hq * D, "attn_bwd: dq_acc");
  TORCH_CHECK(tiles.is_contiguous() && tiles.dim() == 2 && tiles.size(1) == 4, "attn_bwd: tiles [n,4]");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(tiles.data_ptr()) & 15) == 0, "attn_bwd: tile table must be 16-byte aligned");
  TORCH_CHECK(qkv.stride(0) % 8 == 0 && dout.stride(0) % 8 == 0 && dqkv.stride(0) % 8 == 0, "attn_bwd: pitches");
  const c10::cuda::CUDAGuard guard(qkv.device());
  agrpo::launch_attn_varlen_bwd(qkv.data_ptr(), qkv.stride(0), (int)C, qkv.data_ptr(), qkv.stride(0), (int)C, qkv.data_ptr(),
                                qkv.stride(0), (int)C, 0, (int)(Hq * D), (int)((Hq + Hkv) * D), out.data_ptr(), out.stride(0),
                                dout.data_ptr(), dout.stride(0), lse.data_ptr<float>(), delta.data_ptr<float>(),
                                dq_acc.data_ptr<float>(), dqkv.data_ptr(), dqkv.stride(0), dqkv.data_ptr(), dqkv.stride(0),
                                (int)(Hq * D), dqkv.data_ptr(), dqkv.stride(0), (int)((Hq + Hkv) * D), tiles.data_ptr<int>(),
                                (int)tiles.size(0), (int)T, (int)Hq, (int)Hkv, (int)D, (float)softmax_scale,
                                opt_ptr<int>(status), cur_stream());
}

int64_t lmhead_num_groups(int64_t V, int64_t T) { return agrpo::lmhead_num_groups((int)V, (int)T); }
int64_t grpo_num_loss_stats() { return agrpo::grpo_num_loss_stats(); }

void lmhead_logprob(const Tensor& hidden, const Tensor& weight, const Tensor& labels, double temperature, Tensor& partials,
                    Tensor& label_logit, const OptTensor& logp, const OptTensor& entropy, const OptTensor& lse,
                    const OptTensor& status) {
  check_bf16(hidden, "hidden"); check_bf16(weight, "weight"); check_i32(labels, "labels");
  check_f32(partials, "partials"); check_f32(label_logit, "label_logit");
  TORCH_CHECK(hidden.dim() == 2 && weight.dim() == 2 && hidden.stride(1) == 1 && weight.stride(1) == 1, "lmhead: 2-D");
  const int64_t T = hidden.size(0), H = hidden.size(1), V = weight.size(0);
  TORCH_CHECK(weight.size(1) == H && labels.numel() == T && labels.is_contiguous(), "lmhead: shapes");
  TORCH_CHECK(hidden.stride(0) % 8 == 0 && weight.stride(0) % 8 == 0, "lmhead: pitches");
  TORCH_CHECK(partials.numel() >= 3 * agrpo::lmhead_num_groups((int)V, (int)T) * T && label_logit.numel() >= T, "lmhead: scratch");
  for (const OptTensor* o : {&logp, &entropy, &lse})
    if (o->has_value() && (*o)->defined()) { check_f32(**o, "lmhead out"); TORCH_CHECK((*o)->numel() == T && (*o)->is_contiguous(), "lmhead out [T]"); }
  const c10::cuda::CUDAGuard guard(hidden.device());
  agrpo::launch_lmhead_logprob(hidden.data_ptr(), hidden.stride(0), weight.data_ptr(), weight.stride(0), labels.data_ptr<int>(),
                               (int)T, (int)H, (int)V, (float)temperature, partials.data_ptr<float>(),
                               label_logit.data_ptr<float>(), opt_ptr<float>(logp), opt_ptr<float>(entropy), opt_ptr<float>(lse),
                               opt_ptr<int>(status), num_sms(), cur_stream());
}

void grpo_token_loss(const Tensor& logp, const OptTensor& old_logp, const OptTensor& ref_logp, const Tensor& adv,
                     const Tensor& labels, const OptTensor& entropy, const OptTensor& old_entropy, double clip_low,
                     double clip_high, double clip_c, double kl_beta, double grad_weight, const OptTensor& dlogp,
                     Tensor& stats) {
  check_f32(logp, "logp"); check_f32(adv, "adv"); check_i32(labels, "labels"); check_f32(stats, "stats");
  const int64_t T = logp.numel();
  TORCH_CHECK(adv.numel() == T && labels.numel() == T && stats.numel() >= agrpo::grpo_num_loss_stats(), "grpo_token_loss shapes");
  for (const OptTensor* o : {&old_logp, &ref_logp, &entropy, &old_entropy, &dlogp})
    if (o->has_value() && (*o)->defined()) { check_f32(**o, "grpo_token_loss opt"); TORCH_CHECK((*o)->numel() == T, "grpo_token_loss opt [T]"); }
  const c10::cuda::CUDAGuard guard(logp.device());
  agrpo::launch_grpo_token_loss(logp.data_ptr<float>(), opt_ptr<float>(old_logp), opt_ptr<float>(ref_logp), adv.data_ptr<float>(),
                                labels.data_ptr<int>(), opt_ptr<float>(entropy), opt_ptr<float>(old_entropy), (int)T,
                                (float)clip_low, (float)clip_high, (float)clip_c, (float)kl_beta, (float)grad_weight,
                                opt_ptr<float>(dlogp), stats.data_ptr<float>(), cur_stream());
}

void lmhead_backward(const Tensor& hidden, const Tensor& weight, const Tensor& labels, const Tensor& lse, const Tensor& dlogp,
                     double temperature, Tensor& dz_chunk, Tensor& dh_acc, const OptTensor& dweight, const OptTensor& status) {
  check_bf16(hidden, "hidden"); check_bf16(weight, "weight"); check_i32(labels, "labels"); check_f32(lse, "lse");
  check_f32(dlogp, "dlogp"); check_bf16(dz_chunk, "dz_chunk"); check_f32(dh_acc, "dh_acc");
  const int64_t T = hidden.size(0), H = hidden.size(1), V = weight.size(0);
  TORCH_CHECK(dz_chunk.dim() == 2 && dz_chunk.is_contiguous() && dz_chunk.size(0) >= T && dz_chunk.size(1) % 256 == 0, "lmhead_bwd: dz_chunk [T, 256k]");
  TORCH_CHECK(dh_acc.is_contiguous() && dh_acc.numel() == T * H, "lmhead_bwd: dh_acc");
  TORCH_CHECK(hidden.stride(1) == 1 && weight.stride(1) == 1 && hidden.stride(0) % 8 == 0 && weight.stride(0) % 8 == 0, "lmhead_bwd: layout");
  float* dw = nullptr; long long ld_dw = 0;
  if (dweight.has_value() && dweight->defined()) {
    check_f32(*dweight, "dweight");
    TORCH_CHECK(dweight->dim() == 2 && dweight->size(0) == V && dweight->size(1) == H && dweight->stride(1) == 1, "lmhead_bwd: dweight");
    dw = dweight->data_ptr<float>(); ld_dw = dweight->stride(0);
  }
  const c10::cuda::CUDAGuard guard(hidden.device());
  agrpo::launch_lmhead_backward(hidden.data_ptr(), hidden.stride(0), weight.data_ptr(), weight.stride(0), labels.data_ptr<int>(),
                                lse.data_ptr<float>(), dlogp.data_ptr<float>(), (int)T, (int)H, (int)V, (float)temperature,
                                dz_chunk.data_ptr(), (int)dz_chunk.size(1), dh_acc.data_ptr<float>(), dw, ld_dw,
                                opt_ptr<int>(status), num_sms(), cur_stream());
}

void kv_cache_write(const Tensor& qkv, const Tensor& slots, Tensor& k_cache, Tensor& v_cache, int64_t Hq, int64_t Hkv, int64_t D,
                    const OptTensor& status, int64_t kv_head0) {
  check_bf16(qkv, "qkv"); check_i32(slots, "slots"); check_bf16(k_cache, "k_cache"); check_bf16(v_cache, "v_cache");
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.size(1) == (Hq + 2 * Hkv) * D && qkv.stride(0) % 8 == 0, "kv_cache_write: qkv");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous() && k_cache.size(1) + kv_head0 <= Hkv && kv_head0 >= 0 && k_cache.size(3) == D,
              "kv_cache_write: cache [blocks, kv heads of this rank, bs, D]");
  TORCH_CHECK(slots.numel() == qkv.size(0), "kv_cache_write: slots");
  const c10::cuda::CUDAGuard guard(qkv.device());
  // a tensor-parallel rank caches kv heads [kv_head0, kv_head0 + k_cache.size(1)) of the Hkv heads in qkv
  agrpo::launch_kv_cache_write(qkv.data_ptr(), qkv.stride(0), (int)((Hq + kv_head0) * D), (int)((Hq + Hkv + kv_head0) * D), slots.data_ptr<int>(),
                               k_cache.data_ptr(), v_cache.data_ptr(), (int)qkv.size(0), (int)k_cache.size(1), (int)D, (int)k_cache.size(2),
                               (int)k_cache.size(0), opt_ptr<int>(status), cur_stream());
}

void kv_cache_write_decode(const Tensor& qkv, const Tensor& block_tables, const Tensor& seq_lens, Tensor& k_cache,
                           Tensor& v_cache, int64_t Hq, int64_t Hkv, int64_t D, const OptTensor& status) {
  check_bf16(qkv, "qkv"); check_i32(block_tables, "block_tables"); check_i32(seq_lens, "seq_lens");
  check_bf16(k_cache, "k_cache"); check_bf16(v_cache, "v_cache");
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.size(1) == (Hq + 2 * Hkv) * D && qkv.stride(0) % 8 == 0, "kv_write_decode: qkv");
  TORCH_CHECK(block_tables.dim() == 2 && block_tables.stride(1) == 1 && block_tables.size(0) >= qkv.size(0) && seq_lens.numel() >= qkv.size(0), "kv_write_decode: tables");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous(), "kv_write_decode: cache");
  const c10::cuda::CUDAGuard guard(qkv.device());
  agrpo::launch_kv_cache_write_decode(qkv.data_ptr(), qkv.stride(0), (int)(Hq * D), (int)((Hq + Hkv) * D),
                                      block_tables.data_ptr<int>(), (int)block_tables.stride(0), seq_lens.data_ptr<int>(),
                                      k_cache.data_ptr(), v_cache.data_ptr(), (int)qkv.size(0), (int)Hkv, (int)D,
                                      (int)k_cache.size(2), (int)k_cache.size(0), opt_ptr<int>(status), cur_stream());
}

void rope_kv_write_decode(Tensor& qkv, const Tensor& cos_t, const Tensor& sin_t, const Tensor& block_tables, const Tensor& seq_lens,
                          Tensor& k_cache, Tensor& v_cache, int64_t Hq, int64_t Hkv, int64_t D, const OptTensor& status) {
  check_bf16(qkv, "qkv"); check_f32(cos_t, "cos"); check_f32(sin_t, "sin"); check_i32(block_tables, "block_tables");
  check_i32(seq_lens, "seq_lens"); check_bf16(k_cache, "k_cache"); check_bf16(v_cache, "v_cache");
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.size(1) == (Hq + 2 * Hkv) * D && qkv.stride(0) % 8 == 0, "rope_kv_write: qkv");
  TORCH_CHECK(cos_t.is_contiguous() && sin_t.is_contiguous() && cos_t.size(1) == D / 2, "rope_kv_write: tables");
  TORCH_CHECK(block_tables.dim() == 2 && block_tables.stride(1) == 1 && block_tables.size(0) >= qkv.size(0) && seq_lens.numel() >= qkv.size(0), "rope_kv_write: block tables");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous(), "rope_kv_write: cache");
  const c10::cuda::CUDAGuard guard(qkv.device());
  agrpo::launch_rope_kv_write_decode(qkv.data_ptr(), qkv.stride(0), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), (int)cos_t.size(0),
                                     block_tables.data_ptr<int>(), (int)block_tables.stride(0), seq_lens.data_ptr<int>(),
                                     k_cache.data_ptr(), v_cache.data_ptr(), (int)qkv.size(0), (int)Hq, (int)Hkv, (int)D,
                                     (int)k_cache.size(2), (int)k_cache.size(0), opt_ptr<int>(status), cur_stream());
}

void decode_step_inputs(const Tensor& stage, int64_t S, Tensor& seq_lens, Tensor& positions, Tensor& block_tables,
                        const Tensor& base_seeds, Tensor& step_seeds, const OptTensor& status) {
  check_i32(stage, "stage"); check_i32(seq_lens, "seq_lens"); check_i32(positions, "positions"); check_i32(block_tables, "block_tables");
  check_i64(base_seeds, "base_seeds"); check_i64(step_seeds, "step_seeds");
  TORCH_CHECK(stage.is_contiguous() && stage.numel() >= 3 * S + 4 && seq_lens.numel() >= S && positions.numel() >= S &&
              base_seeds.numel() >= S && step_seeds.numel() >= S && block_tables.is_contiguous(), "decode_step_inputs: sizes");
  if (status.has_value() && status->defined()) check_i32(*status, "status");
  const c10::cuda::CUDAGuard guard(stage.device());
  agrpo::launch_decode_step_inputs(stage.data_ptr<int>(), (int)S, seq_lens.data_ptr<int>(), positions.data_ptr<int>(),
                                   block_tables.data_ptr<int>(), block_tables.numel(),
                                   reinterpret_cast<const long long*>(base_seeds.data_ptr<int64_t>()),
                                   reinterpret_cast<long long*>(step_seeds.data_ptr<int64_t>()), opt_ptr<int>(status), cur_stream());
}

// Decode-step qkv projection with everything that used to follow it: folded-norm row scale, bias, rotary embedding at
// position seq_lens[row] - 1 and the write of the new k / v into the paged cache, all in the split-K GEMM's epilogue.
// Returns false, having launched nothing, when the shape is not served (more than 128 rows, head_dim != 128, ...).
bool gemm_decode_rope(const Tensor& a, const Tensor& b, Tensor& qkv, const OptTensor& bias, const OptTensor& ss_in, double eps,
                      const Tensor& cos_t, const Tensor& sin_t, const Tensor& block_tables, const Tensor& seq_lens, Tensor& k_cache,
                      Tensor& v_cache, int64_t Hq, int64_t Hkv, const OptTensor& status) {
  check_bf16(a, "a"); check_bf16(b, "b"); check_bf16(qkv, "qkv"); check_f32(cos_t, "cos"); check_f32(sin_t, "sin");
  check_i32(block_tables, "block_tables"); check_i32(seq_lens, "seq_lens"); check_bf16(k_cache, "k_cache"); check_bf16(v_cache, "v_cache");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && qkv.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && qkv.stride(1) == 1, "gemm_decode_rope: 2-D");
  const int64_t M = a.size(0), K = a.size(1), N = b.size(0);
  TORCH_CHECK(b.size(1) == K && qkv.size(0) == M && qkv.size(1) == N, "gemm_decode_rope: shape mismatch");
  TORCH_CHECK(a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0 && qkv.stride(0) % 8 == 0, "gemm_decode_rope: row pitch multiple of 8");
  TORCH_CHECK(cos_t.is_contiguous() && sin_t.is_contiguous() && cos_t.dim() == 2 && cos_t.size(1) == 64 && sin_t.sizes() == cos_t.sizes(),
              "gemm_decode_rope: cos / sin tables [max_pos, 64] (head_dim 128)");
  TORCH_CHECK(block_tables.dim() == 2 && block_tables.stride(1) == 1 && block_tables.size(0) >= M && seq_lens.numel() >= M, "gemm_decode_rope: block tables");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous() && k_cache.size(3) == 128 && k_cache.size(1) == Hkv &&
              v_cache.sizes() == k_cache.sizes(), "gemm_decode_rope: cache [blocks, Hkv, block_size, 128]");
  if (bias.has_value() && bias->defined()) { check_bf16(*bias, "bias"); TORCH_CHECK(bias->numel() == N && bias->is_contiguous(), "bias [N]"); }
  if (ss_in.has_value() && ss_in->defined()) { check_i64(*ss_in, "ss_in"); TORCH_CHECK(ss_in->numel() >= M && ss_in->is_contiguous(), "ss_in [M]"); }
  if (status.has_value() && status->defined()) check_i32(*status, "status");
  agrpo::DecodeRopeArgs r;
  r.cos_t = cos_t.data_ptr<float>(); r.sin_t = sin_t.data_ptr<float>(); r.max_pos = (int)cos_t.size(0);
  r.block_tables = block_tables.data_ptr<int>(); r.max_blocks = (int)block_tables.stride(0); r.seq_lens = seq_lens.data_ptr<int>();
  r.k_cache = k_cache.data_ptr(); r.v_cache = v_cache.data_ptr();
  r.Hq = (int)Hq; r.Hkv = (int)Hkv; r.block_size = (int)k_cache.size(2); r.num_cache_blocks = (int)k_cache.size(0);
  const c10::cuda::CUDAGuard guard(a.device());
  return agrpo::launch_gemm_skinny(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), qkv.data_ptr(), qkv.stride(0), (int)M, (int)N,
                                   (int)K, opt_ptr<void>(bias), nullptr, 0, opt_ptr<int>(status), num_sms(), cur_stream(), nullptr,
                                   opt_i64(ss_in), nullptr, (float)eps, &r);
}

// All decoder layers of one decode step in one persistent launch (csrc/kernels/decode_mega.cu). Weights are given as
// the layer-0 matrices ([rows, K] views into flat buffers) plus the element stride from one layer to the next.
bool decode_layers_supported(int64_t rows, int64_t H, int64_t Q, int64_t QD, int64_t F, int64_t Hq, int64_t Hkv, int64_t D) {
  return agrpo::decode_layers_supported((int)rows, (int)H, (int)Q, (int)QD, (int)F, (int)Hq, (int)Hkv, (int)D);
}
int64_t decode_layers_scratch_bytes(int64_t rows, int64_t H, int64_t Q, int64_t QD, int64_t F) {
  return agrpo::decode_layers_scratch_bytes((int)rows, (int)H, (int)Q, (int)QD, (int)F, num_sms());
}
int64_t decode_layers_counter_words() { return agrpo::decode_layers_counter_words(); }
void decode_layers(int64_t L, int64_t B, const Tensor& wqkv0, int64_t wqkv_stride, const Tensor& wo0, int64_t wo_stride,
                   const Tensor& wgu0, int64_t wgu_stride, const Tensor& wd0, int64_t wd_stride, const OptTensor& bqkv0,
                   int64_t bqkv_stride, Tensor& x, Tensor& x1, Tensor& qkv, Tensor& attn, Tensor& act, Tensor& ss, double eps,
                   const Tensor& cos_t, const Tensor& sin_t, const Tensor& block_tables, const Tensor& seq_lens, Tensor& cache,
                   int64_t Hq, int64_t Hkv, double softmax_scale, int64_t splits, Tensor& part_o, Tensor& part_ml, Tensor& tickets,
                   Tensor& partials, Tensor& counters, const OptTensor& status, const OptTensor& trace, int64_t trace_layer) {
  check_bf16(wqkv0, "wqkv"); check_bf16(wo0, "wo"); check_bf16(wgu0, "wgu"); check_bf16(wd0, "wd");
  check_bf16(x, "x"); check_bf16(x1, "x1"); check_bf16(qkv, "qkv"); check_bf16(attn, "attn"); check_bf16(act, "act");
  check_i64(ss, "ss"); check_f32(cos_t, "cos"); check_f32(sin_t, "sin"); check_i32(block_tables, "block_tables");
  check_i32(seq_lens, "seq_lens"); check_bf16(cache, "cache"); check_f32(part_o, "part_o"); check_f32(part_ml, "part_ml");
  check_i32(tickets, "tickets"); check_f32(partials, "partials"); check_i32(counters, "counters");
  const int64_t H = x.size(1), Q = qkv.size(1), QD = attn.size(1), F = act.size(1), rows_alloc = x.size(0);
  TORCH_CHECK(x.is_contiguous() && x1.is_contiguous() && qkv.is_contiguous() && attn.is_contiguous() && act.is_contiguous(),
              "decode_layers: activation buffers must be contiguous");
  TORCH_CHECK(x1.size(0) == rows_alloc && qkv.size(0) == rows_alloc && attn.size(0) == rows_alloc && act.size(0) == rows_alloc &&
              x1.size(1) == H, "decode_layers: activation buffers must have the same number of rows");
  const int64_t BT = B <= 32 ? 32 : B <= 64 ? 64 : B <= 128 ? 128 : 256;
  TORCH_CHECK(B >= 1 && rows_alloc >= BT, "decode_layers: buffers must hold the row tile that covers the batch");
  TORCH_CHECK(agrpo::decode_layers_supported((int)B, (int)H, (int)Q, (int)QD, (int)F, (int)Hq, (int)Hkv, 128), "decode_layers: shape not served");
  TORCH_CHECK(wqkv0.dim() == 2 && wqkv0.is_contiguous() && wqkv0.size(0) == Q && wqkv0.size(1) == H, "decode_layers: wqkv [Q, H]");
  TORCH_CHECK(wo0.dim() == 2 && wo0.is_contiguous() && wo0.size(0) == H && wo0.size(1) == QD, "decode_layers: wo [H, q_dim]");
  TORCH_CHECK(wgu0.dim() == 2 && wgu0.is_contiguous() && wgu0.size(0) == 2 * F && wgu0.size(1) == H, "decode_layers: wgu [2F, H]");
  TORCH_CHECK(wd0.dim() == 2 && wd0.is_contiguous() && wd0.size(0) == H && wd0.size(1) == F, "decode_layers: wd [H, F]");
  TORCH_CHECK(wqkv_stride % 8 == 0 && wo_stride % 8 == 0 && wgu_stride % 8 == 0 && wd_stride % 8 == 0, "decode_layers: layer strides");
  TORCH_CHECK(ss.dim() == 2 && ss.stride(1) == 1 && ss.size(0) >= 2 * L + 1 && ss.size(1) >= B, "decode_layers: ss [2L+1, >= rows]");
  TORCH_CHECK(cos_t.is_contiguous() && sin_t.is_contiguous() && cos_t.dim() == 2 && cos_t.size(1) == 64 && sin_t.sizes() == cos_t.sizes(),
              "decode_layers: cos / sin tables [max_pos, 64]");
  TORCH_CHECK(block_tables.dim() == 2 && block_tables.stride(1) == 1 && block_tables.size(0) >= B && seq_lens.numel() >= B, "decode_layers: tables");
  TORCH_CHECK(cache.dim() == 6 && cache.is_contiguous() && cache.size(0) == L && cache.size(1) == 2 && cache.size(3) == Hkv &&
              cache.size(4) == 16 && cache.size(5) == 128, "decode_layers: cache [L, 2, blocks, Hkv, 16, 128]");
  TORCH_CHECK(splits >= 1 && splits <= 64, "decode_layers: splits");
  TORCH_CHECK(part_o.numel() >= B * Hkv * splits * 8 * 128 && part_ml.numel() >= B * Hkv * splits * 16 && tickets.numel() >= B * Hkv,
              "decode_layers: split-KV scratch");
  TORCH_CHECK(counters.numel() >= agrpo::decode_layers_counter_words(), "decode_layers: counters");
  agrpo::DecodeLayersArgs a;
  a.L = (int)L; a.B = (int)B; a.rows_alloc = (int)rows_alloc; a.H = (int)H; a.Q = (int)Q; a.QD = (int)QD; a.F = (int)F;
  a.Hq = (int)Hq; a.Hkv = (int)Hkv; a.num_sms = num_sms(); a.splits = (int)splits;
  a.wqkv = wqkv0.data_ptr(); a.wo = wo0.data_ptr(); a.wgu = wgu0.data_ptr(); a.wd = wd0.data_ptr();
  a.wqkv_stride = wqkv_stride; a.wo_stride = wo_stride; a.wgu_stride = wgu_stride; a.wd_stride = wd_stride;
  a.bqkv = nullptr; a.bqkv_stride = bqkv_stride;
  if (bqkv0.has_value() && bqkv0->defined()) { check_bf16(*bqkv0, "bqkv"); TORCH_CHECK(bqkv0->numel() == Q, "bqkv [Q]"); a.bqkv = bqkv0->data_ptr(); }
  a.x = x.data_ptr(); a.x1 = x1.data_ptr(); a.qkv = qkv.data_ptr(); a.attn = attn.data_ptr(); a.act = act.data_ptr();
  a.ss = reinterpret_cast<long long*>(ss.data_ptr<int64_t>()); a.ss_stride = (int)ss.stride(0); a.eps = (float)eps;
  a.cos_t = cos_t.data_ptr<float>(); a.sin_t = sin_t.data_ptr<float>(); a.max_pos = (int)cos_t.size(0);
  a.block_tables = block_tables.data_ptr<int>(); a.max_blocks = (int)block_tables.stride(0); a.seq_lens = seq_lens.data_ptr<int>();
  a.cache = cache.data_ptr(); a.cache_layer_stride = cache.stride(0); a.cache_v_off = cache.stride(1);
  a.num_cache_blocks = (int)cache.size(2);
  a.softmax_scale = (float)softmax_scale;
  a.part_o = part_o.data_ptr<float>(); a.part_ml = part_ml.data_ptr<float>(); a.att_tickets = tickets.data_ptr<int>();
  a.partials = partials.data_ptr<float>(); a.partials_bytes = partials.numel() * 4;
  a.counters = reinterpret_cast<unsigned int*>(counters.data_ptr<int>());
  a.status = opt_ptr<int>(status);
  {
    static const int pf = [] { const char* e = std::getenv("AGRPO_MEGA_PREFETCH"); return e ? std::atoi(e) : 8; }();
    a.prefetch_tiles = pf;
  }
  if (trace.has_value() && trace->defined()) {
    check_i64(*trace, "trace");
    TORCH_CHECK(trace->numel() >= 32 && trace->is_contiguous(), "decode_layers: trace [32]");
    a.trace = reinterpret_cast<long long*>(trace->data_ptr<int64_t>());
    a.trace_layer = (int)trace_layer;
    a.trace_words = trace->numel();
  }
  const c10::cuda::CUDAGuard guard(x.device());
  agrpo::launch_decode_layers(a, cur_stream());
}

void paged_decode_attn(const Tensor& qkv, const Tensor& k_cache, const Tensor& v_cache, const Tensor& block_tables,
                       const Tensor& seq_lens, Tensor& out, int64_t Hq, int64_t Hkv, int64_t D, double softmax_scale,
                       int64_t splits, const OptTensor& part_o, const OptTensor& part_ml, const OptTensor& status,
                       const OptTensor& tickets) {
  check_bf16(qkv, "qkv"); check_bf16(k_cache, "k_cache"); check_bf16(v_cache, "v_cache"); check_bf16(out, "out");
  check_i32(block_tables, "block_tables"); check_i32(seq_lens, "seq_lens");
  const int64_t B = qkv.size(0);
  if (tickets.has_value() && tickets->defined()) {
    check_i32(*tickets, "tickets");
    TORCH_CHECK(tickets->is_contiguous() && tickets->numel() >= B * Hkv, "decode: tickets [B, Hkv]");
  }
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.size(1) >= Hq * D, "decode: qkv");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == B && out.size(1) == Hq * D && out.stride(1) == 1, "decode: out");
  TORCH_CHECK(block_tables.dim() == 2 && block_tables.stride(1) == 1 && block_tables.size(0) >= B && seq_lens.numel() >= B, "decode: tables");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous(), "decode: cache");
  if (splits > 1) {
    TORCH_CHECK(part_o.has_value() && part_ml.has_value(), "decode: split scratch required");
    check_f32(*part_o, "part_o"); check_f32(*part_ml, "part_ml");
    TORCH_CHECK(part_o->numel() >= B * Hkv * splits * 8 * D && part_ml->numel() >= B * Hkv * splits * 16, "decode: scratch size");
  }
  const c10::cuda::CUDAGuard guard(qkv.device());
  agrpo::launch_paged_decode_attn(qkv.data_ptr(), qkv.stride(0), 0, k_cache.data_ptr(), v_cache.data_ptr(),
                                  block_tables.data_ptr<int>(), seq_lens.data_ptr<int>(), (int)B, (int)block_tables.stride(0),
                                  (int)k_cache.size(0), (int)Hq, (int)Hkv, (int)D, (int)k_cache.size(2), (float)softmax_scale,
                                  (int)splits, out.data_ptr(), out.stride(0), opt_ptr<float>(part_o), opt_ptr<float>(part_ml),
                                  opt_ptr<int>(status), cur_stream(), opt_ptr<int>(tickets));
}

int64_t lm_sample_num_groups(int64_t V, int64_t rows) { return agrpo::lm_sample_num_groups((int)V, (int)rows); }

void lm_sample(const Tensor& hidden, const Tensor& weight, double temperature, const Tensor& seeds, Tensor& part_f,
               Tensor& part_i, Tensor& tokens, const OptTensor& logprobs, const OptTensor& status) {
  check_bf16(hidden, "hidden"); check_bf16(weight, "weight"); check_f32(part_f, "part_f"); check_i32(part_i, "part_i");
  check_i32(tokens, "tokens");
  TORCH_CHECK(seeds.is_cuda() && seeds.scalar_type() == torch::kInt64 && seeds.is_contiguous(), "lm_sample: seeds int64");
  const int64_t R = hidden.size(0), H = hidden.size(1), V = weight.size(0);
  TORCH_CHECK(hidden.stride(1) == 1 && weight.stride(1) == 1 && hidden.stride(0) % 8 == 0 && weight.stride(0) % 8 == 0 && weight.size(1) == H, "lm_sample: layout");
  const int64_t groups = agrpo::lm_sample_num_groups((int)V, (int)R);
  TORCH_CHECK(seeds.numel() >= R && tokens.numel() >= R && part_f.numel() >= 4 * groups * R && part_i.numel() >= groups * R, "lm_sample: sizes");
  if (logprobs.has_value() && logprobs->defined()) { check_f32(*logprobs, "logprobs"); TORCH_CHECK(logprobs->numel() >= R, "lm_sample: logprobs"); }
  const c10::cuda::CUDAGuard guard(hidden.device());
  agrpo::launch_lm_sample(hidden.data_ptr(), hidden.stride(0), weight.data_ptr(), weight.stride(0), (int)R, (int)H, (int)V,
                          (float)temperature, reinterpret_cast<const unsigned long long*>(seeds.data_ptr<int64_t>()),
                          part_f.data_ptr<float>(), part_i.data_ptr<int>(), tokens.data_ptr<int>(), opt_ptr<float>(logprobs),
                          opt_ptr<int>(status), num_sms(), cur_stream());
}

// ---- peer-memory kernels ----
using PtrList = std::vector<int64_t>;
inline const long long* lptr(const PtrList& v) { return reinterpret_cast<const long long*>(v.data()); }

void wait_flag_probe(const Tensor& flag, int64_t want, double budget_s, Tensor& status) {
  TORCH_CHECK(flag.is_cuda() && flag.scalar_type() == torch::kInt64, "flag: int64 cuda");
  check_i32(status, "status");
  const c10::cuda::CUDAGuard guard(flag.device());
  agrpo::launch_wait_flag_probe(flag.data_ptr(), (unsigned long long)want, budget_s, status.data_ptr<int>(), cur_stream());
}
void flag_barrier(const PtrList& flag_ptrs, int64_t my_rank, int64_t epoch, double budget_s, Tensor& status) {
  check_i32(status, "status");
  const c10::cuda::CUDAGuard guard(status.device());
  agrpo::launch_flag_barrier(lptr(flag_ptrs), (int)flag_ptrs.size(), (int)my_rank, (unsigned long long)epoch, budget_s,
                             status.data_ptr<int>(), cur_stream());
}
agrpo::GatherArgs gather_args(const PtrList& src_ptrs, int64_t my_rank, Tensor& staging, int64_t n_per_owner, Tensor& flags,
                              int64_t epoch, int64_t chunk_elems) {
  check_bf16(staging, "gather staging");
  TORCH_CHECK(staging.is_contiguous(), "gather: staging must be contiguous");
  TORCH_CHECK(flags.is_cuda() && flags.scalar_type() == torch::kInt64 && flags.is_contiguous(), "gather: flags int64 cuda");
  const int64_t world = (int64_t)src_ptrs.size();
  TORCH_CHECK(world >= 1 && world <= 8, "gather: 1..8 owners");
  TORCH_CHECK(n_per_owner > 0 && n_per_owner % 8 == 0 && chunk_elems > 0 && chunk_elems % 8 == 0, "gather: sizes must be multiples of 8");
  TORCH_CHECK(staging.numel() >= world * n_per_owner, "gather: staging too small");
  TORCH_CHECK(flags.numel() >= (world * n_per_owner + chunk_elems - 1) / chunk_elems, "gather: too few flags");
  for (auto p : src_ptrs) TORCH_CHECK(p != 0 && (p & 15) == 0, "gather: shard pointers must be 16-byte aligned");
  agrpo::GatherArgs g{};
  for (int64_t r = 0; r < world; ++r) g.src[r] = reinterpret_cast<const void*>(src_ptrs[r]);
  g.dst = staging.data_ptr();
  g.n_per_owner = n_per_owner;
  g.world = (int)world;
  g.my_rank = (int)my_rank;
  g.flags = flags.data_ptr();
  g.epoch = (unsigned long long)epoch;
  g.chunk_elems = (int)chunk_elems;
  return g;
}
// d = a . b^T (+ bias, + residual) with an all-gather of one sharded unit in the same launch. When b is a view of
// `staging` the GEMM consumes what the launch gathers; otherwise the gather is a prefetch for later launches.
void ag_gemm(const Tensor& a, const Tensor& b, Tensor& d, bool a_mn, bool b_mn, const OptTensor& bias, bool accumulate,
             const OptTensor& status, const OptTensor& residual, const PtrList& src_ptrs, int64_t my_rank, Tensor& staging,
             int64_t n_per_owner, Tensor& flags, int64_t epoch, int64_t chunk_elems, int64_t n_copy) {
  check_bf16(a, "ag_gemm a"); check_bf16(b, "ag_gemm b");
  TORCH_CHECK(d.is_cuda() && (d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat32), "ag_gemm d");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && d.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && d.stride(1) == 1, "ag_gemm: 2-D, inner stride 1");
  const c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a_mn ? a.size(1) : a.size(0), K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0), Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb && d.size(0) == M && d.size(1) == N && M > 0 && N > 0 && K > 0, "ag_gemm: shape mismatch");
  TORCH_CHECK(a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0, "ag_gemm: row pitch must be a multiple of 8 elements");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(a.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(b.data_ptr()) & 15) == 0, "ag_gemm: 16-byte alignment");
  if (status.has_value() && status->defined()) check_i32(*status, "ag_gemm status");
  long long ldr = 0;
  if (residual.has_value() && residual->defined()) { check_bf16(*residual, "ag_gemm residual"); ldr = residual->stride(0); }
  agrpo::GatherArgs g = gather_args(src_ptrs, my_rank, staging, n_per_owner, flags, epoch, chunk_elems);
  const char* sb = reinterpret_cast<const char*>(staging.data_ptr());
  const char* bb = reinterpret_cast<const char*>(b.data_ptr());
  long long b_off = -1;
  if (bb >= sb && bb < sb + staging.numel() * 2) b_off = (bb - sb) / 2;
  const bool ok = agrpo::launch_ag_gemm_bf16(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), d.data_ptr(), d.stride(0), (int)M,
                                             (int)N, (int)K, a_mn, b_mn, opt_ptr<void>(bias), 1.f, d.scalar_type() == torch::kFloat32,
                                             accumulate, opt_ptr<int>(status), num_sms(), cur_stream(), opt_ptr<void>(residual), ldr,
                                             g, (int)n_copy, b_off);
  TORCH_CHECK(ok, "ag_gemm: arguments not served");
}
agrpo::ScatterArgs scatter_args(const PtrList& dst_ptrs, int64_t n_per_owner) {
  TORCH_CHECK(dst_ptrs.size() >= 1 && dst_ptrs.size() <= 8, "scatter: 1..8 owners");
  TORCH_CHECK(n_per_owner > 0 && n_per_owner % 128 == 0, "scatter: n_per_owner must be a positive multiple of 128");
  agrpo::ScatterArgs sc{};
  for (size_t r = 0; r < dst_ptrs.size(); ++r) {
    TORCH_CHECK(dst_ptrs[r] != 0 && (dst_ptrs[r] & 15) == 0, "scatter: shard pointers must be 16-byte aligned");
    sc.dst[r] = reinterpret_cast<void*>(dst_ptrs[r]);
  }
  sc.n_per_owner = n_per_owner;
  sc.world = (int)dst_ptrs.size();
  return sc;
}
// owners' gradient shards += op(a) . op(b)^T, the [M, N] result living unit_rel elements into an evenly sharded unit
// with row pitch ldd (see ScatterReduceEpilogue).
void gemm_rs(const Tensor& a, const Tensor& b, bool a_mn, bool b_mn, double alpha, const PtrList& dst_ptrs, int64_t n_per_owner,
             int64_t unit_rel, int64_t ldd, const OptTensor& status) {
  check_bf16(a, "gemm_rs a"); check_bf16(b, "gemm_rs b");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1, "gemm_rs: 2-D, inner stride 1");
  const c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a_mn ? a.size(1) : a.size(0), K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0), Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb && M > 0 && N > 0 && K > 0 && ldd >= N, "gemm_rs: shape mismatch");
  TORCH_CHECK(a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0, "gemm_rs: row pitch must be a multiple of 8 elements");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(a.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(b.data_ptr()) & 15) == 0, "gemm_rs: 16-byte alignment");
  if (status.has_value() && status->defined()) check_i32(*status, "gemm_rs status");
  const agrpo::ScatterArgs sc = scatter_args(dst_ptrs, n_per_owner);
  TORCH_CHECK(agrpo::launch_gemm_rs_bf16(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), (int)M, (int)N, (int)K, a_mn, b_mn,
                                         (float)alpha, sc, unit_rel, ldd, opt_ptr<int>(status), num_sms(), cur_stream()),
              "gemm_rs: arguments not served (offsets must be multiples of 4 and inside the unit)");
}
void scatter_add_f32(Tensor& src, int64_t unit_rel, const PtrList& dst_ptrs, int64_t n_per_owner, bool zero_src) {
  check_f32(src, "scatter_add src");
  TORCH_CHECK(src.is_contiguous() && unit_rel >= 0 && unit_rel % 4 == 0, "scatter_add: contiguous source, offset multiple of 4");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(src.data_ptr()) & 15) == 0, "scatter_add: 16-byte alignment");
  TORCH_CHECK(unit_rel + src.numel() <= n_per_owner * (int64_t)dst_ptrs.size(), "scatter_add: range exceeds the unit");
  const c10::cuda::CUDAGuard guard(src.device());
  agrpo::launch_scatter_add_f32(src.data_ptr<float>(), src.numel(), unit_rel, scatter_args(dst_ptrs, n_per_owner), zero_src,
                                cur_stream());
}
void unit_gather(const PtrList& src_ptrs, int64_t my_rank, Tensor& staging, int64_t n_per_owner, Tensor& flags, int64_t epoch,
                 int64_t chunk_elems, int64_t n_ctas, const OptTensor& status) {
  if (status.has_value() && status->defined()) check_i32(*status, "unit_gather status");
  const c10::cuda::CUDAGuard guard(staging.device());
  agrpo::GatherArgs g = gather_args(src_ptrs, my_rank, staging, n_per_owner, flags, epoch, chunk_elems);
  TORCH_CHECK(agrpo::launch_unit_gather(g, (int)n_ctas, opt_ptr<int>(status), cur_stream()), "unit_gather: arguments not served");
}
void weight_push(const Tensor& src, int64_t local_off, int64_t global_off, int64_t n, const PtrList& dst_ptrs) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && (src.scalar_type() == torch::kFloat32 || src.scalar_type() == torch::kBFloat16), "weight_push: src");
  TORCH_CHECK(local_off >= 0 && local_off + n <= src.numel() && local_off % 8 == 0 && global_off % 8 == 0, "weight_push: range");
  const c10::cuda::CUDAGuard guard(src.device());
  agrpo::launch_weight_push(src.data_ptr(), src.scalar_type() == torch::kFloat32, local_off, global_off, n, lptr(dst_ptrs),
                            (int)dst_ptrs.size(), cur_stream());
}
void weight_push_mc(const Tensor& src, int64_t local_off, int64_t global_off, int64_t n, int64_t mc_ptr) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && (src.scalar_type() == torch::kFloat32 || src.scalar_type() == torch::kBFloat16), "weight_push_mc: src");
  TORCH_CHECK(local_off >= 0 && local_off + n <= src.numel() && local_off % 8 == 0 && global_off % 8 == 0 && n % 8 == 0, "weight_push_mc: range");
  TORCH_CHECK(mc_ptr != 0 && (mc_ptr & 15) == 0, "weight_push_mc: multicast address");
  const c10::cuda::CUDAGuard guard(src.device());
  agrpo::launch_weight_push_mc(src.data_ptr(), src.scalar_type() == torch::kFloat32, local_off, global_off, n,
                               reinterpret_cast<void*>(mc_ptr), cur_stream());
}
void rs_pull_sumsq_mc(int64_t mc_ptr, int64_t global_off, int64_t local_off, int64_t n, Tensor& out, Tensor& norm_sq) {
  check_f32(out, "out"); check_f32(norm_sq, "norm_sq");
  TORCH_CHECK(out.is_contiguous() && local_off + n <= out.numel() && local_off % 4 == 0 && global_off % 4 == 0 && n % 4 == 0, "rs_pull_mc: range");
  TORCH_CHECK(mc_ptr != 0 && (mc_ptr & 15) == 0, "rs_pull_mc: multicast address");
  const c10::cuda::CUDAGuard guard(out.device());
  agrpo::launch_rs_pull_sumsq_mc(reinterpret_cast<const void*>(mc_ptr), global_off, local_off, n, out.data_ptr<float>(),
                                 norm_sq.data_ptr<float>(), cur_stream());
}
void rs_pull_sumsq(const PtrList& grad_ptrs, int64_t my_rank, int64_t global_off, int64_t local_off, int64_t n, Tensor& out,
                   Tensor& norm_sq) {
  check_f32(out, "out"); check_f32(norm_sq, "norm_sq");
  TORCH_CHECK(out.is_contiguous() && local_off + n <= out.numel() && local_off % 4 == 0 && global_off % 4 == 0 && n % 4 == 0, "rs_pull: range");
  const c10::cuda::CUDAGuard guard(out.device());
  agrpo::launch_rs_pull_sumsq(lptr(grad_ptrs), (int)grad_ptrs.size(), (int)my_rank, global_off, local_off, n,
                              out.data_ptr<float>(), norm_sq.data_ptr<float>(), cur_stream());
}
void tp_allreduce_residual(const PtrList& partial_ptrs, const PtrList& flag_ptrs, int64_t my_rank, Tensor& epoch_counter,
                           Tensor& arrive, const Tensor& residual, Tensor& out, const OptTensor& ss, double budget_s, Tensor& status) {
  check_bf16(residual, "residual"); check_bf16(out, "out"); check_i64(epoch_counter, "epoch_counter"); check_i32(arrive, "arrive");
  check_i32(status, "status");
  TORCH_CHECK(residual.dim() == 2 && residual.is_contiguous() && out.is_contiguous() && out.sizes() == residual.sizes(), "tp_allreduce: [rows, H]");
  TORCH_CHECK(residual.size(1) % 8 == 0 && (reinterpret_cast<uintptr_t>(residual.data_ptr()) & 15) == 0 &&
              (reinterpret_cast<uintptr_t>(out.data_ptr()) & 15) == 0, "tp_allreduce: alignment");
  TORCH_CHECK(partial_ptrs.size() == flag_ptrs.size() && my_rank >= 0 && my_rank < (int64_t)partial_ptrs.size(), "tp_allreduce: members");
  for (auto ptr : partial_ptrs) TORCH_CHECK(ptr != 0 && (ptr & 15) == 0, "tp_allreduce: partial buffers");
  for (auto ptr : flag_ptrs) TORCH_CHECK(ptr != 0 && (ptr & 7) == 0, "tp_allreduce: flag rows");
  if (ss.has_value() && ss->defined()) { check_i64(*ss, "ss"); TORCH_CHECK(ss->is_contiguous() && ss->numel() >= residual.size(0), "ss [rows]"); }
  const c10::cuda::CUDAGuard guard(residual.device());
  agrpo::launch_tp_allreduce_residual(lptr(partial_ptrs), lptr(flag_ptrs), (int)partial_ptrs.size(), (int)my_rank,
                                      reinterpret_cast<unsigned long long*>(epoch_counter.data_ptr<int64_t>()),
                                      reinterpret_cast<unsigned int*>(arrive.data_ptr<int>()), residual.data_ptr(), out.data_ptr(),
                                      opt_i64(ss), (int)residual.size(0), (int)residual.size(1), budget_s, status.data_ptr<int>(),
                                      cur_stream());
}
void set_comm_guard(const c10::optional<Tensor>& status) {
  if (status.has_value()) {
    TORCH_CHECK(status->is_cuda() && status->scalar_type() == torch::kInt32 && status->numel() >= 1, "set_comm_guard: int32 CUDA status word");
    agrpo::set_comm_guard(status->data_ptr<int>());
  } else {
    agrpo::set_comm_guard(nullptr);
  }
}
void publish_norm(const Tensor& norm_sq, const PtrList& table_ptrs, int64_t my_rank) {
  check_f32(norm_sq, "norm_sq");
  const c10::cuda::CUDAGuard guard(norm_sq.device());
  agrpo::launch_publish_norm(norm_sq.data_ptr<float>(), lptr(table_ptrs), (int)table_ptrs.size(), (int)my_rank, cur_stream());
}
void adamw_push(Tensor& p, Tensor& m, Tensor& v, Tensor& g, int64_t local_off, int64_t global_off, int64_t n, double lr,
                double beta1, double beta2, double eps, double wd, int64_t step, double grad_scale, const OptTensor& partials,
                double max_norm, const PtrList& dst_ptrs) {
  check_f32(p, "p"); check_f32(m, "m"); check_f32(v, "v"); check_f32(g, "g");
  TORCH_CHECK(local_off + n <= p.numel() && n % 2 == 0 && local_off % 2 == 0 && global_off % 2 == 0, "adamw_push: range");
  int np = 0;
  if (partials.has_value() && partials->defined()) { check_f32(*partials, "partials"); np = (int)partials->numel(); }
  const c10::cuda::CUDAGuard guard(p.device());
  agrpo::launch_adamw_push(p.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), g.data_ptr<float>(), local_off,
                           global_off, n, (float)lr, (float)beta1, (float)beta2, (float)eps, (float)wd, (int)step,
                           (float)grad_scale, opt_ptr<float>(partials), np, (float)max_norm, lptr(dst_ptrs),
                           (int)dst_ptrs.size(), cur_stream());
}

// ---- host packer (CPU tensors) ----
inline void check_cpu(const Tensor& t, torch::ScalarType st, const char* name) {
  TORCH_CHECK(!t.is_cuda() && t.scalar_type() == st && t.is_contiguous(), name, ": contiguous CPU tensor of the right dtype");
}
int64_t pack_count_tiles(const Tensor& in_lens, const Tensor& out_lens, int64_t tile) {
  check_cpu(in_lens, torch::kInt32, "in_lens"); check_cpu(out_lens, torch::kInt32, "out_lens");
  return agrpo::count_tiles(in_lens.data_ptr<int>(), out_lens.data_ptr<int>(), (int)in_lens.numel(), (int)tile);
}
void pack_microbatch(const Tensor& ids, const Tensor& in_lens, const Tensor& out_lens, const Tensor& adv,
                     const OptTensor& logprobs, const OptTensor& entropies, const OptTensor& ref_logprobs, int64_t tile,
                     Tensor& out_int, Tensor& out_float) {
  check_cpu(ids, torch::kInt32, "ids"); check_cpu(in_lens, torch::kInt32, "in_lens"); check_cpu(out_lens, torch::kInt32, "out_lens");
  check_cpu(adv, torch::kFloat32, "adv"); check_cpu(out_int, torch::kInt32, "out_int"); check_cpu(out_float, torch::kFloat32, "out_float");
  const int n = (int)in_lens.numel();
  const long long T = ids.numel();
  long long total_out = 0, total = 0;
  for (int i = 0; i < n; ++i) { total_out += out_lens.data_ptr<int>()[i]; total += in_lens.data_ptr<int>()[i] + out_lens.data_ptr<int>()[i]; }
  TORCH_CHECK(total == T, "pack: lengths do not add up to the number of ids");
  const long long n_tiles = agrpo::count_tiles(in_lens.data_ptr<int>(), out_lens.data_ptr<int>(), n, (int)tile);
  TORCH_CHECK(out_int.numel() >= agrpo::pack_tiles_offset(T, n, total_out) + 4 * n_tiles, "pack: out_int too small");
  TORCH_CHECK(out_float.numel() >= 5 * T, "pack: out_float too small");
  auto fp = [&](const OptTensor& t, const char* name) -> const float* {
    if (!t.has_value() || !t->defined()) return nullptr;
    check_cpu(*t, torch::kFloat32, name);
    TORCH_CHECK(t->numel() == T, name, ": expected one value per token");
    return t->data_ptr<float>();
  };
  agrpo::pack_microbatch(ids.data_ptr<int>(), in_lens.data_ptr<int>(), out_lens.data_ptr<int>(), adv.data_ptr<float>(),
                         fp(logprobs, "logprobs"), fp(entropies, "entropies"), fp(ref_logprobs, "ref_logprobs"), n, (int)tile,
                         out_int.data_ptr<int>(), out_float.data_ptr<float>(), T, total_out, n_tiles);
}
Tensor normalize_rewards_cpu(const Tensor& rewards) {
  check_cpu(rewards, torch::kFloat32, "rewards");
  Tensor out = torch::empty_like(rewards);
  agrpo::normalize_rewards(rewards.data_ptr<float>(), (int)rewards.numel(), out.data_ptr<float>());
  return out;
}

}  // namespace

namespace {
py::dict prefill_plan_to_dict(const agrpo::PrefillPlan& p) {
  py::dict d;
  d["group_ids"] = p.group_ids;
  d["prompt_lens"] = p.prompt_lens;
  d["slot_mapping"] = p.slot_mapping;
  d["cached_lens"] = p.cached_lens;
  d["prefix_slots"] = p.prefix_slots;
  d["seq_ids"] = p.seq_ids;
  d["seq_slots"] = p.seq_slots;
  d["copy_src"] = p.copy_src;
  d["copy_dst"] = p.copy_dst;
  std::vector<int> us, ui, ub;
  for (const auto& u : p.updates) { us.push_back(u.slot); ui.push_back(u.index); ub.push_back(u.block); }
  d["upd_slot"] = us; d["upd_index"] = ui; d["upd_block"] = ub;
  return d;
}
py::dict decode_plan_to_dict(const agrpo::DecodePlan& p) {
  py::dict d;
  d["batch_rows"] = p.batch_rows;
  d["num_active"] = p.num_active;
  // numpy arrays: the engine's per-step bookkeeping is vectorised, no Python loop over sequences
  py::array_t<int> act((py::ssize_t)p.active_slots.size());
  std::copy(p.active_slots.begin(), p.active_slots.end(), act.mutable_data());
  d["active_slots"] = act;
  d["preempted"] = p.preempted;
  const py::ssize_t n = (py::ssize_t)p.updates.size();
  py::array_t<int> us(n), ui(n), ub(n);
  for (py::ssize_t i = 0; i < n; ++i) {
    us.mutable_data()[i] = p.updates[i].slot;
    ui.mutable_data()[i] = p.updates[i].index;
    ub.mutable_data()[i] = p.updates[i].block;
  }
  d["upd_slot"] = us; d["upd_index"] = ui; d["upd_block"] = ub;
  return d;
}
}  // namespace

// Kernel launchers run without the interpreter lock: the trainer, logprob and rollout threads of one process launch
// concurrently, and a decode step must not wait for another thread's launch sequence to yield.
#define NOGIL py::call_guard<py::gil_scoped_release>()

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  py::class_<agrpo::BlockAllocator>(m, "BlockAllocator")
      .def(py::init<int>())
      .def("alloc", &agrpo::BlockAllocator::alloc)
      .def("incref", &agrpo::BlockAllocator::incref)
      .def("release", &agrpo::BlockAllocator::release)
      .def("refcount", &agrpo::BlockAllocator::refcount)
      .def_property_readonly("num_free", &agrpo::BlockAllocator::num_free)
      .def_property_readonly("num_blocks", &agrpo::BlockAllocator::num_blocks);
  py::class_<agrpo::Scheduler>(m, "Scheduler")
      .def(py::init<int, int, int, int, int>(), py::arg("num_blocks"), py::arg("block_size"), py::arg("max_seqs"),
           py::arg("max_blocks_per_seq"), py::arg("max_prefill_tokens"))
      .def("add_group",
           [](agrpo::Scheduler& s, long long group_id, int prompt_len, int n, int max_new_tokens, std::vector<int> forced,
              std::vector<unsigned long long> block_hashes) {
             agrpo::GroupRequest g{group_id, prompt_len, n, max_new_tokens, std::move(forced), std::move(block_hashes)};
             s.add_group(g);
           },
           py::arg("group_id"), py::arg("prompt_len"), py::arg("n"), py::arg("max_new_tokens"),
           py::arg("forced_new_tokens") = std::vector<int>(), py::arg("block_hashes") = std::vector<unsigned long long>())
      .def("plan_prefill", [](agrpo::Scheduler& s) { return prefill_plan_to_dict(s.plan_prefill()); })
      .def("plan_decode", [](agrpo::Scheduler& s) { return decode_plan_to_dict(s.plan_decode()); })
      .def("finish", &agrpo::Scheduler::finish)
      .def("compact_slots", &agrpo::Scheduler::compact_slots)
      .def_property_readonly("highest_slot", &agrpo::Scheduler::highest_slot)
      .def("seq_info",
           [](const agrpo::Scheduler& s, long long id) -> py::object {
             const agrpo::SeqState* q = s.seq(id);
             if (!q) return py::none();
             py::dict d;
             d["seq_id"] = q->seq_id; d["group_id"] = q->group_id; d["child"] = q->child; d["slot"] = q->slot;
             d["prompt_len"] = q->prompt_len; d["len"] = q->len; d["max_len"] = q->max_len; d["forced_len"] = q->forced_len;
             d["blocks"] = q->blocks;
             return d;
           })
      .def_property_readonly("num_waiting", &agrpo::Scheduler::num_waiting)
      .def_property_readonly("num_running", &agrpo::Scheduler::num_running)
      .def_property_readonly("num_free_blocks", &agrpo::Scheduler::num_free_blocks)
      .def_property_readonly("num_free_slots", &agrpo::Scheduler::num_free_slots)
      .def_property_readonly("num_cached_blocks", &agrpo::Scheduler::num_cached_blocks)
      .def("clear_prefix_cache", &agrpo::Scheduler::clear_prefix_cache);

  m.def("gemm_bf16", &gemm_bf16, py::arg("a"), py::arg("b"), py::arg("d"), py::arg("a_mn") = false,
        py::arg("b_mn") = false, py::arg("bias") = py::none(), py::arg("alpha") = 1.0, py::arg("accumulate") = false,
        py::arg("status") = py::none(), py::arg("residual") = py::none(), NOGIL);
  m.def("gemm_skinny_trace", &gemm_skinny_trace);
  m.def("embedding_fwd", &embedding_fwd, NOGIL);
  m.def("embedding_bwd", &embedding_bwd, NOGIL);
  m.def("set_sm_limit", [](int n) { sm_limit() = n; },
        "Cap (0 = none) on the SMs filled by persistent kernels that this THREAD launches.");
  m.def("set_pdl", [](bool on) { agrpo::pdl_flag() = on; },
        "Programmatic dependent launch for the kernels this THREAD launches next (used around the decode step).");
  m.def("embedding_sumsq", &embedding_sumsq, NOGIL);
  m.def("fold_norm_weight", &fold_norm_weight, NOGIL);
  m.def("gemm_decode", &gemm_decode, py::arg("a"), py::arg("b"), py::arg("d"), py::arg("bias") = py::none(),
        py::arg("residual") = py::none(), py::arg("ss_in") = py::none(), py::arg("ss_out") = py::none(), py::arg("eps") = 1e-6,
        py::arg("status") = py::none(), NOGIL);
  m.def("gemm_skinny_splits", &gemm_skinny_splits);
  m.def("gemm_decode_rope", &gemm_decode_rope, NOGIL);
  m.def("decode_step_inputs", &decode_step_inputs, NOGIL);
  m.def("decode_layers", &decode_layers, py::arg("L"), py::arg("B"), py::arg("wqkv0"), py::arg("wqkv_stride"), py::arg("wo0"),
        py::arg("wo_stride"), py::arg("wgu0"), py::arg("wgu_stride"), py::arg("wd0"), py::arg("wd_stride"), py::arg("bqkv0"),
        py::arg("bqkv_stride"), py::arg("x"), py::arg("x1"), py::arg("qkv"), py::arg("attn"), py::arg("act"), py::arg("ss"),
        py::arg("eps"), py::arg("cos_t"), py::arg("sin_t"), py::arg("block_tables"), py::arg("seq_lens"), py::arg("cache"),
        py::arg("Hq"), py::arg("Hkv"), py::arg("softmax_scale"), py::arg("splits"), py::arg("part_o"), py::arg("part_ml"),
        py::arg("tickets"), py::arg("partials"), py::arg("counters"), py::arg("status") = py::none(),
        py::arg("trace") = py::none(), py::arg("trace_layer") = 0, NOGIL);
  m.def("decode_layers_supported", &decode_layers_supported);
  m.def("decode_layers_scratch_bytes", &decode_layers_scratch_bytes);
  m.def("decode_layers_counter_words", &decode_layers_counter_words);
  m.def("gemm_swiglu", &gemm_swiglu, py::arg("a"), py::arg("b"), py::arg("d"), py::arg("ss_in") = py::none(), py::arg("eps") = 1e-6,
        py::arg("status") = py::none(), NOGIL);
  m.def("rmsnorm_fwd", &rmsnorm_fwd, py::arg("x"), py::arg("w"), py::arg("y"), py::arg("rstd") = py::none(),
        py::arg("eps") = 1e-6, NOGIL);
  m.def("rmsnorm_bwd", &rmsnorm_bwd, py::arg("dy"), py::arg("x"), py::arg("w"), py::arg("rstd"), py::arg("dx"),
        py::arg("dw") = py::none(), py::arg("accumulate_dx") = false, NOGIL);
  m.def("colsum", &colsum, NOGIL);
  m.def("rope_inplace", &rope_inplace, NOGIL);
  m.def("swiglu_fwd", &swiglu_fwd, NOGIL);
  m.def("swiglu_bwd", &swiglu_bwd, NOGIL);
  m.def("add_bf16", &add_bf16, NOGIL);
  m.def("attn_varlen_fwd", &attn_varlen_fwd, py::arg("qkv"), py::arg("out"), py::arg("lse"), py::arg("tiles"),
        py::arg("Hq"), py::arg("Hkv"), py::arg("D"), py::arg("softmax_scale"), py::arg("status") = py::none(), NOGIL);
  m.def("attn_varlen_bwd", &attn_varlen_bwd, py::arg("qkv"), py::arg("out"), py::arg("dout"), py::arg("lse"),
        py::arg("delta"), py::arg("dq_acc"), py::arg("dqkv"), py::arg("tiles"), py::arg("Hq"), py::arg("Hkv"), py::arg("D"),
        py::arg("softmax_scale"), py::arg("status") = py::none(), NOGIL);
  m.def("lmhead_num_groups", &lmhead_num_groups);
  m.def("grpo_num_loss_stats", &grpo_num_loss_stats);
  m.def("lmhead_logprob", &lmhead_logprob, py::arg("hidden"), py::arg("weight"), py::arg("labels"), py::arg("temperature"),
        py::arg("partials"), py::arg("label_logit"), py::arg("logp") = py::none(), py::arg("entropy") = py::none(),
        py::arg("lse") = py::none(), py::arg("status") = py::none(), NOGIL);
  m.def("grpo_token_loss", &grpo_token_loss, py::arg("logp"), py::arg("old_logp"), py::arg("ref_logp"), py::arg("adv"),
        py::arg("labels"), py::arg("entropy"), py::arg("old_entropy"), py::arg("clip_low"), py::arg("clip_high"),
        py::arg("clip_c"), py::arg("kl_beta"), py::arg("grad_weight"), py::arg("dlogp"), py::arg("stats"), NOGIL);
  m.def("lmhead_backward", &lmhead_backward, py::arg("hidden"), py::arg("weight"), py::arg("labels"), py::arg("lse"),
        py::arg("dlogp"), py::arg("temperature"), py::arg("dz_chunk"), py::arg("dh_acc"), py::arg("dweight") = py::none(),
        py::arg("status") = py::none(), NOGIL);
  m.def("kv_cache_write", &kv_cache_write, py::arg("qkv"), py::arg("slots"), py::arg("k_cache"), py::arg("v_cache"), py::arg("Hq"),
        py::arg("Hkv"), py::arg("D"), py::arg("status") = py::none(), py::arg("kv_head0") = 0, NOGIL);
  m.def("kv_cache_write_decode", &kv_cache_write_decode, py::arg("qkv"), py::arg("block_tables"), py::arg("seq_lens"),
        py::arg("k_cache"), py::arg("v_cache"), py::arg("Hq"), py::arg("Hkv"), py::arg("D"), py::arg("status") = py::none(), NOGIL);
  m.def("rope_kv_write_decode", &rope_kv_write_decode, py::arg("qkv"), py::arg("cos"), py::arg("sin"), py::arg("block_tables"),
        py::arg("seq_lens"), py::arg("k_cache"), py::arg("v_cache"), py::arg("Hq"), py::arg("Hkv"), py::arg("D"),
        py::arg("status") = py::none(), NOGIL);
  m.def("paged_decode_attn", &paged_decode_attn, py::arg("qkv"), py::arg("k_cache"), py::arg("v_cache"),
        py::arg("block_tables"), py::arg("seq_lens"), py::arg("out"), py::arg("Hq"), py::arg("Hkv"), py::arg("D"),
        py::arg("softmax_scale"), py::arg("splits") = 1, py::arg("part_o") = py::none(), py::arg("part_ml") = py::none(),
        py::arg("status") = py::none(), py::arg("tickets") = py::none(), NOGIL);
  m.def("lm_sample_num_groups", &lm_sample_num_groups);
  m.def("lm_sample", &lm_sample, py::arg("hidden"), py::arg("weight"), py::arg("temperature"), py::arg("seeds"),
        py::arg("part_f"), py::arg("part_i"), py::arg("tokens"), py::arg("logprobs") = py::none(),
        py::arg("status") = py::none(), NOGIL);
  m.def("pack_count_tiles", &pack_count_tiles);
  m.def("pack_microbatch", &pack_microbatch);
  m.def("normalize_rewards", &normalize_rewards_cpu);
  m.def("wait_flag_probe", &wait_flag_probe);
  m.def("flag_barrier", &flag_barrier, NOGIL);
  m.def("weight_push", &weight_push, NOGIL);
  m.def("ag_gemm", &ag_gemm, py::arg("a"), py::arg("b"), py::arg("d"), py::arg("a_mn") = false, py::arg("b_mn") = false,
        py::arg("bias") = py::none(), py::arg("accumulate") = false, py::arg("status") = py::none(),
        py::arg("residual") = py::none(), py::arg("src_ptrs"), py::arg("my_rank"), py::arg("staging"),
        py::arg("n_per_owner"), py::arg("flags"), py::arg("epoch"), py::arg("chunk_elems") = 262144, py::arg("n_copy") = 16, NOGIL);
  m.def("gemm_rs", &gemm_rs, py::arg("a"), py::arg("b"), py::arg("a_mn"), py::arg("b_mn"), py::arg("alpha"), py::arg("dst_ptrs"),
        py::arg("n_per_owner"), py::arg("unit_rel"), py::arg("ldd"), py::arg("status") = py::none(), NOGIL);
  m.def("scatter_add_f32", &scatter_add_f32, py::arg("src"), py::arg("unit_rel"), py::arg("dst_ptrs"), py::arg("n_per_owner"),
        py::arg("zero_src") = true, NOGIL);
  m.def("unit_gather", &unit_gather, py::arg("src_ptrs"), py::arg("my_rank"), py::arg("staging"), py::arg("n_per_owner"),
        py::arg("flags"), py::arg("epoch"), py::arg("chunk_elems") = 262144, py::arg("n_ctas") = 32, py::arg("status") = py::none(), NOGIL);
  m.def("weight_push_mc", &weight_push_mc, NOGIL);
  m.def("rs_pull_sumsq_mc", &rs_pull_sumsq_mc, NOGIL);
  m.def("rs_pull_sumsq", &rs_pull_sumsq, NOGIL);
  m.def("publish_norm", &publish_norm, NOGIL);
  m.def("set_comm_guard", &set_comm_guard, py::arg("status") = py::none());
  m.def("tp_allreduce_residual", &tp_allreduce_residual, py::arg("partial_ptrs"), py::arg("flag_ptrs"), py::arg("my_rank"),
        py::arg("epoch_counter"), py::arg("arrive"), py::arg("residual"), py::arg("out"), py::arg("ss") = py::none(),
        py::arg("budget_s") = 10.0, py::arg("status"), NOGIL);
  m.def("adamw_push", &adamw_push, NOGIL);
  m.def("sumsq", &sumsq, NOGIL);
  m.def("adamw_step", &adamw_step, py::arg("p"), py::arg("m"), py::arg("v"), py::arg("g"), py::arg("p16") = py::none(),
        py::arg("lr") = 1e-6, py::arg("beta1") = 0.9, py::arg("beta2") = 0.999, py::arg("eps") = 1e-8,
        py::arg("wd") = 0.0, py::arg("step") = 1, py::arg("grad_scale") = 1.0, py::arg("norm_sq") = py::none(),
        py::arg("max_norm") = 0.0, py::arg("zero_grad") = false, NOGIL);
  m.def("cast_f32_bf16", &cast_f32_bf16, NOGIL);
}
