// Raw-pointer launchers implemented in the .cu files. They include no torch header so that nvcc
// only sees CUDA code; bindings.cpp (host compiler) wraps them for Python.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <stdexcept>
#include <string>

namespace agrpo {

inline void check_cuda(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// The GEMM / attention kernels need ~200 KB of shared memory per SM. A kernel that prefers a large L1 instead makes
// the SM re-partition its L1 / shared memory when it follows or precedes them, which costs microseconds per switch in a
// decode step of ~280 short kernels. Every small kernel therefore asks for the same (maximum shared) carve-out once.
template <typename K>
inline void prefer_max_shared(K kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
}
#define AGRPO_PREFER_SMEM(kernel)                        \
  do {                                                    \
    static bool agrpo_once_ = false;                      \
    if (!agrpo_once_) {                                   \
      ::agrpo::prefer_max_shared(kernel);                 \
      agrpo_once_ = true;                                 \
    }                                                     \
  } while (0)

// cudaFuncSetAttribute applies to the device that is current when it is called, and role threads launch concurrently:
// one flag per device (atomic) per call site, so that a second GPU driven from the same process is configured too.
struct PerDeviceOnce {
  std::atomic<bool> done[64];
  PerDeviceOnce() {
    for (auto& d : done) d.store(false);
  }
  static int device() {
    int d = 0;
    return cudaGetDevice(&d) == cudaSuccess && d >= 0 && d < 64 ? d : -1;
  }
  bool need(int d) const { return d < 0 || !done[d].load(std::memory_order_acquire); }
  void set(int d) {
    if (d >= 0) done[d].store(true, std::memory_order_release);
  }
};
#define AGRPO_SET_MAX_DYN_SMEM(kernel, bytes, what)                                                                   \
  do {                                                                                                                \
    static ::agrpo::PerDeviceOnce agrpo_once_;                                                                        \
    const int agrpo_dev_ = ::agrpo::PerDeviceOnce::device();                                                          \
    if (agrpo_once_.need(agrpo_dev_)) {                                                                               \
      ::agrpo::check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(bytes)), what); \
      agrpo_once_.set(agrpo_dev_);                                                                                    \
    }                                                                                                                 \
  } while (0)

// Programmatic dependent launch is a per-thread switch: the rollout engine turns it on around its decode step, whose
// ~170 short kernels then overlap each prologue (barrier set-up, TMEM allocation, first weight loads) with the tail
// of the kernel before. Kernels launched through launch_kernel() contain griddepcontrol.wait, so they are correct
// with the switch on or off.
inline bool& pdl_flag() {
  static thread_local bool on = false;
  return on;
}
template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, const char* what,
                          Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_flag() ? 1 : 0;
  check_cuda(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...), what);
}

// d[M,N] = alpha * A . B^T (+ bias[N]) (+ d). bf16 operands, fp32 accumulation on tcgen05.
//   a_mn = false: a is [M, K] row-major with pitch lda; a_mn = true: a is [K, M] row-major
//   b_mn = false: b is [N, K] row-major with pitch ldb; b_mn = true: b is [K, N] row-major
// Pitches are in elements and must be multiples of 8; base pointers 16-byte aligned.
// residual (bf16 [M, ldr], optional) is added to the result, e.g. the skip connection of a decoder block.
void launch_gemm_bf16(const void* a, long long lda, const void* b, long long ldb, void* d, long long ldd, int M, int N,
                      int K, bool a_mn, bool b_mn, const void* bias, float alpha, bool out_fp32, bool accumulate,
                      int* status, int num_sms, cudaStream_t stream, const void* residual = nullptr, long long ldr = 0);

// All-gather of one sharded parameter unit (FSDP / ZeRO-3: every rank owns n_per_owner contiguous elements of it)
// into a local staging buffer. src[r] is rank r's slice (peer addresses for r != my_rank); flags has one 64-bit word
// per chunk_elems elements of the unit and receives `epoch` when the chunk is staged.
struct GatherArgs {
  const void* src[8];
  void* dst;
  long long n_per_owner;
  int world;
  int my_rank;
  void* flags;
  unsigned long long epoch;
  int chunk_elems;
};
// GEMM whose first n_copy CTAs run the gather while the others compute; b_unit_offset >= 0 when B itself is inside the
// unit being gathered (the element offset of B in the staging buffer), < 0 when the job prefetches for later GEMMs.
// Returns false (nothing launched) for arguments it does not serve.
bool launch_ag_gemm_bf16(const void* a, long long lda, const void* b, long long ldb, void* d, long long ldd, int M,
                         int N, int K, bool a_mn, bool b_mn, const void* bias, float alpha, bool out_fp32,
                         bool accumulate, int* status, int num_sms, cudaStream_t stream, const void* residual,
                         long long ldr, const GatherArgs& g, int n_copy, long long b_unit_offset);
// GEMM -> reduce-scatter: the fp32 result is added element by element into the gradient shard of the rank that owns
// it (vector red over NVLink) instead of being stored. dst[r] is owner r's shard already offset to the unit; the result
// matrix starts unit_rel elements into the unit and has row pitch ldd.
struct ScatterArgs {
  void* dst[8];
  long long n_per_owner;
  int world;
};
bool launch_gemm_rs_bf16(const void* a, long long lda, const void* b, long long ldb, int M, int N, int K, bool a_mn, bool b_mn,
                         float alpha, const ScatterArgs& sc, long long unit_rel, long long ldd, int* status, int num_sms,
                         cudaStream_t stream);
// src[0, n) (fp32, local) is added into the owners' shards at unit offset unit_rel and then zeroed when zero_src is set.
void launch_scatter_add_f32(float* src, long long n, long long unit_rel, const ScatterArgs& sc, bool zero_src,
                            cudaStream_t stream);
// The gather alone, for a unit with no GEMM to ride on.
bool launch_unit_gather(const GatherArgs& g, int n_ctas, int* status, cudaStream_t stream);

// Fused gate/up projection + SwiGLU (+ folded RMSNorm row scale, ss_in = row sums of squares of a, may be nullptr):
// b is the stacked [2F, K] weight, d the [M, F] activation.
bool launch_gemm_swiglu_bf16(const void* a, long long lda, const void* b, long long ldb, void* d, long long ldd, int M, int F,
                             int K, const long long* ss_in, float eps, int* status, int num_sms, cudaStream_t stream);

// Decode-time shapes (M <= 256): split-K over a thread-block cluster, reduction through distributed shared memory.
// Returns false (nothing launched) when the shape is outside what it serves. trace (optional, 16 int64 words on the
// device) receives clock64 stamps of the kernel's phases for the first CTA: a built-in phase tracer.
// Decode-step epilogue of the qkv projection: rotary embedding at position seq_lens[row] - 1 and the write of the new
// token's k / v into the paged cache (head_dim 128; cos / sin tables are [max_pos, 64] fp32).
struct DecodeRopeArgs {
  const float* cos_t;
  const float* sin_t;
  int max_pos;
  const int* block_tables;
  int max_blocks;
  const int* seq_lens;
  void* k_cache;
  void* v_cache;
  int Hq, Hkv, block_size, num_cache_blocks;
};
bool launch_gemm_skinny(const void* a, long long lda, const void* b, long long ldb, void* d, long long ldd, int M, int N, int K,
                        const void* bias, const void* residual, long long ldr, int* status, int num_sms, cudaStream_t stream,
                        long long* trace = nullptr, const long long* ss_in = nullptr, long long* ss_out = nullptr, float eps = 0.f,
                        const DecodeRopeArgs* rope = nullptr);
int gemm_skinny_splits(int M, int N, int K, int num_sms);

// ---- bandwidth-bound decoder ops (elementwise.cu); bf16 activations, H and F multiples of 8 ----
void launch_embedding_fwd(const int* ids, const void* table, void* out, int T, int H, int V, cudaStream_t s);
void launch_embedding_bwd(const int* ids, const void* dout, float* dtable, int T, int H, int V, cudaStream_t s);
// Lookup + ss[0][row] = sum of squares of the row, ss[1..n_ss)[row] = 0. ss is [n_ss, ss_stride] int64: sums of squares
// in fixed point with 30 fractional bits (value * 2^30), which makes their atomic accumulation order-independent.
void launch_embedding_sumsq(const int* ids, const void* table, void* out, long long* ss, int n_ss, int ss_stride, int T, int H,
                            int V, cudaStream_t s);
// out[n, k] = w[n, k] * g[k] (bf16, K a multiple of 8).
void launch_fold_norm_weight(const void* w, const void* g, void* out, long long n_rows, int K, cudaStream_t s);
void launch_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int T, int H, float eps, cudaStream_t s);
// dw (fp32 [H], may be nullptr) is accumulated with atomic adds.
void launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw, int T,
                        int H, bool accumulate_dx, cudaStream_t s);
// out[c] += sum over rows of a[r, c]; a has row pitch lda (elements).
void launch_colsum(const void* a, float* out, int T, int C, long long lda, cudaStream_t s);
void launch_rope(void* qkv, const int* pos, const float* cos_t, const float* sin_t, int T, int n_rot_heads, int D,
                 long long row_pitch, int max_pos, bool backward, cudaStream_t s);
void launch_swiglu_fwd(const void* gu, void* out, int T, int F, cudaStream_t s);
void launch_swiglu_bwd(const void* gu, const void* dout, void* dgu, int T, int F, cudaStream_t s);
void launch_add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t s);

// ---- attention (attn_varlen_*.cu) ----
// Causal varlen attention over packed rows. q/k/v are row-major matrices with T rows (they may be the
// same fused qkv buffer); head h of q occupies columns [q_col0 + h*D, q_col0 + (h+1)*D), likewise
// k / v with kv heads. tiles: int32 [n_tiles, 4] = {seq_start, seq_len, q0, 0}, q0 a multiple of 128.
// lse: fp32 [Hq, T] (natural log), may be nullptr.
void launch_attn_varlen_fwd(const void* q, long long ldq, int q_cols, const void* k, long long ldk, int k_cols,
                            const void* v, long long ldv, int v_cols, int q_col0, int k_col0, int v_col0, void* out,
                            long long ldo, float* lse, const int* tiles, int n_tiles, int T, int Hq, int Hkv, int D,
                            float softmax_scale, int* status, cudaStream_t s);

// Backward of the above. out/dout: [T, Hq*D] rows. delta: fp32 [Hq, T] scratch, dq_acc: fp32 [T, Hq*D]
// scratch (zeroed here). dq (pitch ld_dq, columns [0, Hq*D)), dk / dv (head h at column d*_col0 + h*D)
// are bf16 and may alias one fused [T, (Hq+2Hkv)*D] gradient buffer.
void launch_attn_varlen_bwd(const void* q, long long ldq, int q_cols, const void* k, long long ldk, int k_cols,
                            const void* v, long long ldv, int v_cols, int q_col0, int k_col0, int v_col0, const void* out,
                            long long ldo, const void* dout, long long lddo, const float* lse, float* delta, float* dq_acc,
                            void* dq, long long ld_dq, void* dk, long long ld_dk, int dk_col0, void* dv, long long ld_dv,
                            int dv_col0, const int* tiles, int n_tiles, int T, int Hq, int Hkv, int D, float softmax_scale,
                            int* status, cudaStream_t s);

// ---- fused lm_head + GRPO loss (lmhead_loss.cu) ----
// Number of partial-statistics groups the forward writes for a [T, V] problem.
int lmhead_num_groups(int V, int T);
// logits z = hidden . weight^T / temperature never reach memory. labels[t] is the target token of row t
// (already shifted), negative = masked. partials: fp32 [3 * groups * T] scratch; label_logit: fp32 [T] scratch.
// Outputs (each may be nullptr): logp[t] = z[label] - lse (0 on masked rows), entropy[t], lse[t].
void launch_lmhead_logprob(const void* hidden, long long ldh, const void* weight, long long ldw, const int* labels, int T,
                           int H, int V, float temperature, float* partials, float* label_logit, float* logp,
                           float* entropy, float* lse, int* status, int num_sms, cudaStream_t stream);
// Per-token dual-clip GRPO objective (+ kl_beta * k3 KL against ref_logp), its derivative w.r.t. logp scaled by
// grad_weight, and sums over valid tokens in stats[grpo_num_loss_stats()] (atomic adds; zero it first).
void launch_grpo_token_loss(const float* logp, const float* old_logp, const float* ref_logp, const float* adv,
                            const int* labels, const float* entropy, const float* old_entropy, int T, float clip_low,
                            float clip_high, float clip_c, float kl_beta, float grad_weight, float* dlogp, float* stats,
                            cudaStream_t stream);
int grpo_num_loss_stats();
// dh_acc (fp32 [T, H]) = d loss / d hidden; dweight (fp32, pitch ld_dw, may be nullptr) += d loss / d weight.
// dz_chunk: bf16 [T, chunk_cols] scratch, chunk_cols a multiple of 256.
void launch_lmhead_backward(const void* hidden, long long ldh, const void* weight, long long ldw, const int* labels,
                            const float* lse, const float* dlogp, int T, int H, int V, float temperature, void* dz_chunk,
                            int chunk_cols, float* dh_acc, float* dweight, long long ld_dw, int* status, int num_sms,
                            cudaStream_t stream);

// ---- rollout engine (rollout.cu) ----
// KV cache layout per layer: [num_blocks, Hkv, block_size, D] (K and V separately). slots[t] < 0 skips token t.
void launch_kv_cache_write(const void* qkv, long long row_pitch, int k_col0, int v_col0, const int* slots, void* k_cache,
                           void* v_cache, int T, int Hkv, int D, int block_size, int num_cache_blocks, int* status,
                           cudaStream_t s);
void launch_kv_cache_write_decode(const void* qkv, long long row_pitch, int k_col0, int v_col0, const int* block_tables,
                                  int max_blocks, const int* seq_lens, void* k_cache, void* v_cache, int B, int Hkv, int D,
                                  int block_size, int num_cache_blocks, int* status, cudaStream_t s);
// RoPE on the q / k heads of each row (position seq_lens[b] - 1) and the KV write of that token, in one kernel.
void launch_rope_kv_write_decode(void* qkv, long long row_pitch, const float* cos_t, const float* sin_t, int max_pos,
                                 const int* block_tables, int max_blocks, const int* seq_lens, void* k_cache, void* v_cache, int B,
                                 int Hq, int Hkv, int D, int block_size, int num_cache_blocks, int* status, cudaStream_t s);
// Scatters one staged host buffer into the decode step's device inputs (layout: see decode_step_inputs_kernel).
void launch_decode_step_inputs(const int* stage, int S, int* seq_lens, int* positions, int* block_tables, long long table_elems,
                               const long long* base_seeds, long long* step_seeds, int* status, cudaStream_t s);
// One query token per sequence against the paged cache. part_o: fp32 [B, Hkv, splits, 8, D], part_ml: fp32
// [B, Hkv, splits, 8, 2] (only touched when splits > 1). tickets (int32 [B, Hkv], all zero between launches) lets the
// last split CTA of each (sequence, kv head) merge the partials itself; without it a second kernel does the merge.
void launch_paged_decode_attn(const void* q, long long ldq, int q_col0, const void* k_cache, const void* v_cache,
                              const int* block_tables, const int* seq_lens, int B, int max_blocks, int num_cache_blocks,
                              int Hq, int Hkv, int D, int block_size, float softmax_scale, int splits, void* out,
                              long long ldo, float* part_o, float* part_ml, int* status, cudaStream_t s,
                              int* tickets = nullptr);
int lm_sample_num_groups(int V, int rows);
// tokens[r] ~ softmax(hidden[r] . weight^T / temperature) (argmax when temperature <= 0); logprobs may be nullptr.
// part_f: fp32 [4 * groups * rows], part_i: int32 [groups * rows] scratch.
void launch_lm_sample(const void* hidden, long long ldh, const void* weight, long long ldw, int rows, int H, int V,
                      float temperature, const unsigned long long* seeds, float* part_f, int* part_i, int* tokens,
                      float* logprobs, int* status, int num_sms, cudaStream_t stream);

// ---- peer-memory collectives fused with their compute (symm.cu) ----
// Pointer tables are device addresses (as integers) of the peers' symmetric buffers, one per rank / destination.
void launch_wait_flag_probe(const void* flag, unsigned long long want, double budget_s, int* status, cudaStream_t s);
void launch_flag_barrier(const long long* flag_ptrs, int world, int my_rank, unsigned long long epoch, double budget_s,
                         int* status, cudaStream_t s);
// Barrier whose epoch lives in device memory (graph-replayable), and the tensor-parallel all-reduce + residual + row
// statistic that follows a row-parallel projection of the rollout engine (partials read from peers' symmetric buffers).
void launch_tp_allreduce_residual(const long long* partial_ptrs, const long long* flag_ptrs, int world, int my_rank,
                                  unsigned long long* epoch_counter, unsigned int* arrive, const void* residual, void* out,
                                  long long* ss, int rows, int H, double budget_s, int* status, cudaStream_t s);
void launch_weight_push(const void* src, bool src_fp32, long long local_off, long long global_off, long long n,
                        const long long* dst_ptrs, int n_dst, cudaStream_t s);
// NVSwitch multicast variants (mc = multicast address of the symmetric buffer): the push is replicated by the switch,
// the reduce-scatter adds inside the switch over every rank of the multicast group.
void launch_weight_push_mc(const void* src, bool src_fp32, long long local_off, long long global_off, long long n, void* mc,
                           cudaStream_t s);
void launch_rs_pull_sumsq_mc(const void* mc, long long global_off, long long local_off, long long n, float* out, float* norm_sq,
                             cudaStream_t s);
void launch_rs_pull_sumsq(const long long* grad_ptrs, int world, int my_rank, long long global_off, long long local_off,
                          long long n, float* out, float* norm_sq, cudaStream_t s);
void launch_publish_norm(const float* norm_sq, const long long* table_ptrs, int world, int my_rank, cudaStream_t s);
// Status word (device pointer, or nullptr) that the peer-memory kernels launched from the calling thread test at entry:
// non-zero (a barrier before them ran out of time) makes them return without touching any buffer.
void set_comm_guard(const int* status);
void launch_adamw_push(float* p, float* m, float* v, float* g, long long local_off, long long global_off, long long n, float lr,
                       float beta1, float beta2, float eps, float wd, int step, float grad_scale, const float* partials,
                       int n_partials, float max_norm, const long long* dst_ptrs, int n_dst, cudaStream_t s);

// ---- optimizer (optimizer.cu) ----
// *out += scale^2 * sum(g^2)
void launch_sumsq(const float* g, long long n, float scale, float* out, cudaStream_t s);
void launch_adamw(float* p, float* m, float* v, float* g, void* p16, long long n, float lr, float beta1, float beta2,
                  float eps, float wd, int step, float grad_scale, const float* norm_sq, float max_norm, bool zero_grad,
                  cudaStream_t s);
void launch_cast_f32_bf16(const float* in, void* out, long long n, cudaStream_t s);

// All decoder layers of one decode step in one persistent cooperative launch (csrc/kernels/decode_mega.cu).
// Per-layer weights sit at constant element strides in flat bf16 buffers; wqkv and wgu are the copies with the RMSNorm
// weight folded in. Activation buffers have rows_alloc >= the row tile (32 / 64 / 128 / 256) that covers B rows.
struct DecodeLayersArgs {
  int L, B, rows_alloc, H, Q, QD, F, Hq, Hkv, num_sms, splits;
  const void *wqkv, *wo, *wgu, *wd;
  long long wqkv_stride, wo_stride, wgu_stride, wd_stride;
  const void* bqkv;  // nullptr = no bias
  long long bqkv_stride;
  void *x, *x1, *qkv, *attn, *act;
  long long* ss;     // [2 L + 1, ss_stride] row sums of squares, fixed point; entry 0 filled, the rest zero on entry
  int ss_stride;
  float eps;
  const float *cos_t, *sin_t;
  int max_pos;
  const int* block_tables;
  int max_blocks;
  const int* seq_lens;
  void* cache;       // [L, 2, num_cache_blocks, Hkv, 16, 128]
  long long cache_layer_stride, cache_v_off;
  int num_cache_blocks;
  float softmax_scale;
  float *part_o, *part_ml;
  int* att_tickets;
  float* partials;
  long long partials_bytes;
  unsigned int* counters;  // decode_layers_counter_words() words
  int* status;
  long long* trace = nullptr;  // optional phase tracer: 32 clock64 stamps of CTA 0 in layer trace_layer
  int trace_layer = 0;
  int prefetch_tiles = 0;      // weight tiles per CTA requested into L2 ahead of the shared-memory ring
  long long trace_words = 0;   // >= 32 + 4 * num_sms: four global-timer stamps per CTA are recorded as well
};
bool decode_layers_supported(int rows, int H, int Q, int QD, int F, int Hq, int Hkv, int head_dim);
long long decode_layers_scratch_bytes(int rows, int H, int Q, int QD, int F, int num_sms);
int decode_layers_counter_words();
void launch_decode_layers(const DecodeLayersArgs& a, cudaStream_t stream);

}  // namespace agrpo
