/* Allocation-free C entry point of the fused lm_head log-probability kernel.
 *
 * This entry point has no counterpart in the reference project; it exists for embedders of this library.
 *
 * Who needs it: host programs that must not (or cannot) obtain device memory at call time. Two examples: a
 * rollout server that handed the whole HBM to its KV-cache pool at start-up, so any later cudaMalloc fails; and
 * a latency-bound serving loop in which cudaMalloc's implicit device-wide synchronisation is not acceptable.
 * Such callers own their input and output buffers and only lack a place for the kernel's intermediate data.
 *
 * What it does: for T rows of bf16 hidden states and a bf16 [V, H] projection matrix it returns, per row,
 *   logp[t]    = z[t, labels[t]] - logsumexp(z[t, :])   (0 where labels[t] < 0)
 *   entropy[t] = logsumexp(z[t, :]) - sum_v softmax(z[t, :])[v] * z[t, v]
 *   lse[t]     = logsumexp(z[t, :])
 * with z = hidden . weight^T / temperature, without ever writing the [T, V] logits to memory. It runs the same
 * kernels as the library's regular lm_head log-probability path and returns the same numbers.
 *
 * Where the scratch lives: the per-column-group softmax partials that the regular path keeps in caller-allocated
 * scratch are kept here in ONE array of AGRPO_NOALLOC_SCRATCH_BYTES (8 MiB) that is part of the library image:
 * every GPU that loads the library carries it until the process exits. A problem needs
 *   4 * (3 * groups(V, T) + 1) * T  bytes,   groups(V, T) <= ceil(V / 256),
 * (about 3.8 MB for T = 8192, V = 151936). Larger problems are rejected with AGRPO_NOALLOC_E_TOO_LARGE and
 * nothing is launched.
 *
 * Rules for callers:
 *  - The first call on a device looks up the array's device address (once per device, with that device current).
 *    Make that first call outside of any stream capture.
 *  - All calls on a device share the array and it keeps the previous call's contents. The part that has to
 *    start from zero is cleared by every call. Two calls that can overlap on the GPU (different streams without
 *    an ordering between them) race on it: serialise them.
 *  - The function allocates nothing on the device: no cudaMalloc / cudaFree, no allocating library call.
 *  - Pointers are device pointers on the current device. hidden and weight must be 16-byte aligned, row pitches
 *    (in elements) multiples of 8; H a multiple of 8.
 *  - The work is enqueued on `stream` (a cudaStream_t, may be 0) and the function returns without waiting.
 *  - labels[t] must be below V (or negative = no label). They are device data and are not checked: a label >= V selects
 *    no column, and that row comes back as logp = -lse.
 *  - A return value of AGRPO_NOALLOC_OK says the work was enqueued, not that it ran correctly. The kernels bound every
 *    internal wait; should one run out (a device in trouble), they record it in a status word instead of hanging, and the
 *    outputs of that call are then not valid. Call agrpo_lmhead_noalloc_status(stream) after the call: it waits for the
 *    stream and returns that word (0 = outputs valid).
 *  - Within one process the function may be used on several GPUs: each holds its own copy of the array and is set up on
 *    its own first call.
 */
#ifndef AGRPO_NOALLOC_H_
#define AGRPO_NOALLOC_H_

#ifdef __cplusplus
extern "C" {
#endif

#define AGRPO_NOALLOC_SCRATCH_BYTES (8u << 20)

#define AGRPO_NOALLOC_OK 0
#define AGRPO_NOALLOC_E_BAD_ARGUMENT (-1)
#define AGRPO_NOALLOC_E_TOO_LARGE (-2)
#define AGRPO_NOALLOC_E_CUDA (-3)

/* Returns AGRPO_NOALLOC_OK or a negative error code. When `err_msg` is not NULL a NUL-terminated description of the
 * error is written into it (at most err_cap bytes). entropy and lse may be NULL. */
int agrpo_lmhead_logprob_noalloc(const void* hidden_bf16, long long hidden_pitch, const void* weight_bf16,
                                 long long weight_pitch, const int* labels, int T, int H, int V, float temperature,
                                 float* logp, float* entropy, float* lse, void* stream, char* err_msg, int err_cap);

/* Waits for `stream` and returns the status word that the most recent call on the current device left behind: 0 when its
 * kernels completed normally, a positive code when a bounded wait inside them ran out (discard that call's outputs),
 * AGRPO_NOALLOC_E_CUDA when the word could not be read. Has no counterpart in the reference project. */
int agrpo_lmhead_noalloc_status(void* stream);

#ifdef __cplusplus
}
#endif

#endif /* AGRPO_NOALLOC_H_ */
