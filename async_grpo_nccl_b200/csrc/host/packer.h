// Host-side sample packer (no CUDA, no torch).
#pragma once
#include <cmath>

namespace agrpo {

// Offset (in int32 words) of the tile table inside out_int: rounded up to 4 words so the table can be read as int4.
inline long long pack_tiles_offset(long long T, int n, long long total_out) {
  return (3 * T + n + 1 + total_out + 3) / 4 * 4;
}

long long count_tiles(const int* in_lens, const int* out_lens, int n, int tile);

// out_int  : ids[T] | pos[T] | labels[T] | cu_seqlens[n+1] | output_indices[total_out] | pad to 4 words | tiles[4*n_tiles]
// out_float: advantages[T] | old_logprobs[T] | old_entropies[T] | ref_logprobs[T] | output_len[T]
// labels[t] is the target token of row t (the next token when it is an output token of the same sample, else -100),
// i.e. the reference's left-shifted labels (grpo_loss.py:224, 278). Per-token inputs may be nullptr (zeros).
void pack_microbatch(const int* ids_concat, const int* in_lens, const int* out_lens, const float* advantages,
                     const float* logprobs_concat, const float* entropies_concat, const float* ref_logprobs_concat,
                     int n, int tile, int* out_int, float* out_float, long long T, long long total_out,
                     long long n_tiles);

void broadcast_values(const float* values, const int* lens, int n, float* out);
void normalize_rewards(const float* rewards, int n, float* out);

}  // namespace agrpo
