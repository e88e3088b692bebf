// Host packer: turns n samples (concatenated token ids plus per-sample lengths and scalars) into the
// padding-free 1 x T training layout in ONE pass, writing every field into one caller-provided
// (pinned) buffer so that a single host-to-device copy moves the whole microbatch.
//
// It covers what the reference does with two numba kernels and per-sample torch.tensor(list) copies
// (sample_processing_utils.py:29-105, 159-223; gpu_process_worker.py:1672-1686), and additionally emits
// cu_seqlens and the attention tile table, which removes the max_seqlen host sync of the reference's
// varlen path (gpu_process_worker.py:242-252).
#include "packer.h"

#include <algorithm>
#include <cstring>
#include <vector>

namespace agrpo {

long long count_tiles(const int* in_lens, const int* out_lens, int n, int tile) {
  long long c = 0;
  for (int i = 0; i < n; ++i) c += ((long long)in_lens[i] + out_lens[i] + tile - 1) / tile;
  return c;
}

void pack_microbatch(const int* ids_concat, const int* in_lens, const int* out_lens, const float* advantages,
                     const float* logprobs_concat, const float* entropies_concat, const float* ref_logprobs_concat,
                     int n, int tile, int* out_int, float* out_float, long long T, long long total_out,
                     long long n_tiles) {
  int* ids = out_int;
  int* pos = ids + T;
  int* labels = pos + T;
  int* cu = labels + T;
  int* oidx = cu + (n + 1);
  int* tiles = out_int + pack_tiles_offset(T, n, total_out);
  float* adv = out_float;
  float* oldlp = adv + T;
  float* oldent = oldlp + T;
  float* reflp = oldent + T;
  float* outlen = reflp + T;

  long long off = 0, oo = 0;
  struct TileRec { int start, len, q0; };
  std::vector<TileRec> recs;
  recs.reserve((size_t)n_tiles);
  cu[0] = 0;
  for (int i = 0; i < n; ++i) {
    const int li = in_lens[i], lo = out_lens[i], L = li + lo;
    std::memcpy(ids + off, ids_concat + off, sizeof(int) * (size_t)L);
    for (int p = 0; p < L; ++p) {
      pos[off + p] = p;
      // label of row p = token p + 1 when that token is an output token of this sample
      labels[off + p] = (p + 1 >= li && p + 1 < L) ? ids_concat[off + p + 1] : -100;
      adv[off + p] = advantages[i];
      outlen[off + p] = (float)lo;
    }
    if (logprobs_concat) std::memcpy(oldlp + off, logprobs_concat + off, sizeof(float) * (size_t)L);
    else std::fill(oldlp + off, oldlp + off + L, 0.f);
    if (entropies_concat) std::memcpy(oldent + off, entropies_concat + off, sizeof(float) * (size_t)L);
    else std::fill(oldent + off, oldent + off + L, 0.f);
    if (ref_logprobs_concat) std::memcpy(reflp + off, ref_logprobs_concat + off, sizeof(float) * (size_t)L);
    else std::fill(reflp + off, reflp + off + L, 0.f);
    for (int j = 0; j < lo; ++j) oidx[oo++] = (int)(off + li - 1 + j);
    for (int q0 = 0; q0 < L; q0 += tile) recs.push_back({(int)off, L, q0});
    off += L;
    cu[i + 1] = (int)off;
  }
  // heaviest query tiles first (most keys below the diagonal)
  std::stable_sort(recs.begin(), recs.end(), [](const TileRec& a, const TileRec& b) { return a.q0 > b.q0; });
  for (size_t t = 0; t < recs.size(); ++t) {
    tiles[4 * t + 0] = recs[t].start;
    tiles[4 * t + 1] = recs[t].len;
    tiles[4 * t + 2] = recs[t].q0;
    tiles[4 * t + 3] = 0;
  }
}

void broadcast_values(const float* values, const int* lens, int n, float* out) {
  long long o = 0;
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < lens[i]; ++j) out[o++] = values[i];
}

void normalize_rewards(const float* rewards, int n, float* out) {
  if (n <= 0) return;
  double mean = 0.0;
  for (int i = 0; i < n; ++i) mean += rewards[i];
  mean /= n;
  double var = 0.0;
  for (int i = 0; i < n; ++i) var += (rewards[i] - mean) * (rewards[i] - mean);
  var /= n;
  const double denom = std::sqrt(var) + 1e-4;
  for (int i = 0; i < n; ++i) out[i] = (float)((rewards[i] - mean) / denom);
}

}  // namespace agrpo
