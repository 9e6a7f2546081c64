// Host-side launch arithmetic of the GEMV and the GEMM, free of CUDA so that it can be
// compiled and checked on a machine without a GPU: how the tiles of a weight are dealt out to
// CTAs, how many CTAs share the K loop of a GEMM tile, which activation-tile height is used.
#pragma once
#include <cstdint>

namespace turq {

// Units = tiles (groups of 4 tiles for Q8_0); a row-tile has KU of them. CTA b owns units
// [start(b), start(b + 1)) with start(b) = min(b * split_q + min(b, split_r), total).
struct GemvSplit {
  int grid;
  int split_q, split_r;
  bool aligned;  // every CTA owns whole row-tiles: no partial sums cross CTAs
};

// Whole row-tiles per CTA when that keeps at least 70 % of the CTA slots busy or the problem is
// small (at most 24 units per slot); otherwise an even split in units, where a row-tile cut
// between CTAs is finished by the CTA holding its first unit. Depends on the shape only.
// force: -1 = choose, 0 = even split, 1 = whole row-tiles.
inline GemvSplit plan_gemv_split(int row_tiles, int KU, int slots, int force = -1) {
  GemvSplit p{};
  const int64_t T = (int64_t)row_tiles * KU;
  const int per = (row_tiles + slots - 1) / slots;
  const int ga = per > 0 ? (row_tiles + per - 1) / per : 0;
  bool aligned = (int64_t)ga * 10 >= (int64_t)slots * 7 || T <= (int64_t)slots * 24;
  if (force == 0) aligned = false;
  if (force == 1) aligned = true;
  p.aligned = aligned;
  if (aligned) {
    p.grid = ga;
    p.split_q = per * KU;
    p.split_r = 0;
  } else {
    p.grid = (int64_t)slots > T ? (int)T : slots;
    p.split_q = (int)(T / p.grid);
    p.split_r = (int)(T % p.grid);
  }
  return p;
}

inline int64_t gemv_split_start(const GemvSplit& p, int64_t total_units, int b) {
  const int64_t u = (int64_t)b * p.split_q + (b < p.split_r ? b : p.split_r);
  return u < total_units ? u : total_units;
}

// ---- tcgen05 GEMM (128 weight rows per CTA)

// Activation rows per CTA: 64 for decode batches; 256 for prefill, unless twice as many CTAs
// still fit the SMs in one wave - then 128, which doubles the CTA count for the same work.
inline int plan_gemm_bn(int64_t n_rows, int64_t m, int sm_count, int force = 0) {
  if (force == 64 || force == 128 || force == 256) return force;
  int bn = m <= 64 ? 64 : 256;
  if (bn == 256 && 2 * ((n_rows + 127) / 128) * ((m + 255) / 256) <= sm_count) bn = 128;
  return bn;
}

// Split-K for decode batches (one 64-row activation tile): when the 128-row weight tiles alone
// leave SMs without a CTA, the K loop of every tile is shared out over several CTAs (at least 8
// blocks of 64 each, at most 16 CTAs). The split depends on the weight's shape only, so a row's
// result does not depend on the batch it is in; prefill (more than 64 rows) never splits.
// force: -1 = choose, 0 = never, > 0 = that many (still at least 8 blocks each).
inline int plan_gemm_splits(int64_t n_rows, int64_t m, int64_t k, int sm_count, int force = -1) {
  if (m > 64 || force == 0) return 1;
  const int64_t tiles = (n_rows + 127) / 128;
  int64_t s = tiles > 0 ? sm_count / tiles : 1;
  const int64_t by_k = (k / 64) / 8;
  if (force > 0) s = force;
  if (s > by_k) s = by_k;
  if (s > 16) s = 16;
  return s < 2 ? 1 : (int)s;
}

}  // namespace turq
