// Host-side integer table for the log-bucket relative-position index.
//
// Restates make_log_bucket_position (transformers models/deberta_v2/modeling_deberta_v2.py:56-69) and the clamp at
// :318 / :336, which the reference re-evaluates per score element inside its Triton kernels
// (src/flashdeberta/ops/flash_attention.py:236-254).  Here the function is evaluated once per distance on the host,
// in float32 steps like torch does for an int64 input, and the kernels only ever look rows up.
#include <cmath>
#include <cstdint>
#include <vector>

#include "internal.h"

namespace fdb {

static inline float log_f32(float x) { return static_cast<float>(std::log(static_cast<double>(x))); }

int64_t signed_bucket(int32_t bucket_size, int32_t max_position, int64_t rel) {
  const int64_t mid = bucket_size / 2;
  const int64_t sign = (rel > 0) - (rel < 0);
  const bool inside = (rel < mid) && (rel > -mid);
  const int64_t abs_pos = inside ? (mid - 1) : (rel < 0 ? -rel : rel);
  if (abs_pos <= mid) return rel;
  const float ratio = static_cast<float>(abs_pos) / static_cast<float>(mid);
  const float denom = log_f32(static_cast<float>(static_cast<double>(max_position - 1) / static_cast<double>(mid)));
  const float scaled = (log_f32(ratio) / denom) * static_cast<float>(mid - 1);
  const float log_pos = std::ceil(scaled) + static_cast<float>(mid);
  return static_cast<int64_t>(log_pos * static_cast<float>(sign));
}

int32_t relative_index(int32_t position_buckets, int32_t max_relative_positions, int64_t distance) {
  const int64_t span = position_buckets > 0 ? position_buckets : max_relative_positions;
  int64_t b = distance;
  if (position_buckets > 0 && max_relative_positions > 0) b = signed_bucket(position_buckets, max_relative_positions, distance);
  int64_t idx = b + span;
  if (idx < 0) idx = 0;
  if (idx > 2 * span - 1) idx = 2 * span - 1;
  return static_cast<int32_t>(idx);
}

// The index is monotone non-decreasing in the distance and constant beyond some |d|; find the two ends.
// Entry 0 is the largest distance d_lo with idx(d) == 0 for every d <= d_lo; the last entry is the smallest d_hi
// with idx(d) == 2*span-1 for every d >= d_hi.
bool lut_range(int32_t position_buckets, int32_t max_relative_positions, int32_t* d_min, int32_t* len) {
  const int64_t span = position_buckets > 0 ? position_buckets : max_relative_positions;
  if (span <= 0) return false;
  const int64_t limit = 1 << 22;
  int64_t lo = 0, hi = 0;
  while (lo > -limit && relative_index(position_buckets, max_relative_positions, lo) != 0) --lo;
  while (hi < limit && relative_index(position_buckets, max_relative_positions, hi) != 2 * span - 1) ++hi;
  if (lo <= -limit || hi >= limit) return false;
  *d_min = static_cast<int32_t>(lo);
  *len = static_cast<int32_t>(hi - lo + 1);
  return true;
}

}  // namespace fdb
