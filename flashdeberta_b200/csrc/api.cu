// C ABI of libfdb_b200.so: argument checks, error text, dispatch to the launchers.  See include/fdb_b200.h.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "internal.h"

namespace fdb {

static thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}
void clear_error() { g_error[0] = 0; }

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Checks shared by the fused and the check kernel.  `fused` adds the layout rules TMA imposes.
int validate(const fdb_attn_params* p, bool fused) {
  if (p == nullptr) return fail(FDB_ERR_INVALID_ARGUMENT, "params is NULL");
  if (p->struct_bytes != sizeof(fdb_attn_params))
    return fail(FDB_ERR_INVALID_ARGUMENT, "struct_bytes is %u, this library expects %zu (ABI %d)", p->struct_bytes,
                sizeof(fdb_attn_params), FDB_ABI_VERSION);
  if (p->q == nullptr || p->k == nullptr || p->v == nullptr || p->out == nullptr)
    return fail(FDB_ERR_INVALID_ARGUMENT, "q, k, v and out must not be NULL");
  if (p->batch < 0 || p->max_seqlen < 0 || p->total_rows < 0 || p->heads <= 0 || p->head_dim <= 0)
    return fail(FDB_ERR_INVALID_ARGUMENT, "negative size (batch %d, max_seqlen %d, total_rows %d, heads %d, head_dim %d)",
                p->batch, p->max_seqlen, p->total_rows, p->heads, p->head_dim);
  if (p->dtype != FDB_BF16 && p->dtype != FDB_FP32 && p->dtype != FDB_E4M3)
    return fail(FDB_ERR_INVALID_ARGUMENT, "unknown dtype %d", p->dtype);
  if (p->cu_seqlens != nullptr && p->seq_lens != nullptr)
    return fail(FDB_ERR_INVALID_ARGUMENT, "give cu_seqlens (packed) or seq_lens (dense), not both");
  if (p->cu_seqlens == nullptr && (int64_t)p->batch * p->max_seqlen != p->total_rows)
    return fail(FDB_ERR_INVALID_ARGUMENT, "dense layout needs total_rows == batch * max_seqlen (%d != %d * %d)",
                p->total_rows, p->batch, p->max_seqlen);
  if (!(p->sm_scale > 0.f)) return fail(FDB_ERR_INVALID_ARGUMENT, "sm_scale must be positive");
  if ((p->prepared & ~(FDB_PREPARED_SCHEDULE | FDB_PREPARED_TABLES)) != 0)
    return fail(FDB_ERR_INVALID_ARGUMENT, "unknown bits in prepared: 0x%x", p->prepared);
  if ((p->tune & ~(FDB_TUNE_ONE_LAUNCH | FDB_TUNE_TWO_LAUNCHES)) != 0 ||
      (p->tune & (FDB_TUNE_ONE_LAUNCH | FDB_TUNE_TWO_LAUNCHES)) == (FDB_TUNE_ONE_LAUNCH | FDB_TUNE_TWO_LAUNCHES))
    return fail(FDB_ERR_INVALID_ARGUMENT, "unknown or contradictory bits in tune: 0x%x", p->tune);
  if (p->pos_key != nullptr || p->pos_query != nullptr) {
    const int span = p->position_buckets > 0 ? p->position_buckets : p->max_relative_positions;
    if (span <= 0) return fail(FDB_ERR_INVALID_ARGUMENT, "position tables given but att_span is %d", span);
    if (p->bucket_lut == nullptr || p->lut_len < 2)
      return fail(FDB_ERR_INVALID_ARGUMENT, "position tables given but bucket_lut is missing");
  }
  if (fused) {
    if (p->dtype == FDB_FP32) return fail(FDB_ERR_UNSUPPORTED, "the fused kernel takes bf16 or e4m3 inputs, not fp32");
    if (p->head_dim != kHeadDim) return fail(FDB_ERR_UNSUPPORTED, "the fused kernel is built for head_dim 64, got %d", p->head_dim);
    const int64_t esz = p->dtype == FDB_E4M3 ? 1 : 2;
    const int64_t strides[6] = {p->q_row_stride, p->q_head_stride, p->k_row_stride, p->k_head_stride, p->v_row_stride,
                                p->v_head_stride};
    for (int64_t s : strides)
      if (s <= 0 || (s * esz) % 16 != 0)
        return fail(FDB_ERR_ALIGNMENT, "q/k/v strides must be positive multiples of 16 bytes (got %lld elements)", (long long)s);
    if (p->out_row_stride % 8 != 0 || p->out_head_stride % 8 != 0)
      return fail(FDB_ERR_ALIGNMENT, "out strides must be multiples of 8 elements");
    if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->out) ||
        (p->pos_key && !aligned16(p->pos_key)) || (p->pos_query && !aligned16(p->pos_query)))
      return fail(FDB_ERR_ALIGNMENT, "q, k, v, out and the position tables must be 16-byte aligned");
    if (p->dtype == FDB_E4M3 && (p->q_scale == nullptr || p->k_scale == nullptr || p->v_scale == nullptr ||
                                 (p->pos_key && p->pos_key_scale == nullptr) || (p->pos_query && p->pos_query_scale == nullptr)))
      return fail(FDB_ERR_INVALID_ARGUMENT, "e4m3 inputs need q_scale, k_scale, v_scale and a scale per position table");
  } else {
    if (p->dtype == FDB_E4M3) return fail(FDB_ERR_UNSUPPORTED, "the check kernel takes bf16 or fp32 inputs");
    if (p->head_dim > 128) return fail(FDB_ERR_UNSUPPORTED, "the check kernel handles head_dim <= 128, got %d", p->head_dim);
  }
  return FDB_OK;
}

}  // namespace fdb

using namespace fdb;

extern "C" {

int fdb_abi_version(void) { return FDB_ABI_VERSION; }

const char* fdb_last_error(void) { return g_error; }

const char* fdb_status_string(int code) {
  switch (code) {
    case FDB_OK: return "ok";
    case FDB_ERR_INVALID_ARGUMENT: return "invalid argument";
    case FDB_ERR_UNSUPPORTED: return "unsupported configuration";
    case FDB_ERR_ALIGNMENT: return "misaligned pointer or stride";
    case FDB_ERR_WORKSPACE: return "workspace missing or too small";
    case FDB_ERR_CUDA: return "CUDA call failed";
    case FDB_ERR_LIMIT: return "size above a fixed maximum";
    default: return "unknown status";
  }
}

int fdb_build_bucket_lut(int32_t position_buckets, int32_t max_relative_positions, int16_t* out, int32_t capacity,
                         int32_t* d_min, int32_t* len) {
  clear_error();
  if (d_min == nullptr || len == nullptr) return fail(FDB_ERR_INVALID_ARGUMENT, "d_min and len must not be NULL");
  const int64_t span = position_buckets > 0 ? position_buckets : max_relative_positions;
  if (span <= 0 || 2 * span - 1 > 32767)
    return fail(FDB_ERR_INVALID_ARGUMENT, "att_span %lld outside [1, 16384]", (long long)span);
  if (!lut_range(position_buckets, max_relative_positions, d_min, len))
    return fail(FDB_ERR_LIMIT, "relative index does not saturate within 2^22 positions");
  if (out == nullptr) return FDB_OK;
  if (capacity < *len) return fail(FDB_ERR_INVALID_ARGUMENT, "capacity %d < %d entries", capacity, *len);
  for (int32_t i = 0; i < *len; ++i)
    out[i] = static_cast<int16_t>(relative_index(position_buckets, max_relative_positions, (int64_t)*d_min + i));
  return FDB_OK;
}

int32_t fdb_relative_index(int32_t position_buckets, int32_t max_relative_positions, int64_t distance) {
  return relative_index(position_buckets, max_relative_positions, distance);
}

uint64_t fdb_attn_workspace_bytes(const fdb_attn_params* p) {
  clear_error();
  if (validate(p, true) != FDB_OK) return 0;
  ExpandGeometry g = {0, 0, 0, 0};
  if (p->pos_key != nullptr || p->pos_query != nullptr) g = expand_geometry(p->lut_d_min, p->lut_len);
  return workspace_layout(*p, g).total;
}

int fdb_attn_fwd(const fdb_attn_params* p, void* stream) {
  clear_error();
  int rc = validate(p, true);
  if (rc != FDB_OK) return rc;
  if (p->batch == 0 || p->total_rows == 0) return FDB_OK;
  ExpandGeometry g = {0, 0, 0, 0};
  if (p->pos_key != nullptr || p->pos_query != nullptr) g = expand_geometry(p->lut_d_min, p->lut_len);
  const WorkspaceLayout w = workspace_layout(*p, g);
  if (p->workspace == nullptr || p->workspace_bytes < w.total)
    return fail(FDB_ERR_WORKSPACE, "workspace of %llu bytes needed, %llu given", (unsigned long long)w.total,
                (unsigned long long)(p->workspace ? p->workspace_bytes : 0));
  if ((reinterpret_cast<uintptr_t>(p->workspace) & 255u) != 0) return fail(FDB_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
  if ((rc = launch_prepare(*p, g, w, stream)) != FDB_OK) return rc;
  return launch_attn_fwd_sm100(*p, g, w, stream);
}

int fdb_attn_fwd_check(const fdb_attn_params* p, void* stream) {
  clear_error();
  const int rc = validate(p, false);
  if (rc != FDB_OK) return rc;
  if (p->batch == 0 || p->total_rows == 0) return FDB_OK;
  return launch_attn_check(*p, stream);
}

int fdb_relative_index_matrix(const int16_t* bucket_lut, int32_t lut_d_min, int32_t lut_len, int32_t len_q,
                              int32_t len_k, int32_t* out, void* stream) {
  clear_error();
  if (bucket_lut == nullptr || out == nullptr || lut_len < 1 || len_q < 0 || len_k < 0)
    return fail(FDB_ERR_INVALID_ARGUMENT, "relative_index_matrix: bad argument");
  return launch_relative_index_matrix(bucket_lut, lut_d_min, lut_len, len_q, len_k, out, stream);
}

int fdb_quantize_e4m3(const void* x_bf16, int64_t rows, int64_t row_stride, int64_t head_stride,
                      const int32_t* slab_start, int32_t n_slabs, int32_t heads, int32_t head_dim, void* y_e4m3,
                      float* scale, void* stream) {
  clear_error();
  if (x_bf16 == nullptr || slab_start == nullptr || y_e4m3 == nullptr || scale == nullptr || n_slabs < 0 || heads <= 0 ||
      head_dim <= 0 || head_dim % 8 != 0 || rows < 0 || rows > 2147483647LL)
    return fail(FDB_ERR_INVALID_ARGUMENT, "quantize_e4m3: bad argument");
  // the kernels load 16 bytes at x + row*row_stride + head*head_stride + 8*i and store 8 bytes into y
  if (!aligned16(x_bf16) || (reinterpret_cast<uintptr_t>(y_e4m3) & 7u) != 0 || row_stride <= 0 || head_stride <= 0 ||
      row_stride % 8 != 0 || head_stride % 8 != 0)
    return fail(FDB_ERR_ALIGNMENT, "quantize_e4m3: x must be 16-byte aligned, y 8-byte aligned, strides positive multiples of 8 elements");
  if (n_slabs == 0 || rows == 0) return FDB_OK;
  return launch_quantize_e4m3(x_bf16, rows, row_stride, head_stride, slab_start, n_slabs, heads, head_dim, y_e4m3, scale, stream);
}

}  // extern "C"
