// Declarations shared by the translation units of libfdb_b200.so (not part of the public ABI).
#pragma once

#include <cstdarg>
#include <cstdint>

#include "fdb_b200.h"

namespace fdb {

// ---- error text (thread-local) -------------------------------------------------------------------------------------
int fail(int code, const char* fmt, ...);
void clear_error();
// argument checks shared by the entry points; `fused` adds the layout rules of the tensor-core kernel
int validate(const fdb_attn_params* p, bool fused);

// ---- bucket table (host) -------------------------------------------------------------------------------------------
int64_t signed_bucket(int32_t bucket_size, int32_t max_position, int64_t rel);
int32_t relative_index(int32_t position_buckets, int32_t max_relative_positions, int64_t distance);
bool lut_range(int32_t position_buckets, int32_t max_relative_positions, int32_t* d_min, int32_t* len);

// ---- geometry of the fused kernel ----------------------------------------------------------------------------------
constexpr int kTileM = 128;    // query rows per CTA tile
constexpr int kTileN = 128;    // keys per inner step
constexpr int kHeadDim = 64;   // the only head size the fused kernel is built for
constexpr int kWindow = 256;   // rows of an expanded position table staged for one (query tile, key tile) pair
// In a call that runs as two launches, only sequences of at least this many keys are split between them (shorter ones
// have too few far key tiles to pay for it).  Deciding per sequence keeps a sequence's result independent of the batch
// around it.
constexpr int kSplitSeqlen = 3584;

// Expanded position tables.  Row u of an expanded table holds table row idx(d) for d = d_first + u, so a tile pair
// whose distances are [d0, d0+254] needs the contiguous rows [d0 - d_first, +255): the bucket function never runs
// on the device in the fused kernel.  sat_lo / sat_hi are the last / first distances of the two saturated ends.
struct ExpandGeometry {
  int32_t sat_lo;   // idx(d) == first row for every d <= sat_lo
  int32_t sat_hi;   // idx(d) == last row  for every d >= sat_hi
  int32_t d_first;  // distance of expanded row 0
  int32_t rows;     // rows per head in an expanded table
};
ExpandGeometry expand_geometry(int32_t lut_d_min, int32_t lut_len);

// Workspace layout (all offsets multiples of 256 bytes).
struct WorkspaceLayout {
  uint64_t seq_info;   // int32[batch][2] first row, length
  uint64_t tile_first; // int32[batch+1] exclusive prefix of ceil(len/kTileM)
  uint64_t slot_info;  // int32[slots][4] per query-tile slot: sequence (-1: unused slot), first row within it, the
                       // sequence's first row, its length
  uint64_t exp_key;    // expanded pos_key, (heads, rows, 64) elements of the input type
  uint64_t exp_query;  // expanded pos_query
  uint64_t part_o;     // split launch only: float (total_rows, heads, 64) unnormalised output of the far key tiles
  uint64_t part_ml;    // split launch only: float (total_rows, heads, 2) reference maximum (log2 units), row sum
  bool split;          // far key tiles and band key tiles run as two launches
  uint64_t total;
};
// `allow_split` false keeps every key tile in one launch (no partial-result buffers in the workspace).
WorkspaceLayout workspace_layout(const fdb_attn_params& p, const ExpandGeometry& g, bool allow_split = true);
// Query-tile slots of a call: dense -> every tile of the padded row range; packed -> an upper bound on the tiles of the
// sequences (the exact number is only known on the device).
int64_t tile_slots(const fdb_attn_params& p);

// ---- launchers (defined in the .cu files) --------------------------------------------------------------------------
int launch_attn_check(const fdb_attn_params& p, void* stream);
int launch_prepare(const fdb_attn_params& p, const ExpandGeometry& g, const WorkspaceLayout& w, void* stream);
int launch_attn_fwd_sm100(const fdb_attn_params& p, const ExpandGeometry& g, const WorkspaceLayout& w, void* stream);
int launch_attn_fwd_far1(const void* fwd_args, int64_t slots, int heads, void* stream);  // fwd_args: fwd::FwdArgs
int launch_relative_index_matrix(const int16_t* lut, int32_t d_min, int32_t len, int32_t lq, int32_t lk, int32_t* out,
                                 void* stream);
int launch_quantize_e4m3(const void* x, int64_t rows, int64_t row_stride, int64_t head_stride, const int32_t* slab_start,
                         int32_t n_slabs, int32_t heads, int32_t head_dim, void* y, float* scale, void* stream);

}  // namespace fdb
