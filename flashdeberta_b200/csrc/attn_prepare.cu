// Set-up kernels that run in front of the fused attention kernel, on the same stream.
//
//  * seq_info_kernel   turns cu_seqlens / seq_lens into (first row, length) per sequence and an exclusive prefix of
//                      query tiles per sequence, so the fused kernel's CTAs can find their tile without any host
//                      involvement.  The reference builds the same map in a Python loop with one device->host read per
//                      sequence (src/flashdeberta/ops/flash_attention_varlen.py:71-83) and re-uploads it every layer.
//  * expand_tables_kernel  gathers rows of the projected position tables through the bucket table:
//                      expanded[h][u] = table[h][ idx(d_first + u) ].  After this the relative index of
//                      (query m, key n) is just the row (m - n) - d_first: every tile pair needs a contiguous window
//                      of rows and the fused kernel never evaluates the bucket function.
#include <cuda_runtime.h>

#include "internal.h"

namespace fdb {

ExpandGeometry expand_geometry(int32_t lut_d_min, int32_t lut_len) {
  ExpandGeometry g;
  g.sat_lo = lut_d_min;
  g.sat_hi = lut_d_min + lut_len - 1;
  // A tile pair that is not saturated has distances [d0, d0+254] with sat_lo-253 <= d0 <= sat_hi-1 and loads the
  // kWindow rows starting at d0.
  g.d_first = g.sat_lo - 254;
  g.rows = (g.sat_hi + 254) - g.d_first + 1;
  return g;
}

static inline uint64_t align256(uint64_t x) { return (x + 255) & ~uint64_t(255); }

// Two launches pay off once a query tile has key tiles with saturated position terms on both sides of the band.
static bool want_split(const fdb_attn_params& p) {
  if (p.dtype == FDB_E4M3 || (p.pos_key == nullptr && p.pos_query == nullptr)) return false;
  if (p.tune & FDB_TUNE_ONE_LAUNCH) return false;
  if (p.tune & FDB_TUNE_TWO_LAUNCHES) return true;
  return p.max_seqlen >= kSplitSeqlen;
}

int64_t tile_slots(const fdb_attn_params& p) {
  const int64_t dense_tiles = (int64_t)p.batch * ((p.max_seqlen + kTileM - 1) / kTileM);
  if (p.cu_seqlens == nullptr) return dense_tiles;
  const int64_t bound = (int64_t)(p.total_rows + kTileM - 1) / kTileM + p.batch;
  return dense_tiles < bound ? dense_tiles : bound;
}

WorkspaceLayout workspace_layout(const fdb_attn_params& p, const ExpandGeometry& g, bool allow_split) {
  WorkspaceLayout w;
  const uint64_t esz = p.dtype == FDB_E4M3 ? 1 : 2;
  uint64_t off = 0;
  w.seq_info = off;   off = align256(off + uint64_t(p.batch) * 2 * sizeof(int32_t));
  w.tile_first = off; off = align256(off + uint64_t(p.batch + 1) * sizeof(int32_t));
  w.slot_info = off;  off = align256(off + uint64_t(tile_slots(p)) * 4 * sizeof(int32_t));
  const uint64_t table = uint64_t(p.heads) * g.rows * kHeadDim * esz;
  w.exp_key = off;    off = align256(off + (p.pos_key ? table : 0));
  w.exp_query = off;  off = align256(off + (p.pos_query ? table : 0));
  w.split = allow_split && want_split(p);
  const uint64_t cells = w.split ? uint64_t(p.total_rows) * p.heads : 0;
  w.part_o = off;     off = align256(off + cells * kHeadDim * sizeof(float));
  w.part_ml = off;    off = align256(off + cells * 2 * sizeof(float));
  w.total = off;
  return w;
}

namespace {

constexpr int kScanThreads = 1024;

__global__ void __launch_bounds__(kScanThreads) seq_info_kernel(const int32_t* __restrict__ cu_seqlens,
                                                                const int32_t* __restrict__ seq_lens, int batch,
                                                                int max_seqlen, int total_rows,
                                                                int32_t* __restrict__ seq_info,
                                                                int32_t* __restrict__ tile_first,
                                                                int4* __restrict__ slot_info, int slots,
                                                                int32_t* __restrict__ status) {
  __shared__ int32_t partial[kScanThreads];
  const int t = threadIdx.x;
  const int per = (batch + kScanThreads - 1) / kScanThreads;
  const int b0 = t * per, b1 = min(batch, b0 + per);
  const bool packed = cu_seqlens != nullptr;
  const int dense_tiles = (max_seqlen + kTileM - 1) / kTileM;
  bool bad = false;
  int32_t sum = 0;
  for (int b = b0; b < b1; ++b) {
    int start, len;
    if (packed) {
      start = cu_seqlens[b];
      len = cu_seqlens[b + 1] - start;
      if (start < 0 || len < 0 || len > max_seqlen || start + len > total_rows) { bad = true; len = 0; start = 0; }
    } else {
      start = b * max_seqlen;
      len = seq_lens != nullptr ? seq_lens[b] : max_seqlen;
      if (len < 0 || len > max_seqlen) { bad = true; len = len < 0 ? 0 : max_seqlen; }
    }
    seq_info[2 * b] = start;
    seq_info[2 * b + 1] = len;
    // dense: every tile of the padded row range is visited so padding rows get their zeros
    sum += packed ? (len + kTileM - 1) / kTileM : dense_tiles;
  }
  partial[t] = sum;
  __syncthreads();
  for (int o = 1; o < kScanThreads; o <<= 1) {  // inclusive Hillis-Steele scan
    const int32_t add = t >= o ? partial[t - o] : 0;
    __syncthreads();
    partial[t] += add;
    __syncthreads();
  }
  const int32_t total_tiles = partial[kScanThreads - 1];
  int32_t run = partial[t] - sum;  // exclusive
  for (int b = b0; b < b1; ++b) {
    tile_first[b] = run;
    run += packed ? (seq_info[2 * b + 1] + kTileM - 1) / kTileM : dense_tiles;
  }
  if (t == kScanThreads - 1) tile_first[batch] = total_tiles;
  __syncthreads();

  // Slot table: the order in which the fused kernels' CTAs take the query tiles.  A query tile costs in proportion to its
  // sequence's length, so the sequences go longest first (ties by index): the last CTAs of a ragged batch are then the
  // cheap ones.  With more sequences than threads the order stays that of the batch.
  if (batch <= kScanThreads) {
    __shared__ int32_t tiles_by_rank[kScanThreads];
    int len = 0, start = 0, tiles = 0, rank = 0;
    if (t < batch) {
      start = seq_info[2 * t];
      len = seq_info[2 * t + 1];
      tiles = packed ? (len + kTileM - 1) / kTileM : dense_tiles;
      for (int o = 0; o < batch; ++o) {
        const int lo = seq_info[2 * o + 1];
        rank += (lo > len || (lo == len && o < t)) ? 1 : 0;
      }
    }
    __syncthreads();                 // `partial` is free again
    partial[t] = 0;
    __syncthreads();
    if (t < batch) tiles_by_rank[rank] = tiles;
    __syncthreads();
    partial[t] = t < batch ? tiles_by_rank[t] : 0;
    __syncthreads();
    for (int o = 1; o < kScanThreads; o <<= 1) {
      const int32_t add = t >= o ? partial[t - o] : 0;
      __syncthreads();
      partial[t] += add;
      __syncthreads();
    }
    if (t < batch) {
      // Within a sequence the query tiles away from both ends come first: they have the most band key tiles (the
      // expensive kind), so the CTAs that run last are the cheaper ones.
      const int32_t first = partial[rank] - tiles;  // exclusive prefix in rank order
      int pos = 0;
      auto emit = [&](int i) {
        if (first + pos < slots) slot_info[first + pos] = make_int4(t, i * kTileM, start, len);
        ++pos;
      };
      for (int i = 4; i <= tiles - 5; ++i) emit(i);
      for (int k = 3; k >= 0; --k) {
        const int lo = k, hi = tiles - 1 - k;
        if (lo > hi) continue;
        emit(lo);
        if (hi != lo) emit(hi);
      }
    }
  } else {
    int32_t at = partial[t] - sum;
    for (int b = b0; b < b1; ++b) {
      const int start = seq_info[2 * b], len = seq_info[2 * b + 1];
      const int tiles = packed ? (len + kTileM - 1) / kTileM : dense_tiles;
      for (int i = 0; i < tiles && at + i < slots; ++i) slot_info[at + i] = make_int4(b, i * kTileM, start, len);
      at += tiles;
    }
  }
  for (int i = total_tiles + t; i < slots; i += kScanThreads) slot_info[i] = make_int4(-1, 0, 0, 0);
  if (bad && status != nullptr) atomicOr(reinterpret_cast<unsigned int*>(status), FDB_DEV_BAD_SEQLEN);
}

// One thread copies 16 bytes.  row_bytes is 128 (bf16) or 64 (e4m3).
__global__ void expand_tables_kernel(const uint4* __restrict__ pos_key, const uint4* __restrict__ pos_query,
                                     uint4* __restrict__ exp_key, uint4* __restrict__ exp_query,
                                     const int16_t* __restrict__ lut, int lut_d_min, int lut_len, int d_first, int rows,
                                     int table_rows, int heads, int vec_per_row) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)heads * rows * vec_per_row;
  if (i >= total) return;
  const int c = (int)(i % vec_per_row);
  const int u = (int)((i / vec_per_row) % rows);
  const int h = (int)(i / ((int64_t)vec_per_row * rows));
  int li = d_first + u - lut_d_min;
  li = li < 0 ? 0 : (li >= lut_len ? lut_len - 1 : li);
  const int src = lut[li];
  const int64_t s = ((int64_t)h * table_rows + src) * vec_per_row + c;
  if (pos_key != nullptr) exp_key[i] = pos_key[s];
  if (pos_query != nullptr) exp_query[i] = pos_query[s];
}

}  // namespace

int launch_prepare(const fdb_attn_params& p, const ExpandGeometry& g, const WorkspaceLayout& w, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* ws = static_cast<char*>(p.workspace);
  if ((p.prepared & FDB_PREPARED_SCHEDULE) == 0)
    seq_info_kernel<<<1, kScanThreads, 0, s>>>(p.cu_seqlens, p.seq_lens, p.batch, p.max_seqlen, p.total_rows,
                                               reinterpret_cast<int32_t*>(ws + w.seq_info),
                                               reinterpret_cast<int32_t*>(ws + w.tile_first),
                                               reinterpret_cast<int4*>(ws + w.slot_info), (int)tile_slots(p), p.status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "seq_info launch: %s", cudaGetErrorString(e));
  if ((p.pos_key != nullptr || p.pos_query != nullptr) && (p.prepared & FDB_PREPARED_TABLES) == 0) {
    const int esz = p.dtype == FDB_E4M3 ? 1 : 2;
    const int vec_per_row = kHeadDim * esz / 16;
    const int table_rows = 2 * (p.position_buckets > 0 ? p.position_buckets : p.max_relative_positions);
    const int64_t total = (int64_t)p.heads * g.rows * vec_per_row;
    expand_tables_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(
        static_cast<const uint4*>(p.pos_key), static_cast<const uint4*>(p.pos_query),
        reinterpret_cast<uint4*>(ws + w.exp_key), reinterpret_cast<uint4*>(ws + w.exp_query), p.bucket_lut,
        p.lut_d_min, p.lut_len, g.d_first, g.rows, table_rows, p.heads, vec_per_row);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "expand_tables launch: %s", cudaGetErrorString(e));
  }
  return FDB_OK;
}

}  // namespace fdb
