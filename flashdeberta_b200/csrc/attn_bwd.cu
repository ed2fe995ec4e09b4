// Backward of the disentangled attention: the two steps that are not plain GEMMs.
//
// The host side (flashdeberta_b200/backward.py) walks a group of sequences in blocks of query rows.  Per block the
// library GEMM produces Q.K^T, dO.V^T and Q.pos_key^T (and once per group K.pos_query^T); the kernels here
//   1. rebuild the probabilities of the block and form dS in the same pass (bwd_probs_kernel), and
//   2. sum dS over the score elements that share a row of the position tables: per query row over keys (c2p,
//      bwd_c2p_sums_kernel) and per key over query rows (p2c, bwd_p2c_sums_kernel),
// after which every remaining contraction is a plain GEMM again.  The reference does the same work inside its Triton
// backward kernels and scatters the position-bias gradients with global atomics
// (src/flashdeberta/ops/flash_attention.py:616-797, :770-786, :799-940); here the relative index is non-decreasing in
// the distance, so the elements that share a table row are one run of keys (of queries), and the sums need no global
// atomics at all.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <climits>

#include "internal.h"

namespace fdb {
namespace {

__device__ __forceinline__ int lut_at(const int16_t* __restrict__ lut, int d_min, int len, int d) {
  int i = d - d_min;
  i = i < 0 ? 0 : (i >= len ? len - 1 : i);
  return lut[i];
}

__device__ __forceinline__ int seq_len_of(const fdb_bwd_block& a, int group) {
  int len = a.seq_lens != nullptr ? a.seq_lens[group / a.heads] : a.seqlen;
  return len < 0 ? 0 : (len > a.seqlen ? a.seqlen : len);
}

// ---------------------------------------------------------------------------------------------------------------------
// 1. P and dS of a block.  One CTA per (32 query rows x 64 keys) tile of one group.  The c2p term of a score sits in
// the row of its query, the p2c term in the row of its key, and consecutive keys (queries) address consecutive table
// entries; so the tile is walked twice, once with a warp along the keys (coalesced reads of the scores and of the c2p
// row) and once with a warp along the queries (coalesced reads of the p2c row), with the tile in shared memory between.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kPm = 32, kPn = 64, kPThreads = 256;

__global__ void __launch_bounds__(kPThreads) bwd_probs_kernel(fdb_bwd_block a) {
  __shared__ float s_s[kPm][kPn + 1];
  __shared__ float s_d[kPm][kPn + 1];
  const int g = blockIdx.z;
  const int r0 = blockIdx.y * kPm;   // first row of the tile inside the block
  const int n0 = blockIdx.x * kPn;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = seq_len_of(a, g);
  const int64_t gl = (int64_t)g * a.rows;
  const bool pos = a.table_rows > 0 && a.lut != nullptr;

  // pass 1, a warp along the keys: scores + c2p, and dP - delta
#pragma unroll
  for (int i = 0; i < kPm / 8; ++i) {
    const int r = r0 + warp + 8 * i;
    const int m = a.row0 + r;
#pragma unroll
    for (int j = 0; j < kPn / 32; ++j) {
      const int n = n0 + lane + 32 * j;
      float s = 0.f, d = 0.f;
      if (r < a.rows && n < a.seqlen && m < len && n < len) {
        const int64_t e = (gl + r) * a.seqlen + n;
        s = a.scores[e];
        d = a.dprobs[e] - a.delta[gl + r];
        if (pos && a.c2p != nullptr) s += a.c2p[(gl + r) * a.table_rows + lut_at(a.lut, a.lut_d_min, a.lut_len, m - n)];
      }
      s_s[warp + 8 * i][lane + 32 * j] = s;
      s_d[warp + 8 * i][lane + 32 * j] = d;
    }
  }
  __syncthreads();
  // pass 2, a warp along the queries: + p2c, exponential, dS
  {
    const int r = r0 + lane;
    const int m = a.row0 + r;
    const float lse = r < a.rows ? a.lse[gl + r] : 0.f;
#pragma unroll
    for (int j = 0; j < kPn / 8; ++j) {
      const int c = warp + 8 * j;
      const int n = n0 + c;
      float p = 0.f, ds = 0.f;
      if (r < a.rows && n < a.seqlen && m < len && n < len) {
        float s = s_s[lane][c];
        if (pos && a.p2c != nullptr)
          s += a.p2c[((int64_t)g * a.seqlen + n) * a.table_rows + lut_at(a.lut, a.lut_d_min, a.lut_len, m - n)];
        p = __expf(a.sm_scale * s - lse);
        ds = a.sm_scale * p * s_d[lane][c];
      }
      s_s[lane][c] = p;
      s_d[lane][c] = ds;
    }
  }
  __syncthreads();
  // pass 3, a warp along the keys again: store
  __nv_bfloat16* probs = static_cast<__nv_bfloat16*>(a.probs);
  __nv_bfloat16* dscores = static_cast<__nv_bfloat16*>(a.dscores);
#pragma unroll
  for (int i = 0; i < kPm / 8; ++i) {
    const int r = r0 + warp + 8 * i;
#pragma unroll
    for (int j = 0; j < kPn / 32; ++j) {
      const int n = n0 + lane + 32 * j;
      if (r < a.rows && n < a.seqlen) {
        const int64_t e = (gl + r) * a.seqlen + n;
        probs[e] = __float2bfloat16_rn(s_s[warp + 8 * i][lane + 32 * j]);
        dscores[e] = __float2bfloat16_rn(s_d[warp + 8 * i][lane + 32 * j]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// 2a. c2p sums: GC[m][b] = sum of dS[m][n] over the keys n with idx(m - n) == b, i.e. n in [m - last_b, m - first_b].
// One CTA per (query row, group); thread b walks its own run of keys (short everywhere but at the two saturated ends,
// whose runs the whole CTA sums together afterwards).
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kCThreads = 256;
constexpr int kLongRun = 64;

__global__ void __launch_bounds__(kCThreads) bwd_c2p_sums_kernel(fdb_bwd_block a) {
  __shared__ float red[kCThreads / 32];
  __shared__ int long_rows[8];
  __shared__ int n_long;
  const int r = blockIdx.x, g = blockIdx.y;
  const int m = a.row0 + r;
  const int len = seq_len_of(a, g);
  const int64_t row = (int64_t)g * a.rows + r;
  const __nv_bfloat16* ds = static_cast<const __nv_bfloat16*>(a.dscores) + row * a.seqlen;
  float* out = a.c2p_sums + row * a.table_rows;
  if (threadIdx.x == 0) n_long = 0;
  __syncthreads();
  const int keys = m < len ? len : 0;  // rows of the padding have no keys
  for (int b = threadIdx.x; b < a.table_rows; b += kCThreads) {
    const int first = a.bucket_range[2 * b], last = a.bucket_range[2 * b + 1];
    // n = m - d, d in [first, last]  ->  n in [m - last, m - first]; computed in 64 bits (the open ends are INT_MIN/MAX)
    int64_t lo = (int64_t)m - last, hi = (int64_t)m - first;
    lo = lo < 0 ? 0 : lo;
    hi = hi > keys - 1 ? keys - 1 : hi;
    float acc = 0.f;
    if (first <= last && lo <= hi) {
      if (hi - lo >= kLongRun) {
        const int slot = atomicAdd(&n_long, 1);
        if (slot < 8) long_rows[slot] = b;
        else for (int64_t n = lo; n <= hi; ++n) acc += __bfloat162float(ds[n]);  // cannot happen with two open ends
      } else {
        for (int64_t n = lo; n <= hi; ++n) acc += __bfloat162float(ds[n]);
      }
    }
    out[b] = acc;
  }
  __syncthreads();
  const int todo = n_long < 8 ? n_long : 8;
  for (int t = 0; t < todo; ++t) {
    const int b = long_rows[t];
    const int first = a.bucket_range[2 * b], last = a.bucket_range[2 * b + 1];
    int64_t lo = (int64_t)m - last, hi = (int64_t)m - first;
    lo = lo < 0 ? 0 : lo;
    hi = hi > keys - 1 ? keys - 1 : hi;
    float acc = 0.f;
    for (int64_t n = lo + threadIdx.x; n <= hi; n += kCThreads) acc += __bfloat162float(ds[n]);
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
      for (int w = 0; w < kCThreads / 32; ++w) s += red[w];
      out[b] = s;
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// 2b. p2c sums: GP[n][b] += sum of dS[m][n] over the block's query rows m with idx(m - n) == b.  One CTA per (32 keys,
// group): lane = key (coalesced reads of dS), the eight warps take an eighth of the block's rows each.  Walking down a
// column the index never decreases, so a thread keeps a running sum and hands it over when the index changes; the
// hand-over goes to shared memory (one row of table entries per key), which is added to the global sums at the end,
// only over the entries this block can have touched.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kQKeys = 32, kQThreads = 256;

__global__ void __launch_bounds__(kQThreads) bwd_p2c_sums_kernel(fdb_bwd_block a) {
  extern __shared__ float acc_s[];  // [kQKeys][pitch]
  const int pitch = a.table_rows + 2;  // keys next to each other address entries next to each other: keep them in different banks
  const int g = blockIdx.y;
  const int n0 = blockIdx.x * kQKeys;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = seq_len_of(a, g);
  // table entries this block can touch: distances (row0 - n0 - 31) .. (row0 + rows - 1 - n0)
  const int b_lo = lut_at(a.lut, a.lut_d_min, a.lut_len, a.row0 - n0 - (kQKeys - 1));
  const int b_hi = lut_at(a.lut, a.lut_d_min, a.lut_len, a.row0 + a.rows - 1 - n0);
  const int span = b_hi - b_lo + 1;
  for (int i = threadIdx.x; i < kQKeys * span; i += kQThreads) acc_s[(i / span) * pitch + b_lo + i % span] = 0.f;
  __syncthreads();
  const int n = n0 + lane;
  if (n < len) {
    const int per = (a.rows + 7) / 8;
    const int r_begin = warp * per;
    int r_end = r_begin + per;
    r_end = r_end > a.rows ? a.rows : r_end;
    if (a.row0 + r_end > len) r_end = len - a.row0;  // rows of the padding carry zeros anyway
    const __nv_bfloat16* ds = static_cast<const __nv_bfloat16*>(a.dscores) + (int64_t)g * a.rows * a.seqlen + n;
    int cur = -1;
    float acc = 0.f;
    for (int r = r_begin; r < r_end; ++r) {
      const int b = lut_at(a.lut, a.lut_d_min, a.lut_len, a.row0 + r - n);
      if (b != cur) {
        if (cur >= 0) atomicAdd(&acc_s[lane * pitch + cur], acc);
        cur = b;
        acc = 0.f;
      }
      acc += __bfloat162float(ds[(int64_t)r * a.seqlen]);
    }
    if (cur >= 0) atomicAdd(&acc_s[lane * pitch + cur], acc);
  }
  __syncthreads();
  float* out = a.p2c_sums + ((int64_t)g * a.seqlen + n0) * a.table_rows;
  for (int i = threadIdx.x; i < kQKeys * span; i += kQThreads) {
    const int key = i / span, b = b_lo + i % span;
    if (n0 + key < len) out[(int64_t)key * a.table_rows + b] += acc_s[key * pitch + b];
  }
}

int check_block(const fdb_bwd_block* p) {
  if (p == nullptr || p->struct_bytes != sizeof(fdb_bwd_block))
    return fail(FDB_ERR_INVALID_ARGUMENT, "fdb_bwd_block: NULL or struct_bytes %u != %zu", p ? p->struct_bytes : 0u,
                sizeof(fdb_bwd_block));
  if (p->groups < 0 || p->heads <= 0 || p->groups % p->heads != 0 || p->seqlen < 0 || p->rows < 0 || p->row0 < 0 ||
      p->row0 + (int64_t)p->rows > p->seqlen || p->table_rows < 0)
    return fail(FDB_ERR_INVALID_ARGUMENT, "fdb_bwd_block: bad sizes (groups %d, heads %d, seqlen %d, row0 %d, rows %d)",
                p->groups, p->heads, p->seqlen, p->row0, p->rows);
  if (p->groups > 65535) return fail(FDB_ERR_LIMIT, "fdb_bwd_block: more than 65535 groups in one block");
  if (p->table_rows > 0 && (p->lut == nullptr || p->lut_len <= 0))
    return fail(FDB_ERR_INVALID_ARGUMENT, "fdb_bwd_block: position terms need the bucket table");
  return FDB_OK;
}

int after_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return FDB_OK;
}

}  // namespace
}  // namespace fdb

using namespace fdb;

extern "C" FDB_API int fdb_attn_bwd_probs(const fdb_bwd_block* p, void* stream) {
  clear_error();
  int rc = check_block(p);
  if (rc != FDB_OK) return rc;
  if (p->scores == nullptr || p->dprobs == nullptr || p->lse == nullptr || p->delta == nullptr || p->probs == nullptr ||
      p->dscores == nullptr)
    return fail(FDB_ERR_INVALID_ARGUMENT, "fdb_attn_bwd_probs: scores, dprobs, lse, delta, probs and dscores are required");
  if (p->groups == 0 || p->rows == 0 || p->seqlen == 0) return FDB_OK;
  const dim3 grid((p->seqlen + kPn - 1) / kPn, (p->rows + kPm - 1) / kPm, p->groups);
  if (grid.y > 65535) return fail(FDB_ERR_LIMIT, "fdb_attn_bwd_probs: more than %d rows in one block", 65535 * kPm);
  bwd_probs_kernel<<<grid, kPThreads, 0, static_cast<cudaStream_t>(stream)>>>(*p);
  return after_launch("bwd_probs_kernel");
}

extern "C" FDB_API int fdb_attn_bwd_bucket_sums(const fdb_bwd_block* p, void* stream) {
  clear_error();
  int rc = check_block(p);
  if (rc != FDB_OK) return rc;
  if (p->dscores == nullptr || p->table_rows <= 0 || p->bucket_range == nullptr)
    return fail(FDB_ERR_INVALID_ARGUMENT, "fdb_attn_bwd_bucket_sums: dscores, the bucket table and its ranges are required");
  if (p->groups == 0 || p->rows == 0 || p->seqlen == 0) return FDB_OK;
  if (p->c2p_sums != nullptr) {
    bwd_c2p_sums_kernel<<<dim3(p->rows, p->groups), kCThreads, 0, static_cast<cudaStream_t>(stream)>>>(*p);
    if ((rc = after_launch("bwd_c2p_sums_kernel")) != FDB_OK) return rc;
  }
  if (p->p2c_sums != nullptr) {
    const size_t smem = sizeof(float) * kQKeys * (size_t)(p->table_rows + 2);
    if (smem > 200 * 1024) return fail(FDB_ERR_LIMIT, "fdb_attn_bwd_bucket_sums: position tables of more than 1598 rows");
    if (smem > 48 * 1024) {  // per device and cheap, so asked for on every such launch
      const cudaError_t e = cudaFuncSetAttribute(bwd_p2c_sums_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "cudaFuncSetAttribute(bwd_p2c_sums_kernel): %s", cudaGetErrorString(e));
    }
    bwd_p2c_sums_kernel<<<dim3((p->seqlen + kQKeys - 1) / kQKeys, p->groups), kQThreads, smem, static_cast<cudaStream_t>(stream)>>>(*p);
    if ((rc = after_launch("bwd_p2c_sums_kernel")) != FDB_OK) return rc;
  }
  return FDB_OK;
}
