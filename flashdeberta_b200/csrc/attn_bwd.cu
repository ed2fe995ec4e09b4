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
// 1. P and dS of a block.  One CTA per (32 query rows x 128 keys) tile of one group.  The c2p term of a score sits in
// the row of its query, the p2c term in the row of its key, and consecutive keys (queries) address consecutive table
// entries; so the tile is walked twice, once with a warp along the keys (coalesced reads of the scores and of the c2p
// row) and once with a warp along the queries (coalesced reads of the p2c row), with the tile in shared memory between.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kPm = 32, kPn = 128, kPThreads = 256;

__global__ void __launch_bounds__(kPThreads) bwd_probs_kernel(fdb_bwd_block a) {
  __shared__ float s_s[kPm][kPn + 1];
  __shared__ float s_d[kPm][kPn + 1];
  __shared__ int16_t s_idx[kPm + kPn];  // table row of every distance of the tile: entry (m - n) - d_lo
  const int g = blockIdx.z;
  const int r0 = blockIdx.y * kPm;   // first row of the tile inside the block
  const int n0 = blockIdx.x * kPn;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = seq_len_of(a, g);
  const int64_t gl = (int64_t)g * a.rows;
  const bool pos = a.table_rows > 0 && a.lut != nullptr;
  const int d_lo = a.row0 + r0 - (n0 + kPn - 1);
  if (pos) {
    if (threadIdx.x < kPm + kPn - 1) s_idx[threadIdx.x] = (int16_t)lut_at(a.lut, a.lut_d_min, a.lut_len, d_lo + (int)threadIdx.x);
    __syncthreads();
  }

  // A tile that lies inside the block, inside the sequence and on an even row pitch takes the short way: no bounds
  // checks, two keys per global access.
  if (r0 + kPm <= a.rows && n0 + kPn <= len && a.row0 + r0 + kPm <= len && (a.seqlen & 1) == 0) {
    const bool has_c2p = pos && a.c2p != nullptr, has_p2c = pos && a.p2c != nullptr;
#pragma unroll
    for (int i = 0; i < kPm / 8; ++i) {
      const int rl = warp + 8 * i;
      const int64_t row = gl + r0 + rl;
      const float2* sp = reinterpret_cast<const float2*>(a.scores + row * a.seqlen + n0);
      const float2* dp = reinterpret_cast<const float2*>(a.dprobs + row * a.seqlen + n0);
      const float* cp = has_c2p ? a.c2p + row * a.table_rows : nullptr;
      const float delta = a.delta[row];
      const int16_t* ix = s_idx + (rl + kPn - 1);  // ix[-c] = table row of (row - key c of the tile)
#pragma unroll
      for (int j = 0; j < kPn / 64; ++j) {
        const int c = 2 * lane + 64 * j;
        float2 sv = sp[lane + 32 * j];
        const float2 dv = dp[lane + 32 * j];
        if (has_c2p) {
          sv.x += cp[ix[-c]];
          sv.y += cp[ix[-c - 1]];
        }
        s_s[rl][c] = sv.x;
        s_s[rl][c + 1] = sv.y;
        s_d[rl][c] = dv.x - delta;
        s_d[rl][c + 1] = dv.y - delta;
      }
    }
    __syncthreads();
    {
      const float lse = a.lse[gl + r0 + lane];
      const int16_t* ix = s_idx + (lane + kPn - 1);
      const float* pp = has_p2c ? a.p2c + ((int64_t)g * a.seqlen + n0) * a.table_rows : nullptr;
#pragma unroll
      for (int j = 0; j < kPn / 8; ++j) {
        const int c = warp + 8 * j;
        float sc = s_s[lane][c];
        if (has_p2c) sc += pp[(int64_t)c * a.table_rows + ix[-c]];
        const float pr = __expf(a.sm_scale * sc - lse);
        s_s[lane][c] = pr;
        s_d[lane][c] = a.sm_scale * pr * s_d[lane][c];
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kPm / 8; ++i) {
      const int rl = warp + 8 * i;
      const int64_t row = gl + r0 + rl;
      __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(a.probs) + row * a.seqlen + n0);
      __nv_bfloat162* go = reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(a.dscores) + row * a.seqlen + n0);
#pragma unroll
      for (int j = 0; j < kPn / 64; ++j) {
        const int c = 2 * lane + 64 * j;
        po[lane + 32 * j] = __floats2bfloat162_rn(s_s[rl][c], s_s[rl][c + 1]);
        go[lane + 32 * j] = __floats2bfloat162_rn(s_d[rl][c], s_d[rl][c + 1]);
      }
    }
    return;
  }

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
        if (pos && a.c2p != nullptr) s += a.c2p[(gl + r) * a.table_rows + s_idx[m - n - d_lo]];
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
          s += a.p2c[((int64_t)g * a.seqlen + n) * a.table_rows + s_idx[m - n - d_lo]];
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
// 2a. c2p sums: GC[m][b] = sum of dS[m][n] over the keys n with idx(m - n) == b.  Along a row the index never
// increases, so the keys that share a table row are one run, and its sum is a difference of two running sums of the
// row.  A warp takes a query row, 256 keys at a time: every lane adds up its own eight consecutive keys (one 16-byte
// load), a scan over the lanes turns that into the running sum S(n) of the row, and a key n that ends a run (the next key
// addresses another table row) adds +S(n) to its own table entry and -S(n) to the entry of the run that follows, in
// a shared-memory row of table entries.  Two shared-memory atomics per run, none per key, and no global atomics.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kCThreads = 256;
constexpr int kCWarps = kCThreads / 32;  // query rows per CTA: a warp each
constexpr int kCPer = 8;                 // consecutive keys per lane

__global__ void __launch_bounds__(kCThreads) bwd_c2p_sums_kernel(fdb_bwd_block a) {
  extern __shared__ float acc_c[];  // [kCWarps][table_rows], then the bucket table (int16[lut_len])
  int16_t* lut_s = reinterpret_cast<int16_t*>(acc_c + kCWarps * a.table_rows);
  const int g = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int len = seq_len_of(a, g);
  for (int i = threadIdx.x; i < a.lut_len; i += kCThreads) lut_s[i] = a.lut[i];
  for (int i = threadIdx.x; i < kCWarps * a.table_rows; i += kCThreads) acc_c[i] = 0.f;
  __syncthreads();
  const int r = blockIdx.x * kCWarps + warp;
  if (r >= a.rows) return;
  const int m = a.row0 + r;
  const int64_t row = (int64_t)g * a.rows + r;
  const __nv_bfloat16* ds = static_cast<const __nv_bfloat16*>(a.dscores) + row * a.seqlen;
  float* acc = acc_c + warp * a.table_rows;
  const bool vec = ((row * a.seqlen) & 7) == 0;  // the row starts on a 16-byte boundary
  const int keys = m < len ? len : 0;            // rows of the padding have no keys
  float carry = 0.f;                             // running sum of the row in front of this chunk
  for (int base = 0; base < keys; base += kCPer * 32) {
    const int n_first = base + lane * kCPer;
    float v[kCPer];
    if (vec && n_first + kCPer <= keys) {
      const uint4 w = *reinterpret_cast<const uint4*>(ds + n_first);
      const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        v[2 * u] = __uint_as_float(ww[u] << 16);
        v[2 * u + 1] = __uint_as_float(ww[u] & 0xffff0000u);
      }
    } else {
#pragma unroll
      for (int u = 0; u < kCPer; ++u) v[u] = n_first + u < keys ? __bfloat162float(ds[n_first + u]) : 0.f;
    }
    int ix[kCPer + 1];  // table rows of my keys and of the key after them
#pragma unroll
    for (int u = 0; u <= kCPer; ++u) {
      int i = m - (n_first + u) - a.lut_d_min;
      i = i < 0 ? 0 : (i >= a.lut_len ? a.lut_len - 1 : i);
      ix[u] = lut_s[i];
    }
    float run = 0.f;
#pragma unroll
    for (int u = 0; u < kCPer; ++u) { run += v[u]; v[u] = run; }  // running sum inside my keys
    float inc = run;  // inclusive scan of the lanes' totals
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += up;
    }
    const float before = carry + inc - run;
#pragma unroll
    for (int u = 0; u < kCPer; ++u) {
      const int n = n_first + u;
      if (n < keys && (n == keys - 1 || ix[u + 1] != ix[u])) {  // key n ends a run
        const float upto = before + v[u];
        atomicAdd(&acc[ix[u]], upto);
        if (n < keys - 1) atomicAdd(&acc[ix[u + 1]], -upto);
      }
    }
    carry = __shfl_sync(0xffffffffu, before + run, 31);
  }
  __syncwarp();
  float* out = a.c2p_sums + row * a.table_rows;
  for (int b = lane; b < a.table_rows; b += 32) out[b] = acc[b];
}

// ---------------------------------------------------------------------------------------------------------------------
// 2b. p2c sums: GP[n][b] += sum of dS[m][n] over the block's query rows m with idx(m - n) == b.  One CTA per (16 keys,
// group): half a warp along the keys (32-byte reads of dS), sixteen slices of the block's rows per CTA.  Walking down a
// column the index never decreases, so a thread keeps a running sum and hands it over when the index changes; the
// hand-over goes to shared memory (one row of table entries per key), which is added to the global sums at the end,
// only over the entries this block can have touched.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kQKeys = 16, kQThreads = 256, kQSlices = kQThreads / kQKeys;

__global__ void __launch_bounds__(kQThreads) bwd_p2c_sums_kernel(fdb_bwd_block a) {
  extern __shared__ float acc_s[];  // [kQKeys][pitch], then the table rows of the block's distances (int16)
  const int pitch = a.table_rows + 2;  // keys next to each other address entries next to each other: keep them in different banks
  int16_t* idx_s = reinterpret_cast<int16_t*>(acc_s + kQKeys * pitch);
  const int g = blockIdx.y;
  const int n0 = blockIdx.x * kQKeys;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = seq_len_of(a, g);
  // distances of this CTA: (row0 - n0 - 31) .. (row0 + rows - 1 - n0); idx_s[d - d_lo] is the table row of d
  const int d_lo = a.row0 - n0 - (kQKeys - 1);
  const int n_d = a.rows + kQKeys - 1;
  for (int i = threadIdx.x; i < n_d; i += kQThreads) idx_s[i] = (int16_t)lut_at(a.lut, a.lut_d_min, a.lut_len, d_lo + i);
  __syncthreads();
  const int b_lo = idx_s[0], b_hi = idx_s[n_d - 1];  // the index never decreases with the distance
  const int span = b_hi - b_lo + 1;
  for (int i = threadIdx.x; i < kQKeys * span; i += kQThreads) acc_s[(i / span) * pitch + b_lo + i % span] = 0.f;
  __syncthreads();
  const int key = lane & (kQKeys - 1);         // half a warp along the keys (32-byte reads of dS) ...
  const int slice = 2 * warp + (lane >> 4);    // ... and sixteen slices of the block's rows per CTA
  const int n = n0 + key;
  if (n < len) {
    const int per = (a.rows + kQSlices - 1) / kQSlices;
    const int r_begin = slice * per;
    int r_end = r_begin + per;
    r_end = r_end > a.rows ? a.rows : r_end;
    if (a.row0 + r_end > len) r_end = len - a.row0;  // rows of the padding carry zeros anyway
    const __nv_bfloat16* ds = static_cast<const __nv_bfloat16*>(a.dscores) + (int64_t)g * a.rows * a.seqlen + n;
    const int16_t* my_idx = idx_s + (a.row0 - n - d_lo);  // my_idx[r] = table row of (row0 + r) - n
    int cur = -1;
    float acc = 0.f;
    for (int r = r_begin; r < r_end; r += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)  // eight loads in flight: the walk is bound by their latency otherwise
        v[u] = r + u < r_end ? __bfloat162float(ds[(int64_t)(r + u) * a.seqlen]) : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (r + u < r_end) {
          const int b = my_idx[r + u];
          if (b != cur) {
            if (cur >= 0) atomicAdd(&acc_s[key * pitch + cur], acc);
            cur = b;
            acc = 0.f;
          }
          acc += v[u];
        }
      }
    }
    if (cur >= 0) atomicAdd(&acc_s[key * pitch + cur], acc);
  }
  __syncthreads();
  float* out = a.p2c_sums + ((int64_t)g * a.seqlen + n0) * a.table_rows;
  for (int i = threadIdx.x; i < kQKeys * span; i += kQThreads) {
    const int k2 = i / span, b = b_lo + i % span;
    if (n0 + k2 < len) out[(int64_t)k2 * a.table_rows + b] += acc_s[k2 * pitch + b];
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
  if (p->dscores == nullptr || p->table_rows <= 0)
    return fail(FDB_ERR_INVALID_ARGUMENT, "fdb_attn_bwd_bucket_sums: dscores and the bucket table are required");
  if (p->groups == 0 || p->rows == 0 || p->seqlen == 0) return FDB_OK;
  if (p->c2p_sums != nullptr) {
    if (p->table_rows > 8192) return fail(FDB_ERR_LIMIT, "fdb_attn_bwd_bucket_sums: position tables of more than 8192 rows");
    const size_t smem_c = sizeof(float) * kCWarps * (size_t)p->table_rows + sizeof(int16_t) * (size_t)p->lut_len;
    if (smem_c > 200 * 1024) return fail(FDB_ERR_LIMIT, "fdb_attn_bwd_bucket_sums: 32 * table_rows + 2 * lut_len bytes of shared memory exceed 200 KB");
    if (smem_c > 48 * 1024) {
      const cudaError_t e = cudaFuncSetAttribute(bwd_c2p_sums_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_c);
      if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "cudaFuncSetAttribute(bwd_c2p_sums_kernel): %s", cudaGetErrorString(e));
    }
    bwd_c2p_sums_kernel<<<dim3((p->rows + kCWarps - 1) / kCWarps, p->groups), kCThreads, smem_c, static_cast<cudaStream_t>(stream)>>>(*p);
    if ((rc = after_launch("bwd_c2p_sums_kernel")) != FDB_OK) return rc;
  }
  if (p->p2c_sums != nullptr) {
    const size_t smem = sizeof(float) * kQKeys * (size_t)(p->table_rows + 2) + sizeof(int16_t) * ((size_t)p->rows + kQKeys);
    if (smem > 200 * 1024)
      return fail(FDB_ERR_LIMIT, "fdb_attn_bwd_bucket_sums: 64 * (table_rows + 2) + 2 * (rows + 16) bytes of shared memory exceed 200 KB");
    if (smem > 48 * 1024) {  // per device and cheap, so asked for on every such launch
      const cudaError_t e = cudaFuncSetAttribute(bwd_p2c_sums_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "cudaFuncSetAttribute(bwd_p2c_sums_kernel): %s", cudaGetErrorString(e));
    }
    bwd_p2c_sums_kernel<<<dim3((p->seqlen + kQKeys - 1) / kQKeys, p->groups), kQThreads, smem, static_cast<cudaStream_t>(stream)>>>(*p);
    if ((rc = after_launch("bwd_p2c_sums_kernel")) != FDB_OK) return rc;
  }
  return FDB_OK;
}
