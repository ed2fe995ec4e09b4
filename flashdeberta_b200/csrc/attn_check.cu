// Check kernel: disentangled attention forward in plain fp32 on CUDA cores.
//
// One warp per (row, head).  It evaluates, term by term, what the eager module does
// (transformers modeling_deberta_v2.py:243-264 and :313-343): score = (Q.K + Q.pos_key[idx] + K.pos_query[idx]) * scale,
// softmax over the keys of the row's own sequence, times V.  The table row idx comes from the int16 table built on the
// host, looked up per score element.  No tensor cores, no shared staging of tiles: this exists to validate the fused
// kernel and the host plumbing on the device, not to be fast.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "internal.h"

namespace fdb {
namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxD = 128;

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ void store_out(float* p, float x) { *p = x; }
__device__ __forceinline__ void store_out(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }

__device__ __forceinline__ int lut_lookup(const int16_t* __restrict__ lut, int d_min, int len, int d) {
  int i = d - d_min;
  i = i < 0 ? 0 : (i >= len ? len - 1 : i);
  return lut[i];
}

struct CheckArgs {
  const void *q, *k, *v, *pos_key, *pos_query;
  void* out;
  int64_t q_rs, q_hs, k_rs, k_hs, v_rs, v_hs, o_rs, o_hs;
  const int32_t* cu_seqlens;
  const int32_t* seq_lens;
  const int16_t* lut;
  int lut_d_min, lut_len;
  int batch, max_seqlen, total_rows, heads, head_dim, table_rows;
  float sm_scale;
  float* lse;
  int32_t* status;
};

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) attn_check_kernel(CheckArgs a) {
  __shared__ float q_s[kWarpsPerBlock][kMaxD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerBlock + warp;
  const int h = blockIdx.y;
  if (row >= a.total_rows) return;
  const int D = a.head_dim;

  // which sequence owns this row
  int start, len;
  if (a.cu_seqlens != nullptr) {
    int lo = 0, hi = a.batch;  // find b with cu[b] <= row < cu[b+1]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (a.cu_seqlens[mid] <= row) lo = mid; else hi = mid;
    }
    start = a.cu_seqlens[lo];
    len = a.cu_seqlens[lo + 1] - start;
    // lengths the packed layout cannot hold are reported and cut to what exists, as the set-up kernel of the fused path does
    if (len < 0 || len > a.max_seqlen || start < 0 || (int64_t)start + len > a.total_rows) {
      if (lane == 0 && a.status != nullptr) atomicOr(reinterpret_cast<unsigned int*>(a.status), FDB_DEV_BAD_SEQLEN);
      start = start < 0 ? 0 : (start > a.total_rows ? a.total_rows : start);
      len = len < 0 ? 0 : (len > a.max_seqlen ? a.max_seqlen : len);
      if (len > a.total_rows - start) len = a.total_rows - start;
    }
    if (row < start || row >= start + len) len = 0;  // row past the last sequence, or an empty one
  } else {
    const int b = row / a.max_seqlen;
    start = b * a.max_seqlen;
    len = a.seq_lens != nullptr ? a.seq_lens[b] : a.max_seqlen;
    len = len < 0 ? 0 : (len > a.max_seqlen ? a.max_seqlen : len);
  }
  const int m = row - start;
  T* o_ptr = static_cast<T*>(a.out) + row * a.o_rs + h * a.o_hs;
  if (m >= len) {  // padding row
    for (int d = lane; d < D; d += 32) store_out(o_ptr + d, 0.f);
    if (a.lse != nullptr && lane == 0) a.lse[(int64_t)row * a.heads + h] = 0.f;
    return;
  }

  const T* q_ptr = static_cast<const T*>(a.q) + row * a.q_rs + h * a.q_hs;
  for (int d = lane; d < D; d += 32) q_s[warp][d] = to_f32(q_ptr[d]);
  __syncwarp();
  const T* k_base = static_cast<const T*>(a.k) + (int64_t)start * a.k_rs + h * a.k_hs;
  const T* v_base = static_cast<const T*>(a.v) + (int64_t)start * a.v_rs + h * a.v_hs;
  const T* pk = a.pos_key ? static_cast<const T*>(a.pos_key) + (int64_t)h * a.table_rows * D : nullptr;
  const T* pq = a.pos_query ? static_cast<const T*>(a.pos_query) + (int64_t)h * a.table_rows * D : nullptr;

  auto score = [&](int n) -> float {
    const T* kr = k_base + (int64_t)n * a.k_rs;
    float s = 0.f;
    for (int d = 0; d < D; ++d) s = fmaf(q_s[warp][d], to_f32(kr[d]), s);
    if (pk != nullptr || pq != nullptr) {
      const int idx = lut_lookup(a.lut, a.lut_d_min, a.lut_len, m - n);
      if (pk != nullptr) {
        const T* r = pk + (int64_t)idx * D;
        float c = 0.f;
        for (int d = 0; d < D; ++d) c = fmaf(q_s[warp][d], to_f32(r[d]), c);
        s += c;
      }
      if (pq != nullptr) {
        const T* r = pq + (int64_t)idx * D;
        float c = 0.f;
        for (int d = 0; d < D; ++d) c = fmaf(to_f32(kr[d]), to_f32(r[d]), c);
        s += c;
      }
    }
    return s * a.sm_scale;
  };

  // pass 1: row maximum
  float mx = -INFINITY;
  for (int n = lane; n < len; n += 32) mx = fmaxf(mx, score(n));
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));

  // pass 2: exp, sum, PV.  Lane j owns output dims j, j+32, ...
  float acc[kMaxD / 32] = {0.f, 0.f, 0.f, 0.f};
  float l = 0.f;
  for (int n0 = 0; n0 < len; n0 += 32) {
    const int n = n0 + lane;
    const float p = n < len ? __expf(score(n) - mx) : 0.f;
    l += p;
    const int cnt = min(32, len - n0);
    for (int j = 0; j < cnt; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const T* vr = v_base + (int64_t)(n0 + j) * a.v_rs;
#pragma unroll
      for (int t = 0; t < kMaxD / 32; ++t) {
        const int d = lane + 32 * t;
        if (d < D) acc[t] = fmaf(pj, to_f32(vr[d]), acc[t]);
      }
    }
  }
  for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
  const float inv = 1.f / l;
#pragma unroll
  for (int t = 0; t < kMaxD / 32; ++t) {
    const int d = lane + 32 * t;
    if (d < D) store_out(o_ptr + d, acc[t] * inv);
  }
  if (a.lse != nullptr && lane == 0) a.lse[(int64_t)row * a.heads + h] = mx + logf(l);
}

__global__ void relative_index_matrix_kernel(const int16_t* __restrict__ lut, int d_min, int len, int lq, int lk,
                                             int32_t* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)lq * lk) return;
  const int m = (int)(i / lk), n = (int)(i % lk);
  out[i] = lut_lookup(lut, d_min, len, m - n);
}

}  // namespace

int launch_attn_check(const fdb_attn_params& p, void* stream) {
  CheckArgs a;
  a.q = p.q; a.k = p.k; a.v = p.v; a.pos_key = p.pos_key; a.pos_query = p.pos_query; a.out = p.out;
  a.q_rs = p.q_row_stride; a.q_hs = p.q_head_stride; a.k_rs = p.k_row_stride; a.k_hs = p.k_head_stride;
  a.v_rs = p.v_row_stride; a.v_hs = p.v_head_stride; a.o_rs = p.out_row_stride; a.o_hs = p.out_head_stride;
  a.cu_seqlens = p.cu_seqlens; a.seq_lens = p.seq_lens; a.lut = p.bucket_lut;
  a.lut_d_min = p.lut_d_min; a.lut_len = p.lut_len;
  a.batch = p.batch; a.max_seqlen = p.max_seqlen; a.total_rows = p.total_rows; a.heads = p.heads;
  a.head_dim = p.head_dim;
  a.table_rows = 2 * (p.position_buckets > 0 ? p.position_buckets : p.max_relative_positions);
  a.sm_scale = p.sm_scale; a.lse = p.lse; a.status = p.status;
  if (p.heads > 65535) return fail(FDB_ERR_LIMIT, "the check kernel takes up to 65535 heads, got %d", p.heads);
  dim3 grid((p.total_rows + kWarpsPerBlock - 1) / kWarpsPerBlock, p.heads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p.dtype == FDB_FP32) attn_check_kernel<float><<<grid, kWarpsPerBlock * 32, 0, s>>>(a);
  else attn_check_kernel<__nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, s>>>(a);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "attn_check launch: %s", cudaGetErrorString(e));
  return FDB_OK;
}

int launch_relative_index_matrix(const int16_t* lut, int32_t d_min, int32_t len, int32_t lq, int32_t lk, int32_t* out,
                                 void* stream) {
  const int64_t n = (int64_t)lq * lk;
  if (n == 0) return FDB_OK;
  relative_index_matrix_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      lut, d_min, len, lq, lk, out);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "relative_index_matrix launch: %s", cudaGetErrorString(e));
  return FDB_OK;
}

}  // namespace fdb
