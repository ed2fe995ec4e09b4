// out = LayerNorm(x + residual) over the last dimension, bf16 in and out, fp32 statistics: the tail of both output blocks of
// a DeBERTa layer (transformers' DebertaV2SelfOutput / DebertaV2Output, which the reference's FlashDebertaV2Attention and
// FlashDebertaV2Layer keep as they are, src/flashdeberta/model.py:259-272): dense -> dropout -> LayerNorm(hidden + input).
// In eager mode that is an elementwise add (3 passes over HBM) followed by torch's layer-norm kernel (2 passes, measured
// at 1.2 TB/s on this shape); here it is one kernel with 3 passes at streaming speed.  The sum is rounded to bf16 before
// the statistics, as the eager expression `self.LayerNorm(hidden_states + input_tensor)` does.
//
// One warp per row, 16-byte loads, the row stays in registers (hidden = VEC * 256 elements, VEC <= 8).  HBM-bound:
// 3 * hidden * 2 bytes per row (2 when there is no residual).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "internal.h"

namespace fdb {
namespace {

constexpr int kRowsPerBlock = 4;

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ float round_bf16(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int VEC>
__global__ void __launch_bounds__(32 * kRowsPerBlock) add_layernorm_kernel(const uint4* __restrict__ x,
                                                                          const uint4* __restrict__ residual,
                                                                          const uint4* __restrict__ gamma,
                                                                          const uint4* __restrict__ beta,
                                                                          uint4* __restrict__ out, int64_t rows, float eps,
                                                                          const int64_t* __restrict__ ids, int64_t table_rows,
                                                                          const float* __restrict__ row_scale,
                                                                          int32_t* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kRowsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  constexpr int kVecPerRow = VEC * 32;
  int64_t src = row;
  if (ids != nullptr) {  // embedding form: x is a table, this row is table[ids[row]]
    src = ids[row];
    if (src < 0 || src >= table_rows) {
      if (lane == 0 && status != nullptr) atomicOr(reinterpret_cast<unsigned int*>(status), FDB_DEV_BAD_INDEX);
      src = src < 0 ? 0 : table_rows - 1;
    }
  }
  const uint4* xr = x + src * kVecPerRow;
  const uint4* rr = residual != nullptr ? residual + row * kVecPerRow : nullptr;
  float v[VEC * 8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const uint4 a = __ldg(xr + i * 32 + lane);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
    if (rr != nullptr) {
      const uint4 b = __ldg(rr + i * 32 + lane);
      const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v[i * 8 + 2 * k] = round_bf16(bf16_lo(aw[k]) + bf16_lo(bw[k]));
        v[i * 8 + 2 * k + 1] = round_bf16(bf16_hi(aw[k]) + bf16_hi(bw[k]));
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v[i * 8 + 2 * k] = bf16_lo(aw[k]);
        v[i * 8 + 2 * k + 1] = bf16_hi(aw[k]);
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) sum += v[i * 8 + k];
  }
  constexpr float kInv = 1.f / float(VEC * 256);
  const float mean = warp_sum(sum) * kInv;
  float sq = 0.f;
#pragma unroll
  for (int k = 0; k < VEC * 8; ++k) {
    const float d = v[k] - mean;
    sq = fmaf(d, d, sq);
  }
  const float rstd = rsqrtf(warp_sum(sq) * kInv + eps);
  uint4* orow = out + row * kVecPerRow;
  const float scale = row_scale != nullptr ? row_scale[row] : 1.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const uint4 g = __ldg(gamma + i * 32 + lane), b = __ldg(beta + i * 32 + lane);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, bw[4] = {b.x, b.y, b.z, b.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float lo = fmaf((v[i * 8 + 2 * k] - mean) * rstd, bf16_lo(gw[k]), bf16_lo(bw[k]));
      float hi = fmaf((v[i * 8 + 2 * k + 1] - mean) * rstd, bf16_hi(gw[k]), bf16_hi(bw[k]));
      if (row_scale != nullptr) {  // the normalised row is rounded before it is scaled, as two separate kernels would
        lo = round_bf16(lo) * scale;
        hi = round_bf16(hi) * scale;
      }
      o[k] = pack2(lo, hi);
    }
    orow[i * 32 + lane] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <int VEC>
int launch(const void* x, const void* residual, const void* gamma, const void* beta, void* out, int64_t rows, float eps,
           cudaStream_t s, const int64_t* ids = nullptr, int64_t table_rows = 0, const float* row_scale = nullptr,
           int32_t* status = nullptr) {
  const int64_t blocks = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
  add_layernorm_kernel<VEC><<<(unsigned)blocks, 32 * kRowsPerBlock, 0, s>>>(
      static_cast<const uint4*>(x), static_cast<const uint4*>(residual), static_cast<const uint4*>(gamma),
      static_cast<const uint4*>(beta), static_cast<uint4*>(out), rows, eps, ids, table_rows, row_scale, status);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "add_layernorm launch: %s", cudaGetErrorString(e));
  return FDB_OK;
}

}  // namespace
}  // namespace fdb

using namespace fdb;

extern "C" FDB_API int fdb_add_layernorm(const void* x, const void* residual, const void* gamma, const void* beta, void* out,
                                         int64_t rows, int32_t hidden, float eps, void* stream) {
  clear_error();
  if (x == nullptr || gamma == nullptr || beta == nullptr || out == nullptr)
    return fail(FDB_ERR_INVALID_ARGUMENT, "x, gamma, beta and out must not be NULL");
  if (rows < 0 || rows > (int64_t(1) << 31) * kRowsPerBlock - 1) return fail(FDB_ERR_LIMIT, "rows = %lld", (long long)rows);
  if (hidden <= 0 || hidden % 256 != 0 || hidden > 2048)
    return fail(FDB_ERR_UNSUPPORTED, "hidden = %d: the kernel handles multiples of 256 up to 2048", hidden);
  const uintptr_t all = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(residual) |
                        reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(beta) | reinterpret_cast<uintptr_t>(out);
  if ((all & 15u) != 0) return fail(FDB_ERR_ALIGNMENT, "pointers must be 16-byte aligned");
  if (rows == 0) return FDB_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (hidden / 256) {
    case 1: return launch<1>(x, residual, gamma, beta, out, rows, eps, s);
    case 2: return launch<2>(x, residual, gamma, beta, out, rows, eps, s);
    case 3: return launch<3>(x, residual, gamma, beta, out, rows, eps, s);
    case 4: return launch<4>(x, residual, gamma, beta, out, rows, eps, s);
    case 5: return launch<5>(x, residual, gamma, beta, out, rows, eps, s);
    case 6: return launch<6>(x, residual, gamma, beta, out, rows, eps, s);
    case 7: return launch<7>(x, residual, gamma, beta, out, rows, eps, s);
    default: return launch<8>(x, residual, gamma, beta, out, rows, eps, s);
  }
}

extern "C" FDB_API int fdb_embed_layernorm(const int64_t* ids, const void* table, int64_t table_rows, const void* gamma,
                                           const void* beta, const float* row_scale, void* out, int64_t rows,
                                           int32_t hidden, float eps, int32_t* status, void* stream) {
  clear_error();
  if (ids == nullptr || table == nullptr || gamma == nullptr || beta == nullptr || out == nullptr)
    return fail(FDB_ERR_INVALID_ARGUMENT, "ids, table, gamma, beta and out must not be NULL");
  if (table_rows <= 0) return fail(FDB_ERR_INVALID_ARGUMENT, "table_rows = %lld", (long long)table_rows);
  if (rows < 0 || rows > (int64_t(1) << 31) * kRowsPerBlock - 1) return fail(FDB_ERR_LIMIT, "rows = %lld", (long long)rows);
  if (hidden <= 0 || hidden % 256 != 0 || hidden > 2048)
    return fail(FDB_ERR_UNSUPPORTED, "hidden = %d: the kernel handles multiples of 256 up to 2048", hidden);
  const uintptr_t all = reinterpret_cast<uintptr_t>(table) | reinterpret_cast<uintptr_t>(gamma) |
                        reinterpret_cast<uintptr_t>(beta) | reinterpret_cast<uintptr_t>(out);
  if ((all & 15u) != 0) return fail(FDB_ERR_ALIGNMENT, "table, gamma, beta and out must be 16-byte aligned");
  if (rows == 0) return FDB_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (hidden / 256) {
    case 1: return launch<1>(table, nullptr, gamma, beta, out, rows, eps, s, ids, table_rows, row_scale, status);
    case 2: return launch<2>(table, nullptr, gamma, beta, out, rows, eps, s, ids, table_rows, row_scale, status);
    case 3: return launch<3>(table, nullptr, gamma, beta, out, rows, eps, s, ids, table_rows, row_scale, status);
    case 4: return launch<4>(table, nullptr, gamma, beta, out, rows, eps, s, ids, table_rows, row_scale, status);
    case 5: return launch<5>(table, nullptr, gamma, beta, out, rows, eps, s, ids, table_rows, row_scale, status);
    case 6: return launch<6>(table, nullptr, gamma, beta, out, rows, eps, s, ids, table_rows, row_scale, status);
    case 7: return launch<7>(table, nullptr, gamma, beta, out, rows, eps, s, ids, table_rows, row_scale, status);
    default: return launch<8>(table, nullptr, gamma, beta, out, rows, eps, s, ids, table_rows, row_scale, status);
  }
}
