// Per-slab amax scaling of bf16 rows to float8 e4m3 (the FP8 option; the reference has no FP8 code).
//
// One CTA per (slab, head).  A slab is a run of rows [slab_start[s], slab_start[s+1]) — one sequence, or the whole
// position table — so every (sequence, head) gets its own scale = amax/448 and the stored value times the scale gives
// the input back.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "internal.h"

namespace fdb {
namespace {

constexpr int kQuantThreads = 256;

__global__ void __launch_bounds__(kQuantThreads) quantize_e4m3_kernel(const __nv_bfloat16* __restrict__ x, int64_t row_stride,
                                                                      int64_t head_stride,
                                                                      const int32_t* __restrict__ slab_start, int heads,
                                                                      int head_dim, uint8_t* __restrict__ y,
                                                                      float* __restrict__ scale) {
  __shared__ float red[kQuantThreads / 32];
  __shared__ float s_scale;
  const int slab = blockIdx.x, h = blockIdx.y;
  const int r0 = slab_start[slab], r1 = slab_start[slab + 1];
  const int vec_per_row = head_dim / 8;  // 8 bf16 = 16 bytes
  const int64_t n_vec = (int64_t)max(r1 - r0, 0) * vec_per_row;
  float amax = 0.f;
  for (int64_t i = threadIdx.x; i < n_vec; i += kQuantThreads) {
    const int r = r0 + (int)(i / vec_per_row), c = (int)(i % vec_per_row);
    const uint4 v = *reinterpret_cast<const uint4*>(x + r * row_stride + h * head_stride + c * 8);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(b[k]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = red[0];
    for (int w = 1; w < kQuantThreads / 32; ++w) a = fmaxf(a, red[w]);
    a = fmaxf(a, 1e-12f);
    s_scale = a / 448.f;
    scale[(int64_t)slab * heads + h] = s_scale;
  }
  __syncthreads();
  const float inv = 1.f / s_scale;
  for (int64_t i = threadIdx.x; i < n_vec; i += kQuantThreads) {
    const int r = r0 + (int)(i / vec_per_row), c = (int)(i % vec_per_row);
    const uint4 v = *reinterpret_cast<const uint4*>(x + r * row_stride + h * head_stride + c * 8);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint16_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(b[k]);
      o[k] = __nv_cvt_float2_to_fp8x2(make_float2(f.x * inv, f.y * inv), __NV_SATFINITE, __NV_E4M3);
    }
    uint2 packed;
    packed.x = (uint32_t)o[0] | ((uint32_t)o[1] << 16);
    packed.y = (uint32_t)o[2] | ((uint32_t)o[3] << 16);
    *reinterpret_cast<uint2*>(y + ((int64_t)r * heads + h) * head_dim + c * 8) = packed;
  }
}

}  // namespace

int launch_quantize_e4m3(const void* x, int64_t row_stride, int64_t head_stride, const int32_t* slab_start,
                         int32_t n_slabs, int32_t heads, int32_t head_dim, void* y, float* scale, void* stream) {
  quantize_e4m3_kernel<<<dim3(n_slabs, heads), kQuantThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), row_stride, head_stride, slab_start, heads, head_dim,
      static_cast<uint8_t*>(y), scale);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "quantize_e4m3 launch: %s", cudaGetErrorString(e));
  return FDB_OK;
}

}  // namespace fdb
