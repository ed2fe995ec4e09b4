// Per-slab amax scaling of bf16 rows to float8 e4m3 (the FP8 option; the reference has no FP8 code).
//
// A slab is a run of rows [slab_start[s], slab_start[s+1]) — one sequence, or the whole position table — and every
// (slab, head) gets its own scale = amax/448, so the stored value times the scale gives the input back.
// Three small kernels on the caller's stream, each with enough CTAs to fill the GPU whatever the number of slabs (one CTA
// per (slab, head), the first form of this file, left 8 x 16 = 128 CTAs to stream 100 MB):
//   amax_kernel      a CTA takes 64-row chunks of one slab, all heads; eight lanes share a (row, head), reduce with
//                    shuffles, then per head through shared memory into the scale array (bit pattern of a non-negative
//                    float, so an unsigned atomicMax orders it)
//   quantize_kernel  the same walk, x * 448/amax -> e4m3
//   scale_kernel     amax -> amax/448 in place
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "internal.h"

namespace fdb {
namespace {

constexpr int kQuantThreads = 256;
constexpr int kChunkRows = 64;

constexpr int kUnroll = 4;  // 16-byte loads in flight per thread

// Walks the (row, head) pairs of this CTA's 64-row chunks of its slab, eight lanes (16 bytes each) per pair and kUnroll
// pairs per thread at a time: first all loads, then `body(live, r, h, sub, v)` for each.
template <typename F>
__device__ __forceinline__ void walk_slab(const __nv_bfloat16* __restrict__ x, int total_rows, int64_t row_stride,
                                          int64_t head_stride, const int32_t* __restrict__ slab_start, int heads, F&& body) {
  const int slab = blockIdx.y;
  // slab bounds clamped to the rows that exist
  const int r0 = min(max(slab_start[slab], 0), total_rows);
  const int len = max(min(slab_start[slab + 1], total_rows) - r0, 0);
  const int sub = threadIdx.x & 7;
  constexpr int kStep = kQuantThreads >> 3;  // pairs per pass of the CTA
  for (int chunk = blockIdx.x; chunk * kChunkRows < len; chunk += gridDim.x) {
    const int rows = min(kChunkRows, len - chunk * kChunkRows);
    const int pairs = rows * heads;
    const int first_row = r0 + chunk * kChunkRows;
    for (int p0 = threadIdx.x >> 3; (p0 & ~3) < pairs; p0 += kStep * kUnroll) {  // a warp's four pairs stay together
      uint4 v[kUnroll];
      int r[kUnroll], h[kUnroll];
      bool live[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int p = p0 + u * kStep;
        live[u] = p < pairs;
        r[u] = first_row + (live[u] ? p / heads : 0);
        h[u] = live[u] ? p % heads : 0;
        v[u] = make_uint4(0, 0, 0, 0);
        if (live[u]) v[u] = *reinterpret_cast<const uint4*>(x + r[u] * row_stride + h[u] * head_stride + sub * 8);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) body(live[u], r[u], h[u], sub, v[u]);
    }
  }
}

__global__ void __launch_bounds__(kQuantThreads) amax_kernel(const __nv_bfloat16* __restrict__ x, int total_rows,
                                                             int64_t row_stride, int64_t head_stride,
                                                             const int32_t* __restrict__ slab_start, int heads,
                                                             unsigned int* __restrict__ amax_bits) {
  extern __shared__ unsigned int s_amax[];
  for (int h = threadIdx.x; h < heads; h += kQuantThreads) s_amax[h] = 0u;
  __syncthreads();
  walk_slab(x, total_rows, row_stride, head_stride, slab_start, heads, [&](bool live, int, int h, int sub, const uint4& v) {
    // whole warps get here; a dead pair holds zeros
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
    float a = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(b[k]);
      a = fmaxf(a, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 4));
    if (live && sub == 0 && a > 0.f) atomicMax(&s_amax[h], __float_as_uint(a));
  });
  __syncthreads();
  for (int h = threadIdx.x; h < heads; h += kQuantThreads)
    if (s_amax[h] != 0u) atomicMax(&amax_bits[(int64_t)blockIdx.y * heads + h], s_amax[h]);
}

__device__ __forceinline__ float scale_of(unsigned int amax_bits) { return fmaxf(__uint_as_float(amax_bits), 1e-12f) / 448.f; }

__global__ void __launch_bounds__(kQuantThreads) quantize_kernel(const __nv_bfloat16* __restrict__ x, int total_rows,
                                                                 int64_t row_stride, int64_t head_stride,
                                                                 const int32_t* __restrict__ slab_start, int heads,
                                                                 uint8_t* __restrict__ y,
                                                                 const unsigned int* __restrict__ amax_bits) {
  walk_slab(x, total_rows, row_stride, head_stride, slab_start, heads, [&](bool live, int r, int h, int sub, const uint4& v) {
    if (!live) return;
    const float inv = 1.f / scale_of(amax_bits[(int64_t)blockIdx.y * heads + h]);
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
    *reinterpret_cast<uint2*>(y + ((int64_t)r * heads + h) * 64 + sub * 8) = packed;
  });
}

__global__ void scale_kernel(float* __restrict__ scale, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) scale[i] = scale_of(__float_as_uint(scale[i]));
}

}  // namespace

int launch_quantize_e4m3(const void* x, int64_t rows, int64_t row_stride, int64_t head_stride, const int32_t* slab_start,
                         int32_t n_slabs, int32_t heads, int32_t head_dim, void* y, float* scale, void* stream) {
  if (head_dim != 64) return fail(FDB_ERR_UNSUPPORTED, "quantize_e4m3 is built for head_dim 64, got %d", head_dim);
  if (n_slabs <= 0 || heads <= 0) return FDB_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int n = n_slabs * heads;
  cudaError_t e = cudaMemsetAsync(scale, 0, sizeof(float) * n, s);
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "quantize_e4m3 memset: %s", cudaGetErrorString(e));
  // the slab lengths are on the device: a fixed number of CTAs per slab walks its 64-row chunks (about 1200 CTAs in all)
  int per_slab = (1184 + n_slabs - 1) / n_slabs;
  per_slab = per_slab < 1 ? 1 : (per_slab > 128 ? 128 : per_slab);
  const dim3 grid(per_slab, n_slabs);
  auto* xb = static_cast<const __nv_bfloat16*>(x);
  auto* bits = reinterpret_cast<unsigned int*>(scale);
  amax_kernel<<<grid, kQuantThreads, sizeof(unsigned int) * heads, s>>>(xb, (int)rows, row_stride, head_stride, slab_start, heads, bits);
  quantize_kernel<<<grid, kQuantThreads, 0, s>>>(xb, (int)rows, row_stride, head_stride, slab_start, heads, static_cast<uint8_t*>(y), bits);
  scale_kernel<<<(n + 255) / 256, 256, 0, s>>>(scale, n);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "quantize_e4m3 launch: %s", cudaGetErrorString(e));
  return FDB_OK;
}

}  // namespace fdb
