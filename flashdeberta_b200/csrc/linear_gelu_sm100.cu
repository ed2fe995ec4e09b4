// out = GELU(x . W^T + bias) for sm_100a: the intermediate block of an encoder layer in one kernel.
//
// The reference inherits the block from transformers (DebertaV2Intermediate: dense + erf GELU, reached through
// FlashDebertaV2Layer, src/flashdeberta/model.py:265-272): a cuBLAS GEMM with a bias epilogue, then an elementwise kernel
// that reads and rewrites the (rows, 4 * hidden) activation.  Here the activation never leaves the chip between the two:
// the GEMM accumulates in tensor memory and the epilogue warps apply bias and GELU on the way out.
//
// Persistent grid, one CTA per SM, tiles of 128 rows x 256 output features, K in steps of 64:
//   warp 0  lane 0: TMA, x tile (128 x 64) and W tile (256 x 64) into a ring of four 48 KB stages
//   warp 1  lane 0: tcgen05.mma 128 x 256 x 16, four per stage; allocates the 512 tensor-memory columns = two accumulators,
//           so the epilogue of one tile runs beside the main loop of the next
//   warps 2-9: epilogue, two warps per 32-lane quarter of tensor memory (128 columns each): + bias, rounded to bf16 as the
//           separate GEMM would leave it, GELU in fp32, bf16 out with 16-byte stores
// GELU(v) = v * Phi(v) with Phi from the complementary error function in the rational form of Abramowitz & Stegun 7.1.26
// (absolute error 1.5e-7, far below half a bf16 ulp of the result): one reciprocal, one exponential and nine FMAs per
// element, about half of what erff costs — with erff the epilogue would be longer than the main loop.
// Every wait is bounded; on a timeout the CTA raises FDB_DEV_TIMEOUT in the status word, frees its tensor memory and
// returns.  No TMA multicast.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "internal.h"
#include "sm100_ptx.cuh"
#include "tensor_map.cuh"

namespace fdb {
namespace {

using namespace ptx;

constexpr int kBM = 128, kBN = 256, kBK = 64, kStages = 4;
constexpr int kThreads = 320;
constexpr int kTmaWarp = 0, kMmaWarp = 1, kEpiWarp0 = 2, kEpiThreads = 256;
constexpr uint32_t kBytesA = kBM * kBK * 2, kBytesW = kBN * kBK * 2, kStageBytes = kBytesA + kBytesW;  // 16 + 32 KB
constexpr uint32_t kSmemBars = kStages * kStageBytes;
enum : uint32_t { kBarFull = 0, kBarEmpty = kStages, kBarAccFull = 2 * kStages, kBarAccEmpty = 2 * kStages + 2, kNumBars = 2 * kStages + 4 };
constexpr uint32_t kSmemBytes = kSmemBars + 8 * kNumBars + 16 + 1024;  // + tensor-memory slot, abort flag, alignment slack
constexpr uint32_t kTmemCols = 512;

struct LinearArgs {
  CUtensorMap tm_x, tm_w;
  const __nv_bfloat16* bias;  // may be NULL
  __nv_bfloat16* out;
  int32_t* status;
  int64_t rows;
  int n, k;
  int tiles_m, tiles_n;
};

// v * Phi(v) with Phi(v) = 1/2 erfc(-v / sqrt 2):  v * Phi(v) = v / 2 + |v| * (1/2 - q),  q = 1/2 erfc(|v| / sqrt 2)
__device__ __forceinline__ float gelu_erf(float v) {
  const float z = fabsf(v) * 0.70710678118654752f;
  float t;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, z, 1.f)));
  const float e = ex2(z * z * -1.4426950408889634f);
  float p = fmaf(0.5f * 1.061405429f, t, 0.5f * -1.453152027f);
  p = fmaf(p, t, 0.5f * 1.421413741f);
  p = fmaf(p, t, 0.5f * -0.284496736f);
  p = fmaf(p, t, 0.5f * 0.254829592f);
  const float h = fmaf(-(p * t), e, 0.5f);
  return fmaf(fabsf(v), h, 0.5f * v);
}

// 32 bytes per thread in one store (whole sectors)
__device__ __forceinline__ void st_global_32B(void* p, const uint32_t (&o)[16], int at) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(o[at]), "r"(o[at + 1]), "r"(o[at + 2]),
               "r"(o[at + 3]), "r"(o[at + 4]), "r"(o[at + 5]), "r"(o[at + 6]), "r"(o[at + 7])
               : "memory");
}

__global__ void __launch_bounds__(kThreads, 1) linear_gelu_kernel(const __grid_constant__ LinearArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem - smem_u32(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  auto bar = [&](uint32_t i) -> uint32_t { return smem + kSmemBars + 8u * i; };
  const uint32_t tmem_slot = smem + kSmemBars + 8u * kNumBars;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + kSmemBars + 8u * kNumBars + 8u);

  if (tid == 0) {
    *abort_flag = 0u;
    for (uint32_t i = 0; i < kNumBars; ++i) mbar_init(bar(i), (i >= kBarAccEmpty) ? uint32_t(kEpiThreads) : 1u);
    fence_barrier_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem_gen + kSmemBars + 8u * kNumBars);

  const int num_tiles = args.tiles_m * args.tiles_n;
  const int kblocks = args.k / kBK;
  bool ok = true;
  auto wait = [&](uint32_t b, uint32_t parity) {
    if (ok && !mbar_wait_abortable(b, parity, abort_flag)) { ok = false; *abort_flag = 1u; }
  };

  if (warp == kTmaWarp) {
    if (lane == 0) {
      tma_prefetch_desc(&args.tm_x);
      tma_prefetch_desc(&args.tm_w);
      uint32_t it = 0;
#pragma unroll 1
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile / args.tiles_n) * kBM, n0 = (tile % args.tiles_n) * kBN;
#pragma unroll 1
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t st = it % kStages, use = it / kStages;
          if (use > 0) wait(bar(kBarEmpty + st), (use - 1u) & 1u);
          if (!ok) break;
          mbar_expect_tx(bar(kBarFull + st), kStageBytes);
          tma_load_3d(smem + st * kStageBytes, &args.tm_x, bar(kBarFull + st), 0, kb, m0);
          tma_load_3d(smem + st * kStageBytes + kBytesA, &args.tm_w, bar(kBarFull + st), 0, kb, n0);
        }
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      const uint32_t idesc = instr_desc(kBM, kBN, 1, 0, 0);
      uint32_t it = 0, local = 0;
#pragma unroll 1
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const uint32_t acc = local & 1u, acc_use = local >> 1;
        if (acc_use > 0) wait(bar(kBarAccEmpty + acc), (acc_use - 1u) & 1u);  // the epilogue has read this accumulator
        tc_fence_after();
#pragma unroll 1
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t st = it % kStages, use = it / kStages;
          wait(bar(kBarFull + st), use & 1u);
          if (!ok) break;
          tc_fence_after();
          const uint64_t da = smem_desc_sw128(smem + st * kStageBytes, 1024, 16);
          const uint64_t dw = smem_desc_sw128(smem + st * kStageBytes + kBytesA, 1024, 16);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            mma_bf16(tmem_base + acc * uint32_t(kBN), da + uint64_t((ks * 32) >> 4), dw + uint64_t((ks * 32) >> 4), idesc,
                     (kb > 0 || ks > 0) ? 1u : 0u);
          mma_commit(bar(kBarEmpty + st));
        }
        if (ok) mma_commit(bar(kBarAccFull + acc));
      }
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;            // the 32 tensor-memory lanes this warp may read
    const int half = (warp - kEpiWarp0) >> 2;  // which 128 of the tile's 256 columns
    const uint32_t tmem_lane = tmem_base + (uint32_t(quarter * 32) << 16);
    uint32_t local = 0;
#pragma unroll 1
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int m0 = (tile / args.tiles_n) * kBM, n0 = (tile % args.tiles_n) * kBN + half * 128;
      const uint32_t acc = local & 1u;
      wait(bar(kBarAccFull + acc), (local >> 1) & 1u);
      tc_fence_after();
      const int64_t row = (int64_t)m0 + quarter * 32 + lane;
      const bool live = row < args.rows;
      __nv_bfloat16* orow = args.out + row * args.n + n0;
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t a[32];
        if (ok) {  // whole warps execute the load, whatever their rows
          tmem_ld32(tmem_lane + acc * uint32_t(kBN) + uint32_t(half * 128 + ch * 32), a);
          tmem_wait_ld();
        }
        if (ch == 3) {  // the accumulator is in registers: the next tile but one may overwrite it
          tc_fence_before();
          mbar_arrive(bar(kBarAccEmpty + acc));
        }
        uint32_t o[16];
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
          uint4 bw = make_uint4(0, 0, 0, 0);
          if (args.bias != nullptr) bw = __ldg(reinterpret_cast<const uint4*>(args.bias + n0 + ch * 32 + c));
          const uint32_t b4[4] = {bw.x, bw.y, bw.z, bw.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            // the sum as the separate GEMM would leave it: rounded to bf16
            const uint32_t r = pack_bf16x2(__uint_as_float(a[c + 2 * e]) + __uint_as_float(b4[e] << 16),
                                           __uint_as_float(a[c + 2 * e + 1]) + __uint_as_float(b4[e] & 0xffff0000u));
            o[(c >> 1) + e] = pack_bf16x2(gelu_erf(__uint_as_float(r << 16)), gelu_erf(__uint_as_float(r & 0xffff0000u)));
          }
        }
        if (live && ok) {
          st_global_32B(orow + ch * 32, o, 0);
          st_global_32B(orow + ch * 32 + 16, o, 8);
        }
      }
    }
  }

  // ---- teardown ----
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (tid == 0 && args.status != nullptr) atomicOr(reinterpret_cast<unsigned int*>(args.status), FDB_DEV_TIMEOUT);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // copies and MMAs in flight get a bounded time to land
    __syncthreads();
  }
  if (warp == kMmaWarp) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace
}  // namespace fdb

using namespace fdb;

extern "C" FDB_API int fdb_linear_gelu(const void* x, const void* weight, const void* bias, void* out, int64_t rows,
                                       int32_t in_features, int32_t out_features, int32_t* status, void* stream) {
  clear_error();
  if (x == nullptr || weight == nullptr || out == nullptr)
    return fail(FDB_ERR_INVALID_ARGUMENT, "x, weight and out must not be NULL");
  if (rows < 0 || rows > (int64_t(1) << 31) - kBM) return fail(FDB_ERR_LIMIT, "rows = %lld", (long long)rows);
  if (in_features <= 0 || in_features % kBK != 0)
    return fail(FDB_ERR_UNSUPPORTED, "in_features = %d: the kernel handles multiples of %d", in_features, kBK);
  if (out_features <= 0 || out_features % kBN != 0)
    return fail(FDB_ERR_UNSUPPORTED, "out_features = %d: the kernel handles multiples of %d", out_features, kBN);
  const uintptr_t all = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) |
                        reinterpret_cast<uintptr_t>(bias) | reinterpret_cast<uintptr_t>(out);
  if ((all & 15u) != 0) return fail(FDB_ERR_ALIGNMENT, "pointers must be 16-byte aligned");
  if (rows == 0) return FDB_OK;

  LinearArgs a;
  int rc = make_map_rows(&a.tm_x, x, rows, in_features / kBK, in_features, kBK, kBM, false, "x");
  if (rc != FDB_OK) return rc;
  rc = make_map_rows(&a.tm_w, weight, out_features, in_features / kBK, in_features, kBK, kBN, false, "weight");
  if (rc != FDB_OK) return rc;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.status = status;
  a.rows = rows;
  a.n = out_features;
  a.k = in_features;
  a.tiles_m = (int)((rows + kBM - 1) / kBM);
  a.tiles_n = out_features / kBN;

  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_gelu_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "linear_gelu set-up: %s", cudaGetErrorString(e));
  const int64_t tiles = (int64_t)a.tiles_m * a.tiles_n;
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  linear_gelu_kernel<<<grid, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "linear_gelu launch: %s", cudaGetErrorString(e));
  return FDB_OK;
}
