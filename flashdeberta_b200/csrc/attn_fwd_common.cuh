// Definitions shared by the fused attention kernels (attn_fwd_sm100.cu: all tile kinds or band tiles only;
// attn_fwd_far1_sm100.cu: plain and saturated tiles, half an SM per CTA).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "internal.h"
#include "sm100_ptx.cuh"

namespace fdb {
namespace fwd {

using namespace ptx;

struct alignas(64) FwdArgs {
  CUtensorMap tm_q, tm_k, tm_v, tm_xk, tm_xq;
  CUtensorMap tm_xq_sat;      // expanded pos_query again, 8-row boxes: the saturated rows as an MMA operand
  __nv_bfloat16* out;
  int64_t o_rs, o_hs;
  const int32_t* seq_info;    // [batch][2] first row, length
  const int32_t* tile_first;  // [batch+1]
  const int4* slot_info;      // [slots] (sequence, first query row of the tile within it, sequence's first row, length); sequence < 0: empty slot
  const void* xk;             // expanded pos_key   (heads, xrows, 64) bf16 or e4m3
  const void* xq;             // expanded pos_query
  const float *q_scale, *k_scale, *v_scale;  // e4m3 only: [seq * heads + head]
  const float *xk_scale, *xq_scale;          // e4m3 only: [head]
  float* lse;
  int32_t* status;
  int batch, heads, packed, max_seqlen;
  int sat_lo, sat_hi, d_first, xrows;
  float scale_log2;  // sm_scale * log2(e)
  // Split launch: the far kernel leaves, per (row, head), the unnormalised output accumulator (64 floats), the reference
  // maximum (log2 units) and the row sum of the plain and saturated key tiles; the band kernel starts from them.
  float* part_o;   // (rows, heads, 64)
  float* part_ml;  // (rows, heads, 2)
  int band_only;   // attn_fwd_kernel: 0 = every key tile, 1 = band tiles only (continuing from part_o / part_ml)
  int split_len;   // two-launch calls: sequences shorter than this stay whole in attn_fwd_kernel
  int slots;       // query-tile slots of the launch (work items = slots * heads)
#ifdef FDB_TRACE
  long long* trace;  // [role 0..3][tile 0..63][event 0..7] clock64 stamps of CTA (0, 0)
#endif
};

#ifdef FDB_TRACE
// Development builds only (-DFDB_TRACE): clock stamps of one CTA, read back through a buffer whose address comes from the
// environment.  Compiled out otherwise.
inline long long* trace_buffer_from_env() {
  const char* tp = std::getenv("FDB_TRACE_PTR");
  return tp ? reinterpret_cast<long long*>(std::strtoull(tp, nullptr, 0)) : nullptr;
}
#define FDB_STAMP(role, tile, ev) \
  do { if (blockIdx.x == 0 && blockIdx.y == 0 && args.trace != nullptr && (tile) < 64) \
         args.trace[((role) * 64 + (tile)) * 8 + (ev)] = clock64(); } while (0)
#else
#define FDB_STAMP(role, tile, ev) do {} while (0)
#endif

enum TileKind : int { kPlain = 0, kSatHi = 1, kSatLo = 2, kBand = 3 };

// What changes between the bf16 and the e4m3 build of the kernel: bytes per 64-element row (128 / 64, hence 128-byte or
// 64-byte swizzle and 1024- or 512-byte 8-row groups), elements per MMA along K (16 / 32) and the MMA kind.
template <bool F8> struct Geo {
  static constexpr uint32_t kRow = F8 ? 64u : 128u;          // bytes per row of 64 elements
  static constexpr uint32_t kTile = 128u * kRow;             // a 128-row tile
  static constexpr uint32_t kWin = 256u * kRow;              // a 256-row window
  static constexpr uint32_t kGroup = 8u * kRow;              // 8-row group (stride byte offset)
  static constexpr int kSteps = F8 ? 2 : 4;                  // MMAs along head_dim 64
  static constexpr int kPvSteps = F8 ? 4 : 8;                // MMAs along 128 keys
  static constexpr uint32_t kPColsPerStep = 8u;              // TMEM columns of P one P.V MMA reads (16 bf16 / 32 e4m3)
  static constexpr uint32_t kPCols = F8 ? 16u : 32u;         // TMEM columns of P per softmax group (64 keys)
  static constexpr int kFmt = F8 ? 0 : 1;                    // instruction-descriptor operand format: e4m3 / bf16
  __device__ static __forceinline__ uint64_t desc(uint32_t addr, uint32_t group_stride) {
    return F8 ? smem_desc_sw64(addr, group_stride, 16) : smem_desc_sw128(addr, group_stride, 16);
  }
  __device__ static __forceinline__ void mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    if constexpr (F8) mma_f8(d, a, b, idesc, acc); else mma_bf16(d, a, b, idesc, acc);
  }
  __device__ static __forceinline__ void mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    if constexpr (F8) mma_f8_ts(d, a, b, idesc, acc); else mma_bf16_ts(d, a, b, idesc, acc);
  }
};

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts_u16(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(static_cast<uint16_t>(v)) : "memory");
}
__device__ __forceinline__ void sts_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void sts_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

// dot product of one query row (128-byte-swizzled in shared memory) with one 64-element bf16 row in global memory
__device__ __forceinline__ float dot_q_row(uint32_t q_row_addr, int row, const __nv_bfloat16* __restrict__ g) {
  float acc = 0.f;
  const uint4* g4 = reinterpret_cast<const uint4*>(g);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint4 a = lds_v4(q_row_addr + (uint32_t((c ^ (row & 7))) << 4));
    const uint4 b = __ldg(g4 + c);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc = fmaf(bf16_bits_to_f32(aw[i] & 0xffffu), bf16_bits_to_f32(bw[i] & 0xffffu), acc);
      acc = fmaf(bf16_bits_to_f32(aw[i] >> 16), bf16_bits_to_f32(bw[i] >> 16), acc);
    }
  }
  return acc;
}

// the same for e4m3 rows (64 bytes, 64-byte swizzle: 16-byte chunk c of row r sits at chunk c ^ ((r >> 1) & 3))
__device__ __forceinline__ float dot_q_row_f8(uint32_t q_row_addr, int row, const uint8_t* __restrict__ g) {
  float acc = 0.f;
  const uint4* g4 = reinterpret_cast<const uint4*>(g);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint4 a = lds_v4(q_row_addr + (uint32_t(c ^ ((row >> 1) & 3)) << 4));
    const uint4 b = __ldg(g4 + c);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float fa[4], fb[4];
      unpack_e4m3x4(aw[i], fa);
      unpack_e4m3x4(bw[i], fb);
#pragma unroll
      for (int k = 0; k < 4; ++k) acc = fmaf(fa[k], fb[k], acc);
    }
  }
  return acc;
}


// The band tiles of a query tile are one contiguous run of key tiles [first, first + count): this returns it.
// d0(j) = m0 - 128 j - 127 decreases with j; band <=> sat_lo - 254 < d0 < sat_hi.
__device__ __forceinline__ void band_run(int m0, int num_kt, int sat_lo, int sat_hi, int& first, int& count) {
  // smallest j with d0(j) < sat_hi  <=>  128 j > m0 - 127 - sat_hi
  int lo = m0 - 127 - sat_hi;
  lo = lo < 0 ? 0 : lo / 128 + 1;
  // largest j with d0(j) + 254 > sat_lo  <=>  128 j < m0 + 127 - sat_lo
  int hi = m0 + 127 - sat_lo;  // positive
  hi = (hi - 1) / 128;
  if (hi > num_kt - 1) hi = num_kt - 1;
  first = lo;
  count = hi >= lo ? hi - lo + 1 : 0;
}

}  // namespace fwd
}  // namespace fdb
