// Fused attention forward for sm_100a — key tiles whose position terms are saturated (or absent), one team per CTA and two
// CTAs per SM.
//
// Such a tile is a plain flash-attention step (plus one accumulating MMA for the saturated p2c term), needs no
// position-product area in tensor memory, and so fits in half an SM: 256 tensor-memory columns (O 64 | P 64 | S 128),
// 84 KB of shared memory (Q, K and V in two stages), 32768 registers.  Two CTAs therefore share an SM, and what one of them
// cannot overlap inside itself — the round trips to tensor memory and the maximum search before its exponentials, its
// first loads and its output — runs beside the other one's exponentials.  One softmax thread per query row holds all 128
// keys of a tile, so there is no exchange between threads.
//
//   warps 0-3  softmax, thread r = row r          warp 4  lane 0: score MMAs  S = Q.K^T (+ R.K^T), allocates tensor memory
//   warp 5     lane 0: TMA (Q once, K/V 2 stages)  warp 6  lane 0: O += P.V
//
// When the call has position terms the band tiles are left to attn_fwd_kernel (band_only mode), which runs next on the same
// stream: this kernel then stores, per (row, head), the unnormalised accumulator, reference maximum and row sum instead
// of the final output.  Without position terms it handles every tile and writes the output itself.
// Replaces, together with attn_fwd_kernel, src/flashdeberta/ops/flash_attention.py:146-300 of the reference.
//
// bf16 only (the e4m3 build keeps all tiles in attn_fwd_kernel).  Every wait is bounded as in attn_fwd_sm100.cu; no TMA
// multicast.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "attn_fwd_common.cuh"
#include "internal.h"
#include "sm100_ptx.cuh"
#include "tensor_map.cuh"

namespace fdb {
namespace {

using namespace ptx;
using namespace fwd;

constexpr int kThreads = 256;
constexpr int kScoreWarp = 4, kTmaWarp = 5, kPvWarp = 6;
constexpr int kProducerRegs = 56, kSoftmaxRegs = 200;  // 2 CTAs per SM: 32768 = 56 * 128 + 200 * 128
constexpr int kStages = 2;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColO = 0, kColP = 64, kColS = 128;

constexpr uint32_t kSmemQ = 0;
constexpr uint32_t kSmemK = 16384;                      // 2 stages
constexpr uint32_t kSmemV = kSmemK + kStages * 16384;   // 2 stages
constexpr uint32_t kSmemSat = kSmemV + kStages * 16384; // 2 x (8 x 128 B)
constexpr uint32_t kSmemBars = kSmemSat + 2048;
constexpr uint32_t kSmemBytes = kSmemBars + 256 + 1024;
static_assert(2 * (kSmemBytes + 1024) <= 232448, "two CTAs per SM");

enum Bar : uint32_t {
  kBarQ = 0,
  kBarK = 1,        // 2: K stage landed
  kBarV = 3,        // 2: V stage landed
  kBarKFree = 5,    // 2: the score MMAs that read the stage finished
  kBarVFree = 7,    // 2: the P.V that read the stage finished
  kBarS = 9,        // S is in tensor memory
  kBarSFree = 10,   // (count 128) the softmax threads hold the scores in registers
  kBarP = 11,       // (count 128) P is in tensor memory
  kBarO = 12,       // P.V finished
  kNumBars = 13
};

__global__ void __launch_bounds__(kThreads, 2) attn_fwd_far1_kernel(const __grid_constant__ FwdArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem - smem_u32(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.y;

  const int4 slot = __ldg(args.slot_info + blockIdx.x);  // (sequence, first row of the tile in it, its first row, its length)
  if (slot.x < 0) return;                                  // slot past the last sequence
  const int m0 = slot.y, seq_row0 = slot.z, len = slot.w;
  const int row_limit = args.packed ? len : args.max_seqlen;
  const bool has_c2p = args.xk != nullptr, has_p2c = args.xq != nullptr;
  const bool has_pos = has_c2p || has_p2c;

  if (m0 >= len) {
    // dense padding tile: the band kernel writes its zeros when there are position terms, this one otherwise
    if (!has_pos && tid < kTileM && m0 + tid < row_limit) {
      uint4* o4 = reinterpret_cast<uint4*>(args.out + (int64_t)(seq_row0 + m0 + tid) * args.o_rs + (int64_t)head * args.o_hs);
#pragma unroll
      for (int c = 0; c < 8; ++c) o4[c] = make_uint4(0, 0, 0, 0);
      if (args.lse != nullptr) args.lse[(int64_t)(seq_row0 + m0 + tid) * args.heads + head] = 0.f;
    }
    return;
  }

  const int num_kt = (len + kTileN - 1) / kTileN;
  // this launch's key tiles: everything outside the band run [jb, jb + nb)
  int jb = 0, nb = 0;
  if (has_pos) {
    if (len < args.split_len) return;  // short sequence of a two-launch call: left whole to attn_fwd_kernel
    band_run(m0, num_kt, args.sat_lo, args.sat_hi, jb, nb);
  }
  const int n_far = num_kt - nb;
  if (n_far <= 0) return;  // nothing but band tiles: the band kernel starts from scratch
  auto tile_of = [&](int i) -> int { return i < jb ? i : i + nb; };
  auto kind_of = [&](int j) -> int { return !has_pos ? kPlain : (j < jb ? kSatHi : kSatLo); };

  auto bar = [&](uint32_t i) -> uint32_t { return smem + kSmemBars + 8u * i; };
  const uint32_t tmem_slot = smem + kSmemBars + 8u * kNumBars;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + kSmemBars + 8u * kNumBars + 8u);

  if (tid == 0) {
    *abort_flag = 0u;
    for (uint32_t i = 0; i < kNumBars; ++i) mbar_init(bar(i), (i == kBarSFree || i == kBarP) ? 128u : 1u);
    fence_barrier_init();
  }
  if (warp == kScoreWarp) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem_gen + kSmemBars + 8u * kNumBars);

  bool ok = true;

  if (warp >= kScoreWarp) {
    reg_dealloc<kProducerRegs>();
    auto wait = [&](uint32_t b, uint32_t parity) {
      if (ok && !mbar_wait_abortable(b, parity, abort_flag)) { ok = false; *abort_flag = 1u; }
    };
    if (warp == kTmaWarp) {
      if (lane == 0) {
        tma_prefetch_desc(&args.tm_q); tma_prefetch_desc(&args.tm_k); tma_prefetch_desc(&args.tm_v);
        mbar_expect_tx(bar(kBarQ), 16384u + (has_p2c ? 2048u : 0u));
        tma_load_3d(smem + kSmemQ, &args.tm_q, bar(kBarQ), 0, head, seq_row0 + m0);
        if (has_p2c) {
          // Saturated pos_query rows as MMA operands: the last (first) eight rows of an expanded table are all the row of
          // distances beyond sat_hi (sat_lo), so an 8-row box is the 8 identical rows in the swizzled layout.
          tma_load_3d(smem + kSmemSat, &args.tm_xq_sat, bar(kBarQ), 0, args.xrows - 8, head);
          tma_load_3d(smem + kSmemSat + 1024, &args.tm_xq_sat, bar(kBarQ), 0, 0, head);
        }
#pragma unroll 1
        for (int i = 0; i < n_far; ++i) {
          const int st = i & 1;
          const uint32_t use = uint32_t(i >> 1);
          const int row = seq_row0 + tile_of(i) * kTileN;
          if (use > 0) wait(bar(kBarKFree + st), (use - 1u) & 1u);
          if (!ok) break;
          mbar_expect_tx(bar(kBarK + st), 16384);
          tma_load_3d(smem + kSmemK + st * 16384, &args.tm_k, bar(kBarK + st), 0, head, row);
          if (use > 0) wait(bar(kBarVFree + st), (use - 1u) & 1u);
          if (!ok) break;
          mbar_expect_tx(bar(kBarV + st), 16384);
          tma_load_3d(smem + kSmemV + st * 16384, &args.tm_v, bar(kBarV + st), 0, head, row);
        }
      }
      __syncwarp();
    } else if (warp == kScoreWarp) {
      if (lane == 0) {
        const uint32_t idesc_s = instr_desc(128, 128, 1, 0, 0);
        const uint64_t dq = smem_desc_sw128(smem + kSmemQ, 1024, 16);
        const uint64_t dk0 = smem_desc_sw128(smem + kSmemK, 1024, 16);
        const uint64_t dsat = smem_desc_sw128(smem + kSmemSat, 0, 16);  // group stride 0: 8 identical rows serve all 128
        wait(bar(kBarQ), 0);
#pragma unroll 1
        for (int i = 0; i < n_far; ++i) {
          const int st = i & 1;
          const int kind = kind_of(tile_of(i));
          const uint64_t dk = dk0 + uint64_t(st) * (16384u >> 4);
          if (i > 0) wait(bar(kBarSFree), uint32_t(i - 1) & 1u);  // the softmax threads have pulled the previous scores
          wait(bar(kBarK + st), uint32_t(i >> 1) & 1u);
          tc_fence_after();
          if (ok) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              mma_bf16(tmem_base + kColS, dq + uint64_t((ks * 32) >> 4), dk + uint64_t((ks * 32) >> 4), idesc_s, ks > 0);
            if (has_p2c && kind != kPlain) {
              const uint64_t ds = dsat + uint64_t(kind == kSatHi ? 0u : (1024u >> 4));
#pragma unroll
              for (int ks = 0; ks < 4; ++ks)
                mma_bf16(tmem_base + kColS, ds + uint64_t((ks * 32) >> 4), dk + uint64_t((ks * 32) >> 4), idesc_s, 1);
            }
          }
          mma_commit(bar(kBarS));
          mma_commit(bar(kBarKFree + st));
        }
      }
      __syncwarp();
    } else if (warp == kPvWarp) {
      if (lane == 0) {
        const uint32_t idesc_pv = instr_desc(128, 64, 1, 0, 1);
        const uint64_t dv0 = smem_desc_sw128(smem + kSmemV, 1024, 16);
#pragma unroll 1
        for (int i = 0; i < n_far; ++i) {
          const int st = i & 1;
          const uint64_t dv = dv0 + uint64_t(st) * (16384u >> 4);
          wait(bar(kBarV + st), uint32_t(i >> 1) & 1u);
          wait(bar(kBarP), uint32_t(i) & 1u);
          tc_fence_after();
          if (ok) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              mma_bf16_ts(tmem_base + kColO, tmem_base + kColP + 8 * ks, dv + uint64_t((ks * 2048) >> 4), idesc_pv,
                          (i > 0 || ks > 0) ? 1u : 0u);
          }
          mma_commit(bar(kBarO));
          mma_commit(bar(kBarVFree + st));
        }
      }
      __syncwarp();
    }
  } else {
    // =================================================== softmax ========================================================
    reg_alloc<kSoftmaxRegs>();
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t tmem_lane = tmem_base + (uint32_t(quad * 32) << 16);
    const int my_row = m0 + r;
    auto wait = [&](uint32_t b, uint32_t parity) {
      const bool mine = ok && mbar_wait_abortable(b, parity, abort_flag);
      const bool all = __all_sync(0xffffffffu, mine);
      if (ok && !all) *abort_flag = 1u;
      ok = all;
    };

    wait(bar(kBarQ), 0);
    float rc_lo = 0.f, rc_hi = 0.f;
    if (has_c2p && ok) {
      const __nv_bfloat16* xk_h = static_cast<const __nv_bfloat16*>(args.xk) + (int64_t)head * args.xrows * kHeadDim;
      const uint32_t q_row = smem + kSmemQ + uint32_t(r) * 128u;
      rc_lo = dot_q_row(q_row, r, xk_h);
      rc_hi = dot_q_row(q_row, r, xk_h + (int64_t)(args.xrows - 1) * kHeadDim);
    }

    float m_used = 0.f, l_run = 0.f;
#pragma unroll 1
    for (int i = 0; i < n_far; ++i) {
      const uint32_t u = uint32_t(i);
      const int j = tile_of(i);
      const int n0 = j * kTileN;
      const int kind = kind_of(j);

      wait(bar(kBarS), u & 1u);
      tc_fence_after();
      if (lane == 0 && quad == 0) FDB_STAMP(0, i, 0);
      if (n0 + kTileN > len && ok) {
        // ragged last tile of the sequence: overwrite the scores of keys past its end in tensor memory, 32 columns at a
        // time, so the code below is the same for every tile (a select on the 128 register-resident scores under a
        // data-dependent branch made the compiler keep two copies of them)
        const int valid = len - n0;
#pragma unroll 1
        for (int q = valid >> 5; q < 4; ++q) {
          uint32_t a[32];
          tmem_ld32(tmem_lane + kColS + 32 * q, a);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) a[c] = 32 * q + c < valid ? a[c] : 0xff800000u;
          tmem_st32(tmem_lane + kColS + 32 * q, a);
        }
        tmem_wait_st();
      }
      // pull the 128 scores of this row in four chunks, all on their way at once
      uint32_t a0[32], a1[32], a2[32], a3[32];
      if (ok) {
        tmem_ld32(tmem_lane + kColS, a0);
        tmem_ld32(tmem_lane + kColS + 32, a1);
        tmem_ld32(tmem_lane + kColS + 64, a2);
        tmem_ld32(tmem_lane + kColS + 96, a3);
        tmem_wait_ld();
      }
      tc_fence_before();
      mbar_arrive(bar(kBarSFree));  // the scores are in registers: the next tile's may be computed
      float mx[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) mx[q] = max3(__uint_as_float(a0[q]), __uint_as_float(a0[4 + q]), __uint_as_float(a1[q]));
#pragma unroll
      for (int c = 8; c < 32; c += 8)
#pragma unroll
        for (int q = 0; q < 4; ++q) mx[q] = max3(mx[q], __uint_as_float(a0[c + q]), __uint_as_float(a0[c + 4 + q]));
#pragma unroll
      for (int c = 4; c < 28; c += 8)
#pragma unroll
        for (int q = 0; q < 4; ++q) mx[q] = max3(mx[q], __uint_as_float(a1[c + q]), __uint_as_float(a1[c + 4 + q]));
#pragma unroll
      for (int q = 0; q < 4; ++q) mx[q] = fmaxf(mx[q], __uint_as_float(a1[28 + q]));
      if (lane == 0 && quad == 0) FDB_STAMP(0, i, 1);
#pragma unroll
      for (int c = 0; c < 32; c += 8)
#pragma unroll
        for (int q = 0; q < 4; ++q) mx[q] = max3(mx[q], __uint_as_float(a2[c + q]), __uint_as_float(a2[c + 4 + q]));
#pragma unroll
      for (int c = 0; c < 32; c += 8)
#pragma unroll
        for (int q = 0; q < 4; ++q) mx[q] = max3(mx[q], __uint_as_float(a3[c + q]), __uint_as_float(a3[c + 4 + q]));

      const float row_const = kind == kSatHi ? rc_hi : (kind == kSatLo ? rc_lo : 0.f);
      const float t_max = (max3(mx[0], mx[1], fmaxf(mx[2], mx[3])) + row_const) * args.scale_log2;
      if (lane == 0 && quad == 0) FDB_STAMP(0, i, 2);
      if (u == 0) {
        m_used = t_max;
      } else {
        const bool need = t_max > m_used + 8.f;
        if (__any_sync(0xffffffffu, need)) {
          wait(bar(kBarO), (u - 1u) & 1u);  // O is only touched once the previous P.V has finished
          tc_fence_after();
          const float m_new = fmaxf(m_used, t_max);
          const float alpha = ex2(m_used - m_new);
          l_run *= alpha;
          m_used = m_new;
          if (ok) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t o[32];
              tmem_ld32(tmem_lane + kColO + 32 * h, o);
              tmem_wait_ld();
#pragma unroll
              for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
              tmem_st32(tmem_lane + kColO + 32 * h, o);
            }
          }
        }
      }
      if (lane == 0 && quad == 0) FDB_STAMP(0, i, 3);
      // p = 2^(s * scale + off), two keys per instruction where the hardware has a two-wide form; the first 64 keys go to
      // tensor memory while the other 64 are computed
      const float off = row_const * args.scale_log2 - m_used;
      const uint64_t scale2 = pack_f32x2(args.scale_log2, args.scale_log2), off2 = pack_f32x2(off, off);
      uint64_t l2[2] = {0ull, 0ull};
      auto half = [&](const uint32_t (&x)[32], const uint32_t (&y)[32], uint32_t col, bool first) {
        uint32_t p[32];
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float e0, e1, f0, f1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(x[c]), __uint_as_float(x[c + 1])), scale2, off2), e0, e1);
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(y[c]), __uint_as_float(y[c + 1])), scale2, off2), f0, f1);
          e0 = ex2(e0); e1 = ex2(e1); f0 = ex2(f0); f1 = ex2(f1);
          l2[0] = add_f32x2(l2[0], pack_f32x2(e0, e1));
          l2[1] = add_f32x2(l2[1], pack_f32x2(f0, f1));
          p[c >> 1] = pack_bf16x2(e0, e1);
          p[16 + (c >> 1)] = pack_bf16x2(f0, f1);
        }
        // P is free once the previous P.V has read it.  That P.V was issued when the previous tile's exponentials ended, so
        // it is waited for here, behind the first 64 exponentials of this tile, and not in front of the tile
        if (first && u > 0) { wait(bar(kBarO), (u - 1u) & 1u); tc_fence_after(); }
        if (ok) tmem_st32(tmem_lane + col, p);
      };
      half(a0, a1, kColP, true);
      half(a2, a3, kColP + 32, false);
      {
        float s0, s1, s2, s3;
        unpack_f32x2(l2[0], s0, s1);
        unpack_f32x2(l2[1], s2, s3);
        l_run += (s0 + s1) + (s2 + s3);
      }
      if (lane == 0 && quad == 0) FDB_STAMP(0, i, 4);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(kBarP));
      if (lane == 0 && quad == 0) FDB_STAMP(0, i, 5);
    }


    // ---- output: final (no position terms) or the partial result the band launch starts from ----
    wait(bar(kBarO), uint32_t(n_far - 1) & 1u);
    tc_fence_after();
    if (ok) {
      const bool valid = my_row < len;
      const int64_t rh = (int64_t)(seq_row0 + my_row) * args.heads + head;
      const float inv = valid ? 1.f / l_run : 0.f;
      const bool store = has_pos ? valid : (valid || my_row < row_limit);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t o[32];
        tmem_ld32(tmem_lane + kColO + 32 * h, o);  // whole warps execute this, whatever their rows
        tmem_wait_ld();
        if (!store) continue;
        if (has_pos) {
          float4* po = reinterpret_cast<float4*>(args.part_o + rh * 64 + 32 * h);
#pragma unroll
          for (int q = 0; q < 8; ++q)
            po[q] = make_float4(__uint_as_float(o[4 * q]), __uint_as_float(o[4 * q + 1]), __uint_as_float(o[4 * q + 2]),
                                __uint_as_float(o[4 * q + 3]));
        } else {
          uint4* o4 = reinterpret_cast<uint4*>(args.out + (int64_t)(seq_row0 + my_row) * args.o_rs +
                                               (int64_t)head * args.o_hs + 32 * h);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4)
            o4[q4] = !valid ? make_uint4(0, 0, 0, 0) : make_uint4(pack_bf16x2(__uint_as_float(o[q4 * 8 + 0]) * inv, __uint_as_float(o[q4 * 8 + 1]) * inv),
                                pack_bf16x2(__uint_as_float(o[q4 * 8 + 2]) * inv, __uint_as_float(o[q4 * 8 + 3]) * inv),
                                pack_bf16x2(__uint_as_float(o[q4 * 8 + 4]) * inv, __uint_as_float(o[q4 * 8 + 5]) * inv),
                                pack_bf16x2(__uint_as_float(o[q4 * 8 + 6]) * inv, __uint_as_float(o[q4 * 8 + 7]) * inv));
        }
      }
      if (store) {
        if (has_pos) *reinterpret_cast<float2*>(args.part_ml + rh * 2) = make_float2(m_used, l_run);
        else if (args.lse != nullptr) args.lse[rh] = valid ? (m_used + log2f(l_run)) * 0.6931471805599453f : 0.f;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (tid == 0 && args.status != nullptr) atomicOr(reinterpret_cast<unsigned int*>(args.status), FDB_DEV_TIMEOUT);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == kScoreWarp) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace

int launch_attn_fwd_far1(const void* fwd_args, int64_t slots, int heads, void* stream) {
  const FwdArgs& a = *static_cast<const FwdArgs*>(fwd_args);
  cudaError_t e = cudaFuncSetAttribute(attn_fwd_far1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  attn_fwd_far1_kernel<<<dim3((unsigned)slots, heads), kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "attn_fwd_far1 launch: %s", cudaGetErrorString(e));
  return FDB_OK;
}

}  // namespace fdb
