// Fused DeBERTa disentangled-attention forward for sm_100a — the serial bring-up version.
//
// Kept as a second, independently written tensor-core implementation: FDB_ATTN_KERNEL=serial in the environment makes
// fdb_attn_fwd launch it instead of the warp-specialised kernel (attn_fwd_sm100.cu), which is how the two are compared on
// the device.  Same contract, same results up to rounding; about four times slower.
//
// One CTA = one 128-row query tile of one (sequence, head).  It loops over 128-key tiles; per tile:
//   S   = Q.K^T                      tcgen05.mma, operands staged by TMA (128-byte swizzle), accumulator in TMEM
//   S  += c2p + p2c                  (below)
//   P   = exp2(S*scale*log2e - m)    one thread per row, S read from TMEM with tcgen05.ld
//   O  += P.V                        tcgen05.mma, P written to shared memory in the operand layout, O stays in TMEM and is
//                                    only rescaled when the running maximum moved by more than 2^8
// which replaces the reference's Triton forward kernels (src/flashdeberta/ops/flash_attention.py:146-300 and
// src/flashdeberta/ops/flash_attention_varlen.py:85-225) and the two bias GEMMs in front of them
// (src/flashdeberta/model.py:189-192, :210-214).
//
// Position terms.  The tables arrive already expanded through the bucket function (see attn_prepare.cu), so the row a
// score element (m, n) needs is (m - n) - d_first and a tile pair needs 255 consecutive rows.  Three kinds of tile pair:
//   * every distance at or beyond the upper saturation point: c2p is one dot product per query row (added to the
//     row's exponent offset, no per-element work) and p2c is one dot product per key, obtained on the tensor core by
//     accumulating  R.K^T  into S, where every row of R is the saturated pos_query row;
//   * every distance at or below the lower saturation point: the same with the other end of the tables;
//   * otherwise ("band"): X_k.Q^T (256x128) and K.X_q^T (128x256) are computed on the tensor core from the staged
//     windows X_k, X_q, drained to shared memory as bf16, and each thread picks  c2p[m][m-n]  and  p2c[n][m-n]  with
//     plain indexed shared loads whose offsets are compile-time constants relative to a per-thread base.
// No (rows x 2*span) bias tensor is ever written to global memory.
//
// Every mbarrier wait is bounded; when one gives up the CTA stops issuing work, sets FDB_DEV_TIMEOUT in the status
// word, releases its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "internal.h"
#include "sm100_ptx.cuh"
#include "tensor_map.cuh"

namespace fdb {
namespace {

using namespace ptx;

constexpr int kThreads = 128;
constexpr uint32_t kTmemCols = 512;
// TMEM columns
constexpr uint32_t kColO = 0;       // 64 columns: output accumulator
constexpr uint32_t kColS = 64;      // 128 columns: scores
constexpr uint32_t kColBias = 192;  // 256 columns: position products of a band tile

// shared memory map (bytes from a 1024-aligned base)
constexpr uint32_t kSmemQ = 0;                       // 128 x 128 B
constexpr uint32_t kSmemK = 16384;                   // 128 x 128 B
constexpr uint32_t kSmemV = 32768;                   // 128 x 128 B
constexpr uint32_t kSmemP = 49152;                   // 2 x (128 x 128 B): keys 0-63, keys 64-127
constexpr uint32_t kSmemWinK = 81920;                // 256 x 128 B window of expanded pos_key
constexpr uint32_t kSmemWinQ = kSmemWinK + 32768;    // 256 x 128 B window of expanded pos_query
constexpr uint32_t kStageCPitch = 272;               // c2p stage: [256 positions][128 query rows] bf16, padded rows
constexpr uint32_t kSmemStageC = kSmemWinK;          // overlays both windows (dead once the position MMAs finished)
constexpr uint32_t kStagePPitch = 528;               // p2c stage: [128 keys][256 positions] bf16, padded rows
constexpr uint32_t kSmemStageP = kSmemStageC + 256 * kStageCPitch;  // 151552
constexpr uint32_t kSmemSat = kSmemWinK;             // 128 x 128 B tile whose rows all equal one pos_query row
constexpr uint32_t kSmemBars = kSmemStageP + 128 * kStagePPitch;    // 219136
constexpr uint32_t kSmemBytes = kSmemBars + 128 + 1024;             // + alignment slack
static_assert(kSmemStageP == 151552 && kSmemBars == 219136, "shared memory map");
static_assert(kSmemBytes <= 232448, "exceeds 227 KB");

struct alignas(64) FwdArgs {
  CUtensorMap tm_q, tm_k, tm_v, tm_xk, tm_xq;
  __nv_bfloat16* out;
  int64_t o_rs, o_hs;
  const int32_t* seq_info;    // [batch][2] first row, length
  const int32_t* tile_first;  // [batch+1]
  const __nv_bfloat16* xk;    // expanded pos_key   (heads, xrows, 64)
  const __nv_bfloat16* xq;    // expanded pos_query
  float* lse;
  int32_t* status;
  int batch, heads, packed, max_seqlen;
  int sat_lo, sat_hi, d_first, xrows;
  float scale_log2;  // sm_scale * log2(e)
};

enum TileKind : int { kPlain = 0, kSatHi = 1, kSatLo = 2, kBand = 3 };

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t v) { return __uint_as_float(v << 16); }

__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// dot product of this thread's query row (swizzled in shared memory) with one 64-element bf16 row in global memory
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

__global__ void __launch_bounds__(kThreads, 1) attn_fwd_serial_kernel(const __grid_constant__ FwdArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem - smem_u32(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5;
  const int head = blockIdx.y;

  // ---- which tile ------------------------------------------------------------------------------------------------
  const int tile = blockIdx.x;
  if (tile >= __ldg(args.tile_first + args.batch)) return;
  int lo = 0, hi = args.batch;
  while (hi - lo > 1) {  // largest b with tile_first[b] <= tile
    const int mid = (lo + hi) >> 1;
    if (__ldg(args.tile_first + mid) <= tile) lo = mid; else hi = mid;
  }
  const int seq = lo;
  const int m0 = (tile - __ldg(args.tile_first + seq)) * kTileM;
  const int seq_row0 = __ldg(args.seq_info + 2 * seq);
  const int len = __ldg(args.seq_info + 2 * seq + 1);
  // rows of this tile that may be written: packed -> the sequence's own rows; dense -> the padded row range
  const int row_limit = args.packed ? len : args.max_seqlen;
  const int my_row = m0 + tid;  // position inside the sequence
  __nv_bfloat16* out_ptr = args.out + (int64_t)(seq_row0 + my_row) * args.o_rs + (int64_t)head * args.o_hs;

  if (m0 >= len) {  // dense padding tile: zeros, nothing else (src/flashdeberta/padding.py:30-44)
    if (my_row < row_limit) {
      uint4* o4 = reinterpret_cast<uint4*>(out_ptr);
#pragma unroll
      for (int c = 0; c < 8; ++c) o4[c] = make_uint4(0, 0, 0, 0);
      if (args.lse != nullptr) args.lse[(int64_t)(seq_row0 + my_row) * args.heads + head] = 0.f;
    }
    return;
  }

  const bool has_c2p = args.xk != nullptr, has_p2c = args.xq != nullptr;
  const bool has_pos = has_c2p || has_p2c;
  const int num_kt = (len + kTileN - 1) / kTileN;

  // ---- barriers, TMEM ----------------------------------------------------------------------------------------------
  const uint32_t bar_q = smem + kSmemBars + 0, bar_k = smem + kSmemBars + 8, bar_v = smem + kSmemBars + 16,
                 bar_win = smem + kSmemBars + 24, bar_s = smem + kSmemBars + 32, bar_pv = smem + kSmemBars + 40;
  const uint32_t tmem_slot = smem + kSmemBars + 64;
  if (tid == 0) {
    *reinterpret_cast<volatile uint32_t*>(smem_gen + kSmemBars + 72) = 0u;
    mbar_init(bar_q, 1); mbar_init(bar_k, 1); mbar_init(bar_v, 1);
    mbar_init(bar_win, 1); mbar_init(bar_s, 1); mbar_init(bar_pv, 1);
    fence_barrier_init();
    tma_prefetch_desc(&args.tm_q); tma_prefetch_desc(&args.tm_k); tma_prefetch_desc(&args.tm_v);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem_gen + kSmemBars + 64);
  const uint32_t tmem_lane = tmem_base + (uint32_t(warp * 32) << 16);  // this warp's 32 lanes

  // `ok` turns false once a bounded wait gave up.  It is kept warp-uniform (the collective tcgen05 loads and stores
  // below must be executed by whole warps) and becomes CTA-uniform at every sync_check().
  bool ok = true;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + kSmemBars + 72);
  auto wait_all = [&](uint32_t bar, uint32_t parity) { ok = __all_sync(0xffffffffu, ok && mbar_wait(bar, parity)); };
  auto wait_one = [&](uint32_t bar, uint32_t parity) -> bool {  // used by thread 0 alone; reported at the next sync_check()
    const bool r = mbar_wait(bar, parity);
    if (!r) *abort_flag = 1u;
    return r;
  };
  auto sync_check = [&]() {
    __syncthreads();
    ok = ok && (*abort_flag == 0u);
  };
  uint32_t ph_k = 0, ph_v = 0, ph_win = 0, ph_s = 0, ph_pv = 0;

  // ---- first loads ---------------------------------------------------------------------------------------------------
  if (tid == 0) {
    mbar_expect_tx(bar_q, 16384);
    tma_load_3d(smem + kSmemQ, &args.tm_q, bar_q, 0, head, seq_row0 + m0);
    mbar_expect_tx(bar_k, 16384);
    tma_load_3d(smem + kSmemK, &args.tm_k, bar_k, 0, head, seq_row0);
    mbar_expect_tx(bar_v, 16384);
    tma_load_3d(smem + kSmemV, &args.tm_v, bar_v, 0, head, seq_row0);
  }
  wait_all(bar_q, 0);  // every thread reads its Q row below

  // Saturated c2p terms of this thread's row: Q[m].X_k[first row] and Q[m].X_k[last row].
  float rc_lo = 0.f, rc_hi = 0.f;
  if (has_c2p && ok) {
    const __nv_bfloat16* xk_h = args.xk + (int64_t)head * args.xrows * kHeadDim;
    const uint32_t q_row = smem + kSmemQ + uint32_t(tid) * 128u;
    rc_lo = dot_q_row(q_row, tid, xk_h);
    rc_hi = dot_q_row(q_row, tid, xk_h + (int64_t)(args.xrows - 1) * kHeadDim);
  }

  const uint32_t idesc_s = instr_desc(128, 128, 1, 0, 0);
  const uint32_t idesc_p2c = instr_desc(128, 256, 1, 0, 0);
  const uint32_t idesc_pv = instr_desc(128, 64, 1, 0, 1);

  float m_used = 0.f, l_run = 0.f;
  int sat_built = kPlain;  // which saturated pos_query tile currently sits in kSmemSat

  for (int j = 0; j < num_kt; ++j) {
    const int n0 = j * kTileN;
    const int d0 = m0 - n0 - (kTileN - 1);  // smallest distance of the tile pair; largest is d0 + 254
    int kind = kPlain;
    if (has_pos) kind = d0 >= args.sat_hi ? kSatHi : (d0 + 254 <= args.sat_lo ? kSatLo : kBand);

    if (kind == kBand) {
      // ---- position products on the tensor core, drained to shared memory as bf16 ------------------------------
      // Order matters for shared memory: the c2p stage overlays both windows, so the p2c product (which reads the
      // pos_query window) is computed and drained first.
      if (tid == 0 && ok) {
        const int u0 = d0 - args.d_first;
        mbar_expect_tx(bar_win, (has_c2p ? 32768u : 0u) + (has_p2c ? 32768u : 0u));
        if (has_c2p) tma_load_3d(smem + kSmemWinK, &args.tm_xk, bar_win, 0, u0, head);
        if (has_p2c) tma_load_3d(smem + kSmemWinQ, &args.tm_xq, bar_win, 0, u0, head);
        const bool ready = wait_one(bar_win, ph_win) && wait_one(bar_k, ph_k);
        tc_fence_after();
        if (ready && has_p2c) {
          // p2c[n][j] = K[n].X_q[j]   -> 256 columns of the bias area
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            mma_bf16(tmem_base + kColBias, smem_desc_sw128(smem + kSmemK + ks * 32, 1024, 16),
                     smem_desc_sw128(smem + kSmemWinQ + ks * 32, 1024, 16), idesc_p2c, ks > 0);
        }
        mma_commit(bar_s);
      }
      ph_win ^= 1;
      wait_all(bar_s, ph_s); ph_s ^= 1;
      wait_all(bar_pv, ph_pv ^ 1);  // previous P.V (if any) is done as well: P and the stage area are free
      tc_fence_after();
      if (has_p2c && ok) {
        const uint32_t row_addr = smem + kSmemStageP + uint32_t(tid) * kStagePPitch;
#pragma unroll 1
        for (int c8 = 0; c8 < 8; ++c8) {
          uint32_t r[32];
          tmem_ld32(tmem_lane + kColBias + c8 * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4)
            sts_v4(row_addr + (c8 * 4 + q4) * 16,
                   pack_bf16x2(__uint_as_float(r[q4 * 8 + 0]), __uint_as_float(r[q4 * 8 + 1])),
                   pack_bf16x2(__uint_as_float(r[q4 * 8 + 2]), __uint_as_float(r[q4 * 8 + 3])),
                   pack_bf16x2(__uint_as_float(r[q4 * 8 + 4]), __uint_as_float(r[q4 * 8 + 5])),
                   pack_bf16x2(__uint_as_float(r[q4 * 8 + 6]), __uint_as_float(r[q4 * 8 + 7])));
        }
      }
      tc_fence_before();
      sync_check();
      if (tid == 0 && ok) {
        tc_fence_after();
        if (has_c2p) {
          // c2pT[j][m] = X_k[j].Q[m]   two 128-row blocks of the window -> columns [0,128) and [128,256) of the bias area
#pragma unroll
          for (int blk = 0; blk < 2; ++blk)
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              mma_bf16(tmem_base + kColBias + blk * 128,
                       smem_desc_sw128(smem + kSmemWinK + blk * 16384 + ks * 32, 1024, 16),
                       smem_desc_sw128(smem + kSmemQ + ks * 32, 1024, 16), idesc_s, ks > 0);
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_bf16(tmem_base + kColS, smem_desc_sw128(smem + kSmemQ + ks * 32, 1024, 16),
                   smem_desc_sw128(smem + kSmemK + ks * 32, 1024, 16), idesc_s, ks > 0);
        mma_commit(bar_s);
      }
      wait_all(bar_s, ph_s); ph_s ^= 1;
      tc_fence_after();
      if (has_c2p && ok) {
#pragma unroll 1
        for (int blk = 0; blk < 2; ++blk) {
          const uint32_t row_addr = smem + kSmemStageC + uint32_t(blk * 128 + tid) * kStageCPitch;
#pragma unroll 1
          for (int c4 = 0; c4 < 4; ++c4) {
            uint32_t r[32];
            tmem_ld32(tmem_lane + kColBias + blk * 128 + c4 * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
              sts_v4(row_addr + (c4 * 4 + q4) * 16,
                     pack_bf16x2(__uint_as_float(r[q4 * 8 + 0]), __uint_as_float(r[q4 * 8 + 1])),
                     pack_bf16x2(__uint_as_float(r[q4 * 8 + 2]), __uint_as_float(r[q4 * 8 + 3])),
                     pack_bf16x2(__uint_as_float(r[q4 * 8 + 4]), __uint_as_float(r[q4 * 8 + 5])),
                     pack_bf16x2(__uint_as_float(r[q4 * 8 + 6]), __uint_as_float(r[q4 * 8 + 7])));
          }
        }
      }
      tc_fence_before();
      sync_check();
      sat_built = kPlain;  // the stage area overlays the saturated tile
    } else {
      // ---- plain or saturated tile pair -----------------------------------------------------------------------------
      const bool want_sat = has_p2c && kind != kPlain;
      wait_all(bar_pv, ph_pv ^ 1);  // previous P.V (if any) done: P is free, O may be rescaled
      if (want_sat && sat_built != kind) {
        // every row of the tile = the saturated pos_query row, in the 128-byte-swizzled operand layout
        const __nv_bfloat16* src = args.xq + ((int64_t)head * args.xrows + (kind == kSatHi ? args.xrows - 1 : 0)) * kHeadDim;
        const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 v = __ldg(s4 + c);
          sts_v4(smem + kSmemSat + uint32_t(tid) * 128u + (uint32_t(c ^ (tid & 7)) << 4), v.x, v.y, v.z, v.w);
        }
        fence_proxy_async_smem();
        sync_check();
        sat_built = kind;
      }
      if (tid == 0 && ok) {
        const bool ready = wait_one(bar_k, ph_k);
        tc_fence_after();
        if (ready) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            mma_bf16(tmem_base + kColS, smem_desc_sw128(smem + kSmemQ + ks * 32, 1024, 16),
                     smem_desc_sw128(smem + kSmemK + ks * 32, 1024, 16), idesc_s, ks > 0);
          if (want_sat) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              mma_bf16(tmem_base + kColS, smem_desc_sw128(smem + kSmemSat + ks * 32, 1024, 16),
                       smem_desc_sw128(smem + kSmemK + ks * 32, 1024, 16), idesc_s, 1);
          }
        }
        mma_commit(bar_s);
      }
      wait_all(bar_s, ph_s); ph_s ^= 1;
      tc_fence_after();
    }
    ph_k ^= 1;

    // K is consumed: fetch the next key tile while the softmax runs
    if (tid == 0 && ok && j + 1 < num_kt) {
      mbar_expect_tx(bar_k, 16384);
      tma_load_3d(smem + kSmemK, &args.tm_k, bar_k, 0, head, seq_row0 + n0 + kTileN);
    }

    // ---- softmax on this thread's row -----------------------------------------------------------------------------------
    float s[kTileN];
    if (ok) {
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t r[32];
        tmem_ld32(tmem_lane + kColS + c4 * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[c4 * 32 + i] = __uint_as_float(r[i]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < kTileN; ++i) s[i] = 0.f;
    }
    float row_const = 0.f;
    if (kind == kBand) {
      if (has_c2p) {
        // c2p[m][n] sits at stage_c[(m + 127 - i)][m], i = n - n0
        const uint32_t base = smem + kSmemStageC + uint32_t(tid + 127) * kStageCPitch + uint32_t(tid) * 2u;
#pragma unroll
        for (int i = 0; i < kTileN; ++i) s[i] += bf16_bits_to_f32(lds_u16(base - uint32_t(i) * kStageCPitch));
      }
      if (has_p2c) {
        // p2c[m][n] sits at stage_p[i][(m + 127 - i)]
        const uint32_t base = smem + kSmemStageP + uint32_t(tid + 127) * 2u;
#pragma unroll
        for (int i = 0; i < kTileN; ++i) s[i] += bf16_bits_to_f32(lds_u16(base + uint32_t(i) * (kStagePPitch - 2u)));
      }
    } else if (kind == kSatHi) {
      row_const = rc_hi;
    } else if (kind == kSatLo) {
      row_const = rc_lo;
    }
    if (n0 + kTileN > len) {  // keys past the end of the sequence
      const int valid = len - n0;
#pragma unroll
      for (int i = 0; i < kTileN; ++i) s[i] = i < valid ? s[i] : -INFINITY;
    }
    float mx = s[0];
#pragma unroll
    for (int i = 1; i < kTileN; ++i) mx = fmaxf(mx, s[i]);
    const float t_max = (mx + row_const) * args.scale_log2;
    if (j == 0) {
      m_used = t_max;
    } else {
      const bool need = t_max > m_used + 8.f;
      if (__any_sync(0xffffffffu, need)) {  // warp-uniform: O of these 32 rows is rescaled in TMEM
        const float m_new = fmaxf(m_used, t_max);
        const float alpha = ex2(m_used - m_new);
        l_run *= alpha;
        m_used = m_new;
        if (ok) {
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
            uint32_t r[32];
            tmem_ld32(tmem_lane + kColO + c2 * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(tmem_lane + kColO + c2 * 32, r);
          }
          tmem_wait_st();
        }
      }
    }
    const float off = row_const * args.scale_log2 - m_used;
    float l_add = 0.f;
#pragma unroll
    for (int i = 0; i < kTileN; ++i) {
      s[i] = ex2(fmaf(s[i], args.scale_log2, off));
      l_add += s[i];
    }
    l_run += l_add;
    // P as the bf16 A operand of P.V: two 64-key halves, 128-byte rows, 16-byte chunks XOR-swizzled by (row & 7)
#pragma unroll
    for (int kb = 0; kb < 2; ++kb)
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int b = kb * 64 + c * 8;
        sts_v4(smem + kSmemP + kb * 16384 + uint32_t(tid) * 128u + (uint32_t(c ^ (tid & 7)) << 4),
               pack_bf16x2(s[b + 0], s[b + 1]), pack_bf16x2(s[b + 2], s[b + 3]), pack_bf16x2(s[b + 4], s[b + 5]),
               pack_bf16x2(s[b + 6], s[b + 7]));
      }
    fence_proxy_async_smem();
    tc_fence_before();
    sync_check();

    // ---- O += P.V ------------------------------------------------------------------------------------------------------------
    if (tid == 0 && ok) {
      const bool ready = wait_one(bar_v, ph_v);
      tc_fence_after();
      if (ready) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          mma_bf16(tmem_base + kColO,
                   smem_desc_sw128(smem + kSmemP + (ks >> 2) * 16384 + (ks & 3) * 32, 1024, 16),
                   smem_desc_sw128(smem + kSmemV + ks * 2048, 1024, 1024), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
      }
      mma_commit(bar_pv);
    }
    ph_v ^= 1;
    ph_pv ^= 1;
    if (j + 1 < num_kt) {
      // V may only be overwritten once this P.V has read it
      if (tid == 0 && ok) {
        wait_one(bar_pv, ph_pv ^ 1);
        mbar_expect_tx(bar_v, 16384);
        tma_load_3d(smem + kSmemV, &args.tm_v, bar_v, 0, head, seq_row0 + n0 + kTileN);
      }
    }
  }

  // ---- epilogue -------------------------------------------------------------------------------------------------------------
  wait_all(bar_pv, ph_pv ^ 1);
  tc_fence_after();
  if (ok) {
    const bool valid = my_row < len;
    const bool pad = !valid && my_row < row_limit;  // dense padding rows inside a partly valid tile get zeros
    const float inv = valid ? 1.f / l_run : 0.f;
    uint4* o4 = reinterpret_cast<uint4*>(out_ptr);
#pragma unroll
    for (int c2 = 0; c2 < 2; ++c2) {
      uint32_t r[32];
      tmem_ld32(tmem_lane + kColO + c2 * 32, r);  // whole warps execute this, whatever their rows
      tmem_wait_ld();
      if (valid || pad) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 v = make_uint4(0, 0, 0, 0);
          if (valid)
            v = make_uint4(pack_bf16x2(__uint_as_float(r[q4 * 8 + 0]) * inv, __uint_as_float(r[q4 * 8 + 1]) * inv),
                           pack_bf16x2(__uint_as_float(r[q4 * 8 + 2]) * inv, __uint_as_float(r[q4 * 8 + 3]) * inv),
                           pack_bf16x2(__uint_as_float(r[q4 * 8 + 4]) * inv, __uint_as_float(r[q4 * 8 + 5]) * inv),
                           pack_bf16x2(__uint_as_float(r[q4 * 8 + 6]) * inv, __uint_as_float(r[q4 * 8 + 7]) * inv));
          o4[c2 * 4 + q4] = v;
        }
      }
    }
    if (args.lse != nullptr && (valid || pad))
      args.lse[(int64_t)(seq_row0 + my_row) * args.heads + head] =
          valid ? (m_used + log2f(l_run)) * 0.6931471805599453f : 0.f;
  }
  tc_fence_before();
  __syncthreads();
  if (!ok || *abort_flag != 0u) {
    if (tid == 0 && args.status != nullptr) atomicOr(reinterpret_cast<unsigned int*>(args.status), FDB_DEV_TIMEOUT);
    // give copies and MMAs that may still be in flight a bounded time to land before TMEM and shared memory go away
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace

int launch_attn_fwd_serial(const fdb_attn_params& p, const ExpandGeometry& g, const WorkspaceLayout& w, void* stream) {
  if (p.dtype != FDB_BF16) return fail(FDB_ERR_UNSUPPORTED, "the serial kernel takes bf16 inputs only");
  FwdArgs a;
  char* ws = static_cast<char*>(p.workspace);
  int rc;
  if ((rc = make_map_rows(&a.tm_q, p.q, p.total_rows, p.heads, p.q_row_stride, p.q_head_stride, kTileM, false, "q"))) return rc;
  if ((rc = make_map_rows(&a.tm_k, p.k, p.total_rows, p.heads, p.k_row_stride, p.k_head_stride, kTileN, false, "k"))) return rc;
  if ((rc = make_map_rows(&a.tm_v, p.v, p.total_rows, p.heads, p.v_row_stride, p.v_head_stride, kTileN, false, "v"))) return rc;
  a.xk = p.pos_key ? reinterpret_cast<const __nv_bfloat16*>(ws + w.exp_key) : nullptr;
  a.xq = p.pos_query ? reinterpret_cast<const __nv_bfloat16*>(ws + w.exp_query) : nullptr;
  // a map is always encoded so the kernel argument is well formed; an unused one points at q
  if (a.xk) { if ((rc = make_map_table(&a.tm_xk, a.xk, g.rows, p.heads, false, "expanded pos_key"))) return rc; } else a.tm_xk = a.tm_q;
  if (a.xq) { if ((rc = make_map_table(&a.tm_xq, a.xq, g.rows, p.heads, false, "expanded pos_query"))) return rc; } else a.tm_xq = a.tm_q;
  a.out = static_cast<__nv_bfloat16*>(p.out);
  a.o_rs = p.out_row_stride; a.o_hs = p.out_head_stride;
  a.seq_info = reinterpret_cast<const int32_t*>(ws + w.seq_info);
  a.tile_first = reinterpret_cast<const int32_t*>(ws + w.tile_first);
  a.lse = p.lse; a.status = p.status;
  a.batch = p.batch; a.heads = p.heads; a.packed = p.cu_seqlens != nullptr; a.max_seqlen = p.max_seqlen;
  a.sat_lo = g.sat_lo; a.sat_hi = g.sat_hi; a.d_first = g.d_first; a.xrows = g.rows;
  a.scale_log2 = p.sm_scale * 1.4426950408889634f;

  const int64_t dense_tiles = (int64_t)p.batch * ((p.max_seqlen + kTileM - 1) / kTileM);
  int64_t slots = dense_tiles;
  if (a.packed) slots = std::min<int64_t>(dense_tiles, (int64_t)(p.total_rows + kTileM - 1) / kTileM + p.batch);
  if (slots <= 0) return FDB_OK;
  if (slots > 2147483647LL || p.heads > 65535) return fail(FDB_ERR_LIMIT, "grid too large");


  cudaError_t e = cudaFuncSetAttribute(attn_fwd_serial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));

  attn_fwd_serial_kernel<<<dim3((unsigned)slots, p.heads), kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "attn_fwd launch: %s", cudaGetErrorString(e));
  return FDB_OK;
}

}  // namespace fdb
