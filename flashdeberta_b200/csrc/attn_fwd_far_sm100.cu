// Fused attention forward for sm_100a — the "far" kernel: every key tile whose position terms are saturated (or absent).
//
// A long sequence is mostly such tiles: further than about five tiles from the diagonal, c2p is one number per query row
// and p2c one number per key, so a tile costs a plain flash-attention step plus one extra accumulating MMA.  They need no
// position-product area in tensor memory, which leaves room to keep TWO key tiles in flight: two softmax teams of 128
// threads (one thread per query row, all 128 keys of the tile in registers) take the key tiles alternately, each with its
// own S, P and O columns and its own running maximum, so one team's tensor-memory round trips and its maximum search
// overlap the other team's exponentials.  There is no per-tile exchange between threads at all.
//
//   warps 0-3  team 0: key tiles 0, 2, 4, ... of this launch        warp 8   lane 0: score MMAs  S_t = Q.K^T (+ R.K^T)
//   warps 4-7  team 1: key tiles 1, 3, 5, ...                        warp 9   lane 0: TMA (Q once, K/V three stages)
//                                                                    warp 10  lane 0: O_t += P_t.V
// Tensor memory: O_0 64 | O_1 64 | P_0 64 | P_1 64 | S_0 128 | S_1 128.
//
// When the call has position terms the band tiles are left to attn_fwd_kernel (band_only mode), which runs next on the same
// stream: this kernel then stores, per (row, head), the merged unnormalised accumulator, reference maximum and row sum
// instead of the final output.  Without position terms it handles every tile and writes the output itself.
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

constexpr int kFarThreads = 384;
constexpr int kFarScoreWarp = 8, kFarTmaWarp = 9, kFarPvWarp = 10;
constexpr int kFarProducerRegs = 40, kFarSoftmaxRegs = 232;  // 168 * 384 = 40 * 128 + 232 * 256
constexpr int kStages = 3;
constexpr uint32_t kFarTmemCols = 512;
constexpr uint32_t kFColO = 0;    // + 64 t
constexpr uint32_t kFColP = 128;  // + 64 t
constexpr uint32_t kFColS = 256;  // + 128 t

constexpr uint32_t kFSmemQ = 0;
constexpr uint32_t kFSmemK = 16384;                       // 3 stages
constexpr uint32_t kFSmemV = kFSmemK + kStages * 16384;   // 3 stages
constexpr uint32_t kFSmemSat = kFSmemV + kStages * 16384; // 2 x (8 x 128 B)
constexpr uint32_t kFSmemMl = kFSmemSat + 2048;           // float [2 teams][128 rows][2]: reference maximum, row sum
constexpr uint32_t kFSmemBars = kFSmemMl + 2048;
constexpr uint32_t kFSmemBytes = kFSmemBars + 256 + 1024;

enum FarBar : uint32_t {
  kFBarQ = 0,
  kFBarK = 1,        // 3: K stage landed
  kFBarV = 4,        // 3: V stage landed
  kFBarKFree = 7,    // 3: the score MMAs that read the stage finished
  kFBarVFree = 10,   // 3: the P.V that read the stage finished
  kFBarS = 13,       // 2: S_t is in tensor memory
  kFBarSFree = 15,   // 2 (count 128): team t holds its scores in registers
  kFBarP = 17,       // 2 (count 128): P_t is in tensor memory
  kFBarO = 19,       // 2: P_t.V finished
  kFNumBars = 21
};

__global__ void __launch_bounds__(kFarThreads, 1) attn_fwd_far_kernel(const __grid_constant__ FwdArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem - smem_u32(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.y;

  const int4 slot = __ldg(args.slot_info + blockIdx.x);  // (sequence, first row of the tile in it, its first row, its length)
  if (slot.x < 0) return;                                  // slot past the last sequence
  const int seq = slot.x, m0 = slot.y, seq_row0 = slot.z, len = slot.w;
  (void)seq;
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
  if (has_pos) band_run(m0, num_kt, args.sat_lo, args.sat_hi, jb, nb);
  const int n_far = num_kt - nb;
  if (n_far <= 0) return;  // nothing but band tiles: the band kernel starts from scratch
  auto tile_of = [&](int i) -> int { return i < jb ? i : i + nb; };
  auto kind_of = [&](int j) -> int { return !has_pos ? kPlain : (j < jb ? kSatHi : kSatLo); };

  auto bar = [&](uint32_t i) -> uint32_t { return smem + kFSmemBars + 8u * i; };
  const uint32_t tmem_slot = smem + kFSmemBars + 8u * kFNumBars;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + kFSmemBars + 8u * kFNumBars + 8u);

  if (tid == 0) {
    *abort_flag = 0u;
    for (uint32_t i = 0; i < kFNumBars; ++i) {
      const bool team_wide = (i >= kFBarSFree && i < kFBarSFree + 2) || (i >= kFBarP && i < kFBarP + 2);
      mbar_init(bar(i), team_wide ? 128u : 1u);
    }
    fence_barrier_init();
  }
  if (warp == kFarScoreWarp) {
    tmem_alloc(tmem_slot, kFarTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem_gen + kFSmemBars + 8u * kFNumBars);

  bool ok = true;

  if (warp >= kFarScoreWarp) {
    reg_dealloc<kFarProducerRegs>();
    auto wait = [&](uint32_t b, uint32_t parity) {
      if (ok && !mbar_wait_abortable(b, parity, abort_flag)) { ok = false; *abort_flag = 1u; }
    };
    if (warp == kFarTmaWarp) {
      if (lane == 0) {
        tma_prefetch_desc(&args.tm_q); tma_prefetch_desc(&args.tm_k); tma_prefetch_desc(&args.tm_v);
        mbar_expect_tx(bar(kFBarQ), 16384u + (has_p2c ? 2048u : 0u));
        tma_load_3d(smem + kFSmemQ, &args.tm_q, bar(kFBarQ), 0, head, seq_row0 + m0);
        if (has_p2c) {
          // Saturated pos_query rows as MMA operands: the last (first) eight rows of an expanded table are all the row of
          // distances beyond sat_hi (sat_lo), so an 8-row box is the 8 identical rows in the swizzled layout.
          tma_load_3d(smem + kFSmemSat, &args.tm_xq_sat, bar(kFBarQ), 0, args.xrows - 8, head);
          tma_load_3d(smem + kFSmemSat + 1024, &args.tm_xq_sat, bar(kFBarQ), 0, 0, head);
        }
#pragma unroll 1
        for (int i = 0; i < n_far; ++i) {
          const int st = i % kStages;
          const uint32_t use = uint32_t(i / kStages);
          const int row = seq_row0 + tile_of(i) * kTileN;
          if (use > 0) wait(bar(kFBarKFree + st), (use - 1u) & 1u);
          if (!ok) break;
          mbar_expect_tx(bar(kFBarK + st), 16384);
          tma_load_3d(smem + kFSmemK + st * 16384, &args.tm_k, bar(kFBarK + st), 0, head, row);
          if (use > 0) wait(bar(kFBarVFree + st), (use - 1u) & 1u);
          if (!ok) break;
          mbar_expect_tx(bar(kFBarV + st), 16384);
          tma_load_3d(smem + kFSmemV + st * 16384, &args.tm_v, bar(kFBarV + st), 0, head, row);
        }
      }
      __syncwarp();
    } else if (warp == kFarScoreWarp) {
      if (lane == 0) {
        const uint32_t idesc_s = instr_desc(128, 128, 1, 0, 0);
        const uint64_t dq = smem_desc_sw128(smem + kFSmemQ, 1024, 16);
        const uint64_t dk0 = smem_desc_sw128(smem + kFSmemK, 1024, 16);
        const uint64_t dsat = smem_desc_sw128(smem + kFSmemSat, 0, 16);  // group stride 0: 8 identical rows serve all 128
        wait(bar(kFBarQ), 0);
#pragma unroll 1
        for (int i = 0; i < n_far; ++i) {
          const int t = i & 1, st = i % kStages;
          const uint32_t u = uint32_t(i >> 1);  // how often team t's buffers were used before
          const int kind = kind_of(tile_of(i));
          const uint64_t dk = dk0 + uint64_t(st) * (16384u >> 4);
          FDB_STAMP(2, i, 0);
          if (u > 0) wait(bar(kFBarSFree + t), (u - 1u) & 1u);  // team t has pulled its previous scores
          FDB_STAMP(2, i, 1);
          wait(bar(kFBarK + st), uint32_t(i / kStages) & 1u);
          tc_fence_after();
          FDB_STAMP(2, i, 2);
          if (ok) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              mma_bf16(tmem_base + kFColS + 128 * t, dq + uint64_t((ks * 32) >> 4), dk + uint64_t((ks * 32) >> 4), idesc_s, ks > 0);
            if (has_p2c && kind != kPlain) {
              const uint64_t ds = dsat + uint64_t(kind == kSatHi ? 0u : (1024u >> 4));
#pragma unroll
              for (int ks = 0; ks < 4; ++ks)
                mma_bf16(tmem_base + kFColS + 128 * t, ds + uint64_t((ks * 32) >> 4), dk + uint64_t((ks * 32) >> 4), idesc_s, 1);
            }
          }
          mma_commit(bar(kFBarS + t));
          mma_commit(bar(kFBarKFree + st));
          FDB_STAMP(2, i, 3);
        }
      }
      __syncwarp();
    } else if (warp == kFarPvWarp) {
      if (lane == 0) {
        const uint32_t idesc_pv = instr_desc(128, 64, 1, 0, 1);
        const uint64_t dv0 = smem_desc_sw128(smem + kFSmemV, 1024, 16);
#pragma unroll 1
        for (int i = 0; i < n_far; ++i) {
          const int t = i & 1, st = i % kStages;
          const uint32_t u = uint32_t(i >> 1);
          const uint64_t dv = dv0 + uint64_t(st) * (16384u >> 4);
          wait(bar(kFBarV + st), uint32_t(i / kStages) & 1u);
          FDB_STAMP(3, i, 0);
          wait(bar(kFBarP + t), u & 1u);
          tc_fence_after();
          FDB_STAMP(3, i, 1);
          if (ok) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              mma_bf16_ts(tmem_base + kFColO + 64 * t, tmem_base + kFColP + 64 * t + 8 * ks, dv + uint64_t((ks * 2048) >> 4),
                          idesc_pv, (u > 0 || ks > 0) ? 1u : 0u);
          }
          mma_commit(bar(kFBarO + t));
          mma_commit(bar(kFBarVFree + st));
          FDB_STAMP(3, i, 2);
        }
      }
      __syncwarp();
    }
  } else {
    // =================================================== softmax teams ==================================================
    reg_alloc<kFarSoftmaxRegs>();
    const int t = warp >> 2;
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

    wait(bar(kFBarQ), 0);
    float rc_lo = 0.f, rc_hi = 0.f;
    if (has_c2p && ok) {
      const __nv_bfloat16* xk_h = static_cast<const __nv_bfloat16*>(args.xk) + (int64_t)head * args.xrows * kHeadDim;
      const uint32_t q_row = smem + kFSmemQ + uint32_t(r) * 128u;
      rc_lo = dot_q_row(q_row, r, xk_h);
      rc_hi = dot_q_row(q_row, r, xk_h + (int64_t)(args.xrows - 1) * kHeadDim);
    }

    float m_used = 0.f, l_run = 0.f;
    uint32_t u = 0;  // tiles this team has processed
#pragma unroll 1
    for (int i = t; i < n_far; i += 2, ++u) {
      const int j = tile_of(i);
      const int n0 = j * kTileN;
      const int kind = kind_of(j);

      wait(bar(kFBarS + t), u & 1u);
      tc_fence_after();
      if (lane == 0 && quad == 0) FDB_STAMP(t, i, 0);
      if (n0 + kTileN > len && ok) {
        // ragged last tile of the sequence: overwrite the scores of keys past its end in tensor memory, 32 columns at a
        // time, so the code below is the same for every tile (a select on the 128 register-resident scores under a
        // data-dependent branch made the compiler keep two copies of them)
        const int valid = len - n0;
#pragma unroll 1
        for (int q = valid >> 5; q < 4; ++q) {
          uint32_t a[32];
          tmem_ld32(tmem_lane + kFColS + 128 * t + 32 * q, a);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) a[c] = 32 * q + c < valid ? a[c] : 0xff800000u;
          tmem_st32(tmem_lane + kFColS + 128 * t + 32 * q, a);
        }
        tmem_wait_st();
      }
      // the team's previous P.V has finished (it was issued a whole tile of the other team ago): O_t and P_t are free
      if (u > 0) { wait(bar(kFBarO + t), (u - 1u) & 1u); tc_fence_after(); }

      // pull the 128 scores of this row in four chunks; the maximum of the first two is taken while the rest arrive
      uint32_t a0[32], a1[32], a2[32], a3[32];
      if (ok) {
        tmem_ld32(tmem_lane + kFColS + 128 * t, a0);
        tmem_ld32(tmem_lane + kFColS + 128 * t + 32, a1);
        tmem_wait_ld();
        tmem_ld32(tmem_lane + kFColS + 128 * t + 64, a2);
        tmem_ld32(tmem_lane + kFColS + 128 * t + 96, a3);
      }
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
      if (ok) tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bar(kFBarSFree + t));
      if (lane == 0 && quad == 0) FDB_STAMP(t, i, 1);
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
      if (lane == 0 && quad == 0) FDB_STAMP(t, i, 2);
      if (u == 0) {
        m_used = t_max;
      } else {
        const bool need = t_max > m_used + 8.f;
        if (__any_sync(0xffffffffu, need)) {
          const float m_new = fmaxf(m_used, t_max);
          const float alpha = ex2(m_used - m_new);
          l_run *= alpha;
          m_used = m_new;
          if (ok) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t o[32];
              tmem_ld32(tmem_lane + kFColO + 64 * t + 32 * h, o);
              tmem_wait_ld();
#pragma unroll
              for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
              tmem_st32(tmem_lane + kFColO + 64 * t + 32 * h, o);
            }
          }
        }
      }
      if (lane == 0 && quad == 0) FDB_STAMP(t, i, 3);
      // p = 2^(s * scale + off), two keys per instruction where the hardware has a two-wide form; the first 64 keys go to
      // tensor memory while the other 64 are computed
      const float off = row_const * args.scale_log2 - m_used;
      const uint64_t scale2 = pack_f32x2(args.scale_log2, args.scale_log2), off2 = pack_f32x2(off, off);
      uint64_t l2[2] = {0ull, 0ull};
      auto half = [&](const uint32_t (&x)[32], const uint32_t (&y)[32], uint32_t col) {
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
        if (ok) tmem_st32(tmem_lane + col, p);
      };
      half(a0, a1, kFColP + 64 * t);
      half(a2, a3, kFColP + 64 * t + 32);
      {
        float s0, s1, s2, s3;
        unpack_f32x2(l2[0], s0, s1);
        unpack_f32x2(l2[1], s2, s3);
        l_run += (s0 + s1) + (s2 + s3);
      }
      if (lane == 0 && quad == 0) FDB_STAMP(t, i, 4);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(kFBarP + t));
      if (lane == 0 && quad == 0) FDB_STAMP(t, i, 5);
    }

    // ---- merge the two teams: O = O_0 2^(m_0-m) + O_1 2^(m_1-m), l likewise; team t writes output columns 32t .. 32t+31 ----
    if (u > 0) wait(bar(kFBarO + t), (u - 1u) & 1u);  // this team's last P.V
    const uint32_t ml = smem + kFSmemMl + uint32_t(r) * 8u;
    sts_f32(ml + uint32_t(t) * 1024u, u > 0 ? m_used : -INFINITY);
    sts_f32(ml + uint32_t(t) * 1024u + 4u, l_run);
    tc_fence_before();
    bar_sync(1, 256);
    tc_fence_after();
    const float m_a = lds_f32(ml), l_a = lds_f32(ml + 4u), m_b = lds_f32(ml + 1024u), l_b = lds_f32(ml + 1028u);
    const float m = fmaxf(m_a, m_b);                 // team 0 always has at least one tile
    const float w_a = ex2(m_a - m), w_b = ex2(m_b - m);  // 2^(-inf) = 0 for a team without tiles
    const float l_tot = l_a * w_a + l_b * w_b;
    if (ok) {
      uint32_t oa[32], ob[32];
      tmem_ld32(tmem_lane + kFColO + 32 * t, oa);
      if (n_far > 1) tmem_ld32(tmem_lane + kFColO + 64 + 32 * t, ob);  // O_1 was never written when there is one tile
      tmem_wait_ld();
      float o[32];
#pragma unroll
      for (int c = 0; c < 32; ++c)
        o[c] = __uint_as_float(oa[c]) * w_a + (n_far > 1 ? __uint_as_float(ob[c]) * w_b : 0.f);
      const bool valid = my_row < len;
      if (has_pos) {
        if (valid) {  // partial result for the band kernel
          const int64_t rh = (int64_t)(seq_row0 + my_row) * args.heads + head;
          float4* po = reinterpret_cast<float4*>(args.part_o + rh * 64 + 32 * t);
#pragma unroll
          for (int q = 0; q < 8; ++q) po[q] = make_float4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
          if (t == 0) *reinterpret_cast<float2*>(args.part_ml + rh * 2) = make_float2(m, l_tot);
        }
      } else {
        const bool pad = !valid && my_row < row_limit;
        if (valid || pad) {
          const float inv = valid ? 1.f / l_tot : 0.f;
          uint4* o4 = reinterpret_cast<uint4*>(args.out + (int64_t)(seq_row0 + my_row) * args.o_rs +
                                               (int64_t)head * args.o_hs + 32 * t);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (valid)
              v = make_uint4(pack_bf16x2(o[q4 * 8 + 0] * inv, o[q4 * 8 + 1] * inv), pack_bf16x2(o[q4 * 8 + 2] * inv, o[q4 * 8 + 3] * inv),
                             pack_bf16x2(o[q4 * 8 + 4] * inv, o[q4 * 8 + 5] * inv), pack_bf16x2(o[q4 * 8 + 6] * inv, o[q4 * 8 + 7] * inv));
            o4[q4] = v;
          }
          if (t == 0 && args.lse != nullptr)
            args.lse[(int64_t)(seq_row0 + my_row) * args.heads + head] = valid ? (m + log2f(l_tot)) * 0.6931471805599453f : 0.f;
        }
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
  if (warp == kFarScoreWarp) tmem_dealloc(tmem_base, kFarTmemCols);
}

}  // namespace

int launch_attn_fwd_far(const void* fwd_args, int64_t slots, int heads, void* stream) {
  const FwdArgs& a = *static_cast<const FwdArgs*>(fwd_args);
  cudaError_t e = cudaFuncSetAttribute(attn_fwd_far_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFSmemBytes);
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  attn_fwd_far_kernel<<<dim3((unsigned)slots, heads), kFarThreads, kFSmemBytes, static_cast<cudaStream_t>(stream)>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "attn_fwd_far launch: %s", cudaGetErrorString(e));
  return FDB_OK;
}

}  // namespace fdb
