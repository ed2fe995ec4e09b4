// Fused DeBERTa disentangled-attention forward for sm_100a — warp-specialised kernel.
//
// Replaces the reference's Triton forward kernels (src/flashdeberta/ops/flash_attention.py:146-300 and
// src/flashdeberta/ops/flash_attention_varlen.py:85-225) and the two bias GEMMs in front of them
// (src/flashdeberta/model.py:189-192, :210-214).
//
// One CTA = one 128-row query tile of one (sequence, head); 16 warps in four warpgroups (registers move from the
// producer and drain groups to the softmax groups with setmaxnreg):
//   warps 0-3   softmax group 0: thread r owns row r of the tile, keys   0..63  of every 128-key tile
//   warps 4-7   softmax group 1: thread r owns row r of the tile, keys  64..127
//   warp  8     lane 0 issues the score-side tcgen05.mma: S = Q.K^T and the position products (the warp allocates TMEM)
//   warp  9     lane 0 issues every TMA load: Q once, K/V double-buffered, position-table windows
//   warp  10    lane 0 issues O += P.V
//   warps 12-15 drain group: moves the c2p product of a band tile from tensor memory to shared memory (bf16)
// Tensor memory (512 columns): O 64 | P 64 | S 128 | R 256 (position products of a band tile).
//
// Per key tile j:  S = Q.K^T (tensor core, fp32 in TMEM)  ->  both softmax groups pull their half of S (and of the p2c
// product) into registers and release S and R at once, so the tensor core computes the scores of tile j+1 while the
// softmax of tile j runs  ->  the groups agree on the row maximum through shared memory, write P = exp2(...) as bf16 pairs
// into the P columns  ->  O += P.V with P read from tensor memory and V from shared memory.  O stays in TMEM and is
// rescaled only when the running maximum moved by more than 2^8.
//
// Position terms (tables arrive expanded through the bucket function, see attn_prepare.cu; row of (m, n) is (m-n)-d_first):
//   * saturated tile pair (all distances beyond a saturation point): c2p is one dot product per query row, folded into the
//     row's exponent offset; p2c is one dot product per key, accumulated into S on the tensor core as R.K^T where all rows
//     of R equal the saturated pos_query row (R is 8 rows of shared memory read with a zero group stride);
//   * band tile pair: p2c comes from products X_q[32(3-b+t) .. +128).K[32b .. +32)^T, b = key block, t = 0/1 (issued as three
//     128x64 and two 128x32 MMAs groups), arranged so that the value thread (quadrant w, lane l) needs for key 32b+c sits in
//     its own quadrant at lane (l+31-c)&31 of product t = (l > c): one select on the source side and one warp shuffle per
//     score element, fp32, no shared memory;
//     c2p needs a transpose: X_k[window].Q^T (256x128) is computed into R ahead of the p2c product, the drain group writes it
//     to shared memory as bf16 [position][query] while the softmax of the previous tile is still running, and thread m
//     reads c2p[m][m+127-i] at compile-time offsets from a per-thread base.
// No (rows x 2*span) bias tensor is ever written to global memory.
//
// Every mbarrier wait is bounded and gives up early once another role has raised the abort flag; the CTA then sets
// FDB_DEV_TIMEOUT in the status word, waits a millisecond for copies in flight, releases its TMEM and returns.
// No TMA load uses multicast.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "internal.h"
#include "sm100_ptx.cuh"
#include "tensor_map.cuh"
#include "attn_fwd_common.cuh"

namespace fdb {
namespace {

using namespace ptx;
using namespace fwd;

constexpr int kSoftmaxThreads = 256;
constexpr int kDrainThreads = 128;
constexpr int kThreads = 512;            // four warpgroups: softmax 0, softmax 1, producers (warps 10, 11 idle), drain
constexpr int kMmaWarp = 8, kTmaWarp = 9, kPvWarp = 10, kDrainWarp0 = 12;
// 128 registers per thread at launch; after setmaxnreg: 40 * 128 + 72 * 128 + 200 * 256 = 65536
constexpr int kProducerRegs = 40, kDrainRegs = 72, kSoftmaxRegs = 200;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 0;     // 64 columns: output accumulator
constexpr uint32_t kColP = 64;    // 64 columns: P as bf16 pairs (keys 0..63 in the first 32, keys 64..127 in the last 32)
constexpr uint32_t kColS = 128;   // 128 columns: scores
constexpr uint32_t kColR = 256;   // 256 columns: position products of a band tile

// shared memory map (bytes from a 1024-aligned base)
constexpr uint32_t kSmemQ = 0;                      // 128 x 128 B
constexpr uint32_t kSmemK = 16384;                  // 2 stages
constexpr uint32_t kSmemV = 49152;                  // 2 stages
constexpr uint32_t kSmemWinK = 81920;               // 256 x 128 B window of expanded pos_key
constexpr uint32_t kSmemWinQ = 114688;              // 256 x 128 B window of expanded pos_query
// c2p stage: bf16 [128 query rows][256 window positions], rows padded by 16 B.  Row m is rotated by m: position p of the
// window sits in column (p - m) & 255, so the 64 values a softmax thread needs are one aligned 128-byte run whose place does
// not depend on m.
constexpr uint32_t kStageCPitch = 528;
constexpr uint32_t kSmemStageC = 147456;
constexpr uint32_t kSmemSat = kSmemStageC + 69632;  // 217088: 2 x (8 x 128 B) saturated pos_query rows (hi, lo)
static_assert(128 * kStageCPitch <= 69632, "c2p stage");
constexpr uint32_t kSmemXchg = kSmemSat + 2048;     // float [2 parities][2 groups][128 rows] row maxima
constexpr uint32_t kSmemLsum = kSmemXchg + 2048;    // float [2 groups][128 rows] row sums at the end
constexpr uint32_t kSmemBars = kSmemLsum + 1024;
constexpr uint32_t kSmemBytes = kSmemBars + 256 + 1024;  // + alignment slack
static_assert(kSmemSat == 217088, "shared memory map");
static_assert(kSmemBytes <= 232448, "exceeds 227 KB");

// mbarriers.  "count" = arrivals per phase.
enum Bar : uint32_t {
  kBarQ = 0,         // 1   Q (and the saturated pos_query rows of the head) landed (TMA)
  kBarK = 1,         // 1   K stage s landed (TMA), 2 stages
  kBarV = 3,         // 1   V stage s landed (TMA), 2 stages
  kBarKFree = 5,     // 1   the MMAs that read K stage s finished (tcgen05.commit)
  kBarVFree = 7,     // 1   the P.V that read V stage s finished
  kBarWin = 9,       // 1   position windows landed (TMA)
  kBarWinFree = 10,  // 1   the MMAs that read the windows finished
  kBarS = 11,        // 1   S (and the p2c product) of a tile are in tensor memory
  kBarSFree = 12,    // 256 both softmax groups hold their scores in registers: S and R may be overwritten
  kBarP = 13,        // 256 P of a tile is in tensor memory
  kBarO = 14,        // 1   P.V of a tile finished
  kBarC2p = 15,      // 1   the c2p product of a band tile is in R
  kBarStage = 16,    // 128 the drain group has written the c2p stage (R may be overwritten, the stage may be read)
  kBarGather = 17,   // 256 both softmax groups are done reading the c2p stage
  kNumBars = 18
};

template <bool F8>
__global__ void __launch_bounds__(kThreads, 1) attn_fwd_kernel(const __grid_constant__ FwdArgs args) {
  using G = Geo<F8>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem - smem_u32(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.y;

  // ---- which tile ------------------------------------------------------------------------------------------------
  const int4 slot = __ldg(args.slot_info + blockIdx.x);  // (sequence, first row of the tile in it, its first row, its length)
  if (slot.x < 0) return;                                  // slot past the last sequence
  const int seq = slot.x, m0 = slot.y, seq_row0 = slot.z, len = slot.w;
  // rows of this tile that may be written: packed -> the sequence's own rows; dense -> the padded row range
  const int row_limit = args.packed ? len : args.max_seqlen;

  if (m0 >= len) {  // dense padding tile: zeros, nothing else (src/flashdeberta/padding.py:30-44)
    if (tid < kTileM && m0 + tid < row_limit) {
      uint4* o4 = reinterpret_cast<uint4*>(args.out + (int64_t)(seq_row0 + m0 + tid) * args.o_rs + (int64_t)head * args.o_hs);
#pragma unroll
      for (int c = 0; c < 8; ++c) o4[c] = make_uint4(0, 0, 0, 0);
      if (args.lse != nullptr) args.lse[(int64_t)(seq_row0 + m0 + tid) * args.heads + head] = 0.f;
    }
    return;
  }

  const bool has_c2p = args.xk != nullptr, has_p2c = args.xq != nullptr;
  const bool has_pos = has_c2p || has_p2c;
  const int num_kt = (len + kTileN - 1) / kTileN;
  // key tiles this launch works on: all of them, or (split launch) the contiguous run of band tiles; `jj` counts them
  int j_first = 0, n_proc = num_kt;
  if (args.band_only && len >= args.split_len) band_run(m0, num_kt, args.sat_lo, args.sat_hi, j_first, n_proc);
  const bool resume = args.band_only && n_proc < num_kt;  // the far kernel has left a partial result for this tile
  auto tile_kind = [&](int j) -> int {
    if (!has_pos) return kPlain;
    const int d0 = m0 - j * kTileN - (kTileN - 1);  // smallest distance of the pair; the largest is d0 + 254
    return d0 >= args.sat_hi ? kSatHi : (d0 + 254 <= args.sat_lo ? kSatLo : kBand);
  };

  // When the CTA's very first key tile is a band tile, the output and P columns are still unused: the two c2p blocks of
  // that tile go to the S columns and to O|P instead of R, so its p2c products need not wait for the drain group.
  const bool c2p_outside_r = !resume && n_proc > 0 && tile_kind(j_first) == kBand;

  auto bar = [&](uint32_t i) -> uint32_t { return smem + kSmemBars + 8u * i; };
  const uint32_t tmem_slot = smem + kSmemBars + 8u * kNumBars;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + kSmemBars + 8u * kNumBars + 8u);

  // ---- set-up ---------------------------------------------------------------------------------------------------------
  if (tid == 0) {
    *abort_flag = 0u;
    for (uint32_t i = 0; i < kNumBars; ++i) {
      uint32_t count = 1u;
      if (i == kBarSFree || i == kBarP || i == kBarGather) count = kSoftmaxThreads;
      if (i == kBarStage) count = kDrainThreads;
      mbar_init(bar(i), count);
    }
    fence_barrier_init();
  }
  // e4m3: value = stored * scale.  The three score terms carry different scale products; they are brought to the one of
  // Q.K^T (ratio_c, ratio_p) when they are added, and that product goes into the softmax scale.
  float c_eff = args.scale_log2, ratio_c = 1.f, ratio_p = 1.f, v_scale = 1.f;
  if constexpr (F8) {
    const float sq = __ldg(args.q_scale + (int64_t)seq * args.heads + head);
    const float sk = __ldg(args.k_scale + (int64_t)seq * args.heads + head);
    v_scale = __ldg(args.v_scale + (int64_t)seq * args.heads + head);
    c_eff = args.scale_log2 * sq * sk;
    if (has_c2p) ratio_c = __ldg(args.xk_scale + head) / sk;
    if (has_p2c) ratio_p = __ldg(args.xq_scale + head) / sq;
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem_gen + kSmemBars + 8u * kNumBars);

  bool ok = true;

  if (warp >= kDrainWarp0) {
    // =================================================== drain group ====================================================
    reg_dealloc<kDrainRegs>();
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // TMEM lane = position row inside a 128-position block
    const uint32_t tmem_lane = tmem_base + (uint32_t(quad * 32) << 16);
    auto wait = [&](uint32_t b, uint32_t parity) {  // warp-uniform result
      const bool mine = ok && mbar_wait_abortable(b, parity, abort_flag);
      const bool all = __all_sync(0xffffffffu, mine);
      if (ok && !all) *abort_flag = 1u;
      ok = all;
    };
    uint32_t band_idx = 0;
    for (int jj = 0; jj < n_proc; ++jj) {
      const int j = j_first + jj;
      if (tile_kind(j) != kBand) continue;
      wait(bar(kBarC2p), band_idx & 1u);                               // the product is in R
      if (band_idx > 0) wait(bar(kBarGather), (band_idx - 1u) & 1u);   // nobody reads the previous stage any more
      tc_fence_after();
      if (has_c2p && ok) {
        // The product has query rows in the lanes and window positions in the columns, so this thread holds row r.  The
        // windows of consecutive band tiles overlap by half: only the first tile of the run brings 256 positions, every
        // later one the 128 new ones (block 0), written over the half of the stage the new window no longer covers:
        // position p of the current window is "physical" position p ^ flip, stored in column (physical - r) & 255.
        const int nblk = band_idx == 0 ? 2 : 1;
        const uint32_t flip = (band_idx & 1u) ? 128u : 0u;
        const uint32_t row_addr = smem + kSmemStageC + uint32_t(r) * kStageCPitch;
#pragma unroll 1
        for (int blk = 0; blk < nblk; ++blk) {
          // where the score-issuing warp put the block (see there)
          const uint32_t col = tmem_lane + (band_idx > 0 ? kColS : (c2p_outside_r ? (blk == 0 ? kColS : kColO) : kColR + blk * 128));
          const uint32_t start = ((uint32_t(blk) * 128u) ^ flip) - uint32_t(r);  // column of the block's first position (mod 256)
          // an odd start puts value 2k-1 and 2k into one 32-bit word: funnel shift over consecutive pairs by 16 bits;
          // an even start keeps the pairs (shift "32" = take the upper word)
          const uint32_t sh = (start & 1u) ? 16u : 32u;
          uint32_t prev = 0;
          uint32_t t[32];
          tmem_ld32(col, t);
          tmem_wait_ld();
#pragma unroll 1  // kept rolled: this loop runs beside the softmax warps, whose unrolled code already fills the instruction cache
          for (int c4 = 0; c4 < 4; ++c4) {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(__uint_as_float(t[2 * i]), __uint_as_float(t[2 * i + 1]));
            if (c4 < 3) tmem_ld32(col + (c4 + 1) * 32, t);  // the next 32 columns are in flight while these are stored
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const uint32_t word = ((start + uint32_t(32 * c4 + 2 * k)) >> 1) & 127u;
              const uint32_t v = __funnelshift_rc(k == 0 ? prev : pk[k - 1], pk[k], sh);
              if (c4 == 0 && k == 0 && (start & 1u)) {
                // the low half of this word belongs to the other block's last position: write the upper half only
                sts_u16(row_addr + 4u * word + 2u, pk[0] & 0xffffu);
              } else {
                sts_u32(row_addr + 4u * word, v);
              }
            }
            prev = pk[15];
            if (c4 < 3) tmem_wait_ld();
          }
          if (start & 1u) sts_u16(row_addr + 4u * (((start + 128u) >> 1) & 127u), prev >> 16);  // the block's last value
        }
      }
      tc_fence_before();
      mbar_arrive(bar(kBarStage));
      ++band_idx;
    }
  } else if (warp >= kMmaWarp) {
    reg_dealloc<kProducerRegs>();
    if (warp == kTmaWarp) {
      // ================================================= TMA producer ===================================================
      if (lane == 0) {
        auto wait = [&](uint32_t b, uint32_t parity) {
          if (ok && !mbar_wait_abortable(b, parity, abort_flag)) { ok = false; *abort_flag = 1u; }
        };
        tma_prefetch_desc(&args.tm_q); tma_prefetch_desc(&args.tm_k); tma_prefetch_desc(&args.tm_v);
        mbar_expect_tx(bar(kBarQ), G::kTile + (has_p2c ? 16u * G::kRow : 0u));
        tma_load_3d(smem + kSmemQ, &args.tm_q, bar(kBarQ), 0, head, seq_row0 + m0);
        if (has_p2c) {
          // Saturated pos_query rows as MMA operands: the last (first) eight rows of an expanded table are all the row of
          // distances beyond sat_hi (sat_lo), so an 8-row box is the 8 identical rows in the swizzled layout.
          tma_load_3d(smem + kSmemSat, &args.tm_xq_sat, bar(kBarQ), 0, args.xrows - 8, head);
          tma_load_3d(smem + kSmemSat + 1024, &args.tm_xq_sat, bar(kBarQ), 0, 0, head);
        }
        int band_idx = 0;
        for (int jj = 0; jj < n_proc && ok; ++jj) {
          const int j = j_first + jj;
          const int s = jj & 1;
          const uint32_t use = uint32_t(jj >> 1);  // how often this stage was used before
          FDB_STAMP(3, j, 0);
          if (jj >= 2) wait(bar(kBarKFree + s), (use - 1u) & 1u);
          if (!ok) break;
          FDB_STAMP(3, j, 1);
          mbar_expect_tx(bar(kBarK + s), G::kTile);
          tma_load_3d(smem + kSmemK + s * 16384, &args.tm_k, bar(kBarK + s), 0, head, seq_row0 + j * kTileN);
          if (tile_kind(j) == kBand) {
            if (band_idx > 0) wait(bar(kBarWinFree), uint32_t(band_idx - 1) & 1u);
            if (!ok) break;
            const int u0 = m0 - j * kTileN - (kTileN - 1) - args.d_first;
            mbar_expect_tx(bar(kBarWin), (has_c2p ? G::kWin : 0u) + (has_p2c ? G::kWin : 0u));
            if (has_c2p) tma_load_3d(smem + kSmemWinK, &args.tm_xk, bar(kBarWin), 0, u0, head);
            if (has_p2c) tma_load_3d(smem + kSmemWinQ, &args.tm_xq, bar(kBarWin), 0, u0, head);
            ++band_idx;
          }
          if (jj >= 2) wait(bar(kBarVFree + s), (use - 1u) & 1u);
          if (!ok) break;
          FDB_STAMP(3, j, 2);
          mbar_expect_tx(bar(kBarV + s), G::kTile);
          tma_load_3d(smem + kSmemV + s * 16384, &args.tm_v, bar(kBarV + s), 0, head, seq_row0 + j * kTileN);
        }
      }
      __syncwarp();  // lanes 1-31 wait here for lane 0: the block-wide barrier below must be reached by whole warps
    } else if (warp == kMmaWarp) {
      // ================================================= score MMA issuer ===============================================
      // S = Q.K^T (+ saturated p2c) and the position products of band tiles.  Descriptors are built once; per MMA only the
      // start-address field moves (a 64-bit add), which keeps the single issuing thread short of instructions.
      if (lane == 0) {
        auto wait = [&](uint32_t b, uint32_t parity) {
          if (ok && !mbar_wait_abortable(b, parity, abort_flag)) { ok = false; *abort_flag = 1u; }
        };
        const uint32_t idesc_s = instr_desc(128, 128, G::kFmt, 0, 0);
        const uint32_t idesc_p2c = instr_desc(128, 32, G::kFmt, 0, 0);
        const uint32_t idesc_p2c64 = instr_desc(128, 64, G::kFmt, 0, 0);
        const uint64_t dq = G::desc(smem + kSmemQ, G::kGroup);
        const uint64_t dk0 = G::desc(smem + kSmemK, G::kGroup);
        const uint64_t dwk = G::desc(smem + kSmemWinK, G::kGroup);
        const uint64_t dwq = G::desc(smem + kSmemWinQ, G::kGroup);
        const uint64_t dsat = G::desc(smem + kSmemSat, 0);  // group stride 0: every 8-row group is the same rows
        int band_idx = 0;
        wait(bar(kBarQ), 0);
#pragma unroll 1
        for (int jj = 0; jj < n_proc; ++jj) {
          const int j = j_first + jj;
          const int kind = tile_kind(j);
          const int s = jj & 1;
          const uint64_t dk = dk0 + uint64_t(s) * (16384u >> 4);  // stages are 16 KB apart in either build
          // both softmax groups hold tile j-1 in registers: S and R are free
          if (jj > 0) wait(bar(kBarSFree), uint32_t(jj - 1) & 1u);
          wait(bar(kBarK + s), uint32_t(jj >> 1) & 1u);
          if (kind == kBand) {
            wait(bar(kBarWin), uint32_t(band_idx) & 1u);
            tc_fence_after();
            // Order of issue.  First band tile of the run: c2p (two 128-position blocks) -> R, scores -> S, and once the
            // drain group has emptied R, the p2c products -> R.  Later tiles bring one c2p block, and it goes to the S
            // columns (free until this tile's scores are computed), so the p2c products can be issued into R at once and
            // run while the drain group works; only the four score MMAs wait for the drain.  The same holds for a first
            // band tile that is the CTA's first tile at all (c2p_outside_r).
            const bool first = band_idx == 0;
            if (ok && has_c2p) {
              // c2p[m][p] = Q[m].X_k[p] in 128-position blocks (later tiles reuse the lower half of the previous window
              // from the stage)
              const int nblk = first ? 2 : 1;
#pragma unroll 1
              for (int blk = 0; blk < nblk; ++blk)
#pragma unroll
                for (int ks = 0; ks < G::kSteps; ++ks)
                  G::mma(tmem_base + (!first ? kColS : (c2p_outside_r ? (blk == 0 ? kColS : kColO) : kColR + blk * 128)),
                         dq + uint64_t((ks * 32) >> 4), dwk + uint64_t((blk * G::kTile + ks * 32) >> 4), idesc_s, ks > 0);
            }
            mma_commit(bar(kBarC2p));
            const bool scores_last = !first || c2p_outside_r;  // a c2p block sits in the S columns until it is drained
            if (ok && !scores_last) {
#pragma unroll
              for (int ks = 0; ks < G::kSteps; ++ks)
                G::mma(tmem_base + kColS, dq + uint64_t((ks * 32) >> 4), dk + uint64_t((ks * 32) >> 4), idesc_s, ks > 0);
            }
            if (!scores_last) {
              wait(bar(kBarStage), uint32_t(band_idx) & 1u);  // the drain group has moved the c2p product out of R
              tc_fence_after();
            }
            if (ok && has_p2c) {
              // p2c products.  Key block b (32 keys) needs X_q rows starting at 32(3-b) (t = 0) and 32(4-b) (t = 1); blocks
              // b and b+1 share the start row 32(3-b), so three 128x64 products cover six of the eight (b, t) pairs and
              // two 128x32 products the rest (a narrow MMA costs the tensor pipe about as much as a 64-wide one):
              //   start row 96: keys   0..63  -> R +   0 (b=0,t=0 | b=1,t=1)     start row 128: keys  0..31  -> R + 192 (b=0,t=1)
              //   start row 64: keys  32..95  -> R +  64 (b=1,t=0 | b=2,t=1)     start row   0: keys 96..127 -> R + 224 (b=3,t=0)
              //   start row 32: keys  64..127 -> R + 128 (b=2,t=0 | b=3,t=1)
              const uint64_t blk32 = (32u * G::kRow) >> 4;  // 32 rows of an operand, in descriptor address units
#pragma unroll 1
              for (int q = 0; q < 3; ++q) {
                const uint64_t da = dwq + uint64_t(3 - q) * blk32, db = dk + uint64_t(q) * blk32;
#pragma unroll
                for (int ks = 0; ks < G::kSteps; ++ks)
                  G::mma(tmem_base + kColR + 64 * q, da + uint64_t((ks * 32) >> 4), db + uint64_t((ks * 32) >> 4),
                         idesc_p2c64, ks > 0);
              }
#pragma unroll
              for (int ks = 0; ks < G::kSteps; ++ks)
                G::mma(tmem_base + kColR + 192, dwq + 4 * blk32 + uint64_t((ks * 32) >> 4),
                       dk + uint64_t((ks * 32) >> 4), idesc_p2c, ks > 0);
#pragma unroll
              for (int ks = 0; ks < G::kSteps; ++ks)
                G::mma(tmem_base + kColR + 224, dwq + uint64_t((ks * 32) >> 4),
                       dk + 3 * blk32 + uint64_t((ks * 32) >> 4), idesc_p2c, ks > 0);
            }
            if (scores_last) {
              wait(bar(kBarStage), uint32_t(band_idx) & 1u);  // the drain group has moved the c2p product out of S
              tc_fence_after();
              if (ok) {
#pragma unroll
                for (int ks = 0; ks < G::kSteps; ++ks)
                  G::mma(tmem_base + kColS, dq + uint64_t((ks * 32) >> 4), dk + uint64_t((ks * 32) >> 4), idesc_s, ks > 0);
              }
            }
            ++band_idx;
          } else {
            tc_fence_after();
          }
          if (ok && kind != kBand) {
#pragma unroll
            for (int ks = 0; ks < G::kSteps; ++ks)
              G::mma(tmem_base + kColS, dq + uint64_t((ks * 32) >> 4), dk + uint64_t((ks * 32) >> 4), idesc_s, ks > 0);
            if (has_p2c && (kind == kSatHi || kind == kSatLo)) {
              // bf16: accumulated straight into S.  e4m3: the term has its own scale, so it goes to the (idle) product
              // area and the softmax threads add it with the ratio of the scales.
              const uint64_t ds = dsat + uint64_t(kind == kSatHi ? 0u : (1024u >> 4));
#pragma unroll
              for (int ks = 0; ks < G::kSteps; ++ks)
                G::mma(tmem_base + (F8 ? kColR : kColS), ds + uint64_t((ks * 32) >> 4), dk + uint64_t((ks * 32) >> 4),
                       idesc_s, (F8 ? ks > 0 : 1));
            }
          }
          mma_commit(bar(kBarS));
          mma_commit(bar(kBarKFree + s));
          if (kind == kBand) mma_commit(bar(kBarWinFree));
          FDB_STAMP(2, j, 0);
        }
      }
      __syncwarp();  // as above
    } else if (warp == kPvWarp) {
      // ================================================= P.V MMA issuer =================================================
      if (lane == 0) {
        auto wait = [&](uint32_t b, uint32_t parity) {
          if (ok && !mbar_wait_abortable(b, parity, abort_flag)) { ok = false; *abort_flag = 1u; }
        };
        const uint32_t idesc_pv = instr_desc(128, 64, G::kFmt, 0, 1);
        const uint64_t dv0 = G::desc(smem + kSmemV, G::kGroup);  // V is the MN-major operand: keys run along K
#pragma unroll 1
        for (int jj = 0; jj < n_proc; ++jj) {
          const uint64_t dv = dv0 + uint64_t(jj & 1) * (16384u >> 4);
          wait(bar(kBarV + (jj & 1)), uint32_t(jj >> 1) & 1u);
          wait(bar(kBarP), uint32_t(jj) & 1u);  // both groups have written P
          tc_fence_after();
          FDB_STAMP(2, j_first + jj, 3);
          if (ok) {
#pragma unroll
            for (int ks = 0; ks < G::kPvSteps; ++ks)  // one step = 2048 bytes of V in either build (16 x 128 B, 32 x 64 B)
              G::mma_ts(tmem_base + kColO, tmem_base + kColP + G::kPColsPerStep * ks, dv + uint64_t((ks * 2048) >> 4),
                        idesc_pv, (jj > 0 || ks > 0 || resume) ? 1u : 0u);
          }
          mma_commit(bar(kBarO));
          mma_commit(bar(kBarVFree + (jj & 1)));
          FDB_STAMP(2, j_first + jj, 5);
        }
      }
      __syncwarp();  // as above
    }
  } else {
    // =================================================== softmax groups =================================================
    reg_alloc<kSoftmaxRegs>();
    const int g = warp >> 2;                 // key half
    const int quad = warp & 3;
    const int r = quad * 32 + lane;          // row of the tile
    const uint32_t tmem_lane = tmem_base + (uint32_t(quad * 32) << 16);
    const int my_row = m0 + r;
    auto wait = [&](uint32_t b, uint32_t parity) {  // warp-uniform result
      const bool mine = ok && mbar_wait_abortable(b, parity, abort_flag);
      const bool all = __all_sync(0xffffffffu, mine);
      if (ok && !all) *abort_flag = 1u;
      ok = all;
    };

    wait(bar(kBarQ), 0);
    float rc_lo = 0.f, rc_hi = 0.f;  // saturated c2p terms of this row: Q[m].X_k[first row], Q[m].X_k[last row]
    if (has_c2p && ok) {
      const uint32_t q_row = smem + kSmemQ + uint32_t(r) * G::kRow;
      if constexpr (F8) {
        const uint8_t* xk_h = static_cast<const uint8_t*>(args.xk) + (int64_t)head * args.xrows * kHeadDim;
        rc_lo = ratio_c * dot_q_row_f8(q_row, r, xk_h);
        rc_hi = ratio_c * dot_q_row_f8(q_row, r, xk_h + (int64_t)(args.xrows - 1) * kHeadDim);
      } else {
        const __nv_bfloat16* xk_h = static_cast<const __nv_bfloat16*>(args.xk) + (int64_t)head * args.xrows * kHeadDim;
        rc_lo = dot_q_row(q_row, r, xk_h);
        rc_hi = dot_q_row(q_row, r, xk_h + (int64_t)(args.xrows - 1) * kHeadDim);
      }
    }

    uint32_t band_idx = 0;
    float m_used = 0.f, l_run = 0.f;
    if (resume && ok) {
      // continue from what the far kernel accumulated over the plain and saturated tiles of this row: O goes back into
      // tensor memory (this group's 32 columns), the reference maximum and the row sum into registers
      const int64_t rh = (int64_t)(seq_row0 + (my_row < len ? my_row : len - 1)) * args.heads + head;
      const float4* po = reinterpret_cast<const float4*>(args.part_o + rh * 64 + 32 * g);
      uint32_t o[32];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 v4 = __ldg(po + q);
        o[4 * q + 0] = __float_as_uint(v4.x); o[4 * q + 1] = __float_as_uint(v4.y);
        o[4 * q + 2] = __float_as_uint(v4.z); o[4 * q + 3] = __float_as_uint(v4.w);
      }
      tmem_st32(tmem_lane + kColO + 32 * g, o);
      tmem_wait_st();
      const float2 ml = __ldg(reinterpret_cast<const float2*>(args.part_ml + rh * 2));
      m_used = ml.x;
      l_run = g == 0 ? ml.y : 0.f;
    }

    for (int jj = 0; jj < n_proc; ++jj) {
      const int j = j_first + jj;
      const int n0 = j * kTileN;
      const int kind = tile_kind(j);

      if (lane == 0 && quad == 0) FDB_STAMP(g, j, 0);
      wait(bar(kBarS), uint32_t(jj) & 1u);
      tc_fence_after();
      if (lane == 0 && quad == 0) FDB_STAMP(g, j, 1);

      // ---- this thread's 64 scores (+ p2c through the quadrant shuffle) into registers, then S and R are released ----
      float s[64];
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t a[32];
        if (ok) tmem_ld32(tmem_lane + kColS + 64 * g + 32 * ch, a);
        if (kind == kBand && has_p2c) {
          // key block b = 2g + ch: columns of its two products (see the score-issuing warp)
          const int b = 2 * g + ch;
          const uint32_t c0 = b == 3 ? 224u : 64u * uint32_t(b);
          const uint32_t c1 = b == 0 ? 192u : 64u * uint32_t(b) - 32u;
          if constexpr (F8) {
            // the products 16 columns at a time: the e4m3 build has more live values, and three 32-register runs at once
            // pushed it into spilling
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              uint32_t t0[16], t1[16];
              if (ok) {
                tmem_ld16(tmem_lane + kColR + c0 + 16 * hf, t0);
                tmem_ld16(tmem_lane + kColR + c1 + 16 * hf, t1);
                tmem_wait_ld();  // the first wait also covers the 32 scores
              }
#pragma unroll
              for (int c = 0; c < 16; ++c) {
                const int cc = 16 * hf + c;
                const uint32_t x = (lane + cc <= 30) ? t1[c] : t0[c];
                const uint32_t y = __shfl_sync(0xffffffffu, x, lane + 31 - cc);  // the source lane is taken modulo 32
                s[32 * ch + cc] = fmaf(__uint_as_float(y), ratio_p, __uint_as_float(a[cc]));
              }
            }
          } else {
            uint32_t t0[32], t1[32];
            if (ok) {
              tmem_ld32(tmem_lane + kColR + c0, t0);
              tmem_ld32(tmem_lane + kColR + c1, t1);
              tmem_wait_ld();
            }
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const uint32_t x = (lane + c <= 30) ? t1[c] : t0[c];
              const uint32_t y = __shfl_sync(0xffffffffu, x, lane + 31 - c);  // the source lane is taken modulo 32
              s[32 * ch + c] = fmaf(__uint_as_float(y), ratio_p, __uint_as_float(a[c]));
            }
          }
        } else if (F8 && has_p2c && (kind == kSatHi || kind == kSatLo)) {
          // e4m3: the saturated p2c term of these keys sits in the product area (same value in every row)
          uint32_t t0[32];
          if (ok) {
            tmem_ld32(tmem_lane + kColR + 64 * g + 32 * ch, t0);
            tmem_wait_ld();
          }
#pragma unroll
          for (int c = 0; c < 32; ++c) s[32 * ch + c] = fmaf(__uint_as_float(t0[c]), ratio_p, __uint_as_float(a[c]));
        } else {
          if (ok) tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) s[32 * ch + c] = __uint_as_float(a[c]);
        }
      }
      tc_fence_before();
      mbar_arrive(bar(kBarSFree));
      if (lane == 0 && quad == 0) FDB_STAMP(g, j, 2);

      float row_const = 0.f;
      if (kind == kBand) {
        wait(bar(kBarStage), band_idx & 1u);  // the c2p stage of this tile is complete
        if (has_c2p) {
          // c2p[m][i] is position p = m + 127 - i of the window, stored in column ((p ^ flip) - m) & 255 of row m (see the
          // drain group): for this thread's keys i = 64g .. 64g+63 that is the aligned run of 64 columns ending at
          // 127 - 64g (+ 128 when flipped), read with eight 16-byte loads, key i in column (run start) + 63 - (i - 64g).
          const uint32_t run = smem + kSmemStageC + uint32_t(r) * kStageCPitch +
                               2u * (uint32_t(64 * (1 - g)) + ((band_idx & 1u) ? 128u : 0u));
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint4 w4 = lds_v4(run + 16u * uint32_t(q));
            const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {  // column 8q + e of the run -> key 63 - (8q + e)
              const uint32_t bits = (e & 1) ? (w[e >> 1] & 0xffff0000u) : (w[e >> 1] << 16);
              s[63 - (8 * q + e)] = fmaf(__uint_as_float(bits), ratio_c, s[63 - (8 * q + e)]);
            }
          }
        }
        mbar_arrive(bar(kBarGather));
        ++band_idx;
      } else if (kind == kSatHi) {
        row_const = rc_hi;
      } else if (kind == kSatLo) {
        row_const = rc_lo;
      }
      if (n0 + kTileN > len) {  // keys past the end of the sequence
        const int valid = len - n0 - 64 * g;
#pragma unroll
        for (int i = 0; i < 64; ++i) s[i] = i < valid ? s[i] : -INFINITY;
      }
      float mx4[4] = {max3(s[0], s[4], s[8]), max3(s[1], s[5], s[9]), max3(s[2], s[6], s[10]), max3(s[3], s[7], s[11])};
#pragma unroll
      for (int i = 12; i < 60; i += 8)
#pragma unroll
        for (int q = 0; q < 4; ++q) mx4[q] = max3(mx4[q], s[i + q], s[i + 4 + q]);
#pragma unroll
      for (int q = 0; q < 4; ++q) mx4[q] = fmaxf(mx4[q], s[60 + q]);
      float mx = max3(mx4[0], mx4[1], fmaxf(mx4[2], mx4[3]));
      // the two threads of a row agree on the row maximum
      const uint32_t xch = smem + kSmemXchg + uint32_t(jj & 1) * 1024u;
      sts_f32(xch + uint32_t(g) * 512u + uint32_t(r) * 4u, mx);
      if (lane == 0 && quad == 0) FDB_STAMP(g, j, 3);
      bar_sync(1, kSoftmaxThreads);
      if (lane == 0 && quad == 0) FDB_STAMP(g, j, 4);
      mx = fmaxf(mx, lds_f32(xch + uint32_t(g ^ 1) * 512u + uint32_t(r) * 4u));

      const float t_max = (mx + row_const) * c_eff;
      if (jj == 0 && !resume) {
        m_used = t_max;
      } else {
        // The previous P.V has finished: O may be rescaled and the P columns overwritten.  Observed on every tile (it is
        // long done by now) so that this thread never falls two phases behind the barrier, which a parity wait could
        // not tell apart.
        if (jj > 0) wait(bar(kBarO), uint32_t(jj - 1) & 1u);
        tc_fence_after();
        // bf16: O is rescaled only when the maximum moved by more than 2^8 (P <= 256 is harmless in bf16).
        // e4m3: P is stored as 2^8 * exp2(.), so it has to stay <= 1: rescale whenever the maximum moves.
        const bool need = t_max > m_used + (F8 ? 0.f : 8.f);
        if (__any_sync(0xffffffffu, need)) {  // warp-uniform, and the same in both groups: rescale O of these 32 rows
          const float m_new = fmaxf(m_used, t_max);
          const float alpha = ex2(m_used - m_new);
          l_run *= alpha;
          m_used = m_new;
          if (ok) {
            uint32_t o[32];
            tmem_ld32(tmem_lane + kColO + 32 * g, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(tmem_lane + kColO + 32 * g, o);
            tmem_wait_st();
          }
        }
      }
      if (lane == 0 && quad == 0) FDB_STAMP(g, j, 5);
      const float off = row_const * c_eff - m_used + (F8 ? 8.f : 0.f);
      if constexpr (F8) {
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          s[i] = ex2(fmaf(s[i], c_eff, off));
          l4[i & 3] += s[i];
        }
        l_run += (l4[0] + l4[1]) + (l4[2] + l4[3]);
        if (lane == 0 && quad == 0) FDB_STAMP(g, j, 6);
        if (ok) {  // 16 columns of e4m3 quadruples
          uint32_t p[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) p[i] = pack_e4m3x4(s[4 * i], s[4 * i + 1], s[4 * i + 2], s[4 * i + 3]);
          tmem_st16(tmem_lane + kColP + 16 * g, p);
          tmem_wait_st();
        }
      } else {
        // p = 2^(s * scale + off) with the two-wide fp32 forms; the bf16 pairs of the first 32 keys are on their way to
        // tensor memory while the other 32 are computed
        const uint64_t scale2 = pack_f32x2(c_eff, c_eff), off2 = pack_f32x2(off, off);
        uint64_t l2[2] = {0ull, 0ull};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t p[16];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float e0, e1, e2, e3;
            unpack_f32x2(fma_f32x2(pack_f32x2(s[32 * h + i], s[32 * h + i + 1]), scale2, off2), e0, e1);
            unpack_f32x2(fma_f32x2(pack_f32x2(s[32 * h + i + 2], s[32 * h + i + 3]), scale2, off2), e2, e3);
            e0 = ex2(e0); e1 = ex2(e1); e2 = ex2(e2); e3 = ex2(e3);
            l2[0] = add_f32x2(l2[0], pack_f32x2(e0, e1));
            l2[1] = add_f32x2(l2[1], pack_f32x2(e2, e3));
            p[i >> 1] = pack_bf16x2(e0, e1);
            p[(i >> 1) + 1] = pack_bf16x2(e2, e3);
          }
          if (ok) tmem_st16(tmem_lane + kColP + 32 * g + 16 * h, p);
        }
        float s0, s1, s2, s3;
        unpack_f32x2(l2[0], s0, s1);
        unpack_f32x2(l2[1], s2, s3);
        l_run += (s0 + s1) + (s2 + s3);
        if (lane == 0 && quad == 0) FDB_STAMP(g, j, 6);
        tmem_wait_st();
      }
      tc_fence_before();
      mbar_arrive(bar(kBarP));
      if (lane == 0 && quad == 0) FDB_STAMP(g, j, 7);
    }

    // ---- epilogue: combine the two row sums, O / l, write this group's 32 output columns ----
    sts_f32(smem + kSmemLsum + uint32_t(g) * 512u + uint32_t(r) * 4u, l_run);
    bar_sync(1, kSoftmaxThreads);
    const float l_tot = l_run + lds_f32(smem + kSmemLsum + uint32_t(g ^ 1) * 512u + uint32_t(r) * 4u);
    wait(bar(kBarO), uint32_t(n_proc - 1) & 1u);
    tc_fence_after();
    if (ok) {
      const bool valid = my_row < len;
      const bool pad = !valid && my_row < row_limit;  // dense padding rows inside a partly valid tile get zeros
      const float inv = valid ? v_scale / l_tot : 0.f;
      uint32_t o[32];
      tmem_ld32(tmem_lane + kColO + 32 * g, o);  // whole warps execute this, whatever their rows
      tmem_wait_ld();
      if (valid || pad) {
        uint4* o4 = reinterpret_cast<uint4*>(args.out + (int64_t)(seq_row0 + my_row) * args.o_rs +
                                             (int64_t)head * args.o_hs + 32 * g);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 v = make_uint4(0, 0, 0, 0);
          if (valid)
            v = make_uint4(pack_bf16x2(__uint_as_float(o[q4 * 8 + 0]) * inv, __uint_as_float(o[q4 * 8 + 1]) * inv),
                           pack_bf16x2(__uint_as_float(o[q4 * 8 + 2]) * inv, __uint_as_float(o[q4 * 8 + 3]) * inv),
                           pack_bf16x2(__uint_as_float(o[q4 * 8 + 4]) * inv, __uint_as_float(o[q4 * 8 + 5]) * inv),
                           pack_bf16x2(__uint_as_float(o[q4 * 8 + 6]) * inv, __uint_as_float(o[q4 * 8 + 7]) * inv));
          o4[q4] = v;
        }
        if (g == 0 && args.lse != nullptr)
          args.lse[(int64_t)(seq_row0 + my_row) * args.heads + head] =
              valid ? (m_used + log2f(l_tot) - (F8 ? 8.f : 0.f)) * 0.6931471805599453f : 0.f;
      }
    }
  }

  // ---- teardown -------------------------------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (tid == 0 && args.status != nullptr) atomicOr(reinterpret_cast<unsigned int*>(args.status), FDB_DEV_TIMEOUT);
    // give copies and MMAs that may still be in flight a bounded time to land before TMEM and shared memory go away
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == kMmaWarp) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace

int launch_attn_fwd_sm100(const fdb_attn_params& p, const ExpandGeometry& g, const WorkspaceLayout& w, void* stream) {
  const bool f8 = p.dtype == FDB_E4M3;
  FwdArgs a;
  char* ws = static_cast<char*>(p.workspace);
  int rc;
  if ((rc = make_map_rows(&a.tm_q, p.q, p.total_rows, p.heads, p.q_row_stride, p.q_head_stride, kTileM, f8, "q"))) return rc;
  if ((rc = make_map_rows(&a.tm_k, p.k, p.total_rows, p.heads, p.k_row_stride, p.k_head_stride, kTileN, f8, "k"))) return rc;
  if ((rc = make_map_rows(&a.tm_v, p.v, p.total_rows, p.heads, p.v_row_stride, p.v_head_stride, kTileN, f8, "v"))) return rc;
  a.xk = p.pos_key ? ws + w.exp_key : nullptr;
  a.xq = p.pos_query ? ws + w.exp_query : nullptr;
  a.q_scale = p.q_scale; a.k_scale = p.k_scale; a.v_scale = p.v_scale;
  a.xk_scale = p.pos_key_scale; a.xq_scale = p.pos_query_scale;
  // a map is always encoded so the kernel argument is well formed; an unused one points at q
  if (a.xk) { if ((rc = make_map_table(&a.tm_xk, a.xk, g.rows, p.heads, f8, "expanded pos_key"))) return rc; } else a.tm_xk = a.tm_q;
  if (a.xq) { if ((rc = make_map_table(&a.tm_xq, a.xq, g.rows, p.heads, f8, "expanded pos_query"))) return rc; } else a.tm_xq = a.tm_q;
  if (a.xq) { if ((rc = make_map_table(&a.tm_xq_sat, a.xq, g.rows, p.heads, f8, "saturated pos_query rows", 8))) return rc; } else a.tm_xq_sat = a.tm_q;
  a.out = static_cast<__nv_bfloat16*>(p.out);
  a.o_rs = p.out_row_stride; a.o_hs = p.out_head_stride;
  a.seq_info = reinterpret_cast<const int32_t*>(ws + w.seq_info);
  a.tile_first = reinterpret_cast<const int32_t*>(ws + w.tile_first);
  a.slot_info = reinterpret_cast<const int4*>(ws + w.slot_info);
  a.lse = p.lse; a.status = p.status;
  a.batch = p.batch; a.heads = p.heads; a.packed = p.cu_seqlens != nullptr; a.max_seqlen = p.max_seqlen;
  a.sat_lo = g.sat_lo; a.sat_hi = g.sat_hi; a.d_first = g.d_first; a.xrows = g.rows;
  a.scale_log2 = p.sm_scale * 1.4426950408889634f;
  a.part_o = w.split ? reinterpret_cast<float*>(ws + w.part_o) : nullptr;
  a.part_ml = w.split ? reinterpret_cast<float*>(ws + w.part_ml) : nullptr;
  a.band_only = w.split ? 1 : 0;
  a.split_len = (p.tune & FDB_TUNE_TWO_LAUNCHES) ? 0 : kSplitSeqlen;  // forced two launches: every sequence is split
#ifdef FDB_TRACE
  a.trace = trace_buffer_from_env();
#endif

  const int64_t slots = tile_slots(p);
  a.slots = (int)slots;
  if (slots <= 0) return FDB_OK;
  if (slots > 2147483647LL || p.heads > 65535) return fail(FDB_ERR_LIMIT, "grid too large");

  // bf16: key tiles with saturated (or no) position terms go to the far kernel (half an SM per CTA, two CTAs per SM); with
  // position terms the band tiles follow in attn_fwd_kernel, which picks up the partial result on the same stream.
  const bool no_pos = a.xk == nullptr && a.xq == nullptr;
  if (!f8 && (w.split || (no_pos && !(p.tune & FDB_TUNE_ONE_LAUNCH)))) {
    rc = launch_attn_fwd_far1(&a, slots, p.heads, stream);
    if (rc != FDB_OK) return rc;
    if (no_pos) return FDB_OK;
  }

  auto kernel = f8 ? attn_fwd_kernel<true> : attn_fwd_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  kernel<<<dim3((unsigned)slots, p.heads), kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "attn_fwd launch: %s", cudaGetErrorString(e));
  return FDB_OK;
}

}  // namespace fdb
