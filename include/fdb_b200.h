/*
 * fdb_b200.h — C ABI of libfdb_b200.so: DeBERTa-v2/v3 disentangled self-attention forward for
 * NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain pointers and sizes; no libtorch type crosses this boundary.  The caller
 * owns every buffer (inputs, outputs, workspace, status word); the library allocates no device memory
 * unless an entry point's comment says otherwise.  Functions return 0 (FDB_OK) or a negative fdb_status
 * code; fdb_last_error() gives the text of the calling thread's last failure.  Nothing is launched when
 * an argument check fails.
 *
 * The "reference" cited below is Knowledgator/FlashDeBERTa 0.0.5 (paths relative to its root) and, where
 * marked HF, transformers' models/deberta_v2/modeling_deberta_v2.py, which the reference subclasses.
 */
#ifndef FDB_B200_H_
#define FDB_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FDB_ABI_VERSION 4

#if defined(__GNUC__)
#define FDB_API __attribute__((visibility("default")))
#else
#define FDB_API
#endif

typedef enum fdb_status {
  FDB_OK = 0,
  FDB_ERR_INVALID_ARGUMENT = -1, /* NULL where a pointer is required, bad size, bad enum */
  FDB_ERR_UNSUPPORTED = -2,      /* valid in the reference, not built here (e.g. head_dim != 64 in the fused kernel) */
  FDB_ERR_ALIGNMENT = -3,        /* pointer or stride not 16-byte aligned */
  FDB_ERR_WORKSPACE = -4,        /* workspace missing or too small */
  FDB_ERR_CUDA = -5,             /* a CUDA runtime/driver call failed; see fdb_last_error() */
  FDB_ERR_LIMIT = -6             /* size above a stated fixed maximum */
} fdb_status;

typedef enum fdb_dtype {
  FDB_BF16 = 0,
  FDB_FP32 = 1, /* check kernel only */
  FDB_E4M3 = 2  /* fused kernel, per-head scales */
} fdb_dtype;

/* Bits of the device status word written by kernels (0 = no anomaly). */
#define FDB_DEV_TIMEOUT 1u      /* a bounded wait inside a kernel ran out; the output is invalid */
#define FDB_DEV_BAD_SEQLEN 2u   /* cu_seqlens not monotone / a length below zero or above max_seqlen */
#define FDB_DEV_BAD_INDEX 4u    /* fdb_embed_layernorm met an id outside the table (the row was taken from its edge) */
#define FDB_DEV_BAD_MASK 8u     /* reserved for callers: the Python layer sets it when a dense attention mask on the device is
                                   not a right-padded prefix (dense rows are addressed by length alone) */

/*
 * One attention call.  Replaces, in one launch sequence, what the reference does in
 *   src/flashdeberta/model.py:185-204 (fixed length) and :206-249 (packed),
 *   src/flashdeberta/ops/flash_attention.py:1088-1091 -> :421-488 -> kernel :146-300,
 *   src/flashdeberta/ops/flash_attention_varlen.py:485-511 -> :349-440 -> kernel :85-225,
 * including the two bias GEMMs (model.py:189-192, :210-214) that the reference leaves to cuBLAS.
 *
 * Tensors are addressed as element (row, head, d) = base + row*row_stride + head*head_stride + d, strides in
 * ELEMENTS, d contiguous.  "row" counts tokens over the whole batch:
 *   dense  (cu_seqlens == NULL): sequence b owns rows [b*max_seqlen, b*max_seqlen + len_b),
 *                                len_b = seq_lens ? seq_lens[b] : max_seqlen   (right padding)
 *   packed (cu_seqlens != NULL): sequence b owns rows [cu_seqlens[b], cu_seqlens[b+1]).
 * Output rows that belong to no sequence (dense padding) are written as zeros, as
 * src/flashdeberta/padding.py:30-44 does.  Padding rows of v must hold finite numbers.
 */
typedef struct fdb_attn_params {
  uint32_t struct_bytes; /* sizeof(fdb_attn_params), checked */
  int32_t dtype;         /* fdb_dtype of q, k, v, pos_key, pos_query; out is bf16 (fp32 for FDB_FP32) */

  const void* q;
  const void* k;
  const void* v;
  void* out;
  int64_t q_row_stride, q_head_stride;
  int64_t k_row_stride, k_head_stride;
  int64_t v_row_stride, v_head_stride;
  int64_t out_row_stride, out_head_stride;

  /* Projected relative-position tables, (heads, 2*att_span, head_dim) contiguous, i.e. pos_key_layer and
   * pos_query_layer of model.py:159-177 in head-major order.  NULL switches the term off
   * (c2p needs pos_key, p2c needs pos_query). */
  const void* pos_key;
  const void* pos_query;

  const int32_t* cu_seqlens; /* device, batch+1 entries, or NULL */
  const int32_t* seq_lens;   /* device, batch entries, or NULL (dense only) */

  int32_t batch;
  int32_t max_seqlen; /* dense: padded length L.  packed: an upper bound on every length */
  int32_t total_rows; /* number of rows addressable in q/k/v/out (dense: batch*max_seqlen) */
  int32_t heads;
  int32_t head_dim;

  /* position_buckets / max_relative_positions as in HF:168-174; att_span = buckets > 0 ? buckets : max_rel */
  int32_t position_buckets;
  int32_t max_relative_positions;

  /* Device copy of the table made by fdb_build_bucket_lut (int16, lut_len entries); entry i is the table row for
   * relative distance d = lut_d_min + i; distances outside use the first / last entry. */
  const int16_t* bucket_lut;
  int32_t lut_d_min;
  int32_t lut_len;

  float sm_scale; /* 1/sqrt(head_dim * (1 + [c2p] + [p2c])), model.py:151-157 */

  /* FDB_E4M3 only: device float arrays, value = stored * scale.  q/k/v scales have batch*heads entries
   * (sequence-major), table scales have `heads` entries. */
  const float* q_scale;
  const float* k_scale;
  const float* v_scale;
  const float* pos_key_scale;
  const float* pos_query_scale;

  float* lse; /* optional, (total_rows, heads) fp32 natural-log LSE as flash_attention.py:293 */

  void* workspace; /* device, >= fdb_attn_workspace_bytes(), 256-byte aligned */
  uint64_t workspace_bytes;

  int32_t* status; /* device int32, OR-ed with FDB_DEV_* bits; may be NULL */

  /* FDB_PREPARED_* bits (fdb_attn_fwd only): what the workspace still holds from an earlier fdb_attn_fwd call on it, so
   * that the set-up kernel that writes it is not launched again.  FDB_PREPARED_SCHEDULE: the per-sequence rows and the
   * order of the query tiles — valid while batch, max_seqlen, total_rows and the contents of cu_seqlens / seq_lens are
   * the same.  FDB_PREPARED_TABLES: the position tables gathered through the bucket index — valid while pos_key,
   * pos_query (pointers and contents), heads, dtype and the bucket settings are the same.  Both also need the same
   * workspace size as the call that wrote them (same fdb_attn_workspace_bytes), and nothing else may have used the
   * workspace in between.  The reference recomputes both for every layer of every forward (the tile map in a host loop,
   * flash_attention_varlen.py:71-83; the index arithmetic per score element, flash_attention.py:236-254).  0: nothing
   * is assumed. */
  uint32_t prepared;

  /* FDB_TUNE_* bits: overrides of choices the library otherwise makes from the shapes (which kernels a call is split
   * into).  The result is the same either way; they exist so that a test or a tuning run can reach every kernel at any
   * size.  0: the library chooses. */
  uint32_t tune;
} fdb_attn_params;

#define FDB_PREPARED_SCHEDULE 1u
#define FDB_PREPARED_TABLES 2u

#define FDB_TUNE_ONE_LAUNCH 1u     /* every key tile in the fused kernel, whatever the length */
#define FDB_TUNE_TWO_LAUNCHES 2u   /* far key tiles in the far kernel first, band tiles after (bf16 with position terms) */

/* Library / ABI version (FDB_ABI_VERSION the library was built with). */
FDB_API int fdb_abi_version(void);

/* Text of the calling thread's most recent error ("" if none). */
FDB_API const char* fdb_last_error(void);

/* Text for an fdb_status code. */
FDB_API const char* fdb_status_string(int code);

/*
 * Host-side integer table for the log-bucket relative index: replaces the per-score-element float math at
 * src/flashdeberta/ops/flash_attention.py:236-254 and HF:56-69 + the clamp at HF:318/:336.
 * Writes into out[0..*len) the table row for every distance d in [*d_min, *d_min + *len); the first and last
 * entries are the saturated values that hold for every distance beyond.  Pass out == NULL to query *len and
 * *d_min only.  capacity = entries available in out.
 */
FDB_API int fdb_build_bucket_lut(int32_t position_buckets, int32_t max_relative_positions, int16_t* out, int32_t capacity,
                         int32_t* d_min, int32_t* len);

/* Single distance -> table row, same arithmetic as fdb_build_bucket_lut (host). */
FDB_API int32_t fdb_relative_index(int32_t position_buckets, int32_t max_relative_positions, int64_t distance);

/* Bytes of device workspace fdb_attn_fwd needs for these parameters (0 on invalid parameters, see fdb_last_error). */
FDB_API uint64_t fdb_attn_workspace_bytes(const fdb_attn_params* p);

/*
 * Fused forward: tcgen05/TMEM tensor-core kernel fed by TMA.  bf16 or e4m3 inputs, head_dim 64.
 * Launches on `stream` (a cudaStream_t passed as void*); returns without synchronising.
 * Replaces flash_attention_with_disentangled (flash_attention.py:1088) and its varlen twin
 * (flash_attention_varlen.py:485), plus model.py:189-192/:210-214.
 */
FDB_API int fdb_attn_fwd(const fdb_attn_params* p, void* stream);

/*
 * fdb_attn_fwd for callers that cannot give it a workspace.  (No counterpart in the reference: its launchers
 * allocate through torch on every call.)
 *
 * Some hosts of this library have no way to allocate device memory at the point where they call it: an inference
 * server that handed the whole GPU to its own arena at start-up, a plug-in running inside someone else's stream
 * callback or latency-critical loop where cudaMalloc/cudaFree (which synchronise the device) are forbidden, or a
 * C host that simply has no allocator wired to this GPU.  For them this entry point keeps the scratch that
 * fdb_attn_fwd needs (sequence table, tile prefix, the two expanded position tables) in a fixed array that lives
 * inside the library image on the device: FDB_STATIC_SCRATCH_BYTES per GPU that loads the library, held until the
 * process exits.  p->workspace and p->workspace_bytes are ignored; inputs, output and the status word are still the
 * caller's.  It calls no cudaMalloc, cudaFree or any other allocating routine.
 *
 * Limits and rules:
 *  - this entry point always runs the call as one launch of the fused kernel, so its scratch need is the sequence table,
 *    the tile order and the two gathered tables only: what fdb_attn_workspace_bytes reports with FDB_TUNE_ONE_LAUNCH set
 *    in p->tune (without that bit the query adds, from 3584 keys, the partial-result buffers of the two-launch form, which
 *    are not used here).  Parameters that need more than FDB_STATIC_SCRATCH_BYTES are refused with FDB_ERR_LIMIT and
 *    nothing is launched (DeBERTa-v3 geometry: up to 16 heads and tens of thousands of sequences fit);
 *  - the first call on each device looks the array's device address up once (with that device current); make that
 *    first call outside any stream capture;
 *  - every call on a device uses the same array and leaves its contents behind.  The kernels rewrite every byte
 *    they later read, so nothing has to be cleared between calls, but two calls that overlap on the GPU (different
 *    streams, or different host threads without ordering) race on it: keep calls on one device ordered;
 *  - the looked-up address is kept for the life of the process.  cudaDeviceReset() on a device that has already made a
 *    call leaves that address dangling: do not reset a device between calls to this entry point.
 */
#define FDB_STATIC_SCRATCH_BYTES (8u << 20)
FDB_API int fdb_attn_fwd_static(const fdb_attn_params* p, void* stream);

/*
 * Backward pass, the two steps that are not plain GEMMs.  The reference's backward is three Triton kernels
 * (src/flashdeberta/ops/flash_attention.py:581-614 preprocess, :616-797 dK / dV with the position-bias gradients
 * scattered by atomics at :770-786, :799-940 dQ, launcher :942-1030).  Here the host walks a group of sequences in
 * blocks of query rows; the contractions (Q.K^T, dO.V^T, Q.pos_key^T, K.pos_query^T and every product with P or dS)
 * are the caller's GEMMs, and the two entry points below do what lies between them.  All tensors contiguous, on the
 * device; "group" = (sequence, head), sequence = group / heads; a block holds rows [row0, row0 + rows) of every group.
 */
typedef struct fdb_bwd_block {
  uint32_t struct_bytes;       /* sizeof(fdb_bwd_block) */
  int32_t groups;              /* sequences x heads (at most 65535) */
  int32_t heads;
  int32_t seqlen;              /* padded length: keys per group, row pitch of the score-shaped tensors */
  int32_t row0, rows;          /* the block's query rows */
  int32_t table_rows;          /* 2*att_span rows of the position tables; 0 = no position terms */
  int32_t lut_d_min, lut_len;  /* bucket table as in fdb_attn_params */
  float sm_scale;
  const int32_t* seq_lens;     /* (sequences) valid lengths, right padding; NULL = every sequence full */
  const int16_t* lut;
  const float* scores;         /* (groups, rows, seqlen)  Q.K^T, unscaled */
  const float* dprobs;         /* (groups, rows, seqlen)  dO.V^T */
  const float* c2p;            /* (groups, rows, table_rows)  Q.pos_key^T, or NULL */
  const float* p2c;            /* (groups, seqlen, table_rows)  K.pos_query^T, or NULL */
  const float* lse;            /* (groups, rows) natural-log LSE of the forward */
  const float* delta;          /* (groups, rows) sum over the head dimension of dO * O */
  void* probs;                 /* out, bf16 (groups, rows, seqlen): P; zero outside the valid lengths */
  void* dscores;               /* bf16 (groups, rows, seqlen): sm_scale * P * (dP - delta); written by fdb_attn_bwd_probs,
                                  read by fdb_attn_bwd_bucket_sums */
  float* c2p_sums;             /* out (groups, rows, table_rows): per query row, dscores summed over the keys that
                                  address each table row; or NULL */
  float* p2c_sums;             /* in/out (groups, seqlen, table_rows): per key, the same over this block's query rows,
                                  ADDED to what is there (zero it before the first block); or NULL */
  int32_t* status;             /* reserved (may be NULL) */
} fdb_bwd_block;

/* P = exp(sm_scale * (scores + c2p[m][idx(m-n)] + p2c[n][idx(m-n)]) - lse) and dscores of one block. */
FDB_API int fdb_attn_bwd_probs(const fdb_bwd_block* p, void* stream);
/* c2p_sums and / or p2c_sums of one block from its dscores (whichever pointers are set).  No global atomics: the index is
 * non-decreasing in the distance, so the scores that share a table row are one run of keys (of query rows).
 * table_rows at most 8192;
 * 64 * (table_rows + 2) + 2 * (rows + 16) bytes of shared memory, at most 200 KB (FDB_ERR_LIMIT). */
FDB_API int fdb_attn_bwd_bucket_sums(const fdb_bwd_block* p, void* stream);

/*
 * Check kernel: the same contract computed with fp32 arithmetic on CUDA cores, one warp per (row, head), no
 * tensor cores, bucket index looked up per element from bucket_lut.  bf16 or fp32 inputs, head_dim <= 128.
 * Needs no workspace.  For validation, never for speed.
 */
FDB_API int fdb_attn_fwd_check(const fdb_attn_params* p, void* stream);

/*
 * Device dump of the relative index the kernels use: out[m*len_k + n] = row for distance (m - n), m < len_q,
 * n < len_k, via the same device lookup as the attention kernels.  For the bit-exactness test against
 * HF:72-101 + :318.
 */
FDB_API int fdb_relative_index_matrix(const int16_t* bucket_lut, int32_t lut_d_min, int32_t lut_len, int32_t len_q,
                              int32_t len_k, int32_t* out, void* stream);

/*
 * Per-slab amax scaling to e4m3 (no counterpart in the reference; the FP8 option of this library).
 * x is (rows, heads, head_dim) strided like q; slab s covers rows [slab_start[s], slab_start[s+1]) of one head
 * (slab_start device int32, n_slabs+1 entries; pass the cu_seqlens array); slab bounds are clamped to [0, rows).
 * Writes y (e4m3, contiguous (rows, heads, head_dim)) and scale[s*heads + h] = amax/448.
 * x must be 16-byte aligned, y 8-byte aligned, the strides positive multiples of 8 elements (FDB_ERR_ALIGNMENT).
 */
FDB_API int fdb_quantize_e4m3(const void* x_bf16, int64_t rows, int64_t row_stride, int64_t head_stride,
                      const int32_t* slab_start, int32_t n_slabs, int32_t heads, int32_t head_dim, void* y_e4m3,
                      float* scale, void* stream);

/*
 * out = LayerNorm(x + residual) over the last dimension (eps inside the square root), bf16 in and out, fp32 statistics; the
 * sum is rounded to bf16 first, as the eager expression does.  Replaces the tail of both output blocks of a layer, which
 * the reference inherits from transformers: DebertaV2SelfOutput / DebertaV2Output `LayerNorm(dropout(dense(h)) + input)`
 * behind FlashDebertaV2Attention / FlashDebertaV2Layer (src/flashdeberta/model.py:259-272) — there an elementwise add
 * and a layer-norm kernel, here one pass.  x, residual (may be NULL: plain LayerNorm), out: (rows, hidden) contiguous;
 * gamma, beta: (hidden) bf16; hidden a multiple of 256 up to 2048; every pointer 16-byte aligned.
 */
FDB_API int fdb_add_layernorm(const void* x, const void* residual, const void* gamma, const void* beta, void* out,
                              int64_t rows, int32_t hidden, float eps, void* stream);

/*
 * out[r] = LayerNorm(table[ids[r]]) * row_scale[r]: the embedding stage of the model when the input is word embeddings
 * alone (DeBERTa-v3: position_biased_input off, no token types, no projection).  The reference inherits the stage from
 * transformers (DebertaV2Embeddings inside FlashDebertaV2Model, src/flashdeberta/model.py:394-428): an embedding gather, a
 * zero tensor for the absent position term, a layer norm and a multiplication by the mask — four kernels and seven passes
 * over the (rows, hidden) activation, here one kernel and two.  ids: device int64, rows entries; table: (table_rows,
 * hidden) bf16 contiguous; row_scale: device fp32, rows entries, or NULL; the normalised value is rounded to bf16 before
 * it is scaled.  hidden a multiple of 256 up to 2048.  An id outside [0, table_rows) sets FDB_DEV_BAD_INDEX in *status
 * (may be NULL) and reads the nearest edge of the table.
 */
FDB_API int fdb_embed_layernorm(const int64_t* ids, const void* table, int64_t table_rows, const void* gamma,
                                const void* beta, const float* row_scale, void* out, int64_t rows, int32_t hidden,
                                float eps, int32_t* status, void* stream);

/*
 * out = GELU(x . weight^T + bias), erf form, bf16 in and out, fp32 accumulation in tensor memory; the sum is rounded to bf16
 * before the activation, as the separate GEMM would leave it.  Replaces the intermediate block of an encoder layer, which
 * the reference inherits from transformers (DebertaV2Intermediate: dense + ACT2FN["gelu"], inside FlashDebertaV2Layer,
 * src/flashdeberta/model.py:265-272) — there a GEMM and an elementwise kernel with the (rows, out_features) activation
 * written and read back in between, here one kernel.  x: (rows, in_features) contiguous; weight: (out_features,
 * in_features) contiguous, the layout of torch.nn.Linear; bias: (out_features) or NULL; out: (rows, out_features).
 * in_features a multiple of 64, out_features a multiple of 256, every pointer 16-byte aligned.  status: device word that
 * receives FDB_DEV_TIMEOUT if a wait inside the kernel gives up (may be NULL).
 */
FDB_API int fdb_linear_gelu(const void* x, const void* weight, const void* bias, void* out, int64_t rows,
                            int32_t in_features, int32_t out_features, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FDB_B200_H_ */
