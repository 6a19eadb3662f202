/*
 * compactattn_b200 — C ABI of the B200 (sm_100a) CompactAttention chunked-prefill path.
 *
 * Every entry point takes raw device pointers, element strides and a CUDA stream, enqueues its
 * kernels on that stream and returns immediately: 0 on success, a negative CA_ERR_* code
 * otherwise, with a human-readable reason available from ca_last_error() (thread-local).
 * Unless a function says otherwise it never allocates, never synchronises and never exits.
 * The caller owns every buffer.
 *
 * Citations name the interface of the reference project (jiwonsong-dev/CompactAttention,
 * paths relative to its root) that each entry point stands in for.
 *
 * Vocabulary: B batch, Q chunk tokens, K kv_len (chunk included), P = K - Q past tokens,
 * bs block size, Qb = Q/bs, Kb = K/bs, Pb = P/bs, Hq / Hkv heads, G = Hq/Hkv, D = 128,
 * rows R = B*Hkv (row = b*Hkv + hkv).
 */
#ifndef COMPACTATTN_B200_H_
#define COMPACTATTN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CA_OK 0
#define CA_ERR_INVALID (-1)     /* contract violation (shape, alignment, null pointer) */
#define CA_ERR_UNSUPPORTED (-2) /* valid request this build does not implement */
#define CA_ERR_CUDA (-3)        /* a CUDA runtime/driver call failed */
#define CA_ERR_CAPACITY (-4)    /* a caller-provided buffer is too small */

/* Data types of Q/K/V/O tensors. */
#define CA_DTYPE_BF16 0
#define CA_DTYPE_F16 1
#define CA_DTYPE_F32 2

/* Bits a kernel may set in a caller-provided int32 status word (device memory). */
#define CA_STATUS_TIMEOUT 1   /* a bounded device-side wait expired; output is invalid */
#define CA_STATUS_BAD_INDEX 2 /* a block-table entry or count was out of range and was clamped */

typedef void* ca_stream_t; /* cudaStream_t */

const char* ca_last_error(void);
/* ABI version; bumped when a struct below changes (2: ca_select_params.threshold_ptr). */
int ca_abi_version(void);
/* Number of kernel launches the library has enqueued in this process (all entry points). */
int64_t ca_launch_count(void);
/*
 * Programmatic dependent launch (off by default): when enabled, every kernel is enqueued so that
 * its CTAs may become resident and run their prologue while the previous kernel in the stream
 * drains; each kernel waits (griddepcontrol.wait) before its first global-memory access, so
 * results do not change.  Measured on B200: the selection chain gains 2-3 us per step, the long
 * attention launch gains nothing, so plain launches stay the default.  Returns the previous
 * setting.  No reference counterpart (the reference launches through torch / Triton).
 */
int ca_set_programmatic_launch(int enabled);

/*
 * Source KV cache addressing. A "page" is page_size consecutive tokens of all heads of one
 * sequence; element address of (page p, token t, head h, dim d) =
 *   base + p*page_stride + t*token_stride + h*head_stride + d.
 * A contiguous [B,K,Hkv,D] cache (the reference's key_states layout,
 * compact_attn/modules/attention_forward_chunked_dense.py:2733-2735) is page_size=64,
 * pages_per_seq=K/64, page_stride=64*Hkv*D, token_stride=Hkv*D, head_stride=D, page_table=NULL.
 * A heads-first [B,Hkv,K,D] cache (k_hf, :2751) is page_stride=64*D, token_stride=D,
 * head_stride=K*D with one "sequence" per batch entry.
 * page_table[b*pages_per_seq + logical_page] gives the physical page; NULL means
 * physical = b*pages_per_seq + logical_page.
 */
typedef struct ca_kv_layout {
  const void* k;
  const void* v;
  int64_t page_stride;
  int64_t token_stride;
  int64_t head_stride;
  int32_t page_size;     /* tokens per page, multiple of 64 */
  int32_t num_pages;     /* physical pages addressable from k / v */
  int32_t pages_per_seq; /* logical pages per sequence */
  int32_t head_div;      /* 0 or 1: table row r of a batch entry reads KV head r.  d > 1: row r reads KV head
                            r / d - per-query-head (d = G) or query-sub-group (d = G / sub-group size) block
                            tables, the reference's fi_zero_copy_per_query / fi_zero_copy_subgroup routes
                            (compact_attn/kernels/varlen/flashinfer_zero_copy_prefill.py:761, 930).  Read by
                            ca_attn_compact only; the other entry points require 0 or 1. */
  const int32_t* page_table; /* [B, pages_per_seq] int32 or NULL */
} ca_kv_layout;

/*
 * Dense causal attention over the selected KV blocks, read in place through the block table
 * (no materialised compact cache).
 * Replaces: flash_attn_indexed_prefill_from_paged_kv
 *   (compact_attn/kernels/varlen/indexed_dense_prefill_varlen.py:1473-1613),
 *   flashinfer_prefill_zero_copy (compact_attn/kernels/varlen/flashinfer_zero_copy_prefill.py:1139-1353)
 *   and run_direct_indexed_prefill (compact_attn/kernels/varlen/indexed_dense_prefill_direct_triton.py:244).
 * Semantics per row (b,hkv), q-head g, chunk token t: softmax over the row's selected past
 * blocks (all tokens visible) followed by chunk tokens 0..t, scale softmax_scale, out = P.V.
 * block_idx == NULL means "every past block" (dense causal attention: the comparator,
 * compact_attn/modules/dense_prefill.py:117, and the first-chunk case).
 */
typedef struct ca_attn_params {
  const void* q; /* [B,Q,Hq,D] addressed by strides (elements) */
  int64_t q_stride_b, q_stride_t, q_stride_h;
  void* out; /* [B,Q,Hq,D] addressed by strides (elements) */
  int64_t o_stride_b, o_stride_t, o_stride_h;
  ca_kv_layout kv;
  const int32_t* block_idx; /* [R, block_idx_stride] ascending past block ids, -1 padded; or NULL */
  const int32_t* counts;    /* [R] selected past blocks per row; ignored when block_idx==NULL */
  int32_t block_idx_stride; /* capacity of one row of block_idx */
  int32_t B, Q, Hq, Hkv, D;
  int32_t kv_len;     /* K, chunk included; K-Q and Q must be multiples of block_size */
  int32_t block_size; /* multiple of 64 */
  int32_t dtype;      /* CA_DTYPE_BF16 or CA_DTYPE_F16 */
  float softmax_scale;
  float* lse;          /* optional [B,Hq,Q] natural-log sum-exp, or NULL */
  void* workspace;     /* ca_attn_workspace_bytes() bytes, 256-byte aligned, or NULL if that is 0 */
  size_t workspace_bytes;
  int32_t* status; /* optional device int32, OR-ed with CA_STATUS_* bits */
} ca_attn_params;

int ca_attn_workspace_bytes(const ca_attn_params* p, size_t* bytes_out);
int ca_attn_compact(const ca_attn_params* p, ca_stream_t stream);

/*
 * ca_attn_compact for callers that cannot allocate device memory.  (No counterpart in the
 * reference: it exists for hosts such as a serving engine that has handed all of HBM to its own
 * pool, or a latency-critical loop in which cudaMalloc and its implicit synchronisation are
 * banned, and which therefore cannot obtain the workspace that lets the kernel cut work units
 * across SMs.)  The partial accumulators live in a buffer built into the library instead:
 * 41.6 MiB of device memory per GPU that loads the library, enough for a device of up to 160 SMs;
 * a larger device is refused with CA_ERR_CAPACITY.  The buffer is part of the library's device
 * module: it is reserved on every GPU on which any entry point of the library has run, for every
 * user of the library whether or not this entry point is ever called, and it is reserved when the
 * module is loaded on that GPU - so a host that gives the rest of HBM to its own pool must make its
 * first call into the library on that GPU (any entry point) BEFORE it does so, or the module load
 * fails for lack of memory.  p->workspace and p->workspace_bytes are
 * ignored; inputs and outputs are still the caller's.  Nothing is allocated or freed by this
 * call.  The first call on a device looks up the buffer's device address (one runtime query, no
 * allocation), so make that first call outside any stream capture.  All calls on a device share
 * the one buffer and it keeps what the previous call left (each launch re-initialises the slot
 * descriptors it reads): calls whose kernels may overlap on the GPU (different streams) race and
 * must be ordered by the caller.
 */
int ca_attn_compact_static_scratch(const ca_attn_params* p, ca_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Block selection
 * ---------------------------------------------------------------------------------------- */
#define CA_RULE_THRESHOLD 0    /* keep s > threshold (strict, fp32 compare) */
#define CA_RULE_ALPHA_ROWMAX 1 /* keep s >= alpha * rowmax, optional top-min_budget */
#define CA_RULE_TOPK 2         /* keep the k largest, ties to the lower block index */
#define CA_RULE_CUMMASS 3      /* keep the shortest descending prefix whose mass reaches threshold */
#define CA_RULE_MASK 4         /* score is a bool mask (uint8): keep where non-zero */

/*
 * Per-row selection rule on a score tensor [B,H,Qb,Kb] (any strides; f32/bf16/f16, or uint8 for
 * CA_RULE_MASK) -> packed keep bits [B,H,Qb,W], W = ceil(Kb/32), bit j%32 of word j/32 = block j.
 * Row (b,h,i) sees key block j iff valid[b,*,i,j] (bool, broadcast over h when valid_stride_h==0)
 * or, with valid==NULL, iff j <= Pb + i.  Optional masked softmax over the row first.
 * Blocks j < sink and blocks with 0 <= (Pb+i)-j < local are forced on.  Rows i >= rows_voting
 * (0 = all rows vote) produce empty bits.
 * Replaces, one rule each:
 *  THRESHOLD    _build_keep_block_mask / _build_keep_block_mask_chunked_fast_path
 *               (compact_attn/modules/attention_forward_chunked_dense.py:352-403, 559-638) and kernels
 *               build_keep_past_fast_kernel / build_keep_curr_fast_kernel
 *               (compact_attn/csrc/compactattn/cache_fill_kernel.cu:275-326): OR over rows of
 *               (s > thr) equals (max over rows > thr);
 *  ALPHA_ROWMAX _flashprefill_keep_block_from_scores_rowwise
 *               (compact_attn/modules/flashprefill_prefill.py:596-666) and the fused Triton
 *               _flashprefill_kv_union_from_scores_kernel (:307-376);
 *  TOPK         torch.topk + scatter in sparse_flash_attention_forward
 *               (compact_attn/modules/attention_forward.py:43-50), with the tie order fixed;
 *  CUMMASS      no counterpart in the reference (defined by this library: stable descending sort,
 *               sequential fp32 prefix sum, shortest prefix with mass >= threshold);
 *  MASK         a caller-made block mask.
 * Top-k size: topk_k when > 0, else max(1, (topk_num*n_valid + topk_den/2) / topk_den) with
 * n_valid the number of visible blocks of the row; clamped to n_valid.
 */
typedef struct ca_select_params {
  const void* score;
  int64_t score_stride_b, score_stride_h, score_stride_q, score_stride_k;
  int32_t score_dtype;
  int32_t rule;
  const void* valid; /* optional bool (uint8) mask, strides below; NULL = block-causal */
  int64_t valid_stride_b, valid_stride_h, valid_stride_q, valid_stride_k;
  void* bits;      /* uint32 [B,H,Qb,W] */
  float* prob_out; /* optional f32 [B,H,Qb,Kb]: the row the rule saw (after softmax), 0 where masked */
  int32_t B, H, Qb, Kb, Pb;
  int32_t softmax;
  float threshold;
  float alpha;
  int32_t topk_k, topk_num, topk_den;
  int32_t min_budget;
  int32_t sink, local;
  int32_t rows_voting;
  /* Optional threshold in device memory (f32), read by the kernel instead of `threshold`: element
   * b * threshold_stride_b for batch entry b (stride 0 = one value for all).  The reference accepts a
   * scalar or per-batch threshold tensor (compact_attn/modules/attention_forward_chunked_dense.py:381-392);
   * reading it on the device keeps the call free of a device-to-host synchronisation. */
  const float* threshold_ptr;
  int64_t threshold_stride_b;
  /* Optional per-entry exponents (f32, the same strides as score): when given, the rule sees
   * score[j] * 2^(score_max[j] - max_j score_max[j]) (0 where score_max[j] is -inf) - the numerator of the
   * training-free selector's normalisation (ca_flashprefill_score's score_raw and max_raw) without its division
   * by the row sum, which the alpha * row-max and top-k rules do not depend on
   * (compact_attn/flashprefill_vendor/flashprefill_native_forward.py:365-374 followed by
   * compact_attn/modules/flashprefill_prefill.py:596-666).  score must then be f32 and softmax 0. */
  const float* score_max;
} ca_select_params;

int ca_select_rows(const ca_select_params* p, ca_stream_t stream);

/*
 * Block-Union KV selection and the per-KV-head block table.
 * Input: packed bits [B,Hkv*G,Qin,W] from ca_select_rows, or a bool mask [B,Hkv*G,Qin,Kb] by
 * strides (Qin = 1 for a [B,H,Kb] keep_block; G = 1 for a mask that is already per KV head).
 * keep_kv[b,hkv,j] = OR over the G heads and Qin rows, OR (j >= Kb - keep_recent), OR (j >= Pb).
 * block_idx[row, 0:count] = ascending kept past block ids (j < Pb), rest -1; counts[row];
 * cache_seqlens[row] = (count + Kb - Pb) * block_size; pages_per_row = ceil(cache_seqlens / page_size).
 * Replaces _build_kv_head_union_keep_block_mask, _build_kv_head_union_past_block_indices and
 * _build_kv_head_past_block_indices_from_kv_keep_block
 * (compact_attn/modules/attention_forward_chunked_dense.py:641-683, 737-782, 785-819) and kernel
 * build_past_indices_and_metadata_from_keep_block_kernel
 * (compact_attn/csrc/compactattn/cache_fill_kernel.cu:328-385).
 */
typedef struct ca_union_params {
  const void* bits; /* uint32 [B,Hkv*G,Qin,W] or NULL */
  const void* mask; /* uint8 bool by strides or NULL */
  int64_t mask_stride_b, mask_stride_h, mask_stride_q, mask_stride_k;
  int32_t B, Hkv, G, Qin, Kb, Pb;
  int32_t keep_recent;
  int32_t block_size, page_size;
  int32_t* block_idx; /* [B*Hkv, idx_stride] */
  int32_t idx_stride; /* >= max(Pb, 1) */
  int32_t* counts;        /* [B*Hkv] */
  int32_t* cache_seqlens; /* optional [B*Hkv] */
  int32_t* pages_per_row; /* optional [B*Hkv] */
  void* keep_kv;          /* optional bool (uint8) [B,Hkv,Kb] */
} ca_union_params;

int ca_union_table(const ca_union_params* p, ca_stream_t stream);

/*
 * ca_select_rows and ca_union_table in ONE launch: every row CTA of the selection stores its packed bits
 * (into sel->bits, or into the scratch when sel->bits is NULL) and takes a ticket; the CTA that takes the last
 * ticket of a KV-head row (nobody waits for anybody) ORs that row's G * Qb bit rows and compacts them into the
 * block table.  It replaces the same reference functions as the two calls it fuses, in particular the pair
 * build_keep_past_fast_kernel / build_keep_curr_fast_kernel followed by
 * build_past_indices_and_metadata_from_keep_block_kernel
 * (compact_attn/csrc/compactattn/cache_fill_kernel.cu:275-385) and the fused Triton
 * _flashprefill_kv_union_from_scores_kernel (compact_attn/modules/flashprefill_prefill.py:307-376).
 * un gives the table outputs and Hkv, G (sel->H = Hkv*G), Qin = sel->Qb, Kb, Pb, keep_recent, block_size,
 * page_size; its bits, mask and keep_kv must be NULL.  scratch: ca_select_union_scratch_bytes() bytes of
 * 16-byte aligned device memory whose first ceil4(B*Hkv) words (the tickets) are ZERO on the first call; the
 * kernel leaves them zero, so one buffer serves every later call on the same stream (calls that may overlap on
 * the device need a buffer each).  The rest of the scratch holds the rows' bits when sel->bits is NULL and
 * needs no initialisation.
 */
int ca_select_union_scratch_bytes(int B, int H, int Hkv, int Qb, int Kb, size_t* bytes_out);
int ca_select_union_table(const ca_select_params* sel, const ca_union_params* un, void* scratch, size_t scratch_bytes,
                          ca_stream_t stream);

/*
 * Paged metadata of the compact cache: page_offsets[r] = exclusive prefix of pages_per_row
 * (page_offsets[rows] = total) and block_table[r, slot] = page_offsets[r] + slot for
 * slot < pages_per_row[r], else 0.  Replaces build_block_table_kernel
 * (compact_attn/csrc/compactattn/cache_fill_kernel.cu:163-190).
 */
int ca_paged_metadata(const int32_t* pages_per_row, int rows, int32_t* page_offsets, int32_t* block_table,
                      int max_pages, ca_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Block scoring
 * ---------------------------------------------------------------------------------------- */
#define CA_POOL_MAX 1
#define CA_POOL_MIN 2
#define CA_POOL_AVG 4

/*
 * Block pooling over tokens: x [B,L,H,D] (strides, f32/bf16/f16) -> out[b, out_block_offset + blk,
 * h, :] = [max | min | avg] (the kinds present, in that order) of tokens blk*bs .. min((blk+1)*bs, L),
 * fp32 accumulation, avg divides by the tokens present.  Writing at a block offset appends to a
 * selector cache in place.
 * Replaces AttnGate.compress_query_blocks / compress_key_blocks pooling
 * (compact_attn/prefill_sparse/attn_gate.py:113-130), the Triton compute_mean_vector
 * (compact_attn/flashprefill_vendor/flashprefill_native_forward.py:44-95) and the mean-K cache
 * update (compact_attn/prefill_sparse/llama/modeling_llama_flashprefill_compactattn.py:121-150).
 */
typedef struct ca_pool_params {
  const void* x;
  int64_t x_stride_b, x_stride_t, x_stride_h;
  int32_t x_dtype;
  int32_t out_dtype;
  void* out; /* [B, >= out_block_offset + ceil(L/bs), H, nk*D] by strides */
  int64_t out_stride_b, out_stride_blk, out_stride_h;
  int32_t out_block_offset;
  int32_t B, L, H, D, block_size;
  int32_t kinds; /* CA_POOL_* bits */
} ca_pool_params;

int ca_pool_blocks(const ca_pool_params* p, ca_stream_t stream);

/*
 * Per-head linear projection of pooled blocks, block RoPE (half-rotation form) and write at a
 * block offset of the destination (the gate's K-block cache, or the chunk's Q blocks):
 *   y[b,blk,h,:] = x[b,blk,h / (Hout/Hin),:] @ w[h]   (w == NULL: identity)
 *   out = y*cos + rotate_half(y)*sin                  (cos == NULL: no RoPE)
 * x is contiguous f32 [B,nb,Hin,Cin]; w contiguous [Hout,Cin,Cout]; cos/sin f32 [rope_batch,nb,Cout].
 * Replaces MultiHeadLinear.forward (compact_attn/prefill_sparse/attn_gate.py:29-33),
 * AttnGate.apply_block_position_embeddings (:132-171) and _compactattn_append_cached_k_blocks
 * (compact_attn/prefill_sparse/llama/modeling_llama_seerattn_chunked_dense.py:426-478).
 */
typedef struct ca_project_params {
  const float* x;
  const void* w;
  int32_t w_dtype;
  int32_t out_dtype;
  const float* cos;
  const float* sin;
  int32_t rope_batch;
  int32_t out_block_offset;
  void* out;
  int64_t out_stride_b, out_stride_blk, out_stride_h;
  int32_t B, nb, Hin, Hout, Cin, Cout;
} ca_project_params;

int ca_gate_project(const ca_project_params* p, ca_stream_t stream);

/*
 * Fused gate preparation of one chunk (one launch): for the query side and the key side, pool the
 * chunk's token blocks, project per head, apply block RoPE, and write the result at a block offset
 * of the side's destination (the chunk's Q blocks; the gate's K-block cache, i.e. an append).
 * Both sides share B, L (chunk tokens), D, C (gate hidden size) and block_size; cos/sin are
 * f32 [rope_batch, ceil(L/bs), C] for the chunk's block positions.
 * Replaces _build_chunked_gate_blocks + _gate_k_append as used by _compute_chunked_gate_from_cache
 * (compact_attn/prefill_sparse/llama/modeling_llama_seerattn.py:437-481).
 */
typedef struct ca_gate_side {
  const void* x; /* [B,L,H,D] by strides */
  int64_t x_stride_b, x_stride_t, x_stride_h;
  int32_t x_dtype;
  int32_t H;
  int32_t kinds; /* CA_POOL_* bits */
  int32_t w_dtype;
  const void* w; /* [Hw, nk*D, C] contiguous, or NULL for identity */
  int32_t Hw;
  int32_t rope_batch;
  const float* cos;
  const float* sin;
  void* out; /* [B, >= out_block_offset + ceil(L/bs), Hw, C] by strides */
  int64_t out_stride_b, out_stride_blk, out_stride_h;
  int32_t out_dtype;
  int32_t out_block_offset;
} ca_gate_side;

typedef struct ca_gate_prepare_params {
  ca_gate_side q, k;
  int32_t B, L, D, C, block_size;
} ca_gate_prepare_params;

int ca_gate_prepare(const ca_gate_prepare_params* p, ca_stream_t stream);

/*
 * Gate logits: out[b,h,i,j] = (q[b,i,h,:] . k[b,j,h / (Hq/Hk),:]) * scale for j <= Pb + i, else
 * masked_value; out is contiguous f32 [B,Hq,Qb,Kb].  The softmax of
 * AttnGate.score_compressed_blocks (compact_attn/prefill_sparse/attn_gate.py:173-204) is applied
 * by ca_select_rows (softmax = 1), fused with the selection rule.
 */
typedef struct ca_gate_score_params {
  const void* q; /* [B,Qb,Hq,C] by strides */
  int64_t q_stride_b, q_stride_blk, q_stride_h;
  const void* k; /* [B,Kb,Hk,C] by strides */
  int64_t k_stride_b, k_stride_blk, k_stride_h;
  int32_t q_dtype, k_dtype;
  float* out;
  int32_t B, Hq, Hk, Qb, Kb, Pb, C;
  float scale;
  float masked_value;
} ca_gate_score_params;

int ca_gate_scores(const ca_gate_score_params* p, ca_stream_t stream);

/*
 * Gate scores, row rule, Block-Union and block table behind ONE host call: exactly ca_gate_scores(score)
 * followed by ca_select_union_table(sel, un, scratch) with sel->score == score->out (the gate's contiguous fp32
 * buffer) - two launches (the tensor-core score kernel reads every key block once for all Q-blocks and heads; the
 * rule kernel builds the union and the table), validated together.  write_scores is accepted for callers written
 * against an earlier single-launch form and ignored: the logits always pass through score->out.
 * Same reference lines as ca_gate_scores and ca_select_union_table; replaces the chain
 * AttnGate.score_compressed_blocks -> keep-mask builders -> index builders
 * (compact_attn/prefill_sparse/attn_gate.py:173-204, compact_attn/modules/attention_forward_chunked_dense.py:352-403,
 * 641-683, compact_attn/csrc/compactattn/cache_fill_kernel.cu:275-385).
 */
int ca_gate_score_select(const ca_gate_score_params* score, const ca_select_params* sel, const ca_union_params* un, void* scratch,
                         size_t scratch_bytes, int write_scores, ca_stream_t stream);

/*
 * Training-free block score.  For q-block i, head h, key block j over the tokens t of the q-block
 * with P + t >= (j+1)*bs - 1:  S = (q_t . mean_k_j) * D^-0.5 * log2(e),  max_raw = max_t S,
 * score_raw = sum_t 2^(S - max_raw)  (-inf where no token qualifies); all [B,Qb,Kb,Hq] f32.
 * score_norm (optional) = score_raw * 2^(max_raw - max_j max_raw) / (sum_j ... + 1e-9), 0 where
 * max_raw = -inf.
 * Replaces the Triton compute_block_score_chunked and normalize_scores
 * (compact_attn/flashprefill_vendor/flashprefill_native_forward.py:98-207, 365-374) as driven by
 * flash_prefill_score_chunked_from_mean_k (:541-586).
 */
typedef struct ca_flashprefill_score_params {
  const void* q; /* [B,Q,Hq,D] by strides */
  int64_t q_stride_b, q_stride_t, q_stride_h;
  const void* mean_k; /* [B,Kb,Hkv,D] by strides */
  int64_t k_stride_b, k_stride_blk, k_stride_h;
  int32_t q_dtype, k_dtype;
  float* score_raw;
  float* max_raw;
  float* score_norm; /* optional */
  int32_t B, Q, Hq, Hkv, D, Kb, block_size, kv_len;
} ca_flashprefill_score_params;

int ca_flashprefill_score(const ca_flashprefill_score_params* p, ca_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Compact KV gather (cache fill)
 * ---------------------------------------------------------------------------------------- */
/*
 * For each row r = (b,hkv): copies blocks block_idx[r, 0:counts[r]] (block_size tokens x D each)
 * and then the chunk's Q tokens of K and V from the source cache into the compact cache at token
 * position  base(r) + rank*block_size,  base(r) = page_offsets[r]*dst_page_size  (page_offsets
 * from ca_paged_metadata) or r*dst_row_stride_tokens when page_offsets is NULL.  Destination
 * caches are contiguous [tokens, D] (viewed by the caller as [pages, dst_page_size, 1, D]).
 * Replaces build_paged_kv_cache_from_keep_block_fast / build_paged_kv_cache_from_token_mask
 * (compact_attn/kernels/varlen/indexed_dense_prefill_varlen.py:466-766, 1414-1470) and kernels
 * cache_fill_from_past_indices_compact_kernel + cache_fill_current_tail_kernel
 * (compact_attn/csrc/compactattn/cache_fill_kernel.cu:596-720).
 */
typedef struct ca_gather_params {
  ca_kv_layout kv;
  const int32_t* block_idx;
  const int32_t* counts;
  int32_t block_idx_stride;
  int32_t dtype; /* CA_DTYPE_BF16 or CA_DTYPE_F16 (a byte copy of 16-bit elements) */
  const int32_t* page_offsets; /* optional [B*Hkv + 1] */
  int64_t dst_row_stride_tokens;
  void* k_dst;
  void* v_dst;
  int32_t dst_page_size;
  int32_t B, Hkv, D, Q, kv_len, block_size;
  int32_t* status; /* optional */
} ca_gather_params;

int ca_gather_kv(const ca_gather_params* p, ca_stream_t stream);

/*
 * Chunk append: RoPE on the chunk's queries and keys, the keys and values written into the paged
 * cache at token `position`, and (optionally) the mean of the rotated keys of every block appended
 * to the training-free selector's mean-K cache.  One launch, every element read and written once.
 * Replaces, for one chunk of one layer:
 *   apply_rotary_pos_emb (compact_attn/modules/common.py:49-75; out = x*cos + rotate_half(x)*sin,
 *     half-rotation, products and sum rounded separately as torch does, so the result is
 *     bit-identical for 16-bit tables and for fp32 tables),
 *   the KV cache update behind the _do_kv_cache_update hook
 *     (compact_attn/prefill_sparse/llama/modeling_llama_seerattn_chunked_dense.py:518-536;
 *     DynamicCache.update concatenates the whole layer cache, HeadsFirstDynamicCache adds a
 *     permute, modeling_llama_seerattn_chunked_dense_hf.py:29-82), and
 *   compute_mean_vector over the new keys plus the torch.cat of the mean-K parts
 *     (compact_attn/prefill_sparse/llama/modeling_llama_flashprefill_compactattn.py:121-150).
 * q/k/v are [B, Q, H, D] with element strides (D contiguous); q may be NULL (Hq = 0).  q_out may
 * alias q.  cos/sin are [B or 1, Q, D] (cs_stride_b = 0 broadcasts one table), the full head
 * dimension is rotated.  cache.k / cache.v are written (the struct's const is for the readers).
 * mean_k is [B, blocks, Hkv, D] in the tensors' type; block `position / block_size + i` receives
 * chunk block i; it needs position % block_size == 0.  All strides multiples of 8 elements, all
 * pointers 16-byte aligned.  A page-table entry out of range skips that token and sets
 * CA_STATUS_BAD_INDEX.
 */
typedef struct ca_rope_append_params {
  const void* q;
  void* q_out;
  int64_t q_stride_b, q_stride_t, q_stride_h;
  int64_t qo_stride_b, qo_stride_t, qo_stride_h;
  const void* k;
  int64_t k_stride_b, k_stride_t, k_stride_h;
  const void* v;
  int64_t v_stride_b, v_stride_t, v_stride_h;
  const void* cos;
  const void* sin;
  int64_t cs_stride_b, cs_stride_t;
  int32_t rope_dtype; /* CA_DTYPE_F32 or the tensors' dtype */
  int32_t dtype;      /* CA_DTYPE_BF16 or CA_DTYPE_F16 */
  ca_kv_layout cache;
  void* mean_k; /* optional */
  int64_t mk_stride_b, mk_stride_blk, mk_stride_h;
  int32_t B, Q, Hq, Hkv, D;
  int32_t position;   /* first token of the chunk in its sequence */
  int32_t block_size; /* selector block (mean-K granularity, CTA tile) */
  int32_t reserved;
  int32_t* status; /* optional */
} ca_rope_append_params;

int ca_rope_append(const ca_rope_append_params* p, ca_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Output projection fused with the tensor-parallel reduction
 * ---------------------------------------------------------------------------------------- */
/*
 * out (on every rank) = sum over ranks r of  a_r [M, K_r] . w_r[N, K_r]^T,  16-bit in and out, fp32 accumulate.
 * Rank `rank` of `world` passes its own a and w and, for EVERY rank, the peer-mapped device addresses of that
 * rank's staging buffer, per-tile arrival counters, finished-tile counter and output buffer (symmetric
 * allocations of the same sizes on all ranks, see ca_oproj_scratch_bytes; counters zero before the first
 * call).  Two-shot (any world): three launches - a tcgen05 GEMM whose epilogue stores each 128 x 256 partial
 * tile into the staging buffer of the rank that owns the tile (tile t -> rank t % world) with plain peer stores
 * and bumps the owner's arrival counter; a reduction in which every rank sums the partials of its own tiles and
 * stores the result into every rank's output; a one-thread wait until this rank's output is complete.  One-shot
 * (two ranks): the GEMM stores every partial tile into BOTH ranks' staging buffers and each rank reduces all
 * tiles into its own output - the same bytes over NVLink, one exchange instead of two, no final wait; the
 * staging buffer is used in halves by alternate calls.  Every wait is bounded by wait_limit_ns (0 = 2 s); on
 * expiry *status gets CA_STATUS_TIMEOUT and the output is invalid.  `epoch` is the number of this call on these
 * buffers (1, 2, ...), the same on every rank: counters only grow, nothing is reset.  All ranks must issue the
 * same sequence of calls with the same M, N and mode; M may change from call to call when row_epochs and
 * done_tiles_total are kept (see the fields).  world == 1 is a plain GEMM into out[0].
 * Replaces the row-parallel o_proj of the reference's tensor-parallel plan followed by its all-reduce
 * (compact_attn/prefill_sparse/llama/modeling_llama_seerattn.py:111-120; the deferred wait of
 * modeling_llama_flashprefill_compactattn.py:37-41, 321-322).
 */
typedef struct ca_oproj_params {
  const void* a;      /* [M, K] this rank's attention output, K contiguous */
  int64_t a_stride_m;
  const void* w;      /* [N, K] this rank's input columns of the projection weight, K contiguous; NULL = no GEMM:
                         a is then this rank's partial [M, N] itself (a_stride_m >= N, K ignored) and the call is
                         the sum over the ranks alone, an all-reduce through the same exchange (world > 1) */
  int64_t w_stride_n;
  int32_t M, N, K;    /* N a multiple of 256, K a multiple of 64 */
  int32_t dtype;      /* CA_DTYPE_BF16 or CA_DTYPE_F16 */
  int32_t world, rank;
  void* const* stage;              /* [world] staging buffers (NULL when world == 1) */
  uint32_t* const* tile_counters;  /* [world] per-owned-tile arrival counters */
  uint32_t* const* done_counters;  /* [world] finished-tile counters (one uint32 each) */
  void* const* out;                /* [world] output buffers [M, N] */
  int64_t out_stride_m;
  uint32_t epoch;
  uint32_t phases; /* 0 = all three launches; else a mask: 1 GEMM + push, 2 reduction + broadcast, 4 final wait
                      (several ranks emulated on one device enqueue phase by phase, so that no kernel waits for
                      one that has not been launched) */
  uint64_t wait_limit_ns;
  int32_t* status; /* optional */
  int32_t mode;    /* 0 = auto (one-shot on two ranks, two-shot beyond), 1 = two-shot, 2 = one-shot,
                      3 = through the switch (needs stage_mc and out_mc; measured slower than two-shot at 4 GPUs) */
  size_t stage_bytes;          /* size of each staging buffer (checked against what the call needs) */
  const uint32_t* row_epochs;  /* HOST array [ceil(M/128)], optional: for each block of 128 rows, how many calls on
                                  these buffers (this one included) had at least that many rows.  NULL = `epoch` for
                                  every block, i.e. every call so far had at least this call's number of row blocks */
  void* stage_mc;              /* optional: the NVLink-switch multicast address bound to all ranks' staging buffers ... */
  void* out_mc;                /* ... and to all ranks' output buffers.  Mode 3 reduces through the switch: every rank keeps its partial tile in its own staging buffer, the tile's owner
                                  reads the sum with multimem.ld_reduce and stores it to every rank with multimem.st */
  uint32_t done_tiles_total;   /* two-shot: sum of ca_oproj_tile_count(M, N) over all calls so far, this one included;
                                  0 = epoch * this call's tile count (every call the same M) */
} ca_oproj_params;

/* Bytes of the symmetric staging buffer and of the counter block (per-owned-tile counters followed by the
 * finished-tile counter) for outputs of up to M_max rows. */
int ca_oproj_scratch_bytes(int M_max, int N, int world, size_t* stage_bytes, size_t* counter_bytes);
/* Number of 128 x 256 output tiles of an [M, N] result (what done_tiles_total accumulates). */
int ca_oproj_tile_count(int M, int N);
int ca_oproj_allreduce(const ca_oproj_params* p, ca_stream_t stream);

/*
 * Self-test of the bounded device-side wait (no counterpart in the reference).  Every kernel of the library
 * that waits on an mbarrier (TMA arrivals, tensor-core commits, hand-offs between warp roles) does so through
 * one routine that gives up after a time limit, raises the CTA's abort flag and lets the kernel drain and return
 * with CA_STATUS_TIMEOUT instead of hanging.  This entry point runs that routine on a barrier nothing arrives on:
 * one small CTA waits limit_ns (at most 1 s), then ORs CA_STATUS_TIMEOUT into *status and stores the time it
 * waited (nanoseconds of the GPU's global timer) into *waited_ns (optional).  The context stays usable.
 */
int ca_selftest_bounded_wait(uint64_t limit_ns, int32_t* status, uint64_t* waited_ns, ca_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * One chunk of one layer in one call
 * ---------------------------------------------------------------------------------------- */
/*
 * Enqueues the whole per-layer step of the path with one host call, in this order, each stage exactly
 * as its own entry point would (a stage whose first pointer is NULL is skipped):
 *   append   ca_rope_append          RoPE on q/k, K/V into the paged cache (+ mean-K)      [append.k]
 *   prepare  ca_gate_prepare         pool + project + RoPE the chunk's Q and K blocks      [prepare.q.x]
 *   score    ca_gate_scores          gate logits against every cached K block              [score.q]
 *   fp_score ca_flashprefill_score   training-free block scores                            [fp_score.q]
 *   select + table  ca_select_union_table (one launch) when union_scratch is given, else
 *            ca_select_rows then ca_union_table                                            [select.score]
 *            (score + select + table go through ca_gate_score_select when the score stage is present,
 *            union_scratch is given and select.score == score.out)
 *   attn     ca_attn_compact                                                               [attn.q]
 * It stands where the reference runs its per-layer Python between the KV-cache update and o_proj:
 * _compute_chunked_gate_from_cache, the keep-mask / index builders and the indexed attention call
 * (compact_attn/prefill_sparse/llama/modeling_llama_seerattn_chunked_dense.py:547-938,
 * compact_attn/modules/attention_forward_chunked_dense.py:2732-2912), dozens of host-side launches per
 * layer there.  A caller that keeps the struct between chunks only updates the fields that change
 * (lengths, block offsets, the chunk's tensors).  Returns the first failing stage's code.
 */
typedef struct ca_chunk_step_params {
  ca_rope_append_params append;
  ca_gate_prepare_params prepare;
  ca_gate_score_params score;
  ca_flashprefill_score_params fp_score;
  ca_select_params select;
  ca_union_params table;
  void* union_scratch;
  size_t union_scratch_bytes;
  ca_attn_params attn;
  int32_t write_scores; /* passed to ca_gate_score_select (ignored there: the logits always reach score.out) */
} ca_chunk_step_params;

int ca_chunk_step(const ca_chunk_step_params* p, ca_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* COMPACTATTN_B200_H_ */
