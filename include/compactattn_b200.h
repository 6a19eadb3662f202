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
/* ABI version; bumped when a struct below changes. */
int ca_abi_version(void);
/* Number of kernel launches the library has enqueued in this process (all entry points). */
int64_t ca_launch_count(void);

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
  int32_t reserved;
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

#ifdef __cplusplus
}
#endif
#endif /* COMPACTATTN_B200_H_ */
