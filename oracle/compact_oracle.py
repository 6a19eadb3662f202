"""CPU oracle for the CompactAttention chunked-prefill path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain fp32 torch/numpy on the CPU, what the reference project
(jiwonsong-dev/CompactAttention) computes on the path: block scoring, block selection, Block-Union
KV selection, the per-KV-head block table, the compact KV gather and the dense causal attention
over the gathered KV.  It exists so the CUDA library can be checked against it; only tests, the
smoke check and the benchmark's CPU-baseline leg may import it.  Nothing here is used by, or may be
used as a fallback for, the product path.

Pinning: the reference ships no tests or golden vectors for this path.  The restatements below are
pinned against the reference's own Python functions executed on seeded inputs
(``tests/golden/make_golden.py`` imports them and writes the fixtures that
``tests/test_oracle_golden.py`` replays), RoPE (``apply_rotary_pos_emb``) included.  Two rules have no counterpart in the reference and are
defined here alone ("parity unpinned" for them): the cumulative-mass rule and the tie order of the
per-row top-k rule (lower block index wins).

Every function cites the reference file:line it follows (paths relative to the reference root).
Shapes: B batch, Q chunk tokens, K kv_len (chunk included), P = K - Q, bs block size,
Qb = ceil(Q/bs), Kb = ceil(K/bs), Pb = P // bs, G = Hq // Hkv.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F

LOG2E = 1.4426950408889634


# --------------------------------------------------------------------------------------------
# Training-free selector (FlashPrefill): mean-K pooling, block score, normalisation, row rule
# --------------------------------------------------------------------------------------------
def mean_pool_blocks(x: torch.Tensor, block_size: int) -> torch.Tensor:
    """Per-block mean over tokens, fp32 sum / count, stored in the input dtype.

    Follows ``compute_mean_vector`` (compact_attn/flashprefill_vendor/flashprefill_native_forward.py:77-95).
    x: [B, L, H, D] -> [B, ceil(L/bs), H, D].
    """
    B, L, H, D = x.shape
    nb = (L + block_size - 1) // block_size
    pad = nb * block_size - L
    xf = x.to(torch.float32)
    if pad:
        xf = F.pad(xf, (0, 0, 0, 0, 0, pad))
    sums = xf.view(B, nb, block_size, H, D).sum(dim=2)
    cnt = torch.full((nb,), float(block_size))
    if pad:
        cnt[-1] = float(block_size - pad)
    # the reference divides in the input dtype's fp32 image (q is loaded as 16-bit, summed in fp32)
    return (sums / cnt.view(1, nb, 1, 1)).to(x.dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """``[-x2, x1]`` over the two halves of the last dimension (compact_attn/modules/common.py:36-40)."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``(x * cos) + (rotate_half(x) * sin)`` on ``[B, L, H, D]`` with ``cos/sin [B or 1, L, D]``, in the
    operands' own dtypes exactly as the reference writes it (compact_attn/modules/common.py:49-75 with
    ``unsqueeze_dim=2``); the result is cast back to x's dtype (a no-op for 16-bit tables)."""
    c, s = cos.unsqueeze(2), sin.unsqueeze(2)
    return ((x * c) + (rotate_half(x) * s)).to(x.dtype)


def rope_append(q, k, v, cos, sin, k_pages, v_pages, page_table, position: int, block_size: int):
    """What one chunk does to the per-layer state before attention: RoPE on q and k
    (``apply_rope``), the rotated keys and the values written at tokens ``position ..`` of a paged
    cache ``[pages, page_size, Hkv, D]`` through ``page_table [B, pages_per_seq]`` (the reference
    appends to a contiguous cache, modeling_llama_seerattn_chunked_dense.py:518-536; the page table
    only renames where a token lives), and the per-block mean of the rotated keys
    (``mean_pool_blocks``).  Returns ``(q_rot, mean_k_chunk)`` and updates the page tensors in place."""
    q_rot = apply_rope(q, cos, sin) if q is not None else None
    k_rot = apply_rope(k, cos, sin)
    B, Q = k.shape[0], k.shape[1]
    page_size = k_pages.shape[1]
    for b in range(B):
        for t in range(Q):
            tok = position + t
            page = int(page_table[b, tok // page_size])
            k_pages[page, tok % page_size] = k_rot[b, t]
            v_pages[page, tok % page_size] = v[b, t]
    return q_rot, mean_pool_blocks(k_rot, block_size)


def flashprefill_block_score_raw(
    q: torch.Tensor, mean_k: torch.Tensor, key_len: int, block_size: int
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per (q-block, key block, q-head): m = max_t S, p = sum_t 2^(S - m) with
    S[t, j] = (q_t . meanK_j) * D^-0.5 * log2(e), token t counted iff P + t >= (j+1)*bs - 1.

    Follows ``compute_block_score_chunked``
    (compact_attn/flashprefill_vendor/flashprefill_native_forward.py:156-207) with K_STRIDE = bs.
    q: [B, Q, Hq, D]; mean_k: [B, Kb, Hkv, D] -> score, max: [B, Qb, Kb, Hq] fp32 (-inf where no
    token qualifies, as the reference's torch.full initialisation leaves it, :558-565).
    """
    B, Q, Hq, D = q.shape
    Kb, Hkv = mean_k.shape[1], mean_k.shape[2]
    G = Hq // Hkv
    Qb = (Q + block_size - 1) // block_size
    P = key_len - Q
    sm_scale = (1.0 / math.sqrt(D)) * LOG2E
    qf = q.to(torch.float32)
    kf = mean_k.to(torch.float32).repeat_interleave(G, dim=2)  # [B, Kb, Hq, D]
    score = torch.full((B, Qb, Kb, Hq), float("-inf"), dtype=torch.float32)
    mx = torch.full((B, Qb, Kb, Hq), float("-inf"), dtype=torch.float32)
    k_last = torch.arange(Kb) * block_size + block_size - 1  # last token of each key block
    for i in range(Qb):
        t0, t1 = i * block_size, min((i + 1) * block_size, Q)
        s = torch.einsum("bthd,bjhd->bhtj", qf[:, t0:t1], kf) * sm_scale  # [B, Hq, T, Kb]
        q_abs = P + torch.arange(t0, t1)
        causal = q_abs.view(-1, 1) >= k_last.view(1, -1)  # [T, Kb]
        s = torch.where(causal.view(1, 1, *causal.shape), s, torch.full_like(s, float("-inf")))
        m = s.amax(dim=2)  # [B, Hq, Kb]
        p = torch.exp2(s - m.unsqueeze(2))
        p = torch.where(causal.view(1, 1, *causal.shape), p, torch.zeros_like(p)).sum(dim=2)
        # the reference visits key blocks only up to the q-block's last token (:151-152); beyond
        # that the outputs keep their -inf initialisation
        hi = min((P + t0 + block_size - 1 + 1 + block_size - 1) // block_size, Kb)
        visited = torch.arange(Kb) < hi
        has = torch.isfinite(m) & visited.view(1, 1, -1)
        score[:, i] = torch.where(has, p, torch.full_like(p, float("-inf"))).permute(0, 2, 1)
        mx[:, i] = torch.where(has, m, torch.full_like(m, float("-inf"))).permute(0, 2, 1)
    return score, mx


def flashprefill_normalize_scores(score: torch.Tensor, mx: torch.Tensor) -> torch.Tensor:
    """``normalize_scores`` (compact_attn/flashprefill_vendor/flashprefill_native_forward.py:365-374)."""
    mask = mx != float("-inf")
    max_in_max = torch.max(mx, dim=2, keepdim=True).values
    w = torch.exp2(mx - max_in_max)
    w = torch.where(mask, w, torch.ones_like(w))
    s = torch.where(mask, score, torch.zeros_like(score))
    s = s * w
    return s / (s.sum(dim=2, keepdim=True) + 1e-9)


def flashprefill_keep_rowwise(
    score: torch.Tensor,  # [B, Qb, Kb, Hq] normalised
    q_len: int,
    kv_len: int,
    block_size: int,
    num_key_value_groups: int,
    attention_sink: int,
    window_size: int,
    alpha: float,
    last_n_block: int = 0,
    min_budget: int = 0,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """alpha * row-max rule with sink / window, then Q-union and GQA union.

    Follows ``_flashprefill_keep_block_from_scores_rowwise``
    (compact_attn/modules/flashprefill_prefill.py:596-666).  Returns (keep_row [B,Hq,Qp,Kb] before
    any union, keep_block [B,Hq,Kb], keep_block_kv [B,Hkv,Kb]); the chunk's own blocks are forced on
    in the last two.
    """
    s = score.permute(0, 3, 1, 2).contiguous()
    B, Hq, Qb, Kb = s.shape
    Pb = max((max(kv_len - q_len, 0) + block_size - 1) // block_size, 0)
    Hkv = Hq // num_key_value_groups
    tail = min(max(last_n_block, 0), Qb - 1) if Qb > 1 else 0
    Qp = max(Qb - tail, 1)
    k_ids = torch.arange(Kb).view(1, 1, 1, Kb)
    q_ids = torch.arange(Pb, Pb + Qp).view(1, 1, Qp, 1)
    dist = q_ids - k_ids
    causal = dist >= 0
    sink = k_ids < attention_sink
    window = causal & (dist < window_size)
    row = s[:, :, :Qp, :]
    finite = torch.isfinite(row) & causal
    row = torch.where(finite, row, torch.zeros_like(row))
    if min_budget > 0:
        k = min(int(min_budget), Kb)
        order = stable_desc_order(row)
        top_idx = order[..., :k]
        max_val = torch.gather(row, -1, top_idx[..., :1])
        keep_row = finite & (row >= max_val * alpha)
        keep_row.scatter_(-1, top_idx, True)
    else:
        max_val = row.max(dim=-1, keepdim=True).values
        keep_row = finite & (row >= max_val * alpha)
    keep_row = (keep_row | sink | window) & causal
    keep_q = keep_row.any(dim=2)
    keep_block = keep_q.clone()
    keep_block[..., Pb:] = True
    keep_kv = keep_block.view(B, Hkv, num_key_value_groups, Kb).any(dim=2)
    return keep_row, keep_block, keep_kv


# --------------------------------------------------------------------------------------------
# Learned selector (SeerAttention AttnGate)
# --------------------------------------------------------------------------------------------
def pool_blocks(x: torch.Tensor, block_size: int, kinds: Tuple[str, ...]) -> torch.Tensor:
    """max / min / avg pooling over blocks of tokens with ceil_mode, concatenated on channels.

    Follows ``AttnGate.compress_*_blocks`` (compact_attn/prefill_sparse/attn_gate.py:113-130):
    F.{max,avg}_pool3d(kernel=[bs,1,1], stride=[bs,1,1], ceil_mode=True); avg over a ragged last
    block divides by the number of tokens present.  x: [B, L, H, D] -> [B, ceil(L/bs), H, D*len(kinds)].
    """
    B, L, H, D = x.shape
    nb = (L + block_size - 1) // block_size
    outs = []
    for kind in kinds:
        parts = []
        for i in range(nb):
            seg = x[:, i * block_size : min((i + 1) * block_size, L)].to(torch.float32)
            if kind == "max":
                parts.append(seg.amax(dim=1))
            elif kind == "min":
                parts.append(seg.amin(dim=1))
            elif kind == "avg":
                parts.append(seg.sum(dim=1) / seg.shape[1])
            else:
                raise ValueError(kind)
        outs.append(torch.stack(parts, dim=1))
    return torch.cat(outs, dim=-1).to(x.dtype)


def multi_head_linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``MultiHeadLinear.forward`` (compact_attn/prefill_sparse/attn_gate.py:29-33):
    x [B, S, h, I] (h repeated up to the weight's head count), weight [H, I, O] -> [B, S, H, O]."""
    H = weight.shape[0]
    if x.shape[2] < H:
        x = x.repeat_interleave(H // x.shape[2], dim=2)
    return torch.einsum("bshi,hio->bsho", x.to(torch.float32), weight.to(torch.float32))


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """compact_attn/modules/common.py:29-33."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_block_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-rotation RoPE on block vectors: x [B, S, H, D], cos/sin [B, S, D]
    (``AttnGate.apply_block_position_embeddings`` non-flash branch,
    compact_attn/prefill_sparse/attn_gate.py:154-169 -> compact_attn/modules/common.py:49-75)."""
    c = cos.unsqueeze(2).to(torch.float32)
    s = sin.unsqueeze(2).to(torch.float32)
    xf = x.to(torch.float32)
    return xf * c + rotate_half(xf) * s


def gate_block_causal_mask(q_len: int, kv_len: int, block_size: int, batch: int = 1) -> torch.Tensor:
    """Block-level causal mask for a chunk at the end of the cache, no padding:
    mask[i, j] = j <= floor((P + min((i+1)*bs - 1, Q-1)) / bs).

    Follows ``_seerattn_update_causal_mask``
    (compact_attn/prefill_sparse/llama/modeling_llama_seerattn.py:968-1024).  -> bool [B,1,Qb,Kb]."""
    Qb = (q_len + block_size - 1) // block_size
    Kb = (kv_len + block_size - 1) // block_size
    P = kv_len - q_len
    q_end = torch.minimum((torch.arange(Qb) + 1) * block_size - 1, torch.tensor(q_len - 1)) + P
    m = torch.arange(Kb).view(1, Kb) <= (q_end // block_size).view(Qb, 1)
    return m.view(1, 1, Qb, Kb).expand(batch, 1, Qb, Kb).clone()


def gate_score(
    q_blocks: torch.Tensor,  # [B, Qb, Hq, Dg]
    k_blocks: torch.Tensor,  # [B, Kb, Hk, Dg]  (Hk = Hq or Hkv)
    block_mask: Optional[torch.Tensor],  # bool [B, 1|Hq, Qb, Kb]
    use_softmax: bool = True,
    scale: Optional[float] = None,
) -> torch.Tensor:
    """fp32 restatement of ``AttnGate.score_compressed_blocks``
    (compact_attn/prefill_sparse/attn_gate.py:173-204, the SEERATTN_DEBUG_GATE_SCORE_FP32 branch):
    (q . k^T) * hidden^-0.5, masked_fill(~mask, finfo.min), softmax over key blocks.
    -> [B, Hq, Qb, Kb] fp32."""
    q = q_blocks.to(torch.float32).transpose(1, 2)
    k = k_blocks.to(torch.float32).transpose(1, 2)
    Hq = q.shape[1]
    if k.shape[1] < Hq:
        k = k.repeat_interleave(Hq // k.shape[1], dim=1)
    if scale is None:
        scale = q.shape[-1] ** -0.5
    attn = torch.matmul(q, k.transpose(-1, -2)) * scale
    if block_mask is not None:
        attn = attn.masked_fill(~block_mask.to(torch.bool), torch.finfo(attn.dtype).min)
    if use_softmax:
        attn = F.softmax(attn, dim=-1)
    return attn


# --------------------------------------------------------------------------------------------
# Row rules on [B, H, Qb, Kb] scores -> bool [B, H, Qb, Kb]
# --------------------------------------------------------------------------------------------
def stable_desc_order(x: torch.Tensor) -> torch.Tensor:
    """Indices that sort the last dim descending, ties broken toward the lower index."""
    return torch.sort(x, dim=-1, descending=True, stable=True).indices


def block_valid_mask(q_blocks: int, kv_blocks: int, past_blocks: int) -> torch.Tensor:
    """valid[i, j] = j <= past_blocks + i  (block-granular causal, chunk at the end). [Qb, Kb]."""
    return torch.arange(kv_blocks).view(1, -1) <= (past_blocks + torch.arange(q_blocks)).view(-1, 1)


def forced_mask(q_blocks: int, kv_blocks: int, past_blocks: int, sink: int, local: int) -> torch.Tensor:
    """Blocks forced on for row i: the first `sink` blocks and the `local` blocks ending at the
    diagonal block past_blocks + i (the mask recipe of the CPU configuration: sink block and the
    diagonal/local blocks forced on).  [Qb, Kb] bool."""
    j = torch.arange(kv_blocks).view(1, -1)
    d = (past_blocks + torch.arange(q_blocks)).view(-1, 1) - j
    return ((j < sink) | ((d >= 0) & (d < local))) & (d >= 0)


def threshold_rows(score: torch.Tensor, valid: torch.Tensor, threshold: float) -> torch.Tensor:
    """keep = score > threshold (strict, fp32 compare) on valid entries.  OR over rows reproduces
    the column rule ``max_i score > threshold`` of ``_build_keep_block_mask``
    (compact_attn/modules/attention_forward_chunked_dense.py:352-403)."""
    return (score.to(torch.float32) > threshold) & valid


def topk_rows(score: torch.Tensor, valid: torch.Tensor, k_per_row: torch.Tensor) -> torch.Tensor:
    """Per-row top-k among valid entries; ties go to the lower block index.

    The reference's only top-k selection is ``torch.topk(score, k, dim=-1)`` + scatter
    (compact_attn/modules/attention_forward.py:43-50, compact_attn/modules/common.py:210-221),
    whose tie order is unspecified; this restatement fixes it.  k_per_row: int [Qb] (or broadcastable
    to score.shape[:-1]); k is clamped to the number of valid entries."""
    s = score.to(torch.float32).masked_fill(~valid, float("-inf"))
    order = stable_desc_order(s)
    rank = torch.empty_like(order)
    rank.scatter_(-1, order, torch.arange(s.shape[-1]).expand_as(order).contiguous())
    k = k_per_row.view(*([1] * (s.dim() - 2)), -1, 1) if k_per_row.dim() == 1 else k_per_row.unsqueeze(-1)
    return (rank < k) & valid.expand_as(s)


def cummass_rows(prob: torch.Tensor, valid: torch.Tensor, tau: float) -> torch.Tensor:
    """Cumulative-mass rule: sort each row's probabilities descending (ties -> lower index), take
    the inclusive prefix sum sequentially in float32, keep the shortest prefix whose mass >= tau
    (the whole valid row if it never reaches tau).  No counterpart in the reference."""
    p = prob.to(torch.float32).masked_fill(~valid, -1.0)  # invalid entries sort last
    order = stable_desc_order(p)
    sorted_p = torch.gather(p, -1, order).clamp_min(0.0).numpy()
    csum = np.cumsum(sorted_p.astype(np.float32), axis=-1, dtype=np.float32)  # sequential fp32
    reached = torch.from_numpy(csum >= np.float32(tau))
    # element r is kept iff the mass *before* it is still below tau
    before = torch.cat([torch.zeros_like(reached[..., :1]), reached[..., :-1]], dim=-1)
    keep_sorted = ~before
    keep = torch.zeros_like(keep_sorted)
    keep.scatter_(-1, order, keep_sorted)
    return keep & valid.expand_as(keep)


def masked_softmax_rows(logits: torch.Tensor, valid: torch.Tensor) -> torch.Tensor:
    """fp32 softmax over the valid entries of each row; invalid entries get probability 0."""
    s = logits.to(torch.float32).masked_fill(~valid, float("-inf"))
    return torch.nan_to_num(F.softmax(s, dim=-1), nan=0.0)


# --------------------------------------------------------------------------------------------
# Seer column rule, unions, block table
# --------------------------------------------------------------------------------------------
def seer_keep_block(
    score: torch.Tensor,  # [B, H, Qb, Kb]
    block_mask: Optional[torch.Tensor],  # bool [B, 1, Qb, Kb] or None (lower-triangular)
    threshold: float,
    keep_recent_blocks: int,
) -> torch.Tensor:
    """``_build_keep_block_mask`` (compact_attn/modules/attention_forward_chunked_dense.py:352-403):
    keep[b,h,j] = (max over valid rows i of score) > threshold, plus the last keep_recent valid
    columns.  -> bool [B, H, Kb]."""
    if block_mask is not None:
        valid = block_mask.to(torch.bool).expand_as(score)
    else:
        valid = torch.tril(torch.ones_like(score, dtype=torch.bool))
    col = score.masked_fill(~valid, float("-inf")).amax(dim=2)
    valid_cols = valid.any(dim=2)
    keep = (col > threshold) & valid_cols
    if keep_recent_blocks > 0:
        rev = torch.cumsum(valid_cols.to(torch.int32).flip(-1), dim=-1).flip(-1)
        keep = keep | ((rev > 0) & (rev <= keep_recent_blocks) & valid_cols)
    return keep


def seer_keep_block_fast(
    score: torch.Tensor, threshold: float, keep_recent_blocks: int, q_len: int, kv_len: int, block_size: int
) -> torch.Tensor:
    """``_build_keep_block_mask_chunked_fast_path`` torch branch
    (compact_attn/modules/attention_forward_chunked_dense.py:559-638): past columns use every row,
    chunk columns use rows i >= j - Pb, then the last keep_recent columns are forced on."""
    B, H, Qb, Kb = score.shape
    Pb = (kv_len - q_len) // block_size
    keep = torch.zeros((B, H, Kb), dtype=torch.bool)
    if Pb > 0:
        keep[..., :Pb] = score[..., :Pb].amax(dim=2) > threshold
    cur = score[..., Pb:Kb]
    Cb = Kb - Pb
    causal = torch.arange(Qb).view(-1, 1) >= torch.arange(Cb).view(1, -1)
    keep[..., Pb:] = cur.masked_fill(~causal.view(1, 1, Qb, Cb), float("-inf")).amax(dim=2) > threshold
    if keep_recent_blocks > 0:
        keep[..., Kb - min(keep_recent_blocks, Kb) :] = True
    return keep


def kv_head_union(keep_block: torch.Tensor, q_len: int, kv_len: int, block_size: int, G: int) -> torch.Tensor:
    """GQA intra-group OR over past columns; every chunk column forced on.
    ``_build_kv_head_union_keep_block_mask``
    (compact_attn/modules/attention_forward_chunked_dense.py:641-683).  [B,Hq,Kb] -> [B,Hkv,Kb]."""
    B, Hq, Kb = keep_block.shape
    Pb = (kv_len - q_len) // block_size
    Hkv = Hq // G
    out = torch.ones((B, Hkv, Kb), dtype=torch.bool)
    if Pb > 0:
        out[..., :Pb] = keep_block[..., :Pb].view(B, Hkv, G, Pb).any(dim=2)
    return out


def block_table_from_kv_keep(
    keep_kv: torch.Tensor, q_len: int, kv_len: int, block_size: int, page_size: int = 256
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Ascending kept past block ids per (b, kv head), -1 padded to capacity Pb, plus counts,
    cache_seqlens = (count + Qb) * bs and pages_per_row = ceil(cache_seqlens / page).

    ``_build_kv_head_past_block_indices_from_kv_keep_block``
    (compact_attn/modules/attention_forward_chunked_dense.py:785-819) and kernel
    ``build_past_indices_and_metadata_from_keep_block_kernel``
    (compact_attn/csrc/compactattn/cache_fill_kernel.cu:328-385).
    -> idx int32 [B,Hkv,max(Pb,1)], counts int32 [B,Hkv], cache_seqlens int32 [B,Hkv], pages int32 [B,Hkv]."""
    B, Hkv, Kb = keep_kv.shape
    Pb = (kv_len - q_len) // block_size
    Qb = Kb - Pb
    idx = torch.full((B, Hkv, max(Pb, 1)), -1, dtype=torch.int32)
    counts = torch.zeros((B, Hkv), dtype=torch.int32)
    for b in range(B):
        for h in range(Hkv):
            sel = torch.nonzero(keep_kv[b, h, :Pb]).flatten().to(torch.int32)
            idx[b, h, : sel.numel()] = sel
            counts[b, h] = sel.numel()
    seqlens = (counts + Qb) * block_size
    pages = (seqlens + page_size - 1) // page_size
    return idx, counts, seqlens.to(torch.int32), pages.to(torch.int32)


def block_union_table(keep_block: torch.Tensor, q_len: int, kv_len: int, block_size: int, G: int):
    """[B,Hq,Kb] -> (idx, counts): ``_build_kv_head_union_past_block_indices``
    (compact_attn/modules/attention_forward_chunked_dense.py:737-782)."""
    keep_kv = kv_head_union(keep_block, q_len, kv_len, block_size, G)
    idx, counts, _, _ = block_table_from_kv_keep(keep_kv, q_len, kv_len, block_size)
    return idx, counts


def flashinfer_index_metadata(keep_kv: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """CSR form over all kept blocks (chunk included): pages_per_row, kv_indptr [R+1], kv_indices
    with global page id row*Kb + blk.  ``_build_index_metadata_reference_from_keep_block_kv``
    (compact_attn/kernels/varlen/flashinfer_zero_copy_prefill.py:482-510)."""
    B, Hkv, Kb = keep_kv.shape
    flat = keep_kv.reshape(B * Hkv, Kb)
    pages = flat.sum(dim=1).to(torch.int32)
    indptr = torch.zeros(B * Hkv + 1, dtype=torch.int32)
    indptr[1:] = pages.cumsum(0)
    gid = (torch.arange(B * Hkv).view(-1, 1) * Kb + torch.arange(Kb).view(1, -1)).to(torch.int32)
    return pages, indptr, gid[flat]


# --------------------------------------------------------------------------------------------
# Gather and attention
# --------------------------------------------------------------------------------------------
def gather_compact_kv(
    k: torch.Tensor,  # [B, K, Hkv, D]
    v: torch.Tensor,
    idx: torch.Tensor,  # int32 [B, Hkv, cap]
    counts: torch.Tensor,  # int32 [B, Hkv]
    q_len: int,
    block_size: int,
    page_size: int = 256,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Copies each row's selected past blocks, then the chunk's blocks, into a paged compact cache
    [pages, page_size, 1, D] with block_table[row, slot] = page_off[row] + slot and
    cache_seqlens[row] = (count + Qb) * bs.

    Same result as ``build_paged_kv_cache_from_token_mask``
    (compact_attn/kernels/varlen/indexed_dense_prefill_varlen.py:1414-1470) fed with the expanded
    keep mask, and as kernels ``cache_fill_from_past_indices_compact_kernel`` +
    ``cache_fill_current_tail_kernel`` (compact_attn/csrc/compactattn/cache_fill_kernel.cu:596-720)."""
    B, K, Hkv, D = k.shape
    P = K - q_len
    Qb = q_len // block_size
    rows = B * Hkv
    seqlens = ((counts.reshape(rows) + Qb) * block_size).to(torch.int32)
    pages = (seqlens + page_size - 1) // page_size
    offs = torch.cumsum(pages, 0) - pages
    total = max(int(pages.sum()), 1)
    kc = torch.zeros((total, page_size, 1, D), dtype=k.dtype)
    vc = torch.zeros((total, page_size, 1, D), dtype=v.dtype)
    table = torch.zeros((rows, max(int(pages.max()), 1)), dtype=torch.int32)
    kflat, vflat = kc.view(total * page_size, D), vc.view(total * page_size, D)
    for r in range(rows):
        b, h = divmod(r, Hkv)
        c = int(counts.reshape(rows)[r])
        toks = compact_token_index(idx.reshape(rows, -1)[r, :c], P, K, block_size)
        base = int(offs[r]) * page_size
        kflat[base : base + toks.numel()] = k[b, toks, h]
        vflat[base : base + toks.numel()] = v[b, toks, h]
        table[r, : int(pages[r])] = int(offs[r]) + torch.arange(int(pages[r]), dtype=torch.int32)
    return kc, vc, table, seqlens


def compact_token_index(blocks: torch.Tensor, past_len: int, kv_len: int, block_size: int) -> torch.Tensor:
    """Token ids of the selected past blocks (ascending) followed by the chunk's tokens."""
    past = (blocks.to(torch.long).view(-1, 1) * block_size + torch.arange(block_size).view(1, -1)).reshape(-1)
    return torch.cat([past, torch.arange(past_len, kv_len)])


def compact_attention(
    q: torch.Tensor,  # [B, Q, Hq, D]
    k: torch.Tensor,  # [B, K, Hkv, D]
    v: torch.Tensor,
    idx: Optional[torch.Tensor],  # int32 [B, Hkv, cap] or None (every past block)
    counts: Optional[torch.Tensor],
    block_size: int,
    softmax_scale: Optional[float] = None,
    return_lse: bool = False,
):
    """fp32 softmax attention of each (b, kv head) row over its compact keys with bottom-right
    causal alignment: compact key c is visible to chunk token t iff c <= L - Q + t.

    Semantics of ``_direct_indexed_prefill_kernel``
    (compact_attn/kernels/varlen/indexed_dense_prefill_direct_triton.py:155-241) and of
    ``flash_attn_with_kvcache(..., causal=True)`` over the gathered cache
    (compact_attn/kernels/varlen/indexed_dense_prefill_varlen.py:1563-1571).  -> [B,Q,Hq,D] fp32."""
    B, Q, Hq, D = q.shape
    K, Hkv = k.shape[1], k.shape[2]
    G = Hq // Hkv
    P = K - Q
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty((B, Q, Hq, D), dtype=torch.float32)
    lse = torch.empty((B, Hq, Q), dtype=torch.float32)
    for b in range(B):
        for h in range(Hkv):
            if idx is None:
                toks = torch.arange(K)
            else:
                toks = compact_token_index(idx[b, h, : int(counts[b, h])], P, K, block_size)
            L = toks.numel()
            kk, vv = k[b, toks, h].to(torch.float32), v[b, toks, h].to(torch.float32)
            qq = q[b, :, h * G : (h + 1) * G].to(torch.float32)
            s = torch.einsum("qgd,ld->gql", qq, kk) * scale
            vis = torch.arange(L).view(1, -1) <= (L - Q + torch.arange(Q)).view(-1, 1)
            s = s.masked_fill(~vis.unsqueeze(0), float("-inf"))
            lse[b, h * G : (h + 1) * G] = torch.logsumexp(s, dim=-1)
            out[b, :, h * G : (h + 1) * G] = torch.einsum("gql,ld->qgd", torch.softmax(s, dim=-1), vv)
    return (out, lse) if return_lse else out


def dense_causal_attention(q, k, v, softmax_scale: Optional[float] = None) -> torch.Tensor:
    """The reference's own non-CUDA attention: repeat_kv + explicit causal mask + SDPA
    (``_flashprefill_dense_fallback``, compact_attn/modules/flashprefill_prefill.py:248-304).
    q [B,Q,Hq,D], k/v [B,K,Hkv,D] -> [B,Q,Hq,D] fp32."""
    B, Q, Hq, D = q.shape
    K, Hkv = k.shape[1], k.shape[2]
    G = Hq // Hkv
    qq = q.to(torch.float32).transpose(1, 2)
    kk = k.to(torch.float32).transpose(1, 2).repeat_interleave(G, dim=1)
    vv = v.to(torch.float32).transpose(1, 2).repeat_interleave(G, dim=1)
    causal = torch.arange(K).view(1, K) <= torch.arange(K - Q, K).view(Q, 1)
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    out = F.scaled_dot_product_attention(qq, kk, vv, attn_mask=causal.view(1, 1, Q, K), scale=scale)
    return out.transpose(1, 2).contiguous()
