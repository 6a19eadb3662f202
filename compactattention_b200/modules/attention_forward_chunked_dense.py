"""Chunked-prefill CompactAttention operators with the reference's signatures.

Mirrors ``compact_attn/modules/attention_forward_chunked_dense.py`` of the reference:
``chunked_prefill_column_dense_attention_forward`` (:2732-2912) and
``chunked_prefill_column_dense_attention_from_keep_block`` (:2147-2729) keep their names,
argument meaning, return contract ``(out, stats | None)`` and ``ValueError`` behaviour, but every
stage runs in ``libcompactattn_b200.so``: selection rule -> packed bits, Block-Union + block table,
and the block-table-indexed tcgen05 attention kernel that reads the selected KV blocks in place
(there is no materialised compact cache on this route and no host synchronisation).

Differences a caller can observe, all deliberate:
* ``pack_impl`` / ``indexed_impl`` / ``cache_fill_backend`` are accepted (every value the
  reference accepts, plus ``"b200_native"``) but select nothing: there is one implementation.
  Two values keep their meaning because they change the result, not the backend:
  ``"fi_zero_copy_per_query"`` builds one block table per query head (no GQA union) and
  ``"fi_zero_copy_subgroup"`` one per sub-group of ``SEER_ZC_QUERY_SUBGROUP_SIZE`` query heads
  (reference :863-895, :2185-2196); both run the same attention kernel with several table rows
  per KV head.
* Padded batches (an ``attention_mask`` containing zeros), lengths that are not multiples of the
  block size and head dims other than 128 raise ``NotImplementedError`` instead of falling down the
  reference's ladder of slower paths; the reference only takes its indexed path under the same
  preconditions (:993-999, :2267-2277).
* ``block_attention_mask=None`` selects with block-causal validity for a chunk at the end of the cache
  (row i sees key block j iff j <= Pb + i).  The reference's generic mask builder uses
  ``torch.tril`` over the ``[Qb, Kb]`` slice instead (j <= i, :374), which is only meaningful for a
  first chunk; every model integration passes the mask, and with a mask the two agree.
* ``keep_recent_blocks`` forces the last N columns on; the reference forces the last N *valid*
  columns (:398-401).  The two agree whenever the last columns are visible to some row, which holds
  for every block-causal mask.
* The reference's debug switches ``SEERATTN_DEBUG_COMPACTATTN_QUERY_BLOCK_MODE=last`` (only the chunk's
  last Q-block votes, :377-379), ``..._KV_HEAD_MODE=first`` and ``..._DISABLE_CURRENT_OPEN`` (:127-141)
  are refused with ``NotImplementedError``; ``..._THRESHOLD_OVERRIDE`` and ``..._KEEP_RECENT_OVERRIDE``
  are honoured.
* ``attention_mask`` is assumed all-ones when given (checking would need a device-to-host sync,
  which the reference performs once and caches, :529-543); pass ``None`` for the common case.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple, Union

import torch

from .. import ops

COMPACTATTN_VERSION = "CompactAttn-B200-v0.1"

_INDEXED_IMPLS = {
    "fa2_paged", "triton_direct", "fa2_indexed", "fi_paged", "fi_zero_copy", "fi_zero_copy_per_query",
    "fi_zero_copy_subgroup", "cudnn_one_shot", "b200_native",
}


def _timed(fn, enabled: bool):
    """CUDA-event timing of one stage on the current stream (the reference's ``_cuda_elapsed_ms``, :52-61)."""
    if not enabled:
        return fn(), 0.0
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    out = fn()
    end.record()
    end.synchronize()
    return out, float(start.elapsed_time(end))


def _effective_threshold(threshold):
    """``SEERATTN_DEBUG_COMPACTATTN_THRESHOLD_OVERRIDE`` is honoured like the reference (:139-160)."""
    raw = os.environ.get("SEERATTN_DEBUG_COMPACTATTN_THRESHOLD_OVERRIDE", "")
    if raw:
        try:
            return float(raw)
        except ValueError:
            pass
    return threshold


def _effective_keep_recent(default: int) -> int:
    """``SEERATTN_DEBUG_COMPACTATTN_KEEP_RECENT_OVERRIDE`` is honoured like the reference (:142-150)."""
    raw = os.environ.get("SEERATTN_DEBUG_COMPACTATTN_KEEP_RECENT_OVERRIDE")
    if raw is None:
        return int(default)
    try:
        return max(int(raw), 0)
    except ValueError:
        return int(default)


def _refuse_debug_modes() -> None:
    """The reference's debug switches that change which blocks are selected (:127-141) have no
    counterpart in the kernels; running with one of them set would silently select differently."""
    def mode(name):
        return os.environ.get(name, "").strip().lower()
    if mode("SEERATTN_DEBUG_COMPACTATTN_QUERY_BLOCK_MODE") == "last":
        raise NotImplementedError("SEERATTN_DEBUG_COMPACTATTN_QUERY_BLOCK_MODE=last is not supported by the B200 path")
    if mode("SEERATTN_DEBUG_COMPACTATTN_KV_HEAD_MODE") == "first":
        raise NotImplementedError("SEERATTN_DEBUG_COMPACTATTN_KV_HEAD_MODE=first is not supported by the B200 path")
    if mode("SEERATTN_DEBUG_COMPACTATTN_DISABLE_CURRENT_OPEN") in {"1", "true", "yes", "on"}:
        raise NotImplementedError("SEERATTN_DEBUG_COMPACTATTN_DISABLE_CURRENT_OPEN is not supported by the B200 path")


def _kv_dims(key_states, kv_len: Optional[int]):
    """``(kv_len, num_kv_heads)`` of a ``[B,K,Hkv,D]`` tensor or of a paged ``ops.KvCacheView`` (whose
    logical length must be given by the caller)."""
    if isinstance(key_states, ops.KvCacheView):
        if kv_len is None:
            raise ValueError("kv_len is required when key_states is a KvCacheView")
        return int(kv_len), int(key_states.k.shape[-2])
    return int(key_states.shape[1]), int(key_states.shape[2])


_MASK_VERIFIED: Dict[Tuple[str, int, int], bool] = {}


def clear_fast_path_content_cache() -> None:
    """Forget which (device, batch, kv_len) attention masks were verified all-ones (the reference's
    function of this name, :551-553; call between sequences)."""
    _MASK_VERIFIED.clear()


def _check_attention_mask(attention_mask, kv_len: int) -> None:
    """Token masks must be all ones on this path.  The content check costs a device-to-host read, so it
    runs once per (device, batch, kv_len) - the reference caches its verification the same way."""
    if attention_mask is None:
        return
    key = (str(attention_mask.device), int(attention_mask.shape[0]), int(kv_len))
    if _MASK_VERIFIED.get(key):
        return
    if attention_mask.dim() == 2 and not bool(attention_mask[:, -kv_len:].to(torch.bool).all().item()):
        raise NotImplementedError("padded batches (an attention_mask with zeros) are not supported by the B200 path")
    _MASK_VERIFIED[key] = True


def _check_common(query_states, key_states, value_states, query_length, block_size, indexed_impl, kv_len=None):
    if query_length <= 1:
        raise ValueError("chunked compact attention expects query_length > 1.")
    if block_size <= 0:
        raise ValueError("block_size must be positive.")
    if indexed_impl not in _INDEXED_IMPLS:
        raise ValueError(f"Unsupported indexed_impl: {indexed_impl}")
    k_t = key_states.k if isinstance(key_states, ops.KvCacheView) else key_states
    v_t = value_states.v if isinstance(value_states, ops.KvCacheView) else value_states
    if not (query_states.is_cuda and k_t.is_cuda and v_t.is_cuda):
        raise RuntimeError("compactattention_b200 has no CPU path: tensors must live on a CUDA device")
    if query_states.dtype not in (torch.float16, torch.bfloat16) or k_t.dtype != query_states.dtype \
            or v_t.dtype != query_states.dtype:
        raise NotImplementedError("the B200 path computes in bf16/f16; q, k, v must share one of these dtypes")
    if query_states.shape[-1] != 128:
        raise NotImplementedError("the B200 path supports head_dim 128 only")
    if block_size % 64:
        raise NotImplementedError(f"block_size ({block_size}) must be a multiple of 64")


def _dense_fallback(query_states, key_states, value_states, k_hf, v_hf, kv_len, num_kv_heads, block_size, softmax_scale, timing,
                    path: str):
    """Dense causal attention over the whole cache with the same kernel: the reference's route for a
    past length that is not a block multiple (``_dense_prefill_full_kv``, :2413-2423)."""
    kv = _kv_view(key_states, value_states, k_hf, v_hf)
    out, ms = _timed(lambda: ops.attn_compact(query_states, kv, kv_len, num_kv_heads, None, None, block_size=block_size,
                                              softmax_scale=softmax_scale), timing)
    if not timing:
        return out, None
    return out, {"dense_kernel_ms": ms, "col_indexed_dense_kernel_ms": 0.0, "col_index_build_ms": 0.0, "fallback_used": 1.0,
                 "col_indexed_dense_tail_dense_fallback_calls": 1.0, "path": path, "compactattn_version": COMPACTATTN_VERSION}


def _kv_view(key_states, value_states, k_hf, v_hf) -> ops.KvCacheView:
    """Source KV addressing: a caller-made ``KvCacheView`` (paged cache) passes through; tensors are
    viewed in place, seq-first ``[B,K,Hkv,D]`` or, for B == 1, heads-first ``k_hf [B,Hkv,K,D]``."""
    if isinstance(key_states, ops.KvCacheView):
        return key_states
    if key_states.stride(3) == 1 and (key_states.shape[0] == 1 or key_states.shape[1] % 64 != 0
                                      or key_states.stride(0) == key_states.shape[1] * key_states.stride(1)):
        return ops.KvCacheView.from_seq_first(key_states, value_states)
    if k_hf is not None and v_hf is not None and k_hf.shape[0] == 1:
        return ops.KvCacheView.from_heads_first(k_hf, v_hf)
    return ops.KvCacheView.from_seq_first(key_states.contiguous(), value_states.contiguous())


def chunked_prefill_column_dense_attention_from_keep_block(
    query_states: torch.Tensor,  # [B, Q, Hq, D]
    key_states: torch.Tensor,  # [B, K, Hkv, D]
    value_states: torch.Tensor,  # [B, K, Hkv, D]
    keep_block: Optional[torch.Tensor],  # [B, Hq, Kb]
    attention_mask: Optional[torch.Tensor],  # [B, K]
    query_length: int,
    softmax_scale: float,
    block_size: int = 64,
    num_key_value_groups: int = 1,
    pack_impl: str = "torch",
    indexed_impl: str = "fa2_paged",
    cache_fill_backend: str = "auto",
    return_stats: bool = False,
    valid_block: Optional[torch.Tensor] = None,  # [B, Hq, Kb]
    allow_indexed_dense: bool = False,
    keep_block_kv_preprojected: Optional[torch.Tensor] = None,  # [B, Hkv, Kb]
    attn_module=None,
    k_hf: Optional[torch.Tensor] = None,
    v_hf: Optional[torch.Tensor] = None,
    _row_bits: Optional[torch.Tensor] = None,  # packed bits [B, H, Qin, W] from ops.select_rows (internal)
    _keep_recent: int = 0,
    kv_len: Optional[int] = None,  # logical length when key_states is a paged ops.KvCacheView
) -> Tuple[torch.Tensor, Optional[Dict[str, float]]]:
    """Block-Union KV selection from a keep mask, then dense causal attention over the kept blocks.

    Same contract as the reference function of this name (:2147-2167): ``keep_block`` is the
    per-query-head column mask, ``keep_block_kv_preprojected`` the per-KV-head one (wins when both
    are given); the chunk's own blocks are always attended.
    """
    _check_common(query_states, key_states, value_states, query_length, block_size, indexed_impl, kv_len)
    bsz, q_len, num_q_heads, _ = query_states.shape
    kv_len, num_kv_heads = _kv_dims(key_states, kv_len)
    kv_blocks = (kv_len + block_size - 1) // block_size
    if keep_block is None and keep_block_kv_preprojected is None and _row_bits is None:
        raise ValueError("Either keep_block or keep_block_kv_preprojected must be provided.")
    if keep_block is not None and keep_block.shape != (bsz, num_q_heads, kv_blocks):
        raise ValueError(f"keep_block shape mismatch: expected {(bsz, num_q_heads, kv_blocks)}, got {tuple(keep_block.shape)}")
    # block-table rows per KV head: 1 (Block-Union over the GQA group), G (per query head) or G / sub-group size
    rows_per_kv = 1
    if indexed_impl == "fi_zero_copy_per_query":
        if keep_block is None and _row_bits is None:
            raise ValueError("fi_zero_copy_per_query requires q-head keep_block")
        rows_per_kv = num_key_value_groups
    elif indexed_impl == "fi_zero_copy_subgroup":
        query_subgroup_size = int(os.environ.get("SEER_ZC_QUERY_SUBGROUP_SIZE", "4"))
        if query_subgroup_size <= 0 or num_key_value_groups % query_subgroup_size != 0:
            raise ValueError("SEER_ZC_QUERY_SUBGROUP_SIZE must divide num_key_value_groups: "
                             f"{query_subgroup_size} vs {num_key_value_groups}")
        if keep_block_kv_preprojected is None:
            raise ValueError("fi_zero_copy_subgroup requires subgroup keep_block")
        rows_per_kv = num_key_value_groups // query_subgroup_size
    table_rows = num_kv_heads * rows_per_kv
    expected_kv_projected_shape = (bsz, table_rows if indexed_impl == "fi_zero_copy_subgroup" else num_kv_heads, kv_blocks)
    if keep_block_kv_preprojected is not None and keep_block_kv_preprojected.shape != expected_kv_projected_shape:
        raise ValueError("keep_block_kv_preprojected shape mismatch: "
                         f"expected {expected_kv_projected_shape}, got {tuple(keep_block_kv_preprojected.shape)}")
    if valid_block is not None:
        if keep_block is None:
            raise ValueError("valid_block requires keep_block to be provided.")
        if valid_block.shape != keep_block.shape:
            raise ValueError(f"valid_block shape mismatch: expected {tuple(keep_block.shape)}, got {tuple(valid_block.shape)}")
    if num_q_heads != num_kv_heads * num_key_value_groups:
        raise ValueError("num_key_value_groups does not match the head counts")
    _check_attention_mask(attention_mask, kv_len)
    past_blocks = (kv_len - q_len) // block_size
    timing = bool(return_stats)
    if (kv_len - q_len) % block_size != 0:
        return _dense_fallback(query_states, key_states, value_states, k_hf, v_hf, kv_len, num_kv_heads, block_size,
                               softmax_scale, timing, "dense_misaligned_past")

    def _build():
        if _row_bits is not None:
            return ops.union_table(bits=_row_bits, num_kv_heads=table_rows, kv_blocks=kv_blocks, past_blocks=past_blocks,
                                   block_size=block_size, keep_recent=_keep_recent, want_keep_kv=timing)
        src = keep_block_kv_preprojected if keep_block_kv_preprojected is not None else keep_block
        if indexed_impl == "fi_zero_copy_per_query":
            src = keep_block  # the per-query route ignores a KV-head mask, like the reference (:863-871)
        if valid_block is not None and keep_block_kv_preprojected is None:
            src = src & valid_block.to(torch.bool)
        src = src if src.dtype in (torch.bool, torch.uint8) else src.to(torch.bool)
        return ops.union_table(mask=src, num_kv_heads=table_rows, kv_blocks=kv_blocks, past_blocks=past_blocks,
                               block_size=block_size, keep_recent=_keep_recent, want_keep_kv=timing)

    table, index_ms = _timed(_build, timing)
    kv = _kv_view(key_states, value_states, k_hf, v_hf)
    if rows_per_kv > 1:
        kv = kv.with_head_div(rows_per_kv)
    out, attn_ms = _timed(
        lambda: ops.attn_compact(query_states, kv, kv_len, table_rows, table.block_idx, table.counts,
                                 block_size=block_size, softmax_scale=softmax_scale),
        timing,
    )
    if not return_stats:
        return out, None
    selected = float(table.keep_kv.sum().item())
    valid = float(table.keep_kv.numel())
    stats = {
        "col_index_build_ms": index_ms,
        "col_indexed_dense_kernel_ms": attn_ms,
        "dense_kernel_ms": attn_ms,
        "col_selected_kv_materialize_ms": 0.0,  # blocks are read in place: nothing is materialised
        "gather_pack_ms": 0.0,
        "fallback_used": 0.0,
        "selected_blocks": selected,
        "valid_blocks": valid,
        "select_ratio": selected / valid if valid else 1.0,
        "selected_tokens": selected * block_size,
        "valid_tokens": valid * block_size,
        "col_indexed_dense_calls": 1.0,
        "path": "chunked_selected",
        "compactattn_version": COMPACTATTN_VERSION,
    }
    return out, stats


def chunked_prefill_column_dense_attention_forward(
    query_states: torch.Tensor,  # [B, Q, Hq, D]
    key_states: torch.Tensor,  # [B, K, Hkv, D]
    value_states: torch.Tensor,  # [B, K, Hkv, D]
    attention_mask: Optional[torch.Tensor],  # [B, K]
    query_length: int,
    softmax_scale: Optional[float] = None,
    attn_gate_score: Optional[torch.Tensor] = None,  # [B, Hq|Hkv, Qb, Kb]
    block_attention_mask: Optional[torch.Tensor] = None,  # [B, 1, Qb, Kb]
    threshold: Union[float, torch.Tensor] = 0.0,
    keep_recent_blocks: int = 2,
    block_size: int = 64,
    num_key_value_groups: int = 1,
    attn_gate_is_kv_group_aware: bool = False,
    pack_impl: str = "torch",
    indexed_impl: str = "fa2_paged",
    cache_fill_backend: str = "auto",
    return_stats: bool = False,
    attn_module=None,
    k_hf: Optional[torch.Tensor] = None,
    v_hf: Optional[torch.Tensor] = None,
    kv_len: Optional[int] = None,  # logical length when key_states is a paged ops.KvCacheView
) -> Tuple[torch.Tensor, Optional[Dict[str, float]]]:
    """Threshold selection on gate scores, Block-Union, then compact attention.

    Same contract as the reference function of this name (:2732-2753).  A key block is kept for a
    query head when any valid Q-block row scores above ``threshold`` (strict, fp32 compare, :352-403
    / kernels ``build_keep_*_fast_kernel``); the last ``keep_recent_blocks`` columns are forced on;
    the G heads of a KV head are OR-ed; the chunk's own blocks are always attended.
    """
    if attn_gate_score is None:
        raise ValueError("attn_gate_score is required for chunked column-dense attention.")
    _check_common(query_states, key_states, value_states, query_length, block_size, indexed_impl, kv_len)
    threshold = _effective_threshold(threshold)
    _refuse_debug_modes()
    keep_recent_blocks = _effective_keep_recent(keep_recent_blocks)
    bsz, q_len, num_q_heads, head_dim = query_states.shape
    kv_len, num_kv_heads = _kv_dims(key_states, kv_len)
    if isinstance(threshold, torch.Tensor) and (threshold.dim() > 1 or threshold.numel() not in (1, bsz)):
        raise ValueError(f"Expected scalar or 1D batch threshold tensor, got shape={tuple(threshold.shape)}")
    if softmax_scale is None:
        softmax_scale = head_dim ** -0.5
    if (kv_len - q_len) % block_size != 0:
        _check_attention_mask(attention_mask, kv_len)
        return _dense_fallback(query_states, key_states, value_states, k_hf, v_hf, kv_len, num_kv_heads, block_size,
                               softmax_scale, bool(return_stats), "dense_misaligned_past")
    kv_blocks = (kv_len + block_size - 1) // block_size
    q_blocks = (q_len + block_size - 1) // block_size
    if attn_gate_score.dim() != 4 or attn_gate_score.shape[0] != bsz or attn_gate_score.shape[2] != q_blocks:
        raise ValueError(f"attn_gate_score must be [B, H, {q_blocks}, Kb], got {tuple(attn_gate_score.shape)}")
    gate_heads = attn_gate_score.shape[1]
    expect_heads = num_kv_heads if attn_gate_is_kv_group_aware else num_q_heads
    if gate_heads != expect_heads:
        raise ValueError(f"attn_gate_score has {gate_heads} heads, expected {expect_heads}")
    score_blocks = attn_gate_score.shape[3]
    if score_blocks > kv_blocks:
        raise ValueError(f"short keep_block width {score_blocks} exceeds expected KV blocks {kv_blocks}")
    if softmax_scale is None:
        softmax_scale = head_dim ** -0.5
    timing = bool(return_stats)
    past_blocks = kv_blocks - q_blocks
    # a score tensor narrower than the cache covers its last `score_blocks` key blocks (:708-734)
    missing = kv_blocks - score_blocks
    if missing > past_blocks:
        raise NotImplementedError("gate scores must at least cover the chunk's own key blocks")
    valid = None
    if block_attention_mask is not None:
        # nonzero = visible, the conversion the reference's mask builder applies (:372)
        valid = block_attention_mask[..., -q_blocks:, -score_blocks:].to(torch.bool)

    def _select():
        return ops.select_rows(attn_gate_score, past_blocks - missing, "threshold", valid=valid,
                               threshold=threshold if isinstance(threshold, torch.Tensor) else float(threshold))

    bits, select_ms = _timed(_select, timing)
    if missing:
        # left-pad the packed columns with `missing` never-selected blocks
        full = ops.unpack_bits(bits, score_blocks)
        mask = torch.zeros((*full.shape[:-1], kv_blocks), dtype=torch.bool, device=full.device)
        mask[..., missing:] = full
        keep = mask.any(dim=2)
        if keep_recent_blocks > 0:
            keep[..., kv_blocks - min(int(keep_recent_blocks), kv_blocks):] = True
        out, stats = chunked_prefill_column_dense_attention_from_keep_block(
            query_states, key_states, value_states,
            keep_block=None if attn_gate_is_kv_group_aware else keep,
            attention_mask=attention_mask, query_length=query_length, softmax_scale=softmax_scale, block_size=block_size,
            num_key_value_groups=num_key_value_groups, pack_impl=pack_impl, indexed_impl=indexed_impl,
            cache_fill_backend=cache_fill_backend, return_stats=return_stats, allow_indexed_dense=True,
            keep_block_kv_preprojected=keep if attn_gate_is_kv_group_aware else None, attn_module=attn_module, k_hf=k_hf, v_hf=v_hf, kv_len=kv_len)
    else:
        out, stats = chunked_prefill_column_dense_attention_from_keep_block(
            query_states, key_states, value_states, keep_block=None, attention_mask=attention_mask,
            query_length=query_length, softmax_scale=softmax_scale, block_size=block_size,
            num_key_value_groups=num_key_value_groups, pack_impl=pack_impl, indexed_impl=indexed_impl,
            cache_fill_backend=cache_fill_backend, return_stats=return_stats, allow_indexed_dense=True,
            attn_module=attn_module, k_hf=k_hf, v_hf=v_hf, _row_bits=bits, _keep_recent=max(int(keep_recent_blocks), 0),
            kv_len=kv_len)
    if not return_stats:
        return out, None
    stats.update({
        "col_select_mask_ms": select_ms,
        "col_select_mask_past_ms": select_ms,
        "col_select_mask_curr_ms": 0.0,
        "col_select_mask_fastpath_calls": 1.0,
        "col_select_mask_generic_calls": 0.0,
        "compactattn_version": COMPACTATTN_VERSION,
    })
    return out, stats
