"""Training-free (FlashPrefill) selector driving compact attention, with the reference's signature.

Mirrors ``flashprefill_compactattn_prefill_full_kv``
(``compact_attn/modules/flashprefill_prefill.py:880-1189`` of the reference): mean-K pooling (or a
caller-maintained mean-K cache), per-token Q x mean-K block scores with normalisation, the
alpha * row-max rule with sink / window / min-budget, Block-Union, and compact attention.  Every
stage is a kernel of ``libcompactattn_b200.so``; the first chunk (``kv_len == q_len``) runs the same
attention kernel over every block (dense causal attention).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import ops
from .attention_forward_chunked_dense import (
    COMPACTATTN_VERSION,
    _check_common,
    _kv_dims,
    _kv_view,
    _timed,
    chunked_prefill_column_dense_attention_from_keep_block,
)


def flashprefill_compactattn_prefill_full_kv(
    query_states: torch.Tensor,  # [B, Q, Hq, D] (post-RoPE)
    key_states: torch.Tensor,  # [B, K, Hkv, D]
    value_states: torch.Tensor,
    attention_mask: Optional[torch.Tensor],
    *,
    softmax_scale: float,
    num_key_value_groups: int,
    block_size: int,
    attention_sink: int,
    window_size: int,
    alpha: float,
    last_n_block: int,
    min_budget: int,
    pack_impl: str,
    indexed_impl: str,
    cache_fill_backend: str,
    measure_timing: bool = False,
    attn_module=None,
    k_hf: Optional[torch.Tensor] = None,
    v_hf: Optional[torch.Tensor] = None,
    mean_k_cache: Optional[torch.Tensor] = None,  # [B, Kb, Hkv, D]
    kv_len: Optional[int] = None,  # logical length when key_states is a paged ops.KvCacheView
) -> Tuple[torch.Tensor, Dict[str, float]]:
    q_len = int(query_states.shape[1])
    kv_len, num_kv_heads = _kv_dims(key_states, kv_len)
    if q_len <= 1:
        raise NotImplementedError("decode (q_len == 1) is not on the chunked-prefill path of this library")
    _check_common(query_states, key_states, value_states, q_len, block_size, indexed_impl, kv_len)
    if kv_len <= q_len:
        # first chunk: dense causal attention (the reference takes its dense route here, :904-935)
        kv = _kv_view(key_states, value_states, k_hf, v_hf)
        out, ms = _timed(lambda: ops.attn_compact(query_states, kv, kv_len, num_kv_heads, None, None,
                                                  block_size=block_size, softmax_scale=softmax_scale), measure_timing)
        stats = {"dense_kernel_ms": ms, "fallback_used": 0.0, "flashprefill_select_ms": 0.0,
                 "flashprefill_selected_blocks": 0.0, "flashprefill_query_blocks": 0.0, "flashprefill_key_blocks": 0.0}
        return out, (stats if measure_timing else {})

    if (kv_len - q_len) % block_size != 0:
        # a past that is not a block multiple: dense over the whole cache (the reference's dense fallback, :904-935)
        from .attention_forward_chunked_dense import _dense_fallback
        out, stats = _dense_fallback(query_states, key_states, value_states, k_hf, v_hf, kv_len, num_kv_heads, block_size,
                                     softmax_scale, measure_timing, "dense_misaligned_past")
        return out, (stats or {})
    q_blocks, kv_blocks = -(-q_len // block_size), -(-kv_len // block_size)
    past_blocks = (kv_len - q_len) // block_size

    def _score():
        if mean_k_cache is None and isinstance(key_states, ops.KvCacheView):
            raise ValueError("a paged KvCacheView needs a mean_k_cache (the pooled keys are kept beside the cache)")
        mean_k = mean_k_cache if mean_k_cache is not None else ops.pool_blocks(
            key_states, block_size, ("avg",), out_dtype=key_states.dtype)
        if mean_k.shape[1] != kv_blocks:
            raise ValueError(f"mean_k_cache has {mean_k.shape[1]} blocks, expected {kv_blocks}")
        # The alpha * row-max rule (and its top-k minimum budget) does not depend on the row's normalising sum: the
        # rule kernel takes score_raw and max_raw and forms score_raw * 2^(max_raw - row max) itself, so the
        # normalisation launch and its [B, Qb, Kb, Hq] output are skipped.
        raw, mx, _ = ops.flashprefill_score(query_states, mean_k, kv_len, block_size, normalize=False)
        return raw, mx

    (score, score_max), select_ms = _timed(_score, measure_timing)
    tail = min(max(int(last_n_block), 0), q_blocks - 1) if q_blocks > 1 else 0

    def _rule():
        return ops.select_rows(score.permute(0, 3, 1, 2), past_blocks, "alpha_rowmax", alpha=float(alpha),
                               sink=int(attention_sink), local=int(window_size), min_budget=int(min_budget),
                               rows_voting=max(q_blocks - tail, 1), score_max=score_max.permute(0, 3, 1, 2))

    bits, union_ms = _timed(_rule, measure_timing)
    out, compact_stats = chunked_prefill_column_dense_attention_from_keep_block(
        query_states, key_states, value_states, keep_block=None, attention_mask=attention_mask, query_length=q_len,
        softmax_scale=softmax_scale, block_size=block_size, num_key_value_groups=num_key_value_groups, pack_impl=pack_impl,
        indexed_impl=indexed_impl, cache_fill_backend=cache_fill_backend, return_stats=measure_timing,
        allow_indexed_dense=True, attn_module=attn_module, k_hf=k_hf, v_hf=v_hf, _row_bits=bits, kv_len=kv_len)
    if not measure_timing:
        return out, {}
    stats = dict(compact_stats or {})
    stats.update({
        "flashprefill_select_ms": select_ms,
        "flashprefill_union_ms": union_ms,
        "flashprefill_fused_kv_union_calls": 1.0,
        "flashprefill_mean_k_cache_used": 1.0 if mean_k_cache is not None else 0.0,
        "flashprefill_selected_blocks": stats.get("selected_blocks", 0.0),
        "flashprefill_query_blocks": float(q_blocks),
        "flashprefill_key_blocks": float(kv_blocks),
        "flashprefill_pooled_query_blocks": float(max(q_blocks - tail, 1)),
        "compactattn_version": COMPACTATTN_VERSION,
    })
    return out, stats
