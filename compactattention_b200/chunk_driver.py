"""One attention layer's chunked-prefill step on one GPU: selector -> Block-Union table -> compact
attention, with every buffer pre-allocated so a step is a fixed sequence of kernel launches with no
host synchronisation.  It is what the benchmark times and what the attention modules call.

Selectors (reference anchors in ``compact_attn``):
* ``gate``   learned AttnGate over a growing K-block cache, then a per-row rule
             (prefill_sparse/attn_gate.py:37-222, llama/modeling_llama_seerattn.py:437-481);
* ``flashprefill``  mean-K cache + per-token block score + alpha * row-max rule
             (modules/flashprefill_prefill.py:880-1189).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import ops
from .paged_cache import PagedKVCache
from .prefill_sparse.attn_gate import AttnGate, GateKeyBlockCache


@dataclass
class SelectionRule:
    """Per-row rule applied to the selector's scores (see ``ca_select_rows``)."""

    rule: str = "threshold"  # threshold | topk | cummass | alpha_rowmax
    softmax: bool = True
    threshold: float = 5e-4
    alpha: float = 0.06
    topk_ratio: Optional[Tuple[int, int]] = None
    topk_k: int = 0
    min_budget: int = 0
    sink: int = 0
    local: int = 0
    keep_recent: int = 0
    last_n_block: int = 0


class GateSelectorState:
    """Learned-gate selector state of one layer: the gate, its K-block cache and scratch buffers."""

    def __init__(self, gate: AttnGate, batch: int, device, cache_dtype=torch.bfloat16):
        self.gate = gate
        heads = gate.mask_linear_k.weight.shape[0]
        self.cache = GateKeyBlockCache(batch, heads, gate.hidden_size, device, dtype=cache_dtype)
        self.q_blocks = None  # [B, Qb, Hq, C] scratch of the current chunk
        self.logits = None    # [B, Hq, Qb, Kb] scratch of the current chunk

    def append(self, q_nope: torch.Tensor, k_nope: torch.Tensor, block_rope_q=None, block_rope_k=None) -> int:
        """Pools, projects and ropes the chunk's Q blocks (into scratch) and K blocks (appended to the
        cache): one launch.  Returns the number of blocks appended."""
        gate = self.gate
        nb = (q_nope.shape[1] + gate.block_size - 1) // gate.block_size
        self.cache.reserve(self.cache.length + nb)
        if self.q_blocks is None or self.q_blocks.shape[1] != nb:
            self.q_blocks = torch.empty((q_nope.shape[0], nb, gate.num_q_head, gate.hidden_size), dtype=torch.float32,
                                        device=q_nope.device)
        wq = None if gate.mask_linear_q is None else gate.mask_linear_q.weight.detach()
        ops.gate_prepare(q_nope, k_nope, gate.block_size, gate.q_pooling_funcs, gate.k_pooling_funcs, wq,
                         gate.mask_linear_k.weight.detach(), block_rope_q, block_rope_k, self.q_blocks,
                         self.cache.blocks_view(), self.cache.length)
        self.cache.length += nb
        return nb

    def score(self) -> torch.Tensor:
        """Scores the chunk's Q blocks (from the last ``append``) against every cached block: one launch.
        Returns logits ``[B, Hq, Qb, Kb]`` (float32, acausal entries = finfo.min)."""
        gate, nb = self.gate, self.q_blocks.shape[1]
        kb = self.cache.blocks()
        if self.logits is None or self.logits.shape[3] != kb.shape[1] or self.logits.shape[2] != nb:
            self.logits = torch.empty((self.q_blocks.shape[0], gate.num_q_head, nb, kb.shape[1]), dtype=torch.float32,
                                      device=self.q_blocks.device)
        return ops.gate_scores(self.q_blocks, kb, kb.shape[1] - nb, scale=gate.scale, out=self.logits)

    def append_and_score(self, q_nope: torch.Tensor, k_nope: torch.Tensor, block_rope_q=None, block_rope_k=None) -> torch.Tensor:
        """``append`` then ``score`` (two launches)."""
        self.append(q_nope, k_nope, block_rope_q, block_rope_k)
        return self.score()


class MeanKSelectorState:
    """Training-free selector state of one layer: the mean-K cache ``[B, capacity, Hkv, D]``."""

    def __init__(self, batch: int, max_blocks: int, num_kv_heads: int, head_dim: int, block_size: int, device, dtype):
        self.block_size = block_size
        self.mean_k = torch.empty((batch, max_blocks, num_kv_heads, head_dim), dtype=dtype, device=device)
        self.length = 0

    def append_and_score(self, q: torch.Tensor, k_chunk: torch.Tensor, kv_len: int) -> torch.Tensor:
        nb = -(-k_chunk.shape[1] // self.block_size)
        ops.pool_blocks(k_chunk, self.block_size, ("avg",), out=self.mean_k, out_block_offset=self.length)
        self.length += nb
        _, _, norm = ops.flashprefill_score(q, self.mean_k[:, : self.length], kv_len, self.block_size)
        return norm.permute(0, 3, 1, 2)  # [B, Hq, Qb, Kb] view


def select_and_attend(
    q: torch.Tensor,  # [B, Q, Hq, D] post-RoPE queries of the chunk
    kv: ops.KvCacheView,
    kv_len: int,
    num_kv_heads: int,
    score: torch.Tensor,  # [B, Hq, Qb, Kb] selector scores / logits (any strides)
    rule: SelectionRule,
    block_size: int,
    softmax_scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None,
    table: Optional[ops.BlockTable] = None,
    bits: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
):
    """Row rule + Block-Union table (one launch) -> compact attention.  Returns (out, table).  ``bits`` is
    only written when given (a caller that wants the per-row selection)."""
    Qb, Kb = score.shape[2], score.shape[3]
    rows_voting = 0
    if rule.last_n_block > 0 and Qb > 1:
        rows_voting = max(Qb - min(rule.last_n_block, Qb - 1), 1)
    table = ops.select_union_table(score, Kb - Qb, rule.rule, num_kv_heads=num_kv_heads, block_size=block_size,
                                   keep_recent=rule.keep_recent, softmax=rule.softmax, threshold=rule.threshold, alpha=rule.alpha,
                                   topk_k=rule.topk_k, topk_ratio=rule.topk_ratio, min_budget=rule.min_budget, sink=rule.sink,
                                   local=rule.local, rows_voting=rows_voting, bits=bits, out=table)
    out = ops.attn_compact(q, kv, kv_len, num_kv_heads, table.block_idx, table.counts, block_size=block_size,
                           softmax_scale=softmax_scale, out=out, status=status)
    return out, table


def capture_step(fn, warmup: int = 2) -> "torch.cuda.CUDAGraph":
    """Captures ``fn()`` — a fixed sequence of this library's launches on pre-allocated buffers, e.g.
    selector scores -> row rule -> Block-Union table -> attention at one chunk position — into a CUDA
    graph and returns it; ``graph.replay()`` then enqueues the whole step with one host call.

    The entry points need nothing special for this: they allocate nothing, never synchronise, and
    their per-device attributes and the attention workspace of the capturing stream are set up by
    the warm-up calls, which run on a side stream before the capture as torch requires.  A step is
    only replayable while its shapes hold (the chunk position is baked into the launch parameters),
    which is the case for a layer stack at one chunk position and for a benchmark loop.
    """
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(max(warmup, 1)):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return graph

