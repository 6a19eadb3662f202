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

import ctypes
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

    def score_select(self, rule: "SelectionRule", num_kv_heads: int, block_size: int, *, table=None, bits=None,
                     write_scores: bool = False, rows_voting: int = 0) -> ops.BlockTable:
        """Scores the chunk's Q blocks (from the last ``append``) against every cached block, applies the row
        rule and builds the Block-Union table: one library call (``ca_gate_score_select``), two launches - the
        tensor-core score kernel and the rule + union + table kernel."""
        gate, nb = self.gate, self.q_blocks.shape[1]
        kb = self.cache.blocks()
        if self.logits is None or self.logits.shape[3] != kb.shape[1] or self.logits.shape[2] != nb:
            self.logits = torch.empty((self.q_blocks.shape[0], gate.num_q_head, nb, kb.shape[1]), dtype=torch.float32,
                                      device=self.q_blocks.device)
        return ops.gate_score_select(self.q_blocks, kb, kb.shape[1] - nb, rule.rule, num_kv_heads=num_kv_heads, scores=self.logits,
                                     write_scores=write_scores, scale=gate.scale, block_size=block_size,
                                     keep_recent=rule.keep_recent, softmax=rule.softmax, threshold=rule.threshold, alpha=rule.alpha,
                                     topk_k=rule.topk_k, topk_ratio=rule.topk_ratio, min_budget=rule.min_budget, sink=rule.sink,
                                     local=rule.local, rows_voting=rows_voting, bits=bits, out=table)

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
        self.score_max = None   # exponents of the last ``append_and_score`` (same shape and strides as its return)

    def append_and_score(self, q: torch.Tensor, k_chunk: torch.Tensor, kv_len: int) -> torch.Tensor:
        nb = -(-k_chunk.shape[1] // self.block_size)
        ops.pool_blocks(k_chunk, self.block_size, ("avg",), out=self.mean_k, out_block_offset=self.length)
        self.length += nb
        # score_raw and max_raw: the rule forms score_raw * 2^(max_raw - row max) itself (``score_max``), which is
        # all the alpha * row-max and top-k rules need of the normalisation
        raw, mx, _ = ops.flashprefill_score(q, self.mean_k[:, : self.length], kv_len, self.block_size, normalize=False)
        self.score_max = mx.permute(0, 3, 1, 2)
        return raw.permute(0, 3, 1, 2)  # [B, Hq, Qb, Kb] view


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
    score_max: Optional[torch.Tensor] = None,
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
                                   local=rule.local, rows_voting=rows_voting, bits=bits, out=table, score_max=score_max)
    out = ops.attn_compact(q, kv, kv_len, num_kv_heads, table.block_idx, table.counts, block_size=block_size,
                           softmax_scale=softmax_scale, out=out, status=status)
    return out, table


class StepScratch:
    """Buffers one sequence's layers share for the per-layer step (the layers run one after the other on
    one stream and each consumes them at once): the chunk's gate Q blocks, the logits, the block table and
    the fused selection's union scratch, all sized for the longest context so a chunk allocates nothing."""

    def __init__(self, batch: int, heads: int, kv_heads: int, q_blocks: int, max_blocks: int, channels: int, device):
        self.key = (batch, heads, kv_heads, q_blocks, max_blocks, channels)
        self.q_blocks = torch.empty((batch, q_blocks, heads, channels), dtype=torch.float32, device=device)
        self.logits = torch.empty(batch * heads * q_blocks * max_blocks, dtype=torch.float32, device=device)
        self.table = ops.BlockTable(torch.empty((batch, kv_heads, max_blocks), dtype=torch.int32, device=device),
                                    torch.empty((batch, kv_heads), dtype=torch.int32, device=device),
                                    torch.empty((batch, kv_heads), dtype=torch.int32, device=device),
                                    torch.empty((batch, kv_heads), dtype=torch.int32, device=device))
        self.union = ops.union_scratch(torch.device(device) if not isinstance(device, torch.device) else device, batch, heads,
                                       kv_heads, q_blocks, max_blocks)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)


class GateLayerStep:
    """The learned-gate layer's whole step as ONE library call (``ca_chunk_step``): RoPE + paged append,
    gate preparation, gate logits, row rule + Block-Union table, attention.  The parameter block is kept
    between chunks; a call only rewrites what changed (the chunk's tensors, lengths, block offsets), which
    is what keeps the host side of a layer short when the GPU work per layer shrinks under tensor
    parallelism.  ``dense=True`` skips the selection and attends every past block (first chunk, forced dense)."""

    def __init__(self, gate: AttnGate, selector: GateSelectorState, kv: PagedKVCache, rule: SelectionRule, scratch: StepScratch,
                 num_kv_heads: int, softmax_scale: float):
        from . import _lib
        self._lib = _lib
        self.gate, self.selector, self.kv, self.rule, self.scratch = gate, selector, kv, rule, scratch
        self.num_kv_heads, self.scale = num_kv_heads, float(softmax_scale)
        self.p = _lib.ChunkStepParams()
        self._keep = None
        self._static_done = False

    def _fill_static(self, q_nope, k_nope, v, cos, sin):
        lib, p, gate, sc = self._lib, self.p, self.gate, self.scratch
        B, L, Hq, D = q_nope.shape
        Hkv = k_nope.shape[2]
        dt = ops._DTYPES[q_nope.dtype]
        a = p.append
        a.rope_dtype, a.dtype = ops._DTYPES[cos.dtype], dt
        a.cache = self.kv.view().to_c()
        a.B, a.Q, a.Hq, a.Hkv, a.D = B, L, Hq, Hkv, D
        a.block_size = gate.block_size
        wq = None if gate.mask_linear_q is None else gate.mask_linear_q.weight.detach()
        wk = gate.mask_linear_k.weight.detach()
        g = p.prepare
        g.B, g.L, g.D, g.C, g.block_size = B, L, D, gate.hidden_size, gate.block_size
        for side, x, kinds, w in ((g.q, q_nope, gate.q_pooling_funcs, wq), (g.k, k_nope, gate.k_pooling_funcs, wk)):
            side.x_dtype, side.H = dt, x.shape[2]
            bits = 0
            for kind in kinds:
                bits |= ops._POOL_BITS[kind]
            side.kinds = bits
            if w is not None:
                side.w, side.w_dtype, side.Hw = w.data_ptr(), ops._DTYPES[w.dtype], w.shape[0]
            else:
                side.w, side.Hw = None, x.shape[2]
            side.rope_batch = 1
        qb = sc.q_blocks
        g.q.out, g.q.out_stride_b, g.q.out_stride_blk, g.q.out_stride_h = qb.data_ptr(), qb.stride(0), qb.stride(1), qb.stride(2)
        g.q.out_dtype, g.q.out_block_offset = ops._DTYPES[qb.dtype], 0
        s = p.score
        s.q, s.q_stride_b, s.q_stride_blk, s.q_stride_h = qb.data_ptr(), qb.stride(0), qb.stride(1), qb.stride(2)
        s.q_dtype = ops._DTYPES[qb.dtype]
        s.out = sc.logits.data_ptr()
        s.B, s.Hq, s.C = B, gate.num_q_head, gate.hidden_size
        s.scale, s.masked_value = gate.scale, float(torch.finfo(torch.float32).min)
        r, sel = self.rule, p.select
        sel.score_dtype, sel.rule = lib.CA_DTYPE_F32, ops.RULES[r.rule]
        sel.B, sel.H = B, gate.num_q_head
        sel.softmax, sel.threshold, sel.alpha = int(r.softmax), float(r.threshold), float(r.alpha)
        sel.topk_k = int(r.topk_k)
        sel.topk_num, sel.topk_den = r.topk_ratio if r.topk_ratio is not None else (0, 1)
        sel.min_budget, sel.sink, sel.local = int(r.min_budget), int(r.sink), int(r.local)
        t = p.table
        t.B, t.Hkv, t.G = B, self.num_kv_heads, gate.num_q_head // self.num_kv_heads
        t.keep_recent, t.block_size, t.page_size = int(r.keep_recent), gate.block_size, 256
        t.block_idx, t.idx_stride = sc.table.block_idx.data_ptr(), sc.table.block_idx.shape[-1]
        t.counts, t.cache_seqlens, t.pages_per_row = (sc.table.counts.data_ptr(), sc.table.cache_seqlens.data_ptr(),
                                                      sc.table.pages_per_row.data_ptr())
        p.union_scratch, p.union_scratch_bytes = sc.union.data_ptr(), sc.union.numel() * 4
        at = p.attn
        at.kv = self.kv.view().to_c()
        at.block_idx_stride = sc.table.block_idx.shape[-1]
        at.B, at.Q, at.Hq, at.Hkv, at.D = B, L, Hq, Hkv, D
        at.block_size, at.dtype, at.softmax_scale = gate.block_size, dt, self.scale
        at.status = sc.status.data_ptr()
        at.workspace, at.workspace_bytes = None, 0
        self._static_done = (B, L, Hq, Hkv, q_nope.dtype, cos.dtype)

    def run(self, q_nope, k_nope, v, cos, sin, block_rope, position: int, out: torch.Tensor, dense: bool = False,
            score: Optional[torch.Tensor] = None):
        """Appends the chunk at ``position`` and attends.  ``q_nope/k_nope/v`` are the pre-RoPE projections
        ``[B, L, H, D]``; ``cos/sin [1|B, L, D]``; ``block_rope`` the gate's (cos, sin) for the chunk's
        block positions or None; ``out [B, L, Hq, D]`` receives the attention output.  ``score``
        ``[B, H, Qb, Kb]`` (any strides, float32, H a multiple of the KV heads) replaces the gate logits as
        the rule's input (the gate's K-block cache is still appended).  Returns the rotated queries (a new
        tensor) and the new cache length."""
        B, L, Hq, D = q_nope.shape
        key = (B, L, Hq, k_nope.shape[2], q_nope.dtype, cos.dtype)
        if self._static_done != key:
            self._fill_static(q_nope, k_nope, v, cos, sin)
        p, gate, sel_state, sc = self.p, self.gate, self.selector, self.scratch
        bs = gate.block_size
        nb = -(-L // bs)
        if nb > sc.q_blocks.shape[1]:
            raise ValueError(f"a chunk of {nb} blocks does not fit the step scratch ({sc.q_blocks.shape[1]} blocks)")
        q_rot = torch.empty_like(q_nope)
        a = p.append
        a.q, a.q_out = q_nope.data_ptr(), q_rot.data_ptr()
        a.q_stride_b, a.q_stride_t, a.q_stride_h = q_nope.stride(0), q_nope.stride(1), q_nope.stride(2)
        a.qo_stride_b, a.qo_stride_t, a.qo_stride_h = q_rot.stride(0), q_rot.stride(1), q_rot.stride(2)
        a.k, a.k_stride_b, a.k_stride_t, a.k_stride_h = k_nope.data_ptr(), k_nope.stride(0), k_nope.stride(1), k_nope.stride(2)
        a.v, a.v_stride_b, a.v_stride_t, a.v_stride_h = v.data_ptr(), v.stride(0), v.stride(1), v.stride(2)
        a.cos, a.sin = cos.data_ptr(), sin.data_ptr()
        a.cs_stride_b, a.cs_stride_t = (0 if cos.shape[0] == 1 else cos.stride(0)), cos.stride(1)
        a.position = int(position)
        kv_len = position + L
        # gate preparation: the chunk's K blocks go to the end of the K-block cache
        sel_state.cache.reserve(sel_state.cache.length + nb)
        kview = sel_state.cache.blocks_view()
        g = p.prepare
        g.q.x, g.q.x_stride_b, g.q.x_stride_t, g.q.x_stride_h = a.q, a.q_stride_b, a.q_stride_t, a.q_stride_h
        g.k.x, g.k.x_stride_b, g.k.x_stride_t, g.k.x_stride_h = a.k, a.k_stride_b, a.k_stride_t, a.k_stride_h
        keep = [q_rot]
        if block_rope is not None:
            bcos, bsin = block_rope
            bcos, bsin = bcos.to(torch.float32).contiguous(), bsin.to(torch.float32).contiguous()
            keep += [bcos, bsin]
            for side in (g.q, g.k):
                side.cos, side.sin, side.rope_batch = bcos.data_ptr(), bsin.data_ptr(), bcos.shape[0]
        else:
            for side in (g.q, g.k):
                side.cos, side.sin, side.rope_batch = None, None, 1
        g.k.out, g.k.out_stride_b, g.k.out_stride_blk, g.k.out_stride_h = kview.data_ptr(), kview.stride(0), kview.stride(1), kview.stride(2)
        g.k.out_dtype, g.k.out_block_offset = ops._DTYPES[kview.dtype], sel_state.cache.length
        sel_state.cache.length += nb
        Kb = sel_state.cache.length
        Pb = Kb - nb
        at = p.attn
        at.q, at.q_stride_b, at.q_stride_t, at.q_stride_h = a.q_out, a.qo_stride_b, a.qo_stride_t, a.qo_stride_h
        at.out, at.o_stride_b, at.o_stride_t, at.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
        at.kv_len = kv_len
        if dense:
            p.score.q, p.select.score, at.block_idx, at.counts = None, None, None, None
        elif score is not None:
            if score.dtype != torch.float32 or score.shape[0] != B or score.shape[2] != nb or score.shape[3] != Kb:
                raise ValueError("score must be float32 [B, H, Qb, Kb] for this chunk")
            p.score.q = None
            sl = p.select
            sl.score = score.data_ptr()
            sl.score_stride_b, sl.score_stride_h, sl.score_stride_q, sl.score_stride_k = score.stride()
            sl.H, sl.Qb, sl.Kb, sl.Pb = score.shape[1], nb, Kb, Pb
            p.table.G, p.table.Qin, p.table.Kb, p.table.Pb = score.shape[1] // self.num_kv_heads, nb, Kb, Pb
            at.block_idx, at.counts = sc.table.block_idx.data_ptr(), sc.table.counts.data_ptr()
            keep.append(score)
        else:
            s = p.score
            s.q = sc.q_blocks.data_ptr()
            s.k, s.k_stride_b, s.k_stride_blk, s.k_stride_h = kview.data_ptr(), kview.stride(0), kview.stride(1), kview.stride(2)
            s.k_dtype, s.Hk, s.Qb, s.Kb, s.Pb = ops._DTYPES[kview.dtype], kview.shape[2], nb, Kb, Pb
            if Kb * nb * gate.num_q_head * B > sc.logits.numel():
                raise ValueError("the context outgrew the step scratch")
            sl = p.select
            sl.score = sc.logits.data_ptr()
            sl.score_stride_b, sl.score_stride_h, sl.score_stride_q, sl.score_stride_k = gate.num_q_head * nb * Kb, nb * Kb, Kb, 1
            sl.H, sl.Qb, sl.Kb, sl.Pb = gate.num_q_head, nb, Kb, Pb
            p.table.G, p.table.Qin, p.table.Kb, p.table.Pb = gate.num_q_head // self.num_kv_heads, nb, Kb, Pb
            at.block_idx, at.counts = sc.table.block_idx.data_ptr(), sc.table.counts.data_ptr()
        if at.workspace is None:
            ws = ops.attn_workspace(q_nope.device, at)
            at.workspace, at.workspace_bytes = ws.data_ptr(), ws.numel()
            keep.append(ws)
        self._keep = keep
        self._lib.check(self._lib.load().ca_chunk_step(ctypes.byref(p), ops._stream()), "ca_chunk_step")
        self.kv.length = max(self.kv.length, kv_len)
        return q_rot, kv_len


def capture_step(fn, warmup: int = 2) -> "torch.cuda.CUDAGraph":
    """Captures ``fn()`` — a fixed sequence of this library's launches on pre-allocated buffers, e.g.
    selector scores -> row rule -> Block-Union table -> attention at one chunk position — into a CUDA
    graph and returns it; ``graph.replay()`` then enqueues the whole step with one host call.

    The entry points allocate nothing and never synchronise; what the tensor-level wrappers cache per stream
    (the attention workspace that lets the kernel cut work units, the union scratch of the fused selection) and
    the library's per-device kernel attributes are set up by the warm-up calls.  Warm-up and capture run on
    the SAME side stream, so the capture finds those buffers in the cache instead of allocating them inside
    the graph; their addresses are baked into the graph, and they stay alive in the wrappers' caches.  A step
    is only replayable while its shapes hold (the chunk position is baked into the launch parameters), which
    is the case for a layer stack at one chunk position and for a benchmark loop.
    """
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(max(warmup, 1)):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        fn()
    return graph

