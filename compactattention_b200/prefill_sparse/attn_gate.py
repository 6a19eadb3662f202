"""Learned block selector ("AttnGate") with the reference's interface, computed by the CUDA library.

Mirrors ``compact_attn/prefill_sparse/attn_gate.py`` of the reference: class ``AttnGate`` (:37-222),
``MultiHeadLinear`` (:20-33) and the generated ``ATTNGATE_CLASSES`` (``Q{pools}_K{pools}``, :225-278)
keep their constructor arguments, parameter names (``mask_linear_q.weight``, ``mask_linear_k.weight``
so reference checkpoints load) and method names.  Inference only: pooling, projection, block RoPE and
scoring run as kernels of ``libcompactattn_b200.so`` in fp32 (the reference's
``SEERATTN_DEBUG_GATE_SCORE_FP32`` arithmetic), without autograd.
"""
from __future__ import annotations

from itertools import combinations
from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops


class MultiHeadLinear(nn.Module):
    """Per-head weight ``[num_head, in_channel, hidden]``; applied by ``ops.gate_project``."""

    def __init__(self, in_channel_size: int, hidden_size: int, num_head: int):
        super().__init__()
        self.in_channel = in_channel_size
        self.hidden_size = hidden_size
        self.num_head = num_head
        # N(0, 0.02) like the reference's model initialisation of the gate (initializer_range,
        # prefill_sparse/llama/modeling_llama_seerattn.py:765-777); a checkpoint overwrites it.  Never left
        # uninitialised: stray NaN bit patterns in a fresh allocation would silently deselect every block.
        self.weight = nn.Parameter(torch.empty(num_head, in_channel_size, hidden_size).normal_(mean=0.0, std=0.02))

    def forward(self, x: torch.Tensor) -> torch.Tensor:  # x [B, S, h, I] float32 pooled blocks
        return ops.gate_project(x.to(torch.float32).contiguous(), self.weight.detach().contiguous())


class AttnGate(nn.Module):
    def __init__(
        self,
        block_size,
        in_channel_size,
        hidden_size,
        num_k_head,
        num_q_head,
        q_pooling_funcs,
        k_pooling_funcs,
        force_double=False,
        use_flash_rope=False,
        kv_group_aware_query=False,
    ):
        super().__init__()
        if num_q_head % num_k_head != 0:
            raise ValueError(f"num_q_head ({num_q_head}) must be divisible by num_k_head ({num_k_head}).")
        if kv_group_aware_query:
            raise NotImplementedError("kv_group_aware_query gates are not supported by the B200 path")
        self.block_size = block_size
        self.in_channel = in_channel_size
        self.hidden_size = hidden_size
        self.num_k_head = num_k_head
        self.num_q_head = num_q_head
        self.num_key_value_groups = num_q_head // num_k_head
        self.use_flash_rope = use_flash_rope
        self.kv_group_aware_query = False
        self.q_pooling_funcs = tuple(q_pooling_funcs)  # names: "max" / "min" / "avg"
        self.k_pooling_funcs = tuple(k_pooling_funcs)
        self.scale = hidden_size ** -0.5
        self.q_dup_size = len(self.q_pooling_funcs)
        self.k_dup_size = len(self.k_pooling_funcs)
        q_in = in_channel_size * self.q_dup_size
        k_in = in_channel_size * self.k_dup_size
        if self.q_dup_size > 1 or hidden_size != in_channel_size or force_double:
            self.mask_linear_q = MultiHeadLinear(q_in, hidden_size, num_q_head)
            self.mask_linear_k = MultiHeadLinear(k_in, hidden_size, num_k_head)
        else:  # a single projection on K, per query head
            self.mask_linear_q = None
            self.mask_linear_k = MultiHeadLinear(k_in, hidden_size, num_q_head)

    # -- the reference's method names ---------------------------------------------------------
    def compress_query_blocks(self, q: torch.Tensor) -> torch.Tensor:
        pooled = ops.pool_blocks(q, self.block_size, self.q_pooling_funcs)
        w = None if self.mask_linear_q is None else self.mask_linear_q.weight.detach().contiguous()
        return ops.gate_project(pooled, w)

    def compress_key_blocks(self, k: torch.Tensor) -> torch.Tensor:
        pooled = ops.pool_blocks(k, self.block_size, self.k_pooling_funcs)
        return ops.gate_project(pooled, self.mask_linear_k.weight.detach().contiguous())

    def apply_block_position_embeddings(self, q=None, k=None, position_embeddings=None):
        if position_embeddings is None:
            return q, k
        cos, sin = position_embeddings
        if cos.dim() == 2:  # [S, D/2] tables of the fused-rotary form: expand to the half-rotation form
            cos, sin = torch.cat([cos, cos], dim=-1).unsqueeze(0), torch.cat([sin, sin], dim=-1).unsqueeze(0)
        if q is not None:
            q = ops.gate_project(q.to(torch.float32).contiguous(), None, cos, sin)
        if k is not None:
            k = ops.gate_project(k.to(torch.float32).contiguous(), None, cos, sin)
        return q, k

    @staticmethod
    def block_mask_to_valid(attention_mask: torch.Tensor) -> torch.Tensor:
        """The reference accepts two mask forms (prefill_sparse/attn_gate.py:196-199): bool (True =
        visible) and additive floating point (0 = visible, finfo.min / -inf = masked, added to the
        logits).  Both become a bool validity mask here; an additive mask must therefore hold only
        zeros and large negative values.  Integer masks are refused (their meaning is ambiguous)."""
        if attention_mask.dtype == torch.bool:
            return attention_mask
        if attention_mask.is_floating_point():
            return attention_mask == 0
        raise TypeError(f"block attention mask must be bool or floating point (additive), got {attention_mask.dtype}")

    def score_compressed_blocks(self, q, k, attention_mask, use_softmax: bool = True) -> torch.Tensor:
        """``[B, Hq, Qb, Kb]`` float32 scores; ``attention_mask`` is the block mask ``[B, 1, Qb, Kb]``,
        bool or additive (see ``block_mask_to_valid``).  ``None`` means no masking at all, as in the
        reference (:194-195) - every model integration passes the block-causal mask."""
        Qb, Kb = q.shape[1], k.shape[1]
        fill = torch.finfo(torch.float32).min
        if attention_mask is None:
            logits = ops.gate_scores(q, k, Kb, scale=self.scale)  # past_blocks = Kb: no entry lies above the diagonal
            if not use_softmax:
                return logits
            valid = torch.ones((1, 1, 1, 1), dtype=torch.bool, device=logits.device).expand(q.shape[0], 1, Qb, Kb)
        else:
            logits = ops.gate_scores(q, k, Kb - Qb, scale=self.scale)
            valid = self.block_mask_to_valid(attention_mask[..., -Qb:, -Kb:])
            if valid.dim() == 3:
                valid = valid.unsqueeze(1)
            logits = logits.masked_fill(~valid, fill)
            if not use_softmax:
                return logits
        prob = torch.empty_like(logits)
        ops.select_rows(logits, Kb - Qb, "threshold", softmax=True, valid=valid, prob_out=prob)
        return prob

    def forward(self, q, k, attention_mask, position_embeddings=None, use_softmax=True):
        if q.shape[1] == 1:
            return None
        qb = self.compress_query_blocks(q)
        kb = self.compress_key_blocks(k)
        if position_embeddings is not None:
            cos, sin = position_embeddings
            qb, _ = self.apply_block_position_embeddings(q=qb, position_embeddings=(cos[..., -qb.shape[1]:, :], sin[..., -qb.shape[1]:, :]))
            _, kb = self.apply_block_position_embeddings(k=kb, position_embeddings=(cos, sin))
        return self.score_compressed_blocks(qb, kb, attention_mask, use_softmax=use_softmax)

    # -- chunked operation over a growing K-block cache -----------------------------------------
    def append_key_blocks(self, cache: "GateKeyBlockCache", k_chunk: torch.Tensor,
                          position_embeddings: Optional[Tuple[torch.Tensor, torch.Tensor]]) -> None:
        """Pool + project + RoPE the chunk's K blocks straight into the cache (no intermediate copy):
        the reference's ``_compactattn_append_cached_k_blocks``
        (compact_attn/prefill_sparse/llama/modeling_llama_seerattn_chunked_dense.py:426-478)."""
        pooled = ops.pool_blocks(k_chunk, self.block_size, self.k_pooling_funcs)
        nb = pooled.shape[1]
        cache.reserve(cache.length + nb)
        cos = sin = None
        if position_embeddings is not None:
            cos, sin = position_embeddings
        ops.gate_project(pooled, self.mask_linear_k.weight.detach().contiguous(), cos, sin,
                         out=cache.blocks_view(), out_block_offset=cache.length)
        cache.length += nb


class GateKeyBlockCache:
    """Projected + roped K blocks of every past chunk, heads-first ``[B, H, capacity, C]`` so the
    scoring kernel streams each head's blocks contiguously.  Capacity doubles from 256 blocks like the
    reference's buffer (modeling_llama_seerattn_chunked_dense.py:398-406)."""

    def __init__(self, batch: int, heads: int, channels: int, device, dtype=torch.bfloat16, capacity: int = 256):
        self.buffer = torch.empty((batch, heads, capacity, channels), dtype=dtype, device=device)
        self.length = 0

    def reserve(self, required: int) -> None:
        cap = self.buffer.shape[2]
        if required <= cap:
            return
        while cap < required:
            cap *= 2
        new = torch.empty((self.buffer.shape[0], self.buffer.shape[1], cap, self.buffer.shape[3]),
                          dtype=self.buffer.dtype, device=self.buffer.device)
        new[:, :, : self.length].copy_(self.buffer[:, :, : self.length])
        self.buffer = new

    def blocks_view(self) -> torch.Tensor:
        """``[B, capacity, H, C]`` view (block-major indexing over the heads-first storage)."""
        return self.buffer.transpose(1, 2)

    def blocks(self) -> torch.Tensor:
        return self.blocks_view()[:, : self.length]


POOL_FUNCS = {"max": "max", "min": "min", "avg": "avg"}


def _make_class(q_names, k_names):
    name = f"Q{''.join(q_names)}_K{''.join(k_names)}"

    class _Gate(AttnGate):
        def __init__(self, block_size, in_channel_size, hidden_size, num_k_head, num_q_head, force_double=False,
                     use_flash_rope=False, kv_group_aware_query=False):
            super().__init__(block_size, in_channel_size, hidden_size, num_k_head, num_q_head, q_names, k_names,
                             force_double=force_double, use_flash_rope=use_flash_rope,
                             kv_group_aware_query=kv_group_aware_query)

    _Gate.__name__ = name
    return name, _Gate


def _generate():
    classes = {}
    kinds = ["max", "min", "avg"]
    for qn in range(1, 4):
        for kn in range(1, 4):
            for qc in combinations(kinds, qn):
                for kc in combinations(kinds, kn):
                    name, cls = _make_class(qc, kc)
                    classes[name] = cls
    return classes


ATTNGATE_CLASSES = _generate()
