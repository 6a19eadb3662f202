"""Llama attention modules for chunked-prefill CompactAttention with the reference's forward
signatures, running on the B200 library.

Mirrors, for the path only:
* ``LlamaSeerAttentionChunkedDense.forward`` (learned-gate selector,
  ``compact_attn/prefill_sparse/llama/modeling_llama_seerattn_chunked_dense.py:547-938``) with its two
  documented override hooks ``_do_kv_cache_update`` and ``_do_chunked_compactattn_attention`` (:518-545);
* ``LlamaFlashPrefillCompactAttnAttention.forward`` (training-free selector,
  ``compact_attn/prefill_sparse/llama/modeling_llama_flashprefill_compactattn.py:152-341``).
Both return the reference's 5-tuple ``(attn_output, mask_loss, None, attn_gate_output, ground_truth_mask)``.

What differs by design: the KV cache is a paged cache that is appended in place
(``paged_cache.PagedKVCache``) instead of a ``DynamicCache`` that is concatenated every chunk; the
selector state (gate K-block cache, mean-K cache) lives beside it in ``CompactAttnCache``; inference
only (no distillation loss); decode (``q_len == 1``) appends to the paged cache and runs dense attention
with the same kernel, as the reference runs decode dense (:880-891).  A chunk that is not a block
multiple (a prompt's last chunk) is handled; once the cache length is not a block multiple every later
call is dense.  Under tensor
parallelism a module holds the projections of its rank's heads (``tp.HeadShard``) and the row-parallel
``o_proj`` output is summed with one all-reduce.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from ... import ops, tp
from ...chunk_driver import GateLayerStep, GateSelectorState, MeanKSelectorState, SelectionRule, StepScratch
from ...modules import (
    chunked_prefill_column_dense_attention_forward,
    flashprefill_compactattn_prefill_full_kv,
)
from ...paged_cache import PagedKVCache
from ..attn_gate import ATTNGATE_CLASSES


# the reference's debug switches that the operator route honours or refuses; with one of them set the module
# goes through the operator instead of the one-call step
_DEBUG_ENV = ("SEERATTN_DEBUG_COMPACTATTN_THRESHOLD_OVERRIDE", "SEERATTN_DEBUG_COMPACTATTN_KEEP_RECENT_OVERRIDE",
              "SEERATTN_DEBUG_COMPACTATTN_QUERY_BLOCK_MODE", "SEERATTN_DEBUG_COMPACTATTN_KV_HEAD_MODE",
              "SEERATTN_DEBUG_COMPACTATTN_DISABLE_CURRENT_OPEN")


@dataclass
class CompactAttnLlamaConfig:
    """The attributes of the reference's ``SeerAttnLlamaConfig`` that the path reads
    (``compact_attn/prefill_sparse/llama/configuration_llama_seerattn.py:162-280``), same names."""

    hidden_size: int = 4096
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    vocab_size: int = 128256
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    max_position_embeddings: int = 131072
    initializer_range: float = 0.02
    attention_bias: bool = False
    # selector / path switches
    seerattn_gate_type: str = "Qavg_Kmaxminavg"
    seerattn_gate_block_size: int = 64
    seerattn_gate_hidden_size: int = 128
    seerattn_gate_force_double: bool = False
    # threshold | topk (per-row top-k of the gate scores, ties to the lower block) | synthetic_topk (per-row
    # top-k of a fixed random per-KV-head block importance: imposes an exact union density on
    # random-init stacks, whose gate scores are uncorrelated across heads and Q-blocks)
    seerattn_sparsity_method: str = "threshold"
    seerattn_threshold: float = 5e-4
    seerattn_topk_ratio: Tuple[int, int] = (1, 5)
    seerattn_compactattn_keep_recent_blocks: int = 2
    seerattn_compactattn_pack_impl: str = "indexed_dense"
    seerattn_compactattn_indexed_impl: str = "b200_native"
    seerattn_compactattn_cache_fill_backend: str = "auto"
    seerattn_compactattn_disable_first_chunk_dense: bool = False
    seerattn_chunked_prefill_force_dense: bool = False
    seerattn_flashprefill_block_size: int = 128
    seerattn_flashprefill_attention_sink: int = 2
    seerattn_flashprefill_window_size: int = 4
    seerattn_flashprefill_alpha: float = 0.06
    seerattn_flashprefill_last_n_block: int = 0
    seerattn_flashprefill_min_budget: int = 0
    seerattn_defer_async_collective_wait: bool = False
    # Tensor parallel only: o_proj and its sum over the ranks as this library's fused kernels over peer memory
    # (ca_oproj_allreduce) instead of a library GEMM + NCCL all-reduce; chunks of up to this many rows (0 = off).
    compactattn_fused_oproj_rows: int = 0
    compactattn_debug: bool = False


@dataclass
class _LayerState:
    kv: PagedKVCache
    gate: Optional[GateSelectorState] = None
    mean_k: Optional[MeanKSelectorState] = None
    plan: Optional[GateLayerStep] = None


class CompactAttnCache:
    """``past_key_value`` of the modules: per layer a paged KV cache and the selector's own cache."""

    def __init__(self, batch: int, max_tokens: int, device, dtype=torch.bfloat16, page_table: Optional[torch.Tensor] = None):
        self.batch, self.max_tokens, self.device, self.dtype = batch, max_tokens, device, dtype
        self.page_table = page_table
        self.layers: Dict[int, _LayerState] = {}

    def layer(self, idx: int, num_kv_heads: int, head_dim: int) -> _LayerState:
        st = self.layers.get(idx)
        if st is None:
            st = _LayerState(PagedKVCache(self.batch, self.max_tokens, num_kv_heads, head_dim, self.device, self.dtype,
                                          page_table=self.page_table))
            self.layers[idx] = st
        return st

    def get_seq_length(self, idx: int = 0) -> int:
        st = self.layers.get(idx)
        return 0 if st is None else st.kv.length

    def get_mask_sizes(self, query_length: int, layer_idx: int = 0):
        """``(kv_length, kv_offset)`` the way a HuggingFace cache reports them to the stock model's mask
        builder: the tokens held plus the chunk about to be appended, no offset."""
        return self.get_seq_length(layer_idx) + int(query_length), 0

    def step_scratch(self, heads: int, num_kv_heads: int, q_blocks: int, block_size: int, channels: int) -> StepScratch:
        """Scratch of the one-call layer step, shared by the layers, sized for the longest context; rebuilt
        when a larger chunk arrives."""
        sc = getattr(self, "_step_scratch", None)
        max_blocks = -(-self.max_tokens // block_size)
        if sc is None or sc.key[:3] != (self.batch, heads, num_kv_heads) or sc.key[3] < q_blocks or sc.key[4:] != (max_blocks, channels):
            sc = StepScratch(self.batch, heads, num_kv_heads, q_blocks, max_blocks, channels, self.device)
            self._step_scratch = sc
        return sc

    def selection_scratch(self, heads: int, num_kv_heads: int, q_blocks: int, block_size: int):
        """Keep bits and block table shared by every layer (the layers run one after the other on
        one stream and each consumes its table at once), sized for the longest context, so a chunk
        allocates nothing: returns ``(bits_for(kv_blocks), table)``."""
        key = (heads, num_kv_heads, q_blocks, block_size)
        sc = getattr(self, "_scratch", None)
        if sc is None or sc[0] != key:
            max_blocks = self.max_tokens // block_size
            words = ops.words_for(max_blocks)
            flat = torch.empty(self.batch * heads * q_blocks * words, dtype=torch.int32, device=self.device)
            table = ops.BlockTable(
                torch.empty((self.batch, num_kv_heads, max_blocks), dtype=torch.int32, device=self.device),
                torch.empty((self.batch, num_kv_heads), dtype=torch.int32, device=self.device),
                torch.empty((self.batch, num_kv_heads), dtype=torch.int32, device=self.device),
                torch.empty((self.batch, num_kv_heads), dtype=torch.int32, device=self.device))
            sc = (key, flat, table)
            self._scratch = sc
        _, flat, table = sc

        def bits_for(kv_blocks: int) -> torch.Tensor:
            w = ops.words_for(kv_blocks)
            return flat[: self.batch * heads * q_blocks * w].view(self.batch, heads, q_blocks, w)

        return bits_for, table


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim: int = 2):
    """Half-rotation RoPE on ``[B, L, H, D]`` tensors with ``cos/sin [B, L, D]``
    (the reference's ``compact_attn/modules/common.py:49-75``); plain torch ops, not on the path."""
    cos, sin = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
    return (q * cos + rotate_half(q) * sin).to(q.dtype), (k * cos + rotate_half(k) * sin).to(k.dtype)


class _CompactAttnBase(nn.Module):
    def __init__(self, config: CompactAttnLlamaConfig, layer_idx: int, shard: Optional[tp.HeadShard] = None):
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        self.shard = shard or tp.HeadShard(1, 0, config.num_attention_heads, config.num_key_value_heads)
        self.head_dim = config.head_dim
        self.num_heads = len(self.shard.q_heads)          # local query heads
        self.num_key_value_heads = len(self.shard.kv_heads)  # local KV heads
        self.num_key_value_groups = self.shard.group
        self.scaling = self.head_dim ** -0.5
        bias = config.attention_bias
        self.q_proj = nn.Linear(config.hidden_size, self.num_heads * self.head_dim, bias=bias)
        self.k_proj = nn.Linear(config.hidden_size, self.num_key_value_heads * self.head_dim, bias=bias)
        self.v_proj = nn.Linear(config.hidden_size, self.num_key_value_heads * self.head_dim, bias=bias)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, config.hidden_size, bias=False)
        self.compactattn_debug = bool(config.compactattn_debug)
        self.compactattn_pack_impl = config.seerattn_compactattn_pack_impl
        self.compactattn_indexed_impl = config.seerattn_compactattn_indexed_impl
        self.compactattn_cache_fill_backend = config.seerattn_compactattn_cache_fill_backend
        self._compactattn_last_stats = None
        self._pending_reduce = None

    # -- hook: KV cache update (the reference's _do_kv_cache_update, :518-536) --------------------
    def _do_kv_cache_update(self, key_states, value_states, past_key_value, sin, cos, cache_position, collect_stats):
        """Appends the chunk to this layer's paged cache; returns ``(KvCacheView, kv_len, ms)``."""
        st = past_key_value.layer(self.layer_idx, self.num_key_value_heads, self.head_dim)
        pos = int(cache_position[0]) if cache_position is not None and not torch.is_tensor(cache_position) else None
        if torch.is_tensor(cache_position):
            pos = st.kv.length  # positions are appended in order; no device-to-host read of cache_position
        kv_len = st.kv.append(key_states, value_states, position=pos)
        return st.kv.view(), kv_len, 0.0

    def _do_rope_and_kv_cache_update(self, q_nope, k_nope, value_states, past_key_value, cos, sin, cache_position,
                                     mean_k=None, block_size: int = 64):
        """Default route of both modules: RoPE on q and k, the paged append and (for the training-free
        selector) the mean-K pooling in ONE launch (``ops.rope_append``).  Returns
        ``(q_rotated, KvCacheView, kv_len)``.  A subclass that overrides ``_do_kv_cache_update`` (the
        reference's documented hook, which receives already rotated keys) is routed through that hook
        with the separate torch RoPE instead."""
        st = past_key_value.layer(self.layer_idx, self.num_key_value_heads, self.head_dim)
        if type(self)._do_kv_cache_update is not _CompactAttnBase._do_kv_cache_update:
            q, k = apply_rotary_pos_emb(q_nope, k_nope, cos, sin)
            kv_view, kv_len, _ = self._do_kv_cache_update(k, value_states, past_key_value, sin, cos, cache_position,
                                                          self.compactattn_debug)
            if mean_k is not None:
                ops.pool_blocks(k, block_size, ("avg",), out=mean_k, out_block_offset=(kv_len - k.shape[1]) // block_size)
            return q, kv_view, kv_len
        pos = st.kv.length  # chunks are appended in order; no device-to-host read of cache_position
        if cache_position is not None and not torch.is_tensor(cache_position):
            pos = int(cache_position[0])
        q, kv_len = st.kv.append_rope(q_nope, k_nope, value_states, cos, sin, position=pos, mean_k=mean_k,
                                      block_size=block_size)
        return q, st.kv.view(), kv_len

    def _project(self, hidden_states):
        B, L, _ = hidden_states.shape
        q = self.q_proj(hidden_states).view(B, L, self.num_heads, self.head_dim)
        k = self.k_proj(hidden_states).view(B, L, self.num_key_value_heads, self.head_dim)
        v = self.v_proj(hidden_states).view(B, L, self.num_key_value_heads, self.head_dim)
        return q, k, v

    def _finish(self, attn_output, input_shape):
        x = attn_output.reshape(*input_shape, -1)
        rows = int(getattr(self.config, "compactattn_fused_oproj_rows", 0) or 0)
        if rows and tp.fused_projection_applies(x, self.o_proj.weight, self.o_proj.bias, rows):
            self._pending_reduce = None
            return tp.project_and_reduce(x, self.o_proj.weight, rows)
        out = self.o_proj(x)
        work = tp.reduce_layer_output(out, async_op=bool(self.config.seerattn_defer_async_collective_wait))
        self._pending_reduce = work
        return out

    def wait_pending_reduce(self):
        """Completes a deferred layer-output reduction (``seerattn_defer_async_collective_wait``)."""
        if self._pending_reduce is not None:
            self._pending_reduce.wait()
            self._pending_reduce = None

    def _dense(self, q, kv_view, kv_len, block_size):
        return ops.attn_compact(q, kv_view, kv_len, self.num_key_value_heads, None, None, block_size=block_size,
                                softmax_scale=self.scaling)


class LlamaSeerAttentionChunkedDense(_CompactAttnBase):
    """Learned-gate CompactAttention layer."""

    def __init__(self, config: CompactAttnLlamaConfig, layer_idx: int, shard: Optional[tp.HeadShard] = None):
        super().__init__(config, layer_idx, shard)
        self.attn_gate = ATTNGATE_CLASSES[config.seerattn_gate_type](
            config.seerattn_gate_block_size, self.head_dim, config.seerattn_gate_hidden_size,
            self.num_key_value_heads, self.num_heads, force_double=config.seerattn_gate_force_double)
        self.compactattn_keep_recent_blocks = config.seerattn_compactattn_keep_recent_blocks
        self.compactattn_disable_first_chunk_dense = config.seerattn_compactattn_disable_first_chunk_dense
        self._synthetic_importance = None

    # -- hook: the attention itself (the reference's _do_chunked_compactattn_attention, :538-545) --
    def _do_chunked_compactattn_attention(self, query_states, key_states, value_states, **kwargs):
        return chunked_prefill_column_dense_attention_forward(
            query_states=query_states, key_states=key_states, value_states=value_states, **kwargs)

    def _synthetic_scores(self, hidden_states, max_blocks: int, Qb: int, Kb: int) -> torch.Tensor:
        """A fixed random importance per (KV head, key block), seen alike by every Q-block row: per-row top-k
        of it imposes an exact union density on random-init stacks."""
        if self._synthetic_importance is None or self._synthetic_importance.shape[-1] < Kb:
            g = torch.Generator(device=hidden_states.device).manual_seed(1234 + self.layer_idx)
            self._synthetic_importance = torch.rand((1, self.num_key_value_heads, 1, max(max_blocks, Kb)), generator=g,
                                                    device=hidden_states.device)
        return self._synthetic_importance[..., :Kb].expand(hidden_states.shape[0], self.num_key_value_heads, Qb, Kb)

    # -- the default route: the whole layer step as one library call ---------------------------------
    def _one_call_step_applies(self, q_len, past_len, block_attention_mask, cache_position) -> bool:
        """The one-call step serves the plain case: a chunk (not decode) on a block-aligned past, the
        threshold or top-k method, no caller-made block mask, no statistics, and neither documented hook
        overridden (a subclass that overrides one is served through the hooks)."""
        cls = type(self)
        return (q_len > 1 and past_len % self.config.seerattn_gate_block_size == 0 and block_attention_mask is None
                and not self.compactattn_debug and self.config.seerattn_sparsity_method in ("threshold", "topk", "synthetic_topk")
                and not any(os.environ.get(k) for k in _DEBUG_ENV)
                and cls._do_kv_cache_update is _CompactAttnBase._do_kv_cache_update
                and cls._do_chunked_compactattn_attention is LlamaSeerAttentionChunkedDense._do_chunked_compactattn_attention
                and (cache_position is None or torch.is_tensor(cache_position) or int(cache_position[0]) == past_len))

    def _forward_one_call(self, hidden_states, q_nope, k_nope, v, cos, sin, st, past_key_value, block_position_embeddings,
                          past_len, input_shape):
        cfg, bs = self.config, self.config.seerattn_gate_block_size
        q_len = hidden_states.shape[1]
        if st.gate is None:
            st.gate = GateSelectorState(self.attn_gate, hidden_states.shape[0], hidden_states.device, cache_dtype=hidden_states.dtype)
        if st.plan is None:
            if cfg.seerattn_sparsity_method in ("topk", "synthetic_topk"):
                rule = SelectionRule(rule="topk", softmax=False, topk_ratio=tuple(cfg.seerattn_topk_ratio), sink=1,
                                     local=self.compactattn_keep_recent_blocks)
            else:  # threshold on soft-maxed gate scores, the last keep_recent columns forced on
                rule = SelectionRule(rule="threshold", softmax=True, threshold=float(cfg.seerattn_threshold),
                                     keep_recent=max(int(self.compactattn_keep_recent_blocks), 0))
            scratch = past_key_value.step_scratch(self.num_heads, self.num_key_value_heads, -(-q_len // bs), bs,
                                                  cfg.seerattn_gate_hidden_size)
            st.plan = GateLayerStep(self.attn_gate, st.gate, st.kv, rule, scratch, self.num_key_value_heads, self.scaling)
        elif st.plan.scratch.q_blocks.shape[1] < -(-q_len // bs):
            st.plan.scratch = past_key_value.step_scratch(self.num_heads, self.num_key_value_heads, -(-q_len // bs), bs,
                                                          cfg.seerattn_gate_hidden_size)
            st.plan._static_done = False
        rope_blocks = None
        if block_position_embeddings is not None:
            bcos, bsin = block_position_embeddings
            nb = -(-q_len // bs)
            rope_blocks = (bcos[..., -nb:, :], bsin[..., -nb:, :])
        first_chunk = past_len == 0
        dense = bool(cfg.seerattn_chunked_prefill_force_dense) or (first_chunk and not self.compactattn_disable_first_chunk_dense)
        attn = torch.empty_like(q_nope)
        score = None
        if cfg.seerattn_sparsity_method == "synthetic_topk" and not dense:
            Qb, Kb = -(-q_len // bs), -(-(past_len + q_len) // bs)
            score = self._synthetic_scores(hidden_states, past_key_value.max_tokens // bs, Qb, Kb)
        st.plan.run(q_nope, k_nope, v, cos, sin, rope_blocks, past_len, attn, dense=dense, score=score)
        out = self._finish(attn, input_shape)
        self._compactattn_last_stats = None
        return out, 0.0, None, None, None

    def forward(
        self,
        hidden_states: torch.Tensor,
        position_embeddings: Tuple[torch.Tensor, torch.Tensor],
        attention_mask: Optional[torch.Tensor],
        past_key_value: Optional[CompactAttnCache] = None,
        cache_position: Optional[torch.LongTensor] = None,
        block_position_embeddings: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
        block_attention_mask: Optional[torch.Tensor] = None,
        seer_batch_kv_lens=None,
        seer_batch_query_lens=None,
        seer_batch_query_start=None,
        **kwargs,
    ):
        if seer_batch_kv_lens is not None or seer_batch_query_lens is not None or seer_batch_query_start is not None:
            raise NotImplementedError("ragged batch metadata is not supported by the B200 path")
        if past_key_value is None:
            raise ValueError("the B200 path needs a CompactAttnCache as past_key_value")
        input_shape = hidden_states.shape[:-1]
        q_len = hidden_states.shape[1]
        bs = self.config.seerattn_gate_block_size
        q_nope, k_nope, v = self._project(hidden_states)
        cos, sin = position_embeddings
        st = past_key_value.layer(self.layer_idx, self.num_key_value_heads, self.head_dim)
        past_len = st.kv.length
        if self._one_call_step_applies(q_len, past_len, block_attention_mask, cache_position):
            return self._forward_one_call(hidden_states, q_nope, k_nope, v, cos, sin, st, past_key_value, block_position_embeddings,
                                          past_len, input_shape)
        q, kv_view, kv_len = self._do_rope_and_kv_cache_update(q_nope, k_nope, v, past_key_value, cos, sin, cache_position)
        if q_len == 1 or past_len % bs != 0:
            # decode, or a call after a chunk that ended inside a block: dense, the gate is not consulted
            # (reference :741-742, :880-891)
            out = self._finish(self._dense(q, kv_view, kv_len, bs), input_shape)
            self._compactattn_last_stats = {"path": "other"} if self.compactattn_debug else None
            return out, 0.0, None, None, None
        # the gate sees pre-RoPE q/k pooled to blocks, with RoPE at block positions; its K-block cache
        # is appended for every chunk, also when the chunk itself runs dense
        if st.gate is None:
            st.gate = GateSelectorState(self.attn_gate, hidden_states.shape[0], hidden_states.device,
                                        cache_dtype=hidden_states.dtype)
        rope_blocks = None
        if block_position_embeddings is not None:
            bcos, bsin = block_position_embeddings
            nb = -(-q_len // bs)
            rope_blocks = (bcos[..., -nb:, :], bsin[..., -nb:, :])
        logits = st.gate.append_and_score(q_nope, k_nope, rope_blocks, rope_blocks)
        first_chunk = kv_len == q_len
        force_dense = bool(self.config.seerattn_chunked_prefill_force_dense)
        stats = None
        if force_dense or (first_chunk and not self.compactattn_disable_first_chunk_dense):
            attn = self._dense(q, kv_view, kv_len, bs)
            path = "first_chunk_dense" if first_chunk else "forced_dense"
        elif self.config.seerattn_sparsity_method == "synthetic_topk":
            Qb, Kb = logits.shape[2], logits.shape[3]
            score = self._synthetic_scores(hidden_states, past_key_value.max_tokens // bs, Qb, Kb)
            _, table = past_key_value.selection_scratch(self.num_key_value_heads, self.num_key_value_heads, Qb, bs)
            table = ops.select_union_table(score, Kb - Qb, "topk", num_kv_heads=self.num_key_value_heads, block_size=bs,
                                           topk_ratio=tuple(self.config.seerattn_topk_ratio), sink=1,
                                           local=self.compactattn_keep_recent_blocks, out=table)
            attn = ops.attn_compact(q, kv_view, kv_len, self.num_key_value_heads, table.block_idx, table.counts,
                                    block_size=bs, softmax_scale=self.scaling)
            path = "chunked_selected"
        elif self.config.seerattn_sparsity_method == "topk":
            Qb, Kb = logits.shape[2], logits.shape[3]
            _, table = past_key_value.selection_scratch(self.num_heads, self.num_key_value_heads, Qb, bs)
            table = ops.select_union_table(logits, Kb - Qb, "topk", num_kv_heads=self.num_key_value_heads, block_size=bs,
                                           topk_ratio=tuple(self.config.seerattn_topk_ratio), sink=1,
                                           local=self.compactattn_keep_recent_blocks, out=table)
            attn = ops.attn_compact(q, kv_view, kv_len, self.num_key_value_heads, table.block_idx, table.counts,
                                    block_size=bs, softmax_scale=self.scaling)
            path = "chunked_selected"
        else:
            # threshold on softmax-ed gate scores, exactly the operator the reference calls
            Qb, Kb = logits.shape[2], logits.shape[3]
            prob = torch.empty_like(logits)
            valid = None if block_attention_mask is None else self.attn_gate.block_mask_to_valid(block_attention_mask[..., -Qb:, -Kb:])
            ops.select_rows(logits, Kb - Qb, "threshold", softmax=True, valid=valid, prob_out=prob)
            attn, stats = self._do_chunked_compactattn_attention(
                q, kv_view, kv_view, attention_mask=attention_mask, query_length=q_len, softmax_scale=self.scaling,
                attn_gate_score=prob, block_attention_mask=block_attention_mask, threshold=self.config.seerattn_threshold,
                keep_recent_blocks=self.compactattn_keep_recent_blocks, block_size=bs,
                num_key_value_groups=self.num_key_value_groups, pack_impl=self.compactattn_pack_impl,
                indexed_impl=self.compactattn_indexed_impl, cache_fill_backend=self.compactattn_cache_fill_backend,
                return_stats=self.compactattn_debug, attn_module=self, kv_len=kv_len)
            path = "chunked_selected"
        out = self._finish(attn, input_shape)
        self._compactattn_last_stats = dict(stats or {}, path=path) if self.compactattn_debug else None
        return out, 0.0, None, None, None


class LlamaFlashPrefillCompactAttnAttention(_CompactAttnBase):
    """Training-free (FlashPrefill) CompactAttention layer."""

    def forward(
        self,
        hidden_states: torch.Tensor,
        position_embeddings: Tuple[torch.Tensor, torch.Tensor],
        attention_mask: Optional[torch.Tensor],
        past_key_value: Optional[CompactAttnCache] = None,
        cache_position: Optional[torch.LongTensor] = None,
        **kwargs,
    ):
        if past_key_value is None:
            raise ValueError("the B200 path needs a CompactAttnCache as past_key_value")
        input_shape = hidden_states.shape[:-1]
        q_len = hidden_states.shape[1]
        cfg = self.config
        bs = cfg.seerattn_flashprefill_block_size
        q, k, v = self._project(hidden_states)
        cos, sin = position_embeddings
        st = past_key_value.layer(self.layer_idx, self.num_key_value_heads, self.head_dim)
        if q_len == 1 or st.kv.length % bs != 0:
            # decode, or a call after a chunk that ended inside a block: dense, no selector state is touched
            q, kv_view, kv_len = self._do_rope_and_kv_cache_update(q, k, v, past_key_value, cos, sin, cache_position)
            out = self._finish(self._dense(q, kv_view, kv_len, bs), input_shape)
            self._compactattn_last_stats = {"path": "dense_fallback"} if self.compactattn_debug else None
            return out, 0.0, None, None, None
        # mean-K cache of the post-RoPE keys, appended in place by the same launch that rotates and
        # stores the keys (the reference re-concatenates a list of parts every chunk,
        # modeling_llama_flashprefill_compactattn.py:121-150)
        if st.mean_k is None:
            st.mean_k = MeanKSelectorState(hidden_states.shape[0], past_key_value.max_tokens // bs, self.num_key_value_heads,
                                           self.head_dim, bs, hidden_states.device, hidden_states.dtype)
        q, kv_view, kv_len = self._do_rope_and_kv_cache_update(q, k, v, past_key_value, cos, sin, cache_position,
                                                               mean_k=st.mean_k.mean_k, block_size=bs)
        st.mean_k.length = -(-kv_len // bs)
        if kv_len > q_len and not cfg.seerattn_chunked_prefill_force_dense:
            attn, stats = flashprefill_compactattn_prefill_full_kv(
                q, kv_view, kv_view, attention_mask, softmax_scale=self.scaling,
                num_key_value_groups=self.num_key_value_groups, block_size=bs,
                attention_sink=cfg.seerattn_flashprefill_attention_sink, window_size=cfg.seerattn_flashprefill_window_size,
                alpha=cfg.seerattn_flashprefill_alpha, last_n_block=cfg.seerattn_flashprefill_last_n_block,
                min_budget=cfg.seerattn_flashprefill_min_budget, pack_impl=self.compactattn_pack_impl,
                indexed_impl=self.compactattn_indexed_impl, cache_fill_backend=self.compactattn_cache_fill_backend,
                measure_timing=self.compactattn_debug, attn_module=self,
                mean_k_cache=st.mean_k.mean_k[:, : st.mean_k.length], kv_len=kv_len)
            path = "flashprefill_chunked_selected"
        else:
            attn, stats = self._dense(q, kv_view, kv_len, bs), {}
            path = "dense_fallback"
        out = self._finish(attn, input_shape)
        self._compactattn_last_stats = dict(stats or {}, path=path) if self.compactattn_debug else None
        return out, 0.0, None, None, None
