"""A minimal Llama-3.1-shaped decoder stack around the CompactAttention modules, for chunked prefill
of long prompts with KV-head tensor parallelism (random-init weights; the stack exists to drive and
measure the attention path inside a full layer, not to be a model zoo).

Per layer: RMSNorm -> CompactAttention module (q/k/v/o projections, RoPE, paged cache, selector,
compact attention, all-reduce of the row-parallel o_proj) -> RMSNorm -> SwiGLU MLP (gate/up
column-parallel, down row-parallel + all-reduce).  Everything outside the attention path is plain
torch (cuBLAS GEMMs); it mirrors what the reference loads through HuggingFace with its tensor-parallel
plan (``compact_attn/prefill_sparse/llama/modeling_llama_seerattn.py:111-120``) and drives with
``run_chunked_prefill_once`` (``eval/chunked_prefill/chunked_prefill_runtime.py:1103-1321``).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import tp
from .modeling_llama_compactattn import (
    CompactAttnCache,
    CompactAttnLlamaConfig,
    LlamaFlashPrefillCompactAttnAttention,
    LlamaSeerAttentionChunkedDense,
)


class RMSNorm(nn.Module):
    def __init__(self, hidden: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden))
        self.eps = eps

    def forward(self, x):
        # one fused torch kernel (the norm is outside the attention path; six elementwise launches
        # per norm made a tensor-parallel rank wait for its host)
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


class ShardedMLP(nn.Module):
    def __init__(self, config: CompactAttnLlamaConfig, world: int):
        super().__init__()
        inter = config.intermediate_size // world
        self.gate_proj = nn.Linear(config.hidden_size, inter, bias=False)
        self.up_proj = nn.Linear(config.hidden_size, inter, bias=False)
        self.down_proj = nn.Linear(inter, config.hidden_size, bias=False)
        self.fused_rows = int(getattr(config, "compactattn_fused_oproj_rows", 0) or 0)

    def forward(self, x):
        h = F.silu(self.gate_proj(x)) * self.up_proj(x)
        # the down projection is row-parallel like o_proj: the same fused GEMM + sum over peer memory serves it
        if self.fused_rows and tp.fused_projection_applies(h, self.down_proj.weight, None, self.fused_rows):
            return tp.project_and_reduce(h, self.down_proj.weight, self.fused_rows)
        out = self.down_proj(h)
        tp.reduce_layer_output(out)
        return out


class DecoderLayer(nn.Module):
    _graph_pool = None

    def __init__(self, config, layer_idx, selector, shard):
        super().__init__()
        cls = LlamaSeerAttentionChunkedDense if selector == "gate" else LlamaFlashPrefillCompactAttnAttention
        self.self_attn = cls(config, layer_idx, shard)
        self.mlp = ShardedMLP(config, shard.world)
        self.input_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.graph_mlp = False   # set by the driver: replay the MLP half of the layer from a CUDA graph
        self._mlp_graph = None

    def _mlp_local(self, x, attn):
        """Residual add, norm and this rank's slice of the MLP (no collective): ``(x + attn, partial MLP output)``."""
        x = x + attn
        h = self.post_attention_layernorm(x)
        return x, self.mlp.down_proj(F.silu(self.mlp.gate_proj(h)) * self.mlp.up_proj(h))

    def forward(self, x, position_embeddings, cache, block_position_embeddings):
        kwargs = {}
        if isinstance(self.self_attn, LlamaSeerAttentionChunkedDense):
            kwargs["block_position_embeddings"] = block_position_embeddings
        attn = self.self_attn(self.input_layernorm(x), position_embeddings, None, past_key_value=cache, **kwargs)[0]
        self.self_attn.wait_pending_reduce()
        if not self.graph_mlp:
            x = x + attn
            return x + self.mlp(self.post_attention_layernorm(x))
        # The residual + norm + MLP half of the layer has the same shapes in every chunk: its local part
        # (no collective inside the capture) is captured once per layer and replayed, one host call
        # instead of eight; the all-reduce of the partial MLP output and the last add stay eager.
        g = self._mlp_graph
        if g is None or g[1].shape != x.shape:
            xin, ain = torch.empty_like(x), torch.empty_like(attn)
            xin.copy_(x), ain.copy_(attn)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._mlp_local(xin, ain)   # warm-up outside the capture (cuBLAS workspaces)
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            if DecoderLayer._graph_pool is None:   # the layers replay one after the other: one pool for all
                DecoderLayer._graph_pool = torch.cuda.graph_pool_handle()
            with torch.cuda.graph(graph, pool=DecoderLayer._graph_pool):
                x2, part = self._mlp_local(xin, ain)
            g = self._mlp_graph = (graph, xin, ain, x2, part)
        graph, xin, ain, x2, part = g
        xin.copy_(x), ain.copy_(attn)
        graph.replay()
        tp.reduce_layer_output(part)
        return x2 + part


class LlamaCompactAttnStack(nn.Module):
    def __init__(self, config: CompactAttnLlamaConfig, selector: str = "gate", shard: Optional[tp.HeadShard] = None):
        super().__init__()
        if selector not in ("gate", "flashprefill"):
            raise ValueError("selector must be 'gate' or 'flashprefill'")
        self.config, self.selector = config, selector
        self.shard = shard or tp.HeadShard(1, 0, config.num_attention_heads, config.num_key_value_heads)
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList(DecoderLayer(config, i, selector, self.shard) for i in range(config.num_hidden_layers))
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        inv = 1.0 / (config.rope_theta ** (torch.arange(0, config.head_dim, 2, dtype=torch.float32) / config.head_dim))
        self.register_buffer("inv_freq", inv, persistent=False)
        ginv = 1.0 / (config.rope_theta ** (torch.arange(0, config.seerattn_gate_hidden_size, 2, dtype=torch.float32)
                                            / config.seerattn_gate_hidden_size))
        self.register_buffer("gate_inv_freq", ginv, persistent=False)

    @torch.no_grad()
    def init_weights(self, seed: int = 0):
        """N(0, initializer_range) for every matrix (norm weights stay 1), from a per-rank-independent
        generator so that all ranks of a tensor-parallel group hold slices of the same full matrices."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        std = self.config.initializer_range
        cfg, sh = self.config, self.shard
        D = cfg.head_dim

        def full(*shape):
            return torch.randn(shape, generator=g) * std

        self.embed_tokens.weight.copy_(full(cfg.vocab_size, cfg.hidden_size))
        for layer in self.layers:
            a = layer.self_attn
            wq, wk, wv = full(cfg.num_attention_heads * D, cfg.hidden_size), full(cfg.num_key_value_heads * D, cfg.hidden_size), \
                full(cfg.num_key_value_heads * D, cfg.hidden_size)
            wo = full(cfg.hidden_size, cfg.num_attention_heads * D)
            a.q_proj.weight.copy_(wq[sh.q_heads.start * D: sh.q_heads.stop * D])
            a.k_proj.weight.copy_(wk[sh.kv_heads.start * D: sh.kv_heads.stop * D])
            a.v_proj.weight.copy_(wv[sh.kv_heads.start * D: sh.kv_heads.stop * D])
            a.o_proj.weight.copy_(sh.slice_o_proj(wo, D))
            if hasattr(a, "attn_gate"):
                full_gate_q = cfg.num_attention_heads
                gk = a.attn_gate.mask_linear_k
                heads_k_full = cfg.num_attention_heads if gk.weight.shape[0] == len(sh.q_heads) else cfg.num_key_value_heads
                wgk = full(heads_k_full, gk.weight.shape[1], gk.weight.shape[2])
                gk.weight.copy_(sh.slice_gate_weight(wgk) if sh.world > 1 else wgk)
                if a.attn_gate.mask_linear_q is not None:
                    gq = a.attn_gate.mask_linear_q
                    wgq = full(full_gate_q, gq.weight.shape[1], gq.weight.shape[2])
                    gq.weight.copy_(sh.slice_gate_weight(wgq) if sh.world > 1 else wgq)
            inter, r, w = cfg.intermediate_size, sh.rank, sh.world
            sl = slice(r * inter // w, (r + 1) * inter // w)
            layer.mlp.gate_proj.weight.copy_(full(inter, cfg.hidden_size)[sl])
            layer.mlp.up_proj.weight.copy_(full(inter, cfg.hidden_size)[sl])
            layer.mlp.down_proj.weight.copy_(full(cfg.hidden_size, inter)[:, sl])

    def _rope(self, positions: torch.Tensor, inv_freq: torch.Tensor):
        ang = positions.float().unsqueeze(-1) * inv_freq.unsqueeze(0)
        ang = torch.cat([ang, ang], dim=-1)
        return ang.cos().unsqueeze(0), ang.sin().unsqueeze(0)  # [1, L, D]

    def new_cache(self, batch: int, max_tokens: int, page_table: Optional[torch.Tensor] = None) -> CompactAttnCache:
        p = next(self.parameters())
        return CompactAttnCache(batch, max_tokens, p.device, p.dtype, page_table=page_table)

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, chunk_size: int, cache: Optional[CompactAttnCache] = None):
        """Chunked prefill of ``input_ids [B, L]`` (L a multiple of chunk_size); returns the hidden states
        of the last chunk ``[B, chunk, hidden]`` and the cache."""
        B, L = input_ids.shape
        if L % chunk_size:
            raise ValueError("the prompt length must be a multiple of the chunk size")
        cache = cache or self.new_cache(B, L)
        bs = self.config.seerattn_gate_block_size
        hidden = None
        for start in range(0, L, chunk_size):
            pos = torch.arange(start, start + chunk_size, device=input_ids.device)
            cos, sin = self._rope(pos, self.inv_freq)
            dt = self.embed_tokens.weight.dtype
            bcos, bsin = self._rope(pos[::bs], self.gate_inv_freq)
            x = self.embed_tokens(input_ids[:, start:start + chunk_size])
            for layer in self.layers:
                x = layer(x, (cos.to(dt), sin.to(dt)), cache, (bcos, bsin))
            hidden = self.norm(x)
        return hidden, cache
