"""Stock HuggingFace Llama models with every layer's ``self_attn`` replaced by a CompactAttention module
of this library - the insertion harness of the reference
(``compact_attn/load_attention_replacement.py``: ``load_llama_attention_replacement_model`` :236-336,
``_adapt_attention_return_contract`` :75-93, ``_reuse_attention_projections`` :96-100, the runtime
attribute whitelist :41-72).  The decoder layers, norms, MLPs and the LM head stay the stock
implementation; the replaced module keeps the stock projection modules (so their parameters stay
under ``self_attn.*`` and tensor-parallel sharding of the stock model is preserved) and its forward is
narrowed to HuggingFace's ``(attn_output, attn_weights)``.

The KV cache of the replaced modules is this library's paged cache: pass a ``CompactAttnCache`` as
``past_key_values`` (``new_cache`` builds one for a model); it answers the two questions the stock
model asks a cache (``get_seq_length``, ``get_mask_sizes``).  A stock ``DynamicCache`` handed in by
unchanged calling code is adopted: a paged cache is attached to it and it reports that cache's
length, while its own layers stay empty.

Only the variants on the chunked-prefill CompactAttention path are built: ``seer_compactattn`` /
``seer_compactattn_hf`` (learned gate) and ``flashprefill_compactattn`` (training-free); the
block-sparse variants raise ``NotImplementedError``.
"""
from __future__ import annotations

import copy
from types import MethodType
from typing import Optional

import torch
from torch import nn

from .prefill_sparse.llama.modeling_llama_compactattn import (
    CompactAttnCache,
    CompactAttnLlamaConfig,
    LlamaFlashPrefillCompactAttnAttention,
    LlamaSeerAttentionChunkedDense,
)

# runtime attributes copied onto the stock config, the reference's whitelist (:41-72) restricted to
# what the path reads
_SEER_RUNTIME_ATTRS = (
    "seerattn_threshold",
    "seerattn_sparsity_method",
    "seerattn_gate_type",
    "seerattn_gate_block_size",
    "seerattn_gate_hidden_size",
    "seerattn_gate_force_double",
    "seerattn_compactattn_keep_recent_blocks",
    "seerattn_compactattn_disable_first_chunk_dense",
    "seerattn_compactattn_pack_impl",
    "seerattn_compactattn_indexed_impl",
    "seerattn_compactattn_cache_fill_backend",
    "seerattn_chunked_prefill_force_dense",
    "seerattn_flashprefill_alpha",
    "seerattn_flashprefill_block_size",
    "seerattn_flashprefill_attention_sink",
    "seerattn_flashprefill_window_size",
    "seerattn_flashprefill_last_n_block",
    "seerattn_flashprefill_min_budget",
    "seerattn_defer_async_collective_wait",
)

_VARIANTS = {
    "seer_compactattn": LlamaSeerAttentionChunkedDense,
    "seer_compactattn_hf": LlamaSeerAttentionChunkedDense,
    "flashprefill_compactattn": LlamaFlashPrefillCompactAttnAttention,
}


def adopt_past_key_values(cache, model_config, batch: int, device, dtype) -> CompactAttnCache:
    """The paged cache behind whatever the caller passed as ``past_key_values``: a ``CompactAttnCache``
    passes through; any other cache object gets one attached (sized by the config's
    ``compactattn_max_tokens`` or ``max_position_embeddings``) and is taught to report its length."""
    if isinstance(cache, CompactAttnCache):
        return cache
    if cache is None:
        raise ValueError("the replaced attention modules need a cache: call the model with use_cache=True "
                         "or pass past_key_values=new_cache(model, batch, max_tokens)")
    paged = getattr(cache, "_compactattn_cache", None)
    if paged is None:
        max_tokens = int(getattr(model_config, "compactattn_max_tokens", 0) or model_config.max_position_embeddings)
        paged = CompactAttnCache(batch, max_tokens, device, dtype)
        cache._compactattn_cache = paged
        cache.get_seq_length = lambda layer_idx=0: paged.get_seq_length(layer_idx if layer_idx in paged.layers else 0)
        cache.get_mask_sizes = lambda query_length, layer_idx=0: paged.get_mask_sizes(query_length, layer_idx)
    return paged


def new_cache(model: nn.Module, batch: int, max_tokens: int, page_table: Optional[torch.Tensor] = None) -> CompactAttnCache:
    """A paged cache for ``model`` (every layer allocates ``max_tokens`` tokens of K and V on first use)."""
    p = next(model.parameters())
    return CompactAttnCache(batch, max_tokens, p.device, p.dtype, page_table=page_table)


def _adapt_attention_return_contract(attn: nn.Module) -> None:
    """Keep params under ``self_attn.*`` while returning HF's 2-tuple shape.

    Besides narrowing the module's 5-tuple, the wrapper bridges the stock decoder layer's calling
    convention to the module's: ``past_key_values`` (the stock keyword) becomes ``past_key_value``
    and is adopted as a paged cache, and a learned-gate module that was not given
    ``block_position_embeddings`` computes them from ``position_ids`` (every block_size-th position,
    reference modeling_llama_seerattn.py:896-897) with the model's ``block_rotary_emb``."""
    if hasattr(attn, "_seer_replacement_original_forward"):
        return
    original_forward = attn.forward
    attn._seer_replacement_original_forward = original_forward

    def _forward(self, *args, **kwargs):
        if "past_key_values" in kwargs:
            pkv = kwargs.pop("past_key_values")
            if kwargs.get("past_key_value") is None and len(args) < 4:
                kwargs["past_key_value"] = pkv
        hidden = args[0] if args else kwargs["hidden_states"]
        if len(args) < 4 and not isinstance(kwargs.get("past_key_value"), CompactAttnCache):
            kwargs["past_key_value"] = adopt_past_key_values(kwargs.get("past_key_value"), self.config, hidden.shape[0],
                                                             hidden.device, hidden.dtype)
        rope = getattr(self, "_compactattn_block_rotary_emb", None)
        if (rope is not None and isinstance(self, LlamaSeerAttentionChunkedDense)
                and kwargs.get("block_position_embeddings") is None and len(args) < 6):
            position_ids = kwargs.get("position_ids")
            if position_ids is None:
                start = kwargs["past_key_value"].get_seq_length(self.layer_idx)
                position_ids = torch.arange(start, start + hidden.shape[1], device=hidden.device).unsqueeze(0)
            bs = self.config.seerattn_gate_block_size
            bcos, bsin = rope[0](hidden, position_ids[:, ::bs])
            kwargs["block_position_embeddings"] = (bcos.float(), bsin.float())
        out = self._seer_replacement_original_forward(*args, **kwargs)
        if isinstance(out, tuple):
            attn_output = out[0]
            attn_weights = out[2] if len(out) > 2 else None
        else:
            attn_output = out
            attn_weights = None
        return attn_output, attn_weights

    attn.forward = MethodType(_forward, attn)


def _reuse_attention_projections(dst: nn.Module, src: nn.Module) -> None:
    """Reuse stock projection modules so TP DTensor sharding is preserved."""
    for name in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm"):
        if hasattr(src, name):
            setattr(dst, name, getattr(src, name))


def _copy_seer_attrs_to_stock_config(stock_config, seer_config) -> None:
    for name in _SEER_RUNTIME_ATTRS:
        if hasattr(seer_config, name):
            setattr(stock_config, name, getattr(seer_config, name))


def _build_seer_config(stock_config, *, variant, threshold, compactattn_keep_recent_blocks, compactattn_disable_first_chunk_dense,
                       col_pack_impl, col_indexed_impl, col_cache_fill_backend, flashprefill_alpha, flashprefill_block_size,
                       flashprefill_attention_sink, flashprefill_window_size, flashprefill_last_n_block,
                       flashprefill_min_budget) -> CompactAttnLlamaConfig:
    """The path's configuration from the stock model's shape plus the loader's switches
    (the reference's ``_build_seer_config``, :109-159; gate hyper-parameters come from the gate
    checkpoint's config there and from attributes already present on the stock config here)."""
    head_dim = getattr(stock_config, "head_dim", None) or stock_config.hidden_size // stock_config.num_attention_heads
    rope_theta = getattr(stock_config, "rope_theta", None)
    if rope_theta is None:
        rope_theta = (getattr(stock_config, "rope_parameters", None) or {}).get("rope_theta", 500000.0)
    cfg = CompactAttnLlamaConfig(
        hidden_size=stock_config.hidden_size, num_attention_heads=stock_config.num_attention_heads,
        num_key_value_heads=stock_config.num_key_value_heads, head_dim=head_dim,
        intermediate_size=stock_config.intermediate_size, num_hidden_layers=stock_config.num_hidden_layers,
        vocab_size=stock_config.vocab_size, rms_norm_eps=stock_config.rms_norm_eps, rope_theta=float(rope_theta),
        max_position_embeddings=stock_config.max_position_embeddings,
        initializer_range=getattr(stock_config, "initializer_range", 0.02),
        attention_bias=bool(getattr(stock_config, "attention_bias", False)),
    )
    for name in ("seerattn_gate_type", "seerattn_gate_block_size", "seerattn_gate_hidden_size", "seerattn_gate_force_double",
                 "seerattn_sparsity_method"):
        if hasattr(stock_config, name):
            setattr(cfg, name, getattr(stock_config, name))
    cfg.seerattn_threshold = float(threshold)
    cfg.seerattn_compactattn_keep_recent_blocks = int(compactattn_keep_recent_blocks)
    cfg.seerattn_compactattn_disable_first_chunk_dense = bool(compactattn_disable_first_chunk_dense)
    cfg.seerattn_compactattn_pack_impl = col_pack_impl
    cfg.seerattn_compactattn_indexed_impl = col_indexed_impl
    cfg.seerattn_compactattn_cache_fill_backend = col_cache_fill_backend
    cfg.seerattn_flashprefill_alpha = float(flashprefill_alpha)
    cfg.seerattn_flashprefill_block_size = int(flashprefill_block_size)
    cfg.seerattn_flashprefill_attention_sink = int(flashprefill_attention_sink)
    cfg.seerattn_flashprefill_window_size = int(flashprefill_window_size)
    cfg.seerattn_flashprefill_last_n_block = int(flashprefill_last_n_block)
    cfg.seerattn_flashprefill_min_budget = int(flashprefill_min_budget)
    return cfg


def _load_gate_weights(model: nn.Module, gate_model_id) -> None:
    """Loads ``attn_gate`` weights from a local ``attn_gate_weights.pth`` (the file the reference
    downloads from the gate repository, :227-233) or a state dict; ``None`` keeps the initial weights."""
    if gate_model_id is None:
        return
    state = gate_model_id if isinstance(gate_model_id, dict) else None
    if state is None:
        import os
        path = os.path.join(gate_model_id, "attn_gate_weights.pth") if os.path.isdir(gate_model_id) else gate_model_id
        if not os.path.exists(path):
            raise FileNotFoundError(f"no gate weights at {path} (there is no download route: pass a local file or directory)")
        state = torch.load(path, map_location="cpu", weights_only=True)
    missing = model.load_state_dict(state, strict=False)
    if not any("attn_gate" in k for k in state):
        raise ValueError("the gate checkpoint holds no attn_gate parameters")
    del missing


def load_llama_attention_replacement_model(
    *,
    model_id: str,
    base_model: str,
    variant: str,
    torch_dtype: torch.dtype,
    device_map=None,
    tp_plan: Optional[str] = None,
    dense_backend: str = "flashinfer",
    threshold: float = 3e-4,
    last_block_dense: bool = False,
    final_dense_tail_blocks: int = 0,
    compactattn_keep_recent_blocks: int = 2,
    compactattn_disable_first_chunk_dense: bool = False,
    compactattn_chunked_gate_head_pool: str = "avg",
    col_pack_impl: str = "indexed_dense",
    col_indexed_impl: str = "fa2_paged",
    col_cache_fill_backend: str = "auto",
    flashprefill_alpha: float = 0.01,
    flashprefill_block_size: int = 128,
    flashprefill_attention_sink: int = 2,
    flashprefill_window_size: int = 4,
    flashprefill_last_n_block: int = 2,
    flashprefill_min_budget: int = 0,
) -> nn.Module:
    """Same keyword signature as the reference's loader (:236-260).  ``base_model`` is a local
    checkpoint directory for ``LlamaForCausalLM.from_pretrained`` - or an already built stock
    ``LlamaForCausalLM`` (random-init models, models loaded by the caller).  ``model_id`` is the gate
    checkpoint (local file / directory / state dict) for the learned-gate variants, or ``None``.
    ``dense_backend``, ``last_block_dense``, ``final_dense_tail_blocks`` and
    ``compactattn_chunked_gate_head_pool`` are accepted for call-site compatibility; dense segments run
    the library's own kernel."""
    if variant in {"seer_block_sparse", "flashprefill_block_sparse"}:
        raise NotImplementedError(f"variant {variant!r} is a block-sparse comparator, not on the CompactAttention path")
    if variant not in _VARIANTS:
        raise ValueError(f"Unsupported attention replacement variant: {variant}")
    if isinstance(base_model, nn.Module):
        model = base_model.eval()
    else:
        from transformers import LlamaForCausalLM
        load_kwargs = dict(torch_dtype=torch_dtype)
        if tp_plan is not None:
            load_kwargs["tp_plan"] = tp_plan
        else:
            load_kwargs["device_map"] = device_map
        model = LlamaForCausalLM.from_pretrained(base_model, **load_kwargs).eval()

    seer_cfg = _build_seer_config(
        model.config, variant=variant, threshold=threshold, compactattn_keep_recent_blocks=compactattn_keep_recent_blocks,
        compactattn_disable_first_chunk_dense=compactattn_disable_first_chunk_dense, col_pack_impl=col_pack_impl,
        col_indexed_impl=col_indexed_impl, col_cache_fill_backend=col_cache_fill_backend, flashprefill_alpha=flashprefill_alpha,
        flashprefill_block_size=flashprefill_block_size, flashprefill_attention_sink=flashprefill_attention_sink,
        flashprefill_window_size=flashprefill_window_size, flashprefill_last_n_block=flashprefill_last_n_block,
        flashprefill_min_budget=flashprefill_min_budget)
    _copy_seer_attrs_to_stock_config(model.config, seer_cfg)

    # a block-rope module whose width is the gate's hidden size (reference :330-334)
    block_rotary = None
    if variant in {"seer_compactattn", "seer_compactattn_hf"}:
        block_config = copy.deepcopy(model.config)
        block_config.hidden_size = seer_cfg.seerattn_gate_hidden_size * seer_cfg.num_attention_heads
        block_config.head_dim = seer_cfg.seerattn_gate_hidden_size
        block_rotary = type(model.model.rotary_emb)(config=block_config)
        ref = model.model.embed_tokens.weight
        block_rotary.to(device=ref.device)
        model.model.block_rotary_emb = block_rotary

    for layer in model.model.layers:
        src_attn = layer.self_attn
        impl = _VARIANTS[variant](seer_cfg, layer_idx=src_attn.layer_idx)
        impl.to(device=src_attn.q_proj.weight.device, dtype=src_attn.q_proj.weight.dtype)
        _reuse_attention_projections(impl, src_attn)
        if block_rotary is not None:
            # held in a tuple so the shared rope module is not registered once per layer
            impl._compactattn_block_rotary_emb = (block_rotary,)
        _adapt_attention_return_contract(impl)
        layer.self_attn = impl
    model.eval()

    if variant in {"seer_compactattn", "seer_compactattn_hf"}:
        _load_gate_weights(model, model_id)

    # markers consumed by a chunked-prefill runner (reference :316-328)
    setattr(model.config, "seerattn_attention_harness", "replacement")
    setattr(model.config, "seerattn_replacement_needs_block_gate_metadata", variant in {"seer_compactattn", "seer_compactattn_hf"})
    setattr(model.config, "seerattn_cache_layout", "paged_b200")
    return model
