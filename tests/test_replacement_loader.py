"""The insertion harness on a stock HuggingFace Llama: every ``self_attn`` replaced by a CompactAttention
module, projections reused, forward narrowed to ``(attn_output, attn_weights)``.

CPU: construction, parameter names (a stock checkpoint still loads; the gate's parameters sit under
``self_attn.attn_gate.*`` as in the reference's checkpoints), config markers.
GPU: chunked prefill through the stock model's own ``forward`` with the replaced modules - first with a
selection that keeps every block (must equal the stock model's dense attention within bf16 noise),
then with a real selection, against the stock model's hidden states masked the same way.
"""
import pytest
import torch


def tiny_llama(dtype=torch.bfloat16, layers=2, seed=0):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=1024,
                      num_hidden_layers=layers, vocab_size=1024, max_position_embeddings=8192, rms_norm_eps=1e-5,
                      rope_theta=500000.0, attention_bias=False, tie_word_embeddings=False)
    torch.manual_seed(seed)
    return LlamaForCausalLM(cfg).to(dtype).eval()


def test_replacement_keeps_stock_parameters_and_adds_the_gate():
    from compactattention_b200.load_attention_replacement import load_llama_attention_replacement_model
    from compactattention_b200.prefill_sparse.llama.modeling_llama_compactattn import (
        LlamaFlashPrefillCompactAttnAttention, LlamaSeerAttentionChunkedDense)
    stock = tiny_llama()
    stock_keys = set(stock.state_dict().keys())
    q0 = stock.model.layers[0].self_attn.q_proj
    model = load_llama_attention_replacement_model(model_id=None, base_model=stock, variant="seer_compactattn",
                                                   torch_dtype=torch.bfloat16, threshold=5e-4)
    keys = set(model.state_dict().keys())
    assert stock_keys <= keys  # a stock checkpoint loads unchanged
    extra = keys - stock_keys
    assert extra and all(".self_attn.attn_gate.mask_linear_" in k for k in extra), sorted(extra)[:4]
    for layer in model.model.layers:
        assert isinstance(layer.self_attn, LlamaSeerAttentionChunkedDense)
        assert hasattr(layer.self_attn, "_seer_replacement_original_forward")
    assert model.model.layers[0].self_attn.q_proj is q0  # projections reused, not copied
    assert model.config.seerattn_attention_harness == "replacement"
    assert model.config.seerattn_replacement_needs_block_gate_metadata is True
    assert model.config.seerattn_threshold == 5e-4
    assert not model.training and not model.model.layers[0].self_attn.training
    fp = load_llama_attention_replacement_model(model_id=None, base_model=tiny_llama(), variant="flashprefill_compactattn",
                                                torch_dtype=torch.bfloat16, flashprefill_alpha=0.06)
    assert isinstance(fp.model.layers[1].self_attn, LlamaFlashPrefillCompactAttnAttention)
    assert set(fp.state_dict().keys()) == stock_keys
    assert fp.config.seerattn_flashprefill_alpha == 0.06
    with pytest.raises(NotImplementedError):
        load_llama_attention_replacement_model(model_id=None, base_model=tiny_llama(), variant="seer_block_sparse",
                                               torch_dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="Unsupported attention replacement variant"):
        load_llama_attention_replacement_model(model_id=None, base_model=tiny_llama(), variant="nope", torch_dtype=torch.bfloat16)


def test_gate_checkpoint_loads_by_reference_parameter_names(tmp_path):
    from compactattention_b200.load_attention_replacement import load_llama_attention_replacement_model
    stock = tiny_llama()
    # a gate checkpoint as the reference stores it: only attn_gate parameters, by full module path
    shapes = {"mask_linear_k.weight": (4, 3 * 128, 128)}  # default gate Qavg_Kmaxminavg: one K projection per query head
    state = {f"model.layers.{i}.self_attn.attn_gate.{n}": torch.full(s, 0.5 + i) for i in range(2) for n, s in shapes.items()}
    path = tmp_path / "attn_gate_weights.pth"
    torch.save(state, path)
    model = load_llama_attention_replacement_model(model_id=str(tmp_path), base_model=stock, variant="seer_compactattn_hf",
                                                   torch_dtype=torch.bfloat16)
    w = model.model.layers[1].self_attn.attn_gate.mask_linear_k.weight
    assert w.shape == (4, 384, 128) and torch.all(w == 1.5)
    with pytest.raises(FileNotFoundError):
        load_llama_attention_replacement_model(model_id=str(tmp_path / "missing"), base_model=tiny_llama(),
                                               variant="seer_compactattn", torch_dtype=torch.bfloat16)


@pytest.mark.gpu
@pytest.mark.parametrize("variant", ["seer_compactattn", "flashprefill_compactattn"])
def test_replaced_model_prefills_like_the_stock_model(variant):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from transformers import DynamicCache
    from compactattention_b200.load_attention_replacement import load_llama_attention_replacement_model, new_cache
    L, chunk, decode = 1000, 256, 3  # the last chunk has 232 tokens (not a block multiple); then three decode steps
    ids = torch.randint(0, 1024, (1, L + decode), generator=torch.Generator().manual_seed(5)).cuda()
    stock = tiny_llama(seed=3).cuda()
    with torch.no_grad():
        want = stock.model(input_ids=ids, use_cache=False).last_hidden_state.float()
    # keep-everything selection: a threshold below every probability / alpha 0 keeps all visible blocks
    kw = dict(threshold=-1.0) if variant == "seer_compactattn" else dict(flashprefill_alpha=0.0, flashprefill_last_n_block=0,
                                                                          flashprefill_block_size=64)
    model = load_llama_attention_replacement_model(model_id=None, base_model=tiny_llama(seed=3).cuda(), variant=variant,
                                                   torch_dtype=torch.bfloat16, **kw)
    model.config.compactattn_max_tokens = 1024
    for cache in (new_cache(model, 1, 1024), DynamicCache(config=model.config)):  # the library's cache, and an adopted stock cache
        outs = []
        with torch.no_grad():
            bounds = list(range(0, L, chunk)) + [L] + [L + i + 1 for i in range(decode)]
            for s, e in zip(bounds[:-1], bounds[1:]):
                o = model.model(input_ids=ids[:, s:e], past_key_values=cache, use_cache=True)
                outs.append(o.last_hidden_state.float())
                assert cache.get_seq_length() == e
        got = torch.cat(outs, dim=1)
        err = (got - want).abs()
        scale = want.abs().mean().item()
        per_call = [round(err[:, s:e].mean().item(), 4) for s, e in zip(bounds[:-1], bounds[1:])]
        assert err.mean().item() < 0.02 * scale and err.max().item() < 0.25 * want.abs().max().item(), \
            (type(cache).__name__, per_call, err.max().item(), scale)
