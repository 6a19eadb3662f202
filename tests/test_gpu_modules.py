"""GPU tests of the host-side mirror: the operator functions with the reference's signatures, the
AttnGate mirror, the Llama attention modules and the small decoder stack, against compositions of
the CPU oracle (bit-exact tables, attention within max-abs 2e-2 / mean-abs 2e-3)."""
import math

import numpy as np
import pytest
import torch

from oracle import compact_oracle as co

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


@pytest.fixture(scope="module")
def gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda")


def close(out, want):
    err = (out.float().cpu() - want).abs()
    assert not torch.isnan(out.float()).any()
    assert err.max().item() < MAX_ABS and err.mean().item() < MEAN_ABS, (err.max().item(), err.mean().item())


def test_forward_operator_threshold_path(gpu):
    from compactattention_b200.modules import chunked_prefill_column_dense_attention_forward as fwd
    g = torch.Generator().manual_seed(3)
    B, Q, K, Hq, Hkv, D, bs = 1, 256, 4096, 8, 2, 128, 64
    Qb, Kb = Q // bs, K // bs
    q = torch.randn((B, Q, Hq, D), generator=g).to(torch.bfloat16)
    k = torch.randn((B, K, Hkv, D), generator=g).to(torch.bfloat16)
    v = torch.randn((B, K, Hkv, D), generator=g).to(torch.bfloat16)
    mask = co.gate_block_causal_mask(Q, K, bs)
    score = torch.softmax((torch.randn((B, Hq, Qb, Kb), generator=g) * 2.5).masked_fill(~mask, -1e30), dim=-1)
    out, stats = fwd(q.cuda(), k.cuda(), v.cuda(), None, query_length=Q, attn_gate_score=score.cuda(), block_attention_mask=None,
                     threshold=0.02, keep_recent_blocks=2, block_size=bs, num_key_value_groups=Hq // Hkv,
                     pack_impl="indexed_dense", indexed_impl="b200_native", return_stats=True)
    keep = co.seer_keep_block_fast(score, 0.02, 2, Q, K, bs)
    idx, counts = co.block_union_table(keep, Q, K, bs, Hq // Hkv)
    close(out, co.compact_attention(q, k, v, idx, counts, bs))
    assert stats["selected_blocks"] == float(co.kv_head_union(keep, Q, K, bs, Hq // Hkv).sum())
    assert 0 < stats["select_ratio"] < 1 and stats["compactattn_version"].startswith("CompactAttn-B200")
    for key in ("col_index_build_ms", "col_indexed_dense_kernel_ms", "dense_kernel_ms", "col_select_mask_ms"):
        assert key in stats
    # same result with every accepted backend name, with an explicit block mask, and without stats
    out2, none = fwd(q.cuda(), k.cuda(), v.cuda(), None, query_length=Q, attn_gate_score=score.cuda(),
                     block_attention_mask=mask.cuda(), threshold=0.02, keep_recent_blocks=2, block_size=bs,
                     num_key_value_groups=Hq // Hkv, pack_impl="indexed_dense", indexed_impl="fi_zero_copy")
    assert none is None and torch.equal(out2, out)
    # contract errors mirror the reference's
    with pytest.raises(ValueError, match="attn_gate_score is required"):
        fwd(q.cuda(), k.cuda(), v.cuda(), None, query_length=Q)
    with pytest.raises(ValueError, match="Unsupported indexed_impl"):
        fwd(q.cuda(), k.cuda(), v.cuda(), None, query_length=Q, attn_gate_score=score.cuda(), indexed_impl="nope")
    with pytest.raises(ValueError, match="query_length > 1"):
        fwd(q.cuda(), k.cuda(), v.cuda(), None, query_length=1, attn_gate_score=score.cuda())


def test_from_keep_block_operator(gpu):
    from compactattention_b200.modules import chunked_prefill_column_dense_attention_from_keep_block as fkb
    g = torch.Generator().manual_seed(4)
    B, Q, K, Hq, Hkv, D, bs = 2, 128, 2048, 8, 4, 128, 64
    q = torch.randn((B, Q, Hq, D), generator=g).to(torch.bfloat16)
    k = torch.randn((B, K, Hkv, D), generator=g).to(torch.bfloat16)
    v = torch.randn((B, K, Hkv, D), generator=g).to(torch.bfloat16)
    keep = torch.rand((B, Hq, K // bs), generator=g) < 0.25
    idx, counts = co.block_union_table(keep, Q, K, bs, Hq // Hkv)
    want = co.compact_attention(q, k, v, idx, counts, bs)
    out, _ = fkb(q.cuda(), k.cuda(), v.cuda(), keep.cuda(), None, Q, D ** -0.5, block_size=bs, num_key_value_groups=Hq // Hkv,
                 pack_impl="indexed_dense", allow_indexed_dense=True)
    close(out, want)
    keep_kv = co.kv_head_union(keep, Q, K, bs, Hq // Hkv)
    out2, _ = fkb(q.cuda(), k.cuda(), v.cuda(), None, None, Q, D ** -0.5, block_size=bs, num_key_value_groups=Hq // Hkv,
                  keep_block_kv_preprojected=keep_kv.cuda())
    assert torch.equal(out2, out)
    with pytest.raises(ValueError, match="Either keep_block or keep_block_kv_preprojected"):
        fkb(q.cuda(), k.cuda(), v.cuda(), None, None, Q, D ** -0.5)
    with pytest.raises(ValueError, match="keep_block shape mismatch"):
        fkb(q.cuda(), k.cuda(), v.cuda(), keep[:, :, :-1].cuda(), None, Q, D ** -0.5)


def test_flashprefill_operator(gpu):
    from compactattention_b200.modules import flashprefill_compactattn_prefill_full_kv as fp
    g = torch.Generator().manual_seed(5)
    B, Q, K, Hq, Hkv, D, bs = 1, 256, 4096, 8, 2, 128, 128
    G = Hq // Hkv
    q = torch.randn((B, Q, Hq, D), generator=g).to(torch.bfloat16)
    k = torch.randn((B, K, Hkv, D), generator=g).to(torch.bfloat16)
    # a few key blocks aligned with the queries so the alpha rule has something to select
    u = torch.randn((Hkv, D), generator=g)
    boost = (torch.rand((K // bs, Hkv), generator=g) < 0.15).float().repeat_interleave(bs, dim=0)
    k = (k.float() + 3.0 * boost.view(1, K, Hkv, 1) * u.view(1, 1, Hkv, D)).to(torch.bfloat16)
    q = (q.float() + 1.0 * u.repeat_interleave(G, dim=0).view(1, 1, Hq, D)).to(torch.bfloat16)
    v = torch.randn((B, K, Hkv, D), generator=g).to(torch.bfloat16)
    kw = dict(softmax_scale=D ** -0.5, num_key_value_groups=G, block_size=bs, attention_sink=2, window_size=4, alpha=0.06,
              last_n_block=0, min_budget=0, pack_impl="indexed_dense", indexed_impl="b200_native", cache_fill_backend="auto")
    out, stats = fp(q.cuda(), k.cuda(), v.cuda(), None, measure_timing=True, **kw)
    # The floating-point stage (block scores) is bounded against the oracle per row; the integer
    # stages (rule, union, table) are then checked exactly: the oracle's rule runs on the scores the
    # GPU produced (the same two launches the operator makes, read back), so the table the operator
    # used is known bit for bit and the attention comparison is unconditional.
    from compactattention_b200 import ops
    mean_k = co.mean_pool_blocks(k, bs)
    raw, mx = co.flashprefill_block_score_raw(q, mean_k, K, bs)
    norm = co.flashprefill_normalize_scores(raw, mx)
    mean_k_gpu = ops.pool_blocks(k.cuda(), bs, ("avg",), out_dtype=k.dtype)
    _, _, norm_gpu = ops.flashprefill_score(q.cuda(), mean_k_gpu, K, bs)
    norm_gpu = norm_gpu.cpu()
    row_max = norm.amax(dim=2, keepdim=True).clamp_min(1e-30)  # [B, Qb, 1, Hq]: the maximum the rule cuts against
    assert ((norm_gpu - norm).abs() / row_max).max().item() < 1e-3
    _, _, keep_kv = co.flashprefill_keep_rowwise(norm_gpu, Q, K, bs, G, 2, 4, 0.06, 0, 0)
    idx, counts, _, _ = co.block_table_from_kv_keep(keep_kv, Q, K, bs)
    density = float(keep_kv[..., : (K - Q) // bs].float().mean())
    assert 0.05 < density < 0.9
    assert stats["selected_blocks"] == float(keep_kv.sum())
    close(out, co.compact_attention(q, k, v, idx, counts, bs))
    # first chunk: dense
    out0, _ = fp(q.cuda(), k[:, :Q].contiguous().cuda(), v[:, :Q].contiguous().cuda(), None, **kw)
    close(out0, co.compact_attention(q, k[:, :Q], v[:, :Q], None, None, bs))


def test_attn_gate_module_matches_golden(gpu, golden):
    from compactattention_b200.prefill_sparse.attn_gate import ATTNGATE_CLASSES
    g = golden("attn_gate")
    B, Q, K, Hq, Hkv, D, bs = [int(x) for x in g["meta"]]
    T = lambda a: torch.from_numpy(np.asarray(a))
    for name, kwargs in (("Qavg_Kmaxminavg", {}), ("Qavg_Kavg", {"force_double": True})):
        gate = ATTNGATE_CLASSES[name](bs, D, 128, Hkv, Hq, **kwargs).cuda()
        state = {"mask_linear_k.weight": T(g[f"{name}_wk"]).float()}
        if f"{name}_wq" in g.files:
            state["mask_linear_q.weight"] = T(g[f"{name}_wq"]).float()
        gate.load_state_dict(state)  # the reference's parameter names
        # the reference gate scores the whole sequence's K against the chunk's Q
        q_full = torch.zeros((B, K, Hq, D))
        q_full[:, K - Q:] = T(g["q"]).float()
        cos, sin = T(g["cos"]).cuda(), T(g["sin"]).cuda()
        qb = gate.compress_query_blocks(T(g["q"]).float().cuda())
        kb = gate.compress_key_blocks(T(g["k"]).float().cuda())
        nb = qb.shape[1]
        qb, _ = gate.apply_block_position_embeddings(q=qb, position_embeddings=(cos[:, -nb:], sin[:, -nb:]))
        _, kb = gate.apply_block_position_embeddings(k=kb, position_embeddings=(cos, sin))
        soft = gate.score_compressed_blocks(qb, kb, T(g["mask"]).cuda(), use_softmax=True)
        want = T(g[f"{name}_score_softmax"])
        assert ((soft.cpu() - want).abs().amax(-1) / want.amax(-1)).max().item() < 1e-3


def _tiny_config(**kw):
    from compactattention_b200.prefill_sparse.llama import CompactAttnLlamaConfig
    base = dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=512,
                num_hidden_layers=2, vocab_size=1000, rope_theta=10000.0, seerattn_gate_type="Qavg_Kavg",
                seerattn_gate_force_double=True)
    base.update(kw)
    return CompactAttnLlamaConfig(**base)


def _torch_reference_stack(model, input_ids):
    """fp32 torch re-computation of the stack with dense causal attention (one shot, no chunks)."""
    cfg = model.config
    D = cfg.head_dim
    x = model.embed_tokens.weight.float()[input_ids]
    L = input_ids.shape[1]
    pos = torch.arange(L, device=x.device)
    ang = pos.float().unsqueeze(-1) * model.inv_freq.float().unsqueeze(0)
    ang = torch.cat([ang, ang], -1)
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    rot = lambda t: torch.cat((-t[..., D // 2:], t[..., : D // 2]), -1)
    for layer in model.layers:
        a = layer.self_attn
        h = layer.input_layernorm(x.to(torch.bfloat16)).float()
        q = (h @ a.q_proj.weight.float().T).view(1, L, -1, D)
        k = (h @ a.k_proj.weight.float().T).view(1, L, -1, D)
        v = (h @ a.v_proj.weight.float().T).view(1, L, -1, D)
        q, k = q * cos + rot(q) * sin, k * cos + rot(k) * sin
        G = q.shape[2] // k.shape[2]
        att = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(G, 1), v.transpose(1, 2).repeat_interleave(G, 1), is_causal=True)
        x = x + att.transpose(1, 2).reshape(1, L, -1) @ a.o_proj.weight.float().T
        h2 = layer.post_attention_layernorm(x.to(torch.bfloat16)).float()
        m = layer.mlp
        x = x + (torch.nn.functional.silu(h2 @ m.gate_proj.weight.float().T) * (h2 @ m.up_proj.weight.float().T)) @ m.down_proj.weight.float().T
    return model.norm(x.to(torch.bfloat16)).float()


@pytest.mark.parametrize("selector", ["gate", "flashprefill"])
def test_stack_chunked_prefill_keep_all_equals_dense(gpu, selector):
    """With a rule that keeps every block, chunked compact prefill equals one-shot dense attention."""
    from compactattention_b200.prefill_sparse.llama.harness import LlamaCompactAttnStack
    cfg = _tiny_config(seerattn_threshold=-1.0, seerattn_flashprefill_alpha=0.0)
    model = LlamaCompactAttnStack(cfg, selector).to(gpu).to(torch.bfloat16)
    model.init_weights(seed=1)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, cfg.vocab_size, (1, 1024), generator=g).to(gpu)
    hidden, cache = model.prefill(ids, chunk_size=256)
    want = _torch_reference_stack(model, ids)[:, -256:]
    err = (hidden.float() - want).abs()
    assert not torch.isnan(hidden.float()).any()
    assert err.max().item() < 0.25 and err.mean().item() < 2e-2, (err.max().item(), err.mean().item())  # bf16 stack vs fp32
    assert cache.get_seq_length(0) == 1024 and len(cache.layers) == cfg.num_hidden_layers
    stats_path = model.layers[0].self_attn._compactattn_last_stats
    assert stats_path is None  # stats only in debug mode


def test_seer_module_selects_and_reports(gpu):
    """One layer, four chunks, learned gate with top-k: the module's table equals the oracle's built
    from the module's own gate scores, and its output equals compact attention over that table."""
    from compactattention_b200 import ops
    from compactattention_b200.prefill_sparse.llama import CompactAttnCache, LlamaSeerAttentionChunkedDense
    cfg = _tiny_config(seerattn_sparsity_method="topk", seerattn_topk_ratio=(1, 4), compactattn_debug=True, num_hidden_layers=1)
    torch.manual_seed(0)
    attn = LlamaSeerAttentionChunkedDense(cfg, 0).to(gpu).to(torch.bfloat16)
    for p in attn.parameters():
        torch.nn.init.normal_(p, std=0.05)
    B, L, chunk, bs = 1, 1024, 256, 64
    x = (torch.randn((B, L, cfg.hidden_size), device=gpu) * 1.0).to(torch.bfloat16)
    cache = CompactAttnCache(B, L, gpu, torch.bfloat16)
    inv = 1.0 / (10000.0 ** (torch.arange(0, 128, 2, dtype=torch.float32, device=gpu) / 128))
    outs = []
    for s in range(0, L, chunk):
        pos = torch.arange(s, s + chunk, device=gpu)
        ang = torch.cat([pos.float()[:, None] * inv[None]] * 2, -1)
        cos, sin = ang.cos()[None].to(torch.bfloat16), ang.sin()[None].to(torch.bfloat16)
        bang = torch.cat([pos[::bs].float()[:, None] * inv[None]] * 2, -1)
        out = attn(x[:, s:s + chunk], (cos, sin), None, past_key_value=cache, block_position_embeddings=(bang.cos()[None], bang.sin()[None]))
        assert len(out) == 5 and out[1] == 0.0 and out[2] is None
        outs.append(out[0])
    assert attn._compactattn_last_stats["path"] == "chunked_selected"
    assert not torch.isnan(torch.cat(outs, 1).float()).any()
    # oracle for the last chunk from the module's own tensors
    st = cache.layers[0]
    logits = st.gate.logits.cpu()
    Qb, Kb = logits.shape[2], logits.shape[3]
    Pb = Kb - Qb
    valid = co.block_valid_mask(Qb, Kb, Pb).view(1, 1, Qb, Kb).expand_as(logits)
    n_valid = Pb + torch.arange(Qb) + 1
    kk = torch.minimum(torch.clamp((n_valid + 2) // 4, min=1), n_valid)
    keep = co.topk_rows(logits, valid, kk) | (co.forced_mask(Qb, Kb, Pb, 1, 2) & valid)
    idx, counts = co.block_union_table(keep.any(2), chunk, L, bs, 2)
    k_full = st.kv.k_pages.view(1, L, 2, 128).cpu()
    v_full = st.kv.v_pages.view(1, L, 2, 128).cpu()
    h = x[:, -chunk:]
    qn = (h @ attn.q_proj.weight.T).view(B, chunk, 4, 128)
    pos = torch.arange(L - chunk, L, device=gpu)
    ang = torch.cat([pos.float()[:, None] * inv[None]] * 2, -1)
    cos, sin = ang.cos()[None, :, None].to(torch.bfloat16), ang.sin()[None, :, None].to(torch.bfloat16)
    rot = lambda t: torch.cat((-t[..., 64:], t[..., :64]), -1)
    q = (qn * cos + rot(qn) * sin).to(torch.bfloat16).cpu()
    want_attn = co.compact_attention(q, k_full, v_full, idx, counts, bs)
    want = want_attn.reshape(B, chunk, -1) @ attn.o_proj.weight.float().cpu().T
    err = (outs[-1].float().cpu() - want).abs()
    assert err.max().item() < 5e-2 and err.mean().item() < 5e-3, (err.max().item(), err.mean().item())


@pytest.mark.parametrize("method,kw", [("threshold", dict(seerattn_threshold=2e-3)), ("topk", dict(seerattn_topk_ratio=(1, 4))),
                                        ("synthetic_topk", dict(seerattn_topk_ratio=(1, 3)))])
def test_one_call_layer_step_equals_the_operator_route(gpu, method, kw):
    """The module's default route enqueues the whole layer step with one library call (``ca_chunk_step``:
    RoPE + append, gate preparation, logits, rule + table, attention); with statistics switched on the same
    module goes stage by stage through the operator functions.  Same kernels, same order: identical bits,
    over four chunks the last of which is not a block multiple."""
    from compactattention_b200 import _lib
    from compactattention_b200.prefill_sparse.llama import CompactAttnCache, LlamaSeerAttentionChunkedDense
    B, L, chunk, bs = 1, 1000, 256, 64
    outs = {}
    for debug in (False, True):
        cfg = _tiny_config(seerattn_sparsity_method=method, compactattn_debug=debug, num_hidden_layers=1, **kw)
        torch.manual_seed(0)
        attn = LlamaSeerAttentionChunkedDense(cfg, 0).to(gpu).to(torch.bfloat16)
        for p in attn.parameters():
            torch.nn.init.normal_(p, std=0.05)
        x = torch.randn((B, L, cfg.hidden_size), device=gpu, generator=torch.Generator(device=gpu).manual_seed(1)).to(torch.bfloat16)
        cache = CompactAttnCache(B, 1024, gpu, torch.bfloat16)
        inv = 1.0 / (10000.0 ** (torch.arange(0, 128, 2, dtype=torch.float32, device=gpu) / 128))
        got, calls = [], []
        for s in range(0, L, chunk):
            e = min(s + chunk, L)
            pos = torch.arange(s, e, device=gpu)
            ang = torch.cat([pos.float()[:, None] * inv[None]] * 2, -1)
            bang = torch.cat([pos[::bs].float()[:, None] * inv[None]] * 2, -1)
            n0 = _lib.launch_count()
            got.append(attn(x[:, s:e], (ang.cos()[None].to(torch.bfloat16), ang.sin()[None].to(torch.bfloat16)), None,
                            past_key_value=cache, block_position_embeddings=(bang.cos()[None], bang.sin()[None]))[0])
            calls.append(_lib.launch_count() - n0)
        outs[debug] = torch.cat(got, 1)
        if not debug:
            assert cache.layers[0].plan is not None  # the one-call route ran
            # first chunk (dense): append, gate preparation, attention (+ its merge launch); later chunks add the
            # logits (not for synthetic scores) and the fused rule + table launch
            assert calls[0] in (3, 4) and all(c in (4, 5, 6) for c in calls[1:]), calls
            assert int(cache.layers[0].plan.scratch.status.item()) == 0
        else:
            assert cache.layers[0].plan is None
    assert not torch.isnan(outs[False].float()).any()
    assert torch.equal(outs[False], outs[True])
