"""GPU parity of block scoring: pooling, gate projection + RoPE + cache append, gate logits and
softmax, FlashPrefill block score and normalisation.  Floating point: scores must agree with the
fp32 oracle within 1e-3 relative (the tolerance the path's specification states); pooling of
fp32 inputs within 1e-6."""
import numpy as np
import pytest
import torch

from oracle import compact_oracle as co

pytestmark = pytest.mark.gpu

REL = 1e-3


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from compactattention_b200 import ops as o

    return o


def T(a):
    return torch.from_numpy(np.asarray(a))


def rel_err(got, want):
    scale = want.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
    return ((got - want).abs() / scale).max().item()


def fp_row_err(got, want):
    """Training-free scores are [B, Qb, Kb, Hq]: a row of the selection rule runs over the key blocks
    (dim 2), and the rule cuts at alpha x the row's maximum, so the error is bounded against it."""
    scale = want.abs().amax(dim=2, keepdim=True).clamp_min(1e-30)
    return ((got - want).abs() / scale).max().item()


def check_alpha_rule_on_gpu_scores(ops, norm_gpu, Q, K, bs, G):
    """The alpha x row-max rule on the scores the GPU produced: the kernel's packed bits against the
    oracle's rule on the same (read-back) numbers, bit for bit."""
    Qb, Kb = norm_gpu.shape[1], norm_gpu.shape[2]
    bits = ops.select_rows(norm_gpu.permute(0, 3, 1, 2), Kb - Qb, "alpha_rowmax", alpha=0.06, sink=2, local=4)
    keep_row, _, _ = co.flashprefill_keep_rowwise(norm_gpu.cpu(), Q, K, bs, G, 2, 4, 0.06, 0, 0)
    assert torch.equal(ops.unpack_bits(bits, Kb).cpu(), keep_row)  # [B, Hq, Qb, Kb]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("L,bs", [(1024, 64), (674, 64), (256, 128), (64, 64)])
def test_pool_blocks(ops, dtype, L, bs):
    g = torch.Generator().manual_seed(L + bs)
    x = torch.randn((2, L, 4, 128), generator=g).to(dtype)
    for kinds in (("avg",), ("max", "min", "avg"), ("max",), ("min", "avg")):
        got = ops.pool_blocks(x.cuda(), bs, kinds).cpu()
        want = co.pool_blocks(x.float(), bs, kinds)
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-6), kinds
    # mean-K as the training-free selector stores it, in the input dtype: the fp32 mean rounded once,
    # i.e. bit-identical to rounding the kernel's own fp32 result, which in turn is within fp32
    # summation-order error of the oracle's
    got = ops.pool_blocks(x.cuda(), bs, ("avg",), out_dtype=dtype).cpu()
    got32 = ops.pool_blocks(x.cuda(), bs, ("avg",)).cpu()
    assert got.dtype == dtype
    assert torch.equal(got, got32.to(dtype))
    want = co.mean_pool_blocks(x, bs)
    assert torch.allclose(got32, co.pool_blocks(x.float(), bs, ("avg",)), rtol=1e-5, atol=1e-6)
    if dtype != torch.float32:
        # against the oracle's stored value: equal except where the two fp32 means straddle a rounding
        # boundary of the 16-bit type (then one unit in the last place apart)
        assert (got != want).float().mean().item() < 1e-3
        ulp = want.float().abs().clamp_min(1e-3) * (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10)
        assert ((got.float() - want.float()).abs() <= ulp).all()


def test_pool_append_into_cache(ops):
    g = torch.Generator().manual_seed(3)
    cache = torch.zeros((1, 40, 2, 128), dtype=torch.float32, device="cuda")
    full = torch.randn((1, 40 * 64, 2, 128), generator=g)
    for c in range(5):  # five chunks of 8 blocks
        ops.pool_blocks(full[:, c * 512:(c + 1) * 512].cuda(), 64, ("avg",), out=cache, out_block_offset=c * 8)
    assert torch.allclose(cache.cpu(), co.pool_blocks(full, 64, ("avg",)), rtol=1e-5, atol=1e-6)


def test_mean_k_golden(ops, golden):
    g = golden("flashprefill")
    k = T(g["k"]).float()
    got = ops.pool_blocks(k.cuda(), 64, ("avg",)).cpu()
    assert torch.allclose(got, T(g["mean_k"]), rtol=1e-5, atol=1e-6)
    got_r = ops.pool_blocks(k[:, :674].contiguous().cuda(), 64, ("avg",)).cpu()
    assert torch.allclose(got_r, T(g["mean_k_ragged"]), rtol=1e-5, atol=1e-6)


def test_attn_gate_golden(ops, golden):
    """Whole learned-gate chain against the reference AttnGate's outputs."""
    g = golden("attn_gate")
    B, Q, K, Hq, Hkv, D, bs = [int(x) for x in g["meta"]]
    Qb, Kb = Q // bs, K // bs
    q, k = T(g["q"]).float().cuda(), T(g["k"]).float().cuda()
    cos, sin = T(g["cos"]).cuda(), T(g["sin"]).cuda()
    for name, kk in (("Qavg_Kmaxminavg", ("max", "min", "avg")), ("Qavg_Kavg", ("avg",))):
        wq = T(g[f"{name}_wq"]).float().cuda() if f"{name}_wq" in g.files else None
        wk = T(g[f"{name}_wk"]).float().cuda()
        q_pooled = ops.pool_blocks(q, bs, ("avg",))
        k_pooled = ops.pool_blocks(k, bs, kk)
        qb = ops.gate_project(q_pooled, wq)
        kb = ops.gate_project(k_pooled, wk)
        assert torch.allclose(qb.cpu(), T(g[f"{name}_qb"]), rtol=1e-4, atol=1e-5)
        assert torch.allclose(kb.cpu(), T(g[f"{name}_kb"]), rtol=1e-4, atol=1e-5)
        qb_r = ops.gate_project(q_pooled, wq, cos[:, Kb - Qb:], sin[:, Kb - Qb:])
        # K blocks are projected, roped and appended into a heads-first cache with spare capacity
        cache = torch.zeros((B, wk.shape[0], 16, 128), dtype=torch.float32, device="cuda")
        ops.gate_project(k_pooled[:, :3].contiguous(), wk, cos[:, :3], sin[:, :3], out=cache.transpose(1, 2))
        ops.gate_project(k_pooled[:, 3:].contiguous(), wk, cos[:, 3:], sin[:, 3:], out=cache.transpose(1, 2), out_block_offset=3)
        kb_r = cache.transpose(1, 2)[:, :Kb]
        assert torch.allclose(qb_r.cpu(), T(g[f"{name}_qb_rope"]), rtol=1e-4, atol=1e-5)
        assert torch.allclose(kb_r.cpu(), T(g[f"{name}_kb_rope"]), rtol=1e-4, atol=1e-5)
        logits = ops.gate_scores(qb_r, kb_r, Kb - Qb)
        want_raw = T(g[f"{name}_score_raw"])
        vis = T(g["mask"]).expand_as(want_raw)
        assert rel_err(logits.cpu()[vis], want_raw[vis]) < REL
        assert torch.equal(logits.cpu()[~vis], want_raw[~vis])  # finfo.min fill
        prob = torch.empty_like(logits)
        ops.select_rows(logits, Kb - Qb, "threshold", softmax=True, threshold=5e-4, prob_out=prob)
        assert rel_err(prob.cpu(), T(g[f"{name}_score_softmax"])) < REL


@pytest.mark.parametrize("kk,per_q_head,dtype", [(("max", "min", "avg"), True, torch.bfloat16), (("avg",), False, torch.bfloat16),
                                                 (("avg",), False, torch.float32)])
def test_gate_prepare_fused_matches_oracle(ops, kk, per_q_head, dtype):
    """The one-launch pool + project + RoPE + append against the oracle, chunk by chunk."""
    g = torch.Generator().manual_seed(21)
    B, Hq, Hkv, D, bs, chunks, L = 2, 8, 2, 128, 64, 3, 256
    Hk = Hq if per_q_head else Hkv
    nb = L // bs
    q = torch.randn((B, chunks * L, Hq, D), generator=g).to(dtype)
    k = torch.randn((B, chunks * L, Hkv, D), generator=g).to(dtype)
    wq = None if per_q_head else (torch.randn((Hq, D, 128), generator=g) * 0.05)
    wk = torch.randn((Hk, len(kk) * D, 128), generator=g) * 0.05
    inv = 1.0 / (10000.0 ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))
    ang = torch.cat([torch.arange(0, chunks * L, bs, dtype=torch.float32).view(-1, 1) * inv.view(1, -1)] * 2, dim=-1)
    cos, sin = ang.cos().unsqueeze(0), ang.sin().unsqueeze(0)
    cache = torch.zeros((B, Hk, 16, 128), dtype=torch.float32, device="cuda")
    for c in range(chunks):
        sl = slice(c * L, (c + 1) * L)
        bsl = slice(c * nb, (c + 1) * nb)
        q_out = torch.empty((B, nb, Hq, 128), dtype=torch.float32, device="cuda")
        ops.gate_prepare(q[:, sl].cuda(), k[:, sl].cuda(), bs, ("avg",), kk, None if wq is None else wq.cuda(), wk.cuda(),
                         (cos[:, bsl].cuda(), sin[:, bsl].cuda()), (cos[:, bsl].cuda(), sin[:, bsl].cuda()),
                         q_out, cache.transpose(1, 2), c * nb)
        want_q = co.pool_blocks(q[:, sl].float(), bs, ("avg",))
        if wq is not None:
            want_q = co.multi_head_linear(want_q, wq)
        want_q = co.apply_block_rope(want_q, cos[:, bsl], sin[:, bsl])
        assert torch.allclose(q_out.cpu(), want_q, rtol=1e-4, atol=1e-4)
    want_k = co.apply_block_rope(co.multi_head_linear(co.pool_blocks(k.float(), bs, kk), wk), cos, sin)
    assert torch.allclose(cache.transpose(1, 2)[:, : chunks * nb].cpu(), want_k, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("B,Qb,Kb,Hq,Hk,dtype", [(1, 16, 512, 32, 32, torch.bfloat16), (1, 16, 2048, 8, 2, torch.float32),
                                                 (2, 4, 130, 28, 4, torch.bfloat16), (1, 128, 256, 4, 4, torch.float16)])
def test_gate_scores_random(ops, B, Qb, Kb, Hq, Hk, dtype):
    g = torch.Generator().manual_seed(Kb)
    qb = torch.randn((B, Qb, Hq, 128), generator=g).to(dtype)
    kb = torch.randn((B, Kb, Hk, 128), generator=g).to(dtype)
    Pb = Kb - Qb
    mask = co.gate_block_causal_mask(Qb * 64, Kb * 64, 64, B)
    want = co.gate_score(qb, kb, mask, use_softmax=False)
    got = ops.gate_scores(qb.cuda(), kb.cuda(), Pb).cpu()
    vis = mask.expand_as(want)
    assert rel_err(got.masked_fill(~vis, 0), want.masked_fill(~vis, 0)) < REL
    prob = torch.empty_like(got, device="cuda")
    ops.select_rows(got.cuda(), Pb, "threshold", softmax=True, threshold=5e-4, prob_out=prob)
    assert rel_err(prob.cpu(), co.gate_score(qb, kb, mask, use_softmax=True)) < REL


def test_flashprefill_score_golden(ops, golden):
    g = golden("flashprefill")
    B, Q, K, Hq, Hkv, D, bs = [int(x) for x in g["meta"]]
    q = T(g["q"]).float().cuda()
    mean_k = T(g["mean_k"]).cuda()
    raw, mx, norm = ops.flashprefill_score(q, mean_k, K, bs)
    ref_mx, ref_sc, ref_norm = T(g["max_raw"]), T(g["score_raw"]), T(g["score_norm"])
    fin = torch.isfinite(ref_mx)
    assert torch.equal(torch.isfinite(mx.cpu()), fin)
    assert torch.allclose(mx.cpu()[fin], ref_mx[fin], rtol=1e-4, atol=1e-4)
    assert torch.allclose(raw.cpu()[fin], ref_sc[fin], rtol=1e-3, atol=1e-5)
    assert fp_row_err(norm.cpu(), ref_norm) < REL
    check_alpha_rule_on_gpu_scores(ops, norm, Q, K, bs, Hq // Hkv)


@pytest.mark.parametrize("Q,K,Hq,Hkv,bs,dtype", [(1024, 8192, 8, 2, 64, torch.bfloat16), (512, 4096, 4, 4, 128, torch.bfloat16),
                                                 (192, 704, 28, 4, 64, torch.float16), (100, 1060, 4, 1, 64, torch.float32),
                                                 (100, 1060, 4, 1, 64, torch.bfloat16), (1024, 32768, 32, 8, 128, torch.bfloat16),
                                                 (256, 256, 8, 2, 64, torch.bfloat16)])
def test_flashprefill_score_random(ops, Q, K, Hq, Hkv, bs, dtype):
    g = torch.Generator().manual_seed(Q + K)
    q = torch.randn((1, Q, Hq, 128), generator=g).to(dtype)
    k = torch.randn((1, K, Hkv, 128), generator=g).to(dtype)
    mean_k = co.mean_pool_blocks(k, bs)
    raw, mx, norm = ops.flashprefill_score(q.cuda(), mean_k.cuda(), K, bs)
    o_raw, o_mx = co.flashprefill_block_score_raw(q, mean_k, K, bs)
    o_norm = co.flashprefill_normalize_scores(o_raw, o_mx)
    fin = torch.isfinite(o_mx)
    assert torch.equal(torch.isfinite(mx.cpu()), fin)
    assert torch.allclose(mx.cpu()[fin], o_mx[fin], rtol=1e-4, atol=1e-4)
    assert fp_row_err(norm.cpu(), o_norm) < REL
    if Q % bs == 0 and K % bs == 0:
        check_alpha_rule_on_gpu_scores(ops, norm, Q, K, bs, Hq // Hkv)


@pytest.mark.parametrize("rule,kw", [("alpha_rowmax", dict(alpha=0.06, sink=2, local=4)),
                                     ("alpha_rowmax", dict(alpha=0.3, min_budget=5, sink=1, local=1)),
                                     ("topk", dict(topk_ratio=(1, 5), sink=1, local=2))])
@pytest.mark.parametrize("bs,Q,K", [(128, 1024, 32768), (64, 512, 8192)])
def test_rules_on_raw_scores_and_exponents_equal_rules_on_normalised_scores(ops, rule, kw, bs, Q, K):
    """The training-free selector's normalisation divides a row by its sum; the alpha * row-max and top-k rules
    do not depend on that, so the rule kernel may take score_raw and max_raw (``score_max``) and skip the
    normalisation launch.  Same keep bits as the rule on the normalised scores, and the same table."""
    g = torch.Generator().manual_seed(K + bs)
    Hq, Hkv = 8, 2
    q = torch.randn((1, Q, Hq, 128), generator=g).to(torch.bfloat16).cuda()
    mean_k = torch.randn((1, K // bs, Hkv, 128), generator=g).to(torch.bfloat16).cuda()
    raw, mx, norm = ops.flashprefill_score(q, mean_k, K, bs)
    Pb = (K - Q) // bs
    want = ops.select_rows(norm.permute(0, 3, 1, 2), Pb, rule, **kw)
    got = ops.select_rows(raw.permute(0, 3, 1, 2), Pb, rule, score_max=mx.permute(0, 3, 1, 2), **kw)
    assert torch.equal(got, want)
    t_want = ops.select_union_table(norm.permute(0, 3, 1, 2), Pb, rule, num_kv_heads=Hkv, block_size=bs, **kw)
    t_got = ops.select_union_table(raw.permute(0, 3, 1, 2), Pb, rule, num_kv_heads=Hkv, block_size=bs,
                                   score_max=mx.permute(0, 3, 1, 2), **kw)
    assert torch.equal(t_got.block_idx, t_want.block_idx) and torch.equal(t_got.counts, t_want.counts)
    with pytest.raises(ValueError, match="score_max"):
        ops.select_rows(raw.permute(0, 3, 1, 2), Pb, rule, score_max=mx, **kw)   # strides differ from the score's
