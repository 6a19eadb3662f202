"""The benchmark configurations end to end on the CUDA path, against the CPU oracle.

* 32K paged cache, chunk 1024, training-free selection (mean-pooled block logits, cumulative-softmax
  threshold 0.9 + sink + local), and the reference's own training-free rule (alpha x row-max, sink 2,
  window 4) on the same tensors: floating-point stages bounded at 1e-3 relative, then the integer
  stages (rule, Block-Union, table) compared bit for bit with the oracle fed the numbers the GPU
  produced, then the attention output at max-abs 2e-2 / mean-abs 2e-3.
* 128K context, chunk 1024, all 8 KV heads in one launch (whole work units, no merge): every output
  row against the oracle, head by head.
"""
import pytest
import torch

from oracle import compact_oracle as co

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_ABS, REL = 2e-2, 2e-3, 1e-3


@pytest.fixture(scope="module")
def mods():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from compactattention_b200 import ops
    from compactattention_b200.paged_cache import PagedKVCache

    return ops, PagedKVCache


def low_rank_biased_kv(g, Q, K, Hq, Hkv, D, bs, rank=4, amp=20.0):
    """N(0,1) tensors; K rows carry a per-head rank-`rank` bias whose strength is constant inside a
    key block (a few blocks matter a lot), and the queries lean on the same directions, so pooled
    scores are peaked instead of flat."""
    G = Hq // Hkv
    q = torch.randn((1, Q, Hq, D), generator=g)
    k = torch.randn((1, K, Hkv, D), generator=g)
    v = torch.randn((1, K, Hkv, D), generator=g)
    u = torch.nn.functional.normalize(torch.randn((Hkv, rank, D), generator=g), dim=-1)
    a = amp * torch.rand((K // bs, Hkv, rank), generator=g) ** 4
    k = k + torch.einsum("thr,hrd->thd", a.repeat_interleave(bs, dim=0), u).view(1, K, Hkv, D)
    w = torch.rand((Hq, rank), generator=g) + 0.5
    q = q + torch.einsum("hr,hrd->hd", w, u.repeat_interleave(G, dim=0)).view(1, 1, Hq, D) * 1.5
    return q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)


def check_attention(out, want):
    err = (out.float().cpu() - want).abs()
    assert not torch.isnan(out.float()).any()
    assert err.max().item() < MAX_ABS and err.mean().item() < MEAN_ABS, (err.max().item(), err.mean().item())


def test_32k_paged_cache_training_free_selection_end_to_end(mods):
    ops, PagedKVCache = mods
    g = torch.Generator().manual_seed(1234 + 2)
    Q, K, Hq, Hkv, D, bs = 1024, 32768, 32, 8, 128, 64
    G, Qb, Kb = Hq // Hkv, Q // bs, K // bs
    Pb = Kb - Qb
    q, k, v = low_rank_biased_kv(g, Q, K, Hq, Hkv, D, bs)
    perm = torch.randperm(K // 64, generator=g).to(torch.int32).view(1, -1)
    cache = PagedKVCache(1, K, Hkv, D, "cuda", page_table=perm.cuda())
    cache.append(k.cuda(), v.cuda(), position=0)
    assert not torch.equal(perm, torch.arange(K // 64, dtype=torch.int32).view(1, -1))
    qd = q.cuda()
    valid = co.block_valid_mask(Qb, Kb, Pb).view(1, 1, Qb, Kb).expand(1, Hq, Qb, Kb)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    # ---- mode 1: mean-pooled Q-block x K-block logits, cumulative softmax mass 0.9, sink 1, local 2 ----
    qb = ops.pool_blocks(qd, bs, ("avg",))
    kb = ops.pool_blocks(k.cuda(), bs, ("avg",))
    logits = ops.gate_scores(qb, kb, Pb, scale=D ** -0.5)
    prob = torch.empty_like(logits)
    bits = ops.select_rows(logits, Pb, "cummass", softmax=True, threshold=0.9, sink=1, local=2, prob_out=prob)
    table = ops.union_table(bits=bits, num_kv_heads=Hkv, kv_blocks=Kb, past_blocks=Pb, block_size=bs)
    out = ops.attn_compact(qd, cache.view(), K, Hkv, table.block_idx, table.counts, block_size=bs, status=status)
    # floating point: logits and probabilities against the oracle's chain
    mask = co.gate_block_causal_mask(Q, K, bs)
    want_logits = co.gate_score(co.pool_blocks(q.float(), bs, ("avg",)), co.pool_blocks(k.float(), bs, ("avg",)), mask,
                                use_softmax=False)
    scale = want_logits.masked_fill(~valid, 0).abs().amax(dim=-1, keepdim=True)
    assert (((logits.cpu() - want_logits).abs() / scale)[valid]).max().item() < REL
    want_prob = co.masked_softmax_rows(want_logits, valid)
    assert ((prob.cpu() - want_prob).abs() / want_prob.amax(dim=-1, keepdim=True)).max().item() < REL
    # integers: the oracle's rule on the probabilities the GPU used, then union and table, bit for bit
    keep = co.cummass_rows(prob.cpu(), valid, 0.9) | (co.forced_mask(Qb, Kb, Pb, 1, 2) & valid)
    assert torch.equal(ops.unpack_bits(bits, Kb).cpu(), keep)
    idx, counts = co.block_union_table(keep.any(dim=2), Q, K, bs, G)
    assert torch.equal(table.block_idx.cpu(), idx) and torch.equal(table.counts.cpu(), counts)
    assert torch.equal(table.cache_seqlens.cpu(), (counts + Qb) * bs)
    density = counts.float().mean().item() / Pb
    assert 0.02 < density < 0.9, density  # peaked scores: the rule selects a real subset
    check_attention(out, co.compact_attention(q, k, v, idx, counts, bs))

    # ---- mode 2: the reference's training-free rule on the same tensors (alpha 0.06, sink 2, window 4) ----
    mean_k = ops.pool_blocks(k.cuda(), bs, ("avg",), out_dtype=torch.bfloat16)
    _, _, norm = ops.flashprefill_score(qd, mean_k, K, bs)
    bits2 = ops.select_rows(norm.permute(0, 3, 1, 2), Pb, "alpha_rowmax", alpha=0.06, sink=2, local=4)
    table2 = ops.union_table(bits=bits2, num_kv_heads=Hkv, kv_blocks=Kb, past_blocks=Pb, block_size=bs)
    out2 = ops.attn_compact(qd, cache.view(), K, Hkv, table2.block_idx, table2.counts, block_size=bs, status=status)
    o_mean_k = co.mean_pool_blocks(k, bs)
    o_raw, o_mx = co.flashprefill_block_score_raw(q, o_mean_k, K, bs)
    o_norm = co.flashprefill_normalize_scores(o_raw, o_mx)
    assert ((norm.cpu() - o_norm).abs() / o_norm.amax(dim=2, keepdim=True).clamp_min(1e-30)).max().item() < REL
    keep_row, _, keep_kv = co.flashprefill_keep_rowwise(norm.cpu(), Q, K, bs, G, 2, 4, 0.06, 0, 0)
    assert torch.equal(ops.unpack_bits(bits2, Kb).cpu(), keep_row)
    idx2, counts2, _, _ = co.block_table_from_kv_keep(keep_kv, Q, K, bs)
    assert torch.equal(table2.block_idx.cpu(), idx2) and torch.equal(table2.counts.cpu(), counts2)
    check_attention(out2, co.compact_attention(q, k, v, idx2, counts2, bs))
    torch.cuda.synchronize()
    assert int(status.item()) == 0


def test_128k_context_all_kv_heads_against_oracle(mods):
    """The shape the benchmark times: 32/8 heads, chunk 1024 at the end of a 128K-token paged cache with
    permuted pages, about 20 % of the past blocks per KV head: 128 work units in one launch, whole (one
    unit per SM) and cut over all SMs with the pieces merged (the default at this size)."""
    ops, PagedKVCache = mods
    g = torch.Generator().manual_seed(1234 + 3)
    Q, K, Hq, Hkv, D, bs = 1024, 131072, 32, 8, 128, 64
    G, Pb = Hq // Hkv, (K - Q) // bs
    q = torch.randn((1, Q, Hq, D), generator=g).to(torch.bfloat16)
    k = torch.randn((1, K, Hkv, D), generator=g).to(torch.bfloat16)
    v = torch.randn((1, K, Hkv, D), generator=g).to(torch.bfloat16)
    keep = torch.rand((1, Hkv, Pb), generator=g) < 0.2
    idx = torch.full((1, Hkv, Pb), -1, dtype=torch.int32)
    counts = torch.zeros((1, Hkv), dtype=torch.int32)
    for h in range(Hkv):
        sel = torch.nonzero(keep[0, h]).flatten().to(torch.int32)
        idx[0, h, : sel.numel()], counts[0, h] = sel, sel.numel()
    perm = torch.randperm(K // 64, generator=g).to(torch.int32).view(1, -1)
    cache = PagedKVCache(1, K, Hkv, D, "cuda", page_table=perm.cuda())
    cache.append(k.cuda(), v.cuda(), position=0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lse = torch.empty((1, Hq, Q), dtype=torch.float32, device="cuda")
    from compactattention_b200 import _lib
    n0 = _lib.launch_count()
    whole = ops.attn_compact(q.cuda(), cache.view(), K, Hkv, idx.cuda(), counts.cuda(), block_size=bs, status=status,
                             use_workspace=False).cpu()
    assert _lib.launch_count() - n0 == 1  # without a workspace every unit stays on one SM: no merge launch
    out = ops.attn_compact(q.cuda(), cache.view(), K, Hkv, idx.cuda(), counts.cuda(), block_size=bs, status=status, lse=lse)
    out, lse = out.cpu(), lse.cpu()
    assert int(status.item()) == 0
    for h in range(Hkv):  # one KV head at a time keeps the oracle's score tensor small
        want, want_lse = co.compact_attention(q[:, :, h * G:(h + 1) * G], k[:, :, h:h + 1], v[:, :, h:h + 1], idx[:, h:h + 1],
                                              counts[:, h:h + 1], bs, return_lse=True)
        check_attention(out[:, :, h * G:(h + 1) * G], want)
        check_attention(whole[:, :, h * G:(h + 1) * G], want)
        assert torch.allclose(lse[:, h * G:(h + 1) * G], want_lse, rtol=1e-3, atol=2e-2)
