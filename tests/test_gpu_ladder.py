"""The input classes the reference serves through its fallback ladder, on the CUDA path, against the CPU
oracle: chunks that are not a block multiple (the last chunk of a real prompt), past lengths that are not
a block multiple (dense), decode steps (one query token, dense), scalar and per-batch threshold tensors read
on the device, and the checks that replace the ladder's remaining rungs (padded batches are refused after one
verified read of the mask).  Tables bit-exact, attention within max-abs 2e-2 / mean-abs 2e-3."""
import pytest
import torch

from oracle import compact_oracle as co

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


@pytest.fixture(scope="module")
def mods():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from compactattention_b200 import ops
    from compactattention_b200.paged_cache import PagedKVCache

    return ops, PagedKVCache


def close(out, want):
    err = (out.float().cpu() - want).abs()
    assert not torch.isnan(out.float()).any()
    assert err.max().item() < MAX_ABS and err.mean().item() < MEAN_ABS, (err.max().item(), err.mean().item())


def rand_qkv(g, B, Q, K, Hq, Hkv, dtype=torch.bfloat16):
    return (torch.randn((B, Q, Hq, 128), generator=g).to(dtype), torch.randn((B, K, Hkv, 128), generator=g).to(dtype),
            torch.randn((B, K, Hkv, 128), generator=g).to(dtype))


def table_from_keep(keep_kv, Pb):
    B, Hkv, _ = keep_kv.shape
    idx = torch.full((B, Hkv, max(Pb, 1)), -1, dtype=torch.int32)
    counts = torch.zeros((B, Hkv), dtype=torch.int32)
    for b in range(B):
        for h in range(Hkv):
            sel = torch.nonzero(keep_kv[b, h, :Pb]).flatten().to(torch.int32)
            idx[b, h, : sel.numel()], counts[b, h] = sel, sel.numel()
    return idx, counts


@pytest.mark.parametrize("B,Q,K,Hq,Hkv,bs,layout", [
    (1, 100, 1060, 8, 2, 64, "seq"),      # last chunk of 100 tokens after 15 blocks, contiguous cache of ragged length
    (2, 37, 37 + 640, 4, 4, 64, "seq"),   # batch of two, G = 1
    (1, 200, 200 + 1024, 28, 4, 128, "heads"),  # block 128, G = 7, heads-first cache
    (1, 333, 333 + 2048, 8, 2, 64, "paged"),    # paged cache whose last page is partly filled
    (1, 65, 65, 8, 8, 64, "seq"),         # first chunk that is itself ragged
])
def test_attention_with_a_ragged_last_chunk(mods, B, Q, K, Hq, Hkv, bs, layout):
    ops, PagedKVCache = mods
    g = torch.Generator().manual_seed(Q * 31 + K)
    q, k, v = rand_qkv(g, B, Q, K, Hq, Hkv)
    Pb = (K - Q) // bs
    keep = torch.rand((B, Hkv, max(Pb, 1)), generator=g) < 0.4
    idx, counts = table_from_keep(keep, Pb)
    if layout == "seq":
        kv = ops.KvCacheView.from_seq_first(k.cuda(), v.cuda())
    elif layout == "heads":
        kv = ops.KvCacheView.from_heads_first(k.transpose(1, 2).contiguous().cuda(), v.transpose(1, 2).contiguous().cuda())
    else:
        pages = -(-K // 64)
        perm = torch.randperm(pages, generator=g).to(torch.int32).view(1, -1).cuda()
        cache = PagedKVCache(1, pages * 64, Hkv, 128, "cuda", page_table=perm)
        ones = torch.ones((1, K, 128), dtype=torch.bfloat16, device="cuda")
        cache.append_rope(None, k.cuda(), v.cuda(), ones, torch.zeros_like(ones), position=0)  # identity rotation: a plain append
        kv = cache.view()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lse = torch.empty((B, Hq, Q), dtype=torch.float32, device="cuda")
    out = ops.attn_compact(q.cuda(), kv, K, Hkv, idx.cuda(), counts.cuda(), block_size=bs, status=status, lse=lse)
    want, want_lse = co.compact_attention(q, k, v, idx, counts, bs, return_lse=True)
    close(out, want)
    assert torch.allclose(lse.cpu(), want_lse, rtol=1e-3, atol=2e-2)
    assert int(status.item()) == 0


@pytest.mark.parametrize("B,Q,K,Hq,Hkv", [(1, 1, 777, 8, 2), (2, 1, 4097, 4, 4), (1, 37, 5000, 32, 8), (1, 300, 300 + 70, 8, 2)])
def test_dense_attention_with_an_unaligned_past_and_decode(mods, B, Q, K, Hq, Hkv):
    """No block table: dense causal attention for any Q and K - decode steps and pasts that are not block multiples."""
    ops, _ = mods
    g = torch.Generator().manual_seed(K)
    q, k, v = rand_qkv(g, B, Q, K, Hq, Hkv)
    kv = ops.KvCacheView.from_seq_first(k.cuda(), v.cuda())
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.attn_compact(q.cuda(), kv, K, Hkv, None, None, block_size=64, status=status)
    close(out, co.dense_causal_attention(q, k, v))
    assert int(status.item()) == 0
    # a block table needs an aligned past: refused, not computed
    if (K - Q) % 64:
        idx = torch.zeros((B, Hkv, max((K - Q) // 64, 1)), dtype=torch.int32, device="cuda")
        with pytest.raises(RuntimeError, match="multiple of block_size"):
            ops.attn_compact(q.cuda(), kv, K, Hkv, idx, torch.zeros((B, Hkv), dtype=torch.int32, device="cuda"), block_size=64)


def test_forward_operator_ragged_chunk_tensor_thresholds_and_fallbacks(mods):
    ops, _ = mods
    from compactattention_b200.modules import chunked_prefill_column_dense_attention_forward as fwd
    from compactattention_b200.modules import chunked_prefill_column_dense_attention_from_keep_block as fkb
    from compactattention_b200.modules.attention_forward_chunked_dense import clear_fast_path_content_cache
    g = torch.Generator().manual_seed(11)
    B, Q, P, Hq, Hkv, bs = 2, 150, 1920, 8, 2, 64
    K, G = P + Q, Hq // Hkv
    Qb, Kb, Pb = -(-Q // bs), -(-K // bs), P // bs
    q, k, v = rand_qkv(g, B, Q, K, Hq, Hkv)
    mask = co.gate_block_causal_mask(Q, K, bs, B)
    assert mask.shape[-2:] == (Qb, Kb)
    score = torch.softmax((torch.randn((B, Hq, Qb, Kb), generator=g) * 2.5).masked_fill(~mask, -1e30), dim=-1)
    kw = dict(query_length=Q, attn_gate_score=score.cuda(), block_attention_mask=mask.cuda(), keep_recent_blocks=2, block_size=bs,
              num_key_value_groups=G, pack_impl="indexed_dense", indexed_impl="b200_native")
    # float threshold, ragged chunk: the reference's generic mask builder on the same scores is the oracle
    out, stats = fwd(q.cuda(), k.cuda(), v.cuda(), None, threshold=0.02, return_stats=True, **kw)
    keep = co.seer_keep_block(score, mask, 0.02, 2)
    idx, counts = co.block_union_table(keep, Q, K, bs, G)
    close(out, co.compact_attention(q, k, v, idx, counts, bs))
    assert stats["selected_blocks"] == float(co.kv_head_union(keep, Q, K, bs, G).sum())
    # scalar tensor threshold: same result, read on the device
    out_t, _ = fwd(q.cuda(), k.cuda(), v.cuda(), None, threshold=torch.tensor(0.02, device="cuda"), **kw)
    assert torch.equal(out_t, out)
    # per-batch thresholds
    thr = torch.tensor([0.02, 0.2])
    out_b, _ = fwd(q.cuda(), k.cuda(), v.cuda(), None, threshold=thr.cuda(), **kw)
    keep_b = torch.cat([co.seer_keep_block(score[b:b + 1], mask[b:b + 1], float(thr[b]), 2) for b in range(B)])
    idx_b, counts_b = co.block_union_table(keep_b, Q, K, bs, G)
    assert counts_b[1].sum() < counts_b[0].sum()
    close(out_b, co.compact_attention(q, k, v, idx_b, counts_b, bs))
    with pytest.raises(ValueError, match="scalar or 1D batch threshold"):
        fwd(q.cuda(), k.cuda(), v.cuda(), None, threshold=torch.zeros(3, device="cuda"), **kw)
    # a past that is not a block multiple: dense over the whole cache, reported as a fallback
    k2, v2 = k[:, 7:].contiguous(), v[:, 7:].contiguous()
    K2 = K - 7
    score2 = torch.rand((B, Hq, -(-Q // bs), -(-K2 // bs)), generator=g)
    out_d, stats_d = fwd(q.cuda(), k2.cuda(), v2.cuda(), None, query_length=Q, attn_gate_score=score2.cuda(), threshold=0.5,
                         block_size=bs, num_key_value_groups=G, return_stats=True)
    close(out_d, co.dense_causal_attention(q, k2, v2))
    assert stats_d["fallback_used"] == 1.0 and stats_d["path"] == "dense_misaligned_past"
    # token masks: all ones passes (verified once, then cached); zeros are refused
    clear_fast_path_content_cache()
    ones = torch.ones((B, K), dtype=torch.bool, device="cuda")
    out_m, _ = fwd(q.cuda(), k.cuda(), v.cuda(), ones, threshold=0.02, **kw)
    assert torch.equal(out_m, out)
    clear_fast_path_content_cache()
    padded = ones.clone()
    padded[1, :5] = False
    with pytest.raises(NotImplementedError, match="padded batches"):
        fwd(q.cuda(), k.cuda(), v.cuda(), padded, threshold=0.02, **kw)
    clear_fast_path_content_cache()
    # from_keep_block with a ragged chunk
    keep_q = torch.rand((B, Hq, Kb), generator=g) < 0.3
    out_k, _ = fkb(q.cuda(), k.cuda(), v.cuda(), keep_q.cuda(), None, Q, 128 ** -0.5, block_size=bs, num_key_value_groups=G)
    idx_k, counts_k = co.block_union_table(keep_q, Q, K, bs, G)
    close(out_k, co.compact_attention(q, k, v, idx_k, counts_k, bs))


def test_flashprefill_operator_ragged_chunk(mods):
    ops, _ = mods
    from compactattention_b200.modules import flashprefill_compactattn_prefill_full_kv as fp
    g = torch.Generator().manual_seed(12)
    B, Q, P, Hq, Hkv, bs = 1, 200, 3072, 8, 2, 128
    K, G = P + Q, Hq // Hkv
    q, k, v = rand_qkv(g, B, Q, K, Hq, Hkv)
    u = torch.randn((Hkv, 128), generator=g)
    boost = (torch.rand((-(-K // bs), Hkv), generator=g) < 0.2).float().repeat_interleave(bs, dim=0)[:K]
    k = (k.float() + 3.0 * boost.view(1, K, Hkv, 1) * u.view(1, 1, Hkv, 128)).to(torch.bfloat16)
    q = (q.float() + u.repeat_interleave(G, dim=0).view(1, 1, Hq, 128)).to(torch.bfloat16)
    kw = dict(softmax_scale=128 ** -0.5, num_key_value_groups=G, block_size=bs, attention_sink=2, window_size=4, alpha=0.06,
              last_n_block=0, min_budget=0, pack_impl="indexed_dense", indexed_impl="b200_native", cache_fill_backend="auto")
    out, stats = fp(q.cuda(), k.cuda(), v.cuda(), None, measure_timing=True, **kw)
    mean_k = ops.pool_blocks(k.cuda(), bs, ("avg",), out_dtype=k.dtype)
    _, _, norm = ops.flashprefill_score(q.cuda(), mean_k, K, bs)
    o_raw, o_mx = co.flashprefill_block_score_raw(q, co.mean_pool_blocks(k, bs), K, bs)
    o_norm = co.flashprefill_normalize_scores(o_raw, o_mx)
    assert ((norm.cpu() - o_norm).abs() / o_norm.amax(dim=2, keepdim=True).clamp_min(1e-30)).max().item() < 1e-3
    _, _, keep_kv = co.flashprefill_keep_rowwise(norm.cpu(), Q, K, bs, G, 2, 4, 0.06, 0, 0)
    idx, counts, _, _ = co.block_table_from_kv_keep(keep_kv, Q, K, bs)
    assert stats["selected_blocks"] == float(keep_kv.sum())
    close(out, co.compact_attention(q, k, v, idx, counts, bs))
    # unaligned past: dense
    out_d, _ = fp(q.cuda(), k[:, 5:].contiguous().cuda(), v[:, 5:].contiguous().cuda(), None, **kw)
    close(out_d, co.dense_causal_attention(q, k[:, 5:], v[:, 5:]))
