"""Per-query-head and query-sub-group block tables (several table rows per KV head), the reference's
``fi_zero_copy_per_query`` / ``fi_zero_copy_subgroup`` routes, against the CPU oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from compactattention_b200 import ops as _ops
    return _ops


def _inputs(seed, B, Q, K, Hq, Hkv, D=128, bs=64, density=0.25):
    from oracle import compact_oracle as co
    g = torch.Generator().manual_seed(seed)
    q = torch.randn((B, Q, Hq, D), generator=g).to(torch.bfloat16)
    k = torch.randn((B, K, Hkv, D), generator=g).to(torch.bfloat16)
    v = torch.randn((B, K, Hkv, D), generator=g).to(torch.bfloat16)
    Qb, Kb = Q // bs, K // bs
    Pb = Kb - Qb
    keep = torch.rand((B, Hq, Kb), generator=g) < density                       # per query head, column mask
    keep |= co.forced_mask(Qb, Kb, Pb, 1, 2).any(dim=0).view(1, 1, Kb)
    return q, k, v, keep, Pb, Kb


@pytest.mark.parametrize("sub", [1, 2])   # query heads per table row: 1 = per query head, 2 = sub-groups of two
def test_rows_per_kv_head_match_oracle(ops, sub):
    from oracle import compact_oracle as co
    B, Q, K, Hq, Hkv, bs = 1, 256, 4096, 8, 2, 64
    G = Hq // Hkv
    q, k, v, keep, Pb, Kb = _inputs(11 + sub, B, Q, K, Hq, Hkv)
    rows = Hq // sub
    # oracle: every table row is a "KV head" of its own that reads a copy of its real KV head
    idx, counts = co.block_union_table(keep, Q, K, bs, sub)                      # union inside the sub-group only
    rep = G // sub
    want = co.compact_attention(q, k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2), idx, counts, bs)
    table = ops.union_table(mask=keep.cuda(), num_kv_heads=rows, kv_blocks=Kb, past_blocks=Pb, block_size=bs)
    assert torch.equal(table.block_idx.cpu(), idx) and torch.equal(table.counts.cpu(), counts)
    kv = ops.KvCacheView.from_seq_first(k.cuda(), v.cuda()).with_head_div(rep)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for use_ws in (True, False):
        out = ops.attn_compact(q.cuda(), kv, K, rows, table.block_idx, table.counts, block_size=bs, status=status,
                               use_workspace=use_ws)
        err = (out.float().cpu() - want).abs()
        assert int(status.item()) == 0
        assert err.max().item() < 2e-2 and err.mean().item() < 2e-3, (sub, use_ws, err.max().item(), err.mean().item())
    # the GQA-union table selects a superset, so per-row tables never read more blocks
    full_idx, full_counts = co.block_union_table(keep, Q, K, bs, G)
    assert int(counts.view(B, Hkv, rep).max(dim=2).values.sub(full_counts.view(B, Hkv)).max()) <= 0


def test_module_routes_per_query_and_subgroup(ops, monkeypatch):
    from oracle import compact_oracle as co
    from compactattention_b200.modules import chunked_prefill_column_dense_attention_from_keep_block as from_keep
    B, Q, K, Hq, Hkv, bs = 1, 128, 2048, 8, 2, 64
    G = Hq // Hkv
    q, k, v, keep, Pb, Kb = _inputs(21, B, Q, K, Hq, Hkv)
    scale = 128 ** -0.5
    # per query head
    out, _ = from_keep(q.cuda(), k.cuda(), v.cuda(), keep.cuda(), None, Q, scale, block_size=bs, num_key_value_groups=G,
                       indexed_impl="fi_zero_copy_per_query")
    idx, counts = co.block_union_table(keep, Q, K, bs, 1)
    want = co.compact_attention(q, k.repeat_interleave(G, dim=2), v.repeat_interleave(G, dim=2), idx, counts, bs)
    assert (out.float().cpu() - want).abs().max().item() < 2e-2
    # sub-groups of two query heads: the caller passes the sub-group masks
    monkeypatch.setenv("SEER_ZC_QUERY_SUBGROUP_SIZE", "2")
    keep_sub = keep.view(B, Hq // 2, 2, Kb).any(dim=2)
    out2, stats = from_keep(q.cuda(), k.cuda(), v.cuda(), None, None, Q, scale, block_size=bs, num_key_value_groups=G,
                            indexed_impl="fi_zero_copy_subgroup", keep_block_kv_preprojected=keep_sub.cuda(),
                            return_stats=True)
    idx2, counts2 = co.block_union_table(keep, Q, K, bs, 2)
    want2 = co.compact_attention(q, k.repeat_interleave(2, dim=2), v.repeat_interleave(2, dim=2), idx2, counts2, bs)
    assert (out2.float().cpu() - want2).abs().max().item() < 2e-2
    assert stats["path"] == "chunked_selected"
    # the reference's argument errors
    with pytest.raises(ValueError, match="requires subgroup keep_block"):
        from_keep(q.cuda(), k.cuda(), v.cuda(), keep.cuda(), None, Q, scale, block_size=bs, num_key_value_groups=G,
                  indexed_impl="fi_zero_copy_subgroup")
    monkeypatch.setenv("SEER_ZC_QUERY_SUBGROUP_SIZE", "3")
    with pytest.raises(ValueError, match="must divide num_key_value_groups"):
        from_keep(q.cuda(), k.cuda(), v.cuda(), None, None, Q, scale, block_size=bs, num_key_value_groups=G,
                  indexed_impl="fi_zero_copy_subgroup", keep_block_kv_preprojected=keep_sub.cuda())


def test_head_div_is_rejected_elsewhere(ops):
    k = torch.zeros((1, 256, 2, 128), dtype=torch.bfloat16, device="cuda")
    kv = ops.KvCacheView.from_seq_first(k, k.clone()).with_head_div(2)
    idx = torch.zeros((2, 2), dtype=torch.int32, device="cuda")
    cnt = torch.zeros((2,), dtype=torch.int32, device="cuda")
    dst = torch.zeros((2 * 128, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="head_div"):
        ops.gather_kv(kv, 2, 1, 64, 256, idx, cnt, dst, dst.clone(), dst_row_stride_tokens=128)
    q = torch.zeros((1, 64, 6, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="head_div"):
        ops.attn_compact(q, ops.KvCacheView.from_seq_first(k, k.clone()).with_head_div(4), 256, 6, None, None)
