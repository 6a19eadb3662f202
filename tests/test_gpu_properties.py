"""Size-independent properties at the benchmark configurations' full sizes (32K paged cache, 128K
context), where the CPU oracle would take too long: page-permutation invariance, full selection =
dense, linearity in V, gather followed by dense attention = indexed attention, and structural
properties of the selection rules and the block table."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from compactattention_b200 import ops as o

    return o


def rand_table(Hkv, Pb, density, g):
    n = int(round(Pb * density))
    idx = torch.full((Hkv, Pb), -1, dtype=torch.int32, device="cuda")
    counts = torch.empty((Hkv,), dtype=torch.int32, device="cuda")
    for r in range(Hkv):
        c = max(0, min(Pb, n + int(torch.randint(-n // 4 - 1, n // 4 + 2, (1,), generator=g))))
        idx[r, :c] = torch.randperm(Pb, generator=g)[:c].sort().values.int().cuda()
        counts[r] = c
    return idx, counts


def test_config2_paged_permutation_full_dense_linearity(ops):
    """32K-token paged cache with randomly permuted 64-token pages, chunk 1024, 32/8 heads."""
    g = torch.Generator().manual_seed(1234 + 2)
    Q, K, Hq, Hkv, D, bs = 1024, 32768, 32, 8, 128, 64
    Pb = (K - Q) // bs
    q = torch.randn((1, Q, Hq, D), generator=g).to(torch.bfloat16).cuda()
    k = torch.randn((1, K, Hkv, D), generator=g).to(torch.bfloat16).cuda()
    v = torch.randn((1, K, Hkv, D), generator=g).to(torch.bfloat16).cuda()
    perm = torch.randperm(K // 64, generator=g).cuda()
    kp, vp = torch.empty((K // 64, 64, Hkv, D), dtype=torch.bfloat16, device="cuda"), torch.empty((K // 64, 64, Hkv, D), dtype=torch.bfloat16, device="cuda")
    kp[perm], vp[perm] = k.view(K // 64, 64, Hkv, D), v.view(K // 64, 64, Hkv, D)
    paged = ops.KvCacheView.from_paged(kp, vp, perm.int().view(1, -1).contiguous())
    flat = ops.KvCacheView.from_seq_first(k, v)
    idx, counts = rand_table(Hkv, Pb, 0.2, g)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    a = ops.attn_compact(q, flat, K, Hkv, idx, counts, status=status)
    b = ops.attn_compact(q, paged, K, Hkv, idx, counts, status=status)
    assert int(status.item()) == 0 and torch.equal(a, b)  # a page table only relabels pages
    # heads-first source view
    c = ops.attn_compact(q, ops.KvCacheView.from_heads_first(k.transpose(1, 2).contiguous(), v.transpose(1, 2).contiguous()),
                         K, Hkv, idx, counts)
    assert torch.equal(a, c)
    # every block selected = dense
    full_idx = torch.arange(Pb, dtype=torch.int32, device="cuda").repeat(Hkv, 1).contiguous()
    full_cnt = torch.full((Hkv,), Pb, dtype=torch.int32, device="cuda")
    assert torch.equal(ops.attn_compact(q, paged, K, Hkv, full_idx, full_cnt), ops.attn_compact(q, paged, K, Hkv, None, None))
    # linear in V (a power-of-two scale is exact in bf16)
    flat2 = ops.KvCacheView.from_seq_first(k, (v.float() * 2).to(torch.bfloat16))
    assert torch.equal(ops.attn_compact(q, flat2, K, Hkv, idx, counts).float(), a.float() * 2)
    # with and without cutting work units across SMs: same math, different summation order
    d = ops.attn_compact(q, flat, K, Hkv, idx, counts, use_workspace=False)
    assert (a.float() - d.float()).abs().max().item() < 2e-2


@pytest.mark.parametrize("K,density", [(131072, 0.2), (32768, 0.5)])
def test_gather_then_dense_equals_indexed_attention(ops, K, density):
    """Config 3 size: copying the selected blocks into a compact cache and running the dense kernel on
    each row's compact sequence gives bit-identical output to reading the blocks in place, when both
    runs walk their KV in one piece per work unit (cutting units across SMs changes the fp32
    summation order, so the default launches are compared within one bf16 step)."""
    g = torch.Generator().manual_seed(1234 + 3)
    Q, Hq, Hkv, D, bs = 1024, 32, 8, 128, 64
    G = Hq // Hkv
    Pb = (K - Q) // bs
    q = torch.randn((1, Q, Hq, D), generator=g).to(torch.bfloat16).cuda()
    k = torch.randn((1, K, Hkv, D), generator=g).to(torch.bfloat16).cuda()
    v = torch.randn((1, K, Hkv, D), generator=g).to(torch.bfloat16).cuda()
    kv = ops.KvCacheView.from_seq_first(k, v)
    idx, counts = rand_table(Hkv, Pb, density, g)
    indexed = ops.attn_compact(q, kv, K, Hkv, idx, counts, use_workspace=False)
    indexed_cut = ops.attn_compact(q, kv, K, Hkv, idx, counts)
    assert (indexed.float() - indexed_cut.float()).abs().max().item() < 2e-3
    cap = (Pb + Q // bs) * bs
    kd = torch.zeros((Hkv * cap, D), dtype=torch.bfloat16, device="cuda")
    vd = torch.zeros_like(kd)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.gather_kv(kv, Hkv, 1, Q, K, idx, counts, kd, vd, block_size=bs, dst_row_stride_tokens=cap, status=status)
    assert int(status.item()) == 0
    cnt = counts.cpu().tolist()
    for r in range(Hkv):
        L = (cnt[r] + Q // bs) * bs
        kr = kd[r * cap: r * cap + L].view(1, L, 1, D)
        vr = vd[r * cap: r * cap + L].view(1, L, 1, D)
        # byte-exact gather: first and last selected block, and the chunk
        first = int(idx[r, 0]) if cnt[r] else None
        if first is not None:
            assert torch.equal(kr[0, :bs, 0], k[0, first * bs:(first + 1) * bs, r])
        assert torch.equal(vr[0, L - Q:, 0], v[0, K - Q:, r])
        qr = q[:, :, r * G:(r + 1) * G].contiguous()
        dense = ops.attn_compact(qr, ops.KvCacheView.from_seq_first(kr, vr), L, 1, None, None, use_workspace=False)
        assert torch.equal(dense, indexed[:, :, r * G:(r + 1) * G])
        dense_cut = ops.attn_compact(qr, ops.KvCacheView.from_seq_first(kr, vr), L, 1, None, None)
        assert (dense_cut.float() - dense.float()).abs().max().item() < 2e-3


def test_selection_rule_properties_full_size(ops):
    g = torch.Generator().manual_seed(7)
    H, Qb, Kb = 32, 16, 2048
    Pb = Kb - Qb
    score = torch.randn((1, H, Qb, Kb), generator=g).cuda()
    n_valid = (Pb + torch.arange(Qb) + 1).cuda()
    # top-k: every row keeps exactly k blocks, all causally valid
    bits = ops.select_rows(score, Pb, "topk", topk_ratio=(1, 5))
    keep = ops.unpack_bits(bits, Kb)
    k = torch.clamp((n_valid + 2) // 5, min=1)
    assert torch.equal(keep.sum(-1), k.view(1, 1, Qb).expand(1, H, Qb))
    cols = torch.arange(Kb, device="cuda")
    assert not (keep & (cols.view(1, 1, 1, Kb) > (Pb + torch.arange(Qb, device="cuda")).view(1, 1, Qb, 1))).any()
    # every kept score >= every dropped valid score of its row
    valid = cols.view(1, 1, 1, Kb) <= (Pb + torch.arange(Qb, device="cuda")).view(1, 1, Qb, 1)
    kept_min = torch.where(keep, score, torch.full_like(score, float("inf"))).amin(-1)
    drop_max = torch.where(valid & ~keep, score, torch.full_like(score, float("-inf"))).amax(-1)
    assert (kept_min >= drop_max).all()
    # threshold: monotone in the threshold
    prob = torch.softmax(score.masked_fill(~valid, float("-inf")), -1)
    lo = ops.unpack_bits(ops.select_rows(prob, Pb, "threshold", threshold=2e-4), Kb)
    hi = ops.unpack_bits(ops.select_rows(prob, Pb, "threshold", threshold=1e-3), Kb)
    assert (hi & ~lo).sum() == 0 and hi.sum() < lo.sum()
    # cumulative mass: kept mass reaches tau, and without its smallest kept entry it does not
    cm = ops.unpack_bits(ops.select_rows(score * 3, Pb, "cummass", softmax=True, threshold=0.9), Kb)
    p3 = torch.softmax((score * 3).masked_fill(~valid, float("-inf")), -1)
    mass = (p3 * cm).sum(-1)
    smallest = torch.where(cm, p3, torch.full_like(p3, float("inf"))).amin(-1)
    assert (mass >= 0.9 - 1e-5).all() and ((mass - smallest) < 0.9 + 1e-5).all()
    # union + table: ascending ids, -1 padding, counts = popcount of the union, idempotent re-projection
    t = ops.union_table(bits=bits, num_kv_heads=8, kv_blocks=Kb, past_blocks=Pb, want_keep_kv=True)
    union = keep.view(1, 8, 4, Qb, Kb).any(3).any(2)
    assert torch.equal(t.counts.view(-1), union[..., :Pb].sum(-1).int().view(-1))
    for r in range(8):
        c = int(t.counts.view(-1)[r])
        row = t.block_idx.view(8, -1)[r]
        assert (row[:c][1:] > row[:c][:-1]).all() and (row[c:] == -1).all()
        assert torch.equal(row[:c].long(), torch.nonzero(union[0, r, :Pb]).flatten())
    t2 = ops.union_table(mask=t.keep_kv, num_kv_heads=8, kv_blocks=Kb, past_blocks=Pb)
    assert torch.equal(t2.block_idx, t.block_idx) and torch.equal(t2.counts, t.counts)


def test_edge_shapes(ops):
    """Smallest shapes, empty selections, batches with unequal counts, chunk shorter than a tile pair."""
    g = torch.Generator().manual_seed(11)
    from oracle import compact_oracle as co
    for (B, Q, K, Hq, Hkv) in [(1, 64, 64, 1, 1), (3, 64, 256, 2, 2), (2, 192, 1216, 8, 1), (1, 64, 4160, 4, 4)]:
        q = torch.randn((B, Q, Hq, 128), generator=g).to(torch.bfloat16)
        k = torch.randn((B, K, Hkv, 128), generator=g).to(torch.bfloat16)
        v = torch.randn((B, K, Hkv, 128), generator=g).to(torch.bfloat16)
        Pb = (K - Q) // 64
        keep = torch.rand((B, Hkv, max(Pb, 1)), generator=g) < 0.4
        if Pb:
            keep[0, 0] = False  # a row with nothing selected
        else:
            keep[:] = False
        idx, counts, _, _ = co.block_table_from_kv_keep(torch.cat([keep[..., :Pb], torch.ones((B, Hkv, Q // 64), dtype=torch.bool)], -1), Q, K, 64)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = ops.attn_compact(q.cuda(), ops.KvCacheView.from_seq_first(k.cuda(), v.cuda()), K, Hkv, idx.cuda(), counts.cuda(), status=status)
        want = co.compact_attention(q, k, v, idx, counts, 64)
        err = (out.float().cpu() - want).abs()
        assert int(status.item()) == 0 and err.max().item() < 2e-2 and err.mean().item() < 2e-3, (B, Q, K, Hq, Hkv)


def test_programmatic_launch_does_not_change_results(ops):
    """The same selection + attention chain with dependent launches and with plain launches: every
    kernel waits for its predecessor before touching global memory, so outputs are bit-identical."""
    from compactattention_b200 import _lib
    g = torch.Generator().manual_seed(99)
    Q, K, Hq, Hkv, D, bs = 512, 16384, 16, 4, 128, 64
    Pb, Kb = (K - Q) // bs, K // bs
    q = torch.randn((1, Q, Hq, D), generator=g).to(torch.bfloat16).cuda()
    k = torch.randn((1, K, Hkv, D), generator=g).to(torch.bfloat16).cuda()
    v = torch.randn((1, K, Hkv, D), generator=g).to(torch.bfloat16).cuda()
    score = torch.randn((1, Hq, Q // bs, Kb), generator=g).cuda()
    kv = ops.KvCacheView.from_seq_first(k, v)
    results = []
    try:
        for on in (True, False):
            _lib.set_programmatic_launch(on)
            for _ in range(3):   # back-to-back chains, so launches do overlap when allowed
                bits = ops.select_rows(score, Pb, "topk", topk_ratio=(1, 5), sink=1, local=2)
                table = ops.union_table(bits=bits, num_kv_heads=Hkv, kv_blocks=Kb, past_blocks=Pb, block_size=bs)
                out = ops.attn_compact(q, kv, K, Hkv, table.block_idx, table.counts, use_workspace=False)
            torch.cuda.synchronize()
            results.append((bits.clone(), table.block_idx.clone(), table.counts.clone(), out.clone()))
    finally:
        _lib.set_programmatic_launch(False)
    for a, b in zip(*results):
        assert torch.equal(a, b)


def test_step_replays_from_a_cuda_graph(ops):
    """Selection + table + attention captured once and replayed: same bits, table and output as the
    eager launches, also after the inputs changed in place."""
    from compactattention_b200.chunk_driver import capture_step
    g = torch.Generator().manual_seed(5)
    Q, K, Hq, Hkv, D, bs = 256, 8192, 8, 2, 128, 64
    Pb, Kb = (K - Q) // bs, K // bs
    q = torch.randn((1, Q, Hq, D), generator=g).to(torch.bfloat16).cuda()
    k = torch.randn((1, K, Hkv, D), generator=g).to(torch.bfloat16).cuda()
    v = torch.randn((1, K, Hkv, D), generator=g).to(torch.bfloat16).cuda()
    score = torch.randn((1, Hq, Q // bs, Kb), generator=g).cuda()
    kv = ops.KvCacheView.from_seq_first(k, v)
    bits = ops.select_rows(score, Pb, "topk", topk_ratio=(1, 5), sink=1, local=2)
    table = ops.union_table(bits=bits, num_kv_heads=Hkv, kv_blocks=Kb, past_blocks=Pb, block_size=bs)
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def step():
        ops.select_rows(score, Pb, "topk", topk_ratio=(1, 5), sink=1, local=2, bits=bits)
        ops.union_table(bits=bits, num_kv_heads=Hkv, kv_blocks=Kb, past_blocks=Pb, block_size=bs, out=table)
        ops.attn_compact(q, kv, K, Hkv, table.block_idx, table.counts, out=out, status=status)

    graph = capture_step(step)
    for trial in range(2):
        step()
        torch.cuda.synchronize()
        want = (bits.clone(), table.block_idx.clone(), table.counts.clone(), out.clone())
        bits.zero_(), table.block_idx.zero_(), table.counts.zero_(), out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for a, b in zip(want, (bits, table.block_idx, table.counts, out)):
            assert torch.equal(a, b)
        score.copy_(torch.randn(score.shape, generator=g))   # new scores, same buffers: the graph follows
        q.copy_(torch.randn(q.shape, generator=g).to(torch.bfloat16))


def test_a_bounded_wait_runs_out_and_the_context_stays_usable(ops):
    """The wait routine behind every mbarrier wait of the tcgen05 / TMA kernels, on a barrier nothing arrives on:
    it must give up after the limit (not before, not much later), report CA_STATUS_TIMEOUT, and leave the
    context able to run the attention kernel afterwards."""
    from compactattention_b200 import _lib
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    limit_ns = 3_000_000   # 3 ms
    rc = _lib.load().ca_selftest_bounded_wait(limit_ns, status.data_ptr(), waited.data_ptr(), ops._stream())
    assert rc == 0, _lib.load().ca_last_error()
    torch.cuda.synchronize()
    assert int(status.item()) & _lib.CA_STATUS_TIMEOUT
    assert limit_ns <= int(waited.item()) < 20 * limit_ns
    assert _lib.load().ca_selftest_bounded_wait(0, status.data_ptr(), None, ops._stream()) == -1   # limits are bounded themselves
    # the context is intact: a small attention call still runs and reports no timeout
    q = torch.randn((1, 128, 4, 128), device="cuda").to(torch.bfloat16)
    k = torch.randn((1, 256, 2, 128), device="cuda").to(torch.bfloat16)
    st2 = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.attn_compact(q, ops.KvCacheView.from_seq_first(k, k.clone()), 256, 2, None, None, status=st2)
    torch.cuda.synchronize()
    assert int(st2.item()) == 0 and torch.isfinite(out.float()).all()
