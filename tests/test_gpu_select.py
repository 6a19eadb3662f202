"""GPU parity of block selection: CUDA (through the C ABI) vs the CPU oracle and the golden
fixtures.  Everything here is integer/bool work: the bar is bit-exact."""
import math

import numpy as np
import pytest
import torch

from oracle import compact_oracle as co

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from compactattention_b200 import ops as o

    return o


def T(a):
    return torch.from_numpy(np.asarray(a))


def cuda_table(ops, keep_block, Hkv, Kb, Pb, bs, **kw):
    t = ops.union_table(mask=keep_block.cuda(), num_kv_heads=Hkv, kv_blocks=Kb, past_blocks=Pb, block_size=bs,
                        want_keep_kv=True, **kw)
    return t


def test_union_table_golden(ops, golden):
    g = golden("union_table")
    Hq, Qb, Kb, G, bs, Hq7, Qb7, Kb7 = [int(x) for x in g["meta"]]
    # from the 2-D block mask [Hq, Qb, Kb] of the CPU configuration (Q-block union done by the kernel)
    mask = T(g["mask"]).unsqueeze(0)
    t = cuda_table(ops, mask, Hq // G, Kb, Kb - Qb, bs)
    assert torch.equal(t.block_idx.cpu(), T(g["idx"])) and torch.equal(t.counts.cpu(), T(g["counts"]))
    assert torch.equal(t.keep_kv.cpu(), T(g["keep_kv"]))
    assert torch.equal(t.cache_seqlens.cpu(), (T(g["counts"]) + Qb) * bs)
    # from the [B, Hq, Kb] keep_block
    t2 = cuda_table(ops, T(g["keep_block"]), Hq // G, Kb, Kb - Qb, bs)
    assert torch.equal(t2.block_idx.cpu(), T(g["idx"])) and torch.equal(t2.counts.cpu(), T(g["counts"]))
    # from the already-projected KV-level mask (G = 1)
    t3 = cuda_table(ops, T(g["keep_kv"]), Hq // G, Kb, Kb - Qb, bs)
    assert torch.equal(t3.block_idx.cpu(), T(g["idx"])) and torch.equal(t3.counts.cpu(), T(g["counts"]))
    # G = 7, batch 2, an empty and a full row
    t7 = cuda_table(ops, T(g["keep_block_g7"]), Hq7 // 7, Kb7, Kb7 - Qb7, bs)
    assert torch.equal(t7.block_idx.cpu(), T(g["idx_g7"])) and torch.equal(t7.counts.cpu(), T(g["counts_g7"]))
    assert torch.equal(t7.keep_kv.cpu(), T(g["keep_kv_g7"]))


@pytest.mark.parametrize("B,Hq,G,Qb,Kb,density,seed", [
    (1, 32, 4, 4, 128, 0.2, 0),       # the CPU configuration's shape
    (1, 32, 4, 16, 512, 0.05, 1),     # 32K cache, chunk 1024
    (1, 32, 4, 16, 2048, 0.2, 2),     # 128K cache
    (2, 28, 7, 8, 264, 0.3, 3),       # G = 7, ragged word count
    (1, 8, 1, 2, 33, 0.5, 4),         # no grouping, Kb not a multiple of 32
    (1, 16, 4, 16, 4096, 0.1, 5),     # 256K cache
    (3, 4, 2, 1, 1, 1.0, 6),          # first chunk of one block: no past at all
])
def test_union_table_random(ops, B, Hq, G, Qb, Kb, density, seed):
    g = torch.Generator().manual_seed(seed)
    Pb = Kb - Qb
    bs = 64
    mask = torch.rand((B, Hq, Qb, Kb), generator=g) < density
    keep_block = mask.any(dim=2)
    want_kv = co.kv_head_union(keep_block, Qb * bs, Kb * bs, bs, G)
    idx, counts, seqlens, pages = co.block_table_from_kv_keep(want_kv, Qb * bs, Kb * bs, bs, page_size=256)
    t = cuda_table(ops, mask, Hq // G, Kb, Pb, bs, page_size=256)
    assert torch.equal(t.block_idx.cpu(), idx) and torch.equal(t.counts.cpu(), counts)
    assert torch.equal(t.cache_seqlens.cpu(), seqlens) and torch.equal(t.pages_per_row.cpu(), pages)
    assert torch.equal(t.keep_kv.cpu(), want_kv)
    # packed-bit input gives the same table
    bits = ops.select_rows(mask.cuda(), Pb, "mask", valid=torch.ones((B, 1, Qb, Kb), dtype=torch.bool, device="cuda"))
    assert torch.equal(ops.unpack_bits(bits, Kb).cpu(), mask)
    t2 = ops.union_table(bits=bits, num_kv_heads=Hq // G, kv_blocks=Kb, past_blocks=Pb, block_size=bs)
    assert torch.equal(t2.block_idx.cpu(), idx) and torch.equal(t2.counts.cpu(), counts)
    # paged metadata
    offs, table = ops.paged_metadata(t.pages_per_row, max_pages=int(pages.max()))
    want_offs = torch.cat([torch.zeros(1, dtype=torch.int64), pages.reshape(-1).cumsum(0)]).to(torch.int32)
    assert torch.equal(offs.cpu(), want_offs)
    slot = torch.arange(int(pages.max())).view(1, -1)
    want_table = torch.where(slot < pages.reshape(-1, 1), want_offs[:-1].view(-1, 1) + slot, torch.zeros_like(slot)).to(torch.int32)
    assert torch.equal(table.cpu(), want_table)


def test_seer_threshold_rule_golden(ops, golden):
    g = golden("seer_keep")
    B, H, Qb, Kb, bs = [int(x) for x in g["meta"]]
    score, valid = T(g["score"]), T(g["valid"])
    Pb = Kb - Qb
    for dtype in (torch.float32,):
        for ti, thr in enumerate(g["thresholds"]):
            for kr in (0, 2):
                for v in (None, valid.cuda()):
                    bits = ops.select_rows(score.to(dtype).cuda(), Pb, "threshold", threshold=float(thr), valid=v)
                    t = ops.union_table(bits=bits, num_kv_heads=H, kv_blocks=Kb, past_blocks=Pb, keep_recent=kr,
                                        want_keep_kv=True)
                    want = T(g[f"fast_t{ti}_r{kr}"]).clone()
                    want[..., Pb:] = True  # the KV-level projection opens the whole chunk
                    assert torch.equal(t.keep_kv.cpu(), want)


def test_seer_threshold_bf16_scores(ops):
    """Scores arriving in bf16 are compared in fp32 after widening, like the reference's kernels
    (compact_attn/csrc/compactattn/cache_fill_kernel.cu:291-296)."""
    g = torch.Generator().manual_seed(11)
    B, H, Qb, Kb = 1, 8, 4, 100
    Pb = Kb - Qb
    valid = co.block_valid_mask(Qb, Kb, Pb)
    score = torch.softmax((torch.randn((B, H, Qb, Kb), generator=g) * 3).masked_fill(~valid, -1e30), dim=-1).to(torch.bfloat16)
    bits = ops.select_rows(score.cuda(), Pb, "threshold", threshold=5e-4)
    want = co.threshold_rows(score.float(), valid.expand_as(score), 5e-4)
    assert torch.equal(ops.unpack_bits(bits, Kb).cpu(), want)


def test_flashprefill_alpha_rule_golden(ops, golden):
    g = golden("flashprefill")
    B, Q, K, Hq, Hkv, D, bs = [int(x) for x in g["meta"]]
    G = Hq // Hkv
    Qb, Kb = Q // bs, K // bs
    norm = T(g["score_norm"]).cuda()  # [B, Qb, Kb, Hq]
    for tag in ("a", "b", "c"):
        sink, window, alpha, last_n, budget = g[f"params_{tag}"]
        tail = min(max(int(last_n), 0), Qb - 1) if Qb > 1 else 0
        bits = ops.select_rows(norm.permute(0, 3, 1, 2), Kb - Qb, "alpha_rowmax", alpha=float(alpha), sink=int(sink),
                               local=int(window), min_budget=int(budget), rows_voting=max(Qb - tail, 1))
        t = ops.union_table(bits=bits, num_kv_heads=Hkv, kv_blocks=Kb, past_blocks=Kb - Qb, block_size=bs, want_keep_kv=True)
        assert torch.equal(t.keep_kv.cpu(), T(g[f"keep_kv_{tag}"])), tag
        keep_row, _, _ = co.flashprefill_keep_rowwise(T(g["score_norm"]), Q, K, bs, G, int(sink), int(window),
                                                      float(alpha), int(last_n), int(budget))
        got = ops.unpack_bits(bits, Kb).cpu()[:, :, : keep_row.shape[2]]
        assert torch.equal(got, keep_row), tag


@pytest.mark.parametrize("Kb,Qb,H,num,den,seed", [(128, 4, 8, 1, 5, 0), (2048, 16, 4, 1, 10, 1), (2048, 16, 4, 3, 10, 2),
                                                  (4096, 16, 2, 1, 5, 3), (37, 3, 5, 1, 2, 4)])
def test_topk_rule(ops, Kb, Qb, H, num, den, seed):
    g = torch.Generator().manual_seed(seed)
    Pb = Kb - Qb
    score = torch.randn((1, H, Qb, Kb), generator=g)
    # plant ties, including across the selection boundary
    score[..., ::7] = score[..., :1]
    score = score.to(torch.bfloat16).float()  # many equal values
    valid = co.block_valid_mask(Qb, Kb, Pb).view(1, 1, Qb, Kb).expand_as(score)
    n_valid = Pb + torch.arange(Qb) + 1
    k = torch.clamp((num * n_valid + den // 2) // den, min=1)
    k = torch.minimum(k, n_valid)
    want = co.topk_rows(score, valid, k) | (co.forced_mask(Qb, Kb, Pb, 1, 2) & valid)
    bits = ops.select_rows(score.cuda(), Pb, "topk", topk_ratio=(num, den), sink=1, local=2)
    got = ops.unpack_bits(bits, Kb).cpu()
    assert torch.equal(got, want)
    assert torch.equal(got.sum(-1).min() >= k.min(), torch.tensor(True))
    # absolute k
    bits = ops.select_rows(score.cuda(), Pb, "topk", topk_k=5)
    want5 = co.topk_rows(score, valid, torch.minimum(torch.full((Qb,), 5), n_valid))
    assert torch.equal(ops.unpack_bits(bits, Kb).cpu(), want5)


@pytest.mark.parametrize("Kb,Qb,H,tau,seed", [(512, 16, 8, 0.9, 0), (128, 4, 4, 0.5, 1), (100, 3, 2, 0.99, 2), (2048, 16, 2, 0.9, 3)])
def test_cummass_rule(ops, Kb, Qb, H, tau, seed):
    """Cumulative-mass rule on logits: masked softmax (fp32) then the shortest descending prefix with
    mass >= tau.  The probabilities the kernel used are read back and fed to the oracle's rule, so the
    mask comparison is exact; the probabilities themselves are checked to 1e-5 relative."""
    g = torch.Generator().manual_seed(seed)
    Pb = Kb - Qb
    logits = torch.randn((1, H, Qb, Kb), generator=g) * 4
    valid = co.block_valid_mask(Qb, Kb, Pb).view(1, 1, Qb, Kb).expand_as(logits)
    prob = torch.empty((1, H, Qb, Kb), dtype=torch.float32, device="cuda")
    bits = ops.select_rows(logits.cuda(), Pb, "cummass", softmax=True, threshold=tau, sink=1, local=2, prob_out=prob)
    want_prob = co.masked_softmax_rows(logits, valid)
    assert torch.allclose(prob.cpu(), want_prob, rtol=1e-5, atol=1e-9)
    want = co.cummass_rows(prob.cpu(), valid, tau) | (co.forced_mask(Qb, Kb, Pb, 1, 2) & valid)
    assert torch.equal(ops.unpack_bits(bits, Kb).cpu(), want)


def test_capacity_and_contract_errors(ops):
    mask = torch.ones((1, 4, 1, 16), dtype=torch.bool, device="cuda")
    small = ops.BlockTable(torch.empty((1, 1, 4), dtype=torch.int32, device="cuda"),
                           torch.empty((1, 1), dtype=torch.int32, device="cuda"),
                           torch.empty((1, 1), dtype=torch.int32, device="cuda"),
                           torch.empty((1, 1), dtype=torch.int32, device="cuda"))
    with pytest.raises(RuntimeError, match="capacity"):
        ops.union_table(mask=mask, num_kv_heads=1, kv_blocks=16, past_blocks=12, out=small)
    with pytest.raises(ValueError):
        ops.union_table(mask=mask, num_kv_heads=3, kv_blocks=16, past_blocks=12)


@pytest.mark.parametrize("rule,kw", [
    ("topk", dict(topk_ratio=(1, 5), sink=1, local=2)),
    ("threshold", dict(softmax=True, threshold=2e-3, keep_recent=2)),
    ("alpha_rowmax", dict(alpha=0.3, sink=2, local=4, rows_voting=3)),
    ("cummass", dict(softmax=True, threshold=0.8, sink=1, local=1)),
])
@pytest.mark.parametrize("B,Hkv,G,Qb,Kb", [(1, 8, 4, 16, 2048), (2, 2, 7, 4, 130), (1, 1, 1, 1, 33)])
def test_fused_select_union_table_equals_the_two_launches(ops, rule, kw, B, Hkv, G, Qb, Kb):
    """One launch (row rule + ticketed Block-Union + table) against select_rows followed by union_table:
    bits, table, counts, seqlens and pages bit for bit, on three calls in a row with different scores (the
    kernel must leave its scratch clean), with and without the per-row bits output."""
    Pb = Kb - Qb
    H = Hkv * G
    kw = dict(kw)
    keep_recent = kw.pop("keep_recent", 0)
    if "rows_voting" in kw:
        kw["rows_voting"] = min(kw["rows_voting"], Qb)
    g = torch.Generator().manual_seed(Kb * 7 + Qb)
    for call in range(3):
        score = (torch.randn((B, H, Qb, Kb), generator=g) * 2).cuda()
        bits = ops.select_rows(score, Pb, rule, **kw)
        want = ops.union_table(bits=bits, num_kv_heads=Hkv, kv_blocks=Kb, past_blocks=Pb, block_size=64, keep_recent=keep_recent)
        got_bits = torch.full_like(bits, -1) if call != 1 else None
        got = ops.select_union_table(score, Pb, rule, num_kv_heads=Hkv, block_size=64, keep_recent=keep_recent, bits=got_bits, **kw)
        for name in ("block_idx", "counts", "cache_seqlens", "pages_per_row"):
            assert torch.equal(getattr(got, name), getattr(want, name)), (name, call)
        if got_bits is not None:
            assert torch.equal(got_bits, bits)
    # and against the oracle's union of the rows the kernel selected
    keep_rows = ops.unpack_bits(bits, Kb).cpu()
    keep_block = keep_rows.any(dim=2)
    if keep_recent:
        keep_block[..., Kb - keep_recent:] = True
    idx, counts = co.block_union_table(keep_block, Qb * 64, Kb * 64, 64, G)
    assert torch.equal(got.block_idx.cpu(), idx) and torch.equal(got.counts.cpu(), counts)
    scratch = ops.union_scratch(torch.device("cuda", torch.cuda.current_device()), B, H, Hkv, Qb, Kb)
    assert int(scratch[: B * Hkv].abs().sum().item()) == 0  # the tickets are left clean


def test_fused_select_union_contract_errors(ops):
    score = torch.randn((1, 8, 4, 64), device="cuda")
    with pytest.raises(ValueError, match="multiple"):
        ops.select_union_table(score, 60, "topk", num_kv_heads=3, topk_k=4)
    with pytest.raises(ValueError, match="Kb - past_blocks"):
        ops.select_union_table(score, 50, "topk", num_kv_heads=2, topk_k=4)
    small = torch.zeros(4, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="scratch holds"):
        ops.select_union_table(score, 60, "topk", num_kv_heads=2, topk_k=4, scratch=small)


@pytest.mark.parametrize("rule,kw", [
    ("topk", dict(topk_ratio=(1, 5), sink=1, local=2)),
    ("threshold", dict(softmax=True, threshold=2e-3, keep_recent=2)),
    ("alpha_rowmax", dict(alpha=0.3, sink=2, local=4, rows_voting=3, min_budget=3)),
    ("cummass", dict(softmax=True, threshold=0.8, sink=1, local=1)),
])
@pytest.mark.parametrize("B,Hkv,G,Qb,Kb,C,kdt", [
    (1, 8, 4, 16, 2048, 128, torch.bfloat16),   # the headline shape: tensor-core scores, 128 columns
    (2, 2, 2, 3, 37, 128, torch.float16),       # two heads per KV head, ragged word and column counts
    (1, 3, 1, 1, 5, 128, torch.bfloat16),       # one head per KV head, a single Q-block
    (1, 1, 4, 16, 600, 128, torch.bfloat16),    # a tensor-parallel rank with one KV head
    (1, 2, 8, 2, 70, 128, torch.bfloat16),      # eight heads per KV head
    (1, 1, 4, 40, 300, 128, torch.bfloat16),    # 160 query rows per cache head: beyond the tensor-core form
    (1, 2, 4, 2, 70, 64, torch.float32),        # 64 channels, fp32 cache: the CUDA-core score kernels
])
def test_gate_score_select_equals_scores_then_selection(ops, rule, kw, B, Hkv, G, Qb, Kb, C, kdt):
    """Gate logits + row rule + Block-Union + table behind one host call against ca_gate_scores followed by
    ca_select_union_table: the logits and every table output bit for bit, on three calls in a row (scratch left
    clean); two launches whatever the shape."""
    Pb, Hq = Kb - Qb, Hkv * G
    kw = dict(kw)
    keep_recent = kw.pop("keep_recent", 0)
    if "rows_voting" in kw:
        kw["rows_voting"] = min(kw["rows_voting"], Qb)
    g = torch.Generator().manual_seed(Kb * 11 + Qb + G)
    import compactattention_b200._lib as L
    for call in range(3):
        qb = torch.randn((B, Qb, Hq, C), generator=g).cuda()
        kb = torch.randn((B, Kb, Hkv, C), generator=g).to(kdt).cuda()
        logits = ops.gate_scores(qb, kb, Pb)
        want = ops.select_union_table(logits, Pb, rule, num_kv_heads=Hkv, block_size=64, keep_recent=keep_recent, **kw)
        write = call != 1
        got_scores = torch.full_like(logits, 7.0)
        n0 = L.launch_count()
        got = ops.gate_score_select(qb, kb, Pb, rule, num_kv_heads=Hkv, scores=got_scores, write_scores=write, block_size=64,
                                    keep_recent=keep_recent, **kw)
        launches = L.launch_count() - n0
        assert launches == 2
        for name in ("block_idx", "counts", "cache_seqlens", "pages_per_row"):
            assert torch.equal(getattr(got, name), getattr(want, name)), (name, call)
        assert torch.equal(got_scores, logits), call
    scratch = ops.union_scratch(torch.device("cuda", torch.cuda.current_device()), B, Hq, Hkv, Qb, Kb)
    assert int(scratch[: B * Hkv].abs().sum().item()) == 0
