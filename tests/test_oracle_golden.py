"""The CPU oracle against the fixtures produced by the reference project's own functions
(tests/golden/make_golden.py).  Integer/bool results must be identical; floating-point results
within 1e-5 (both sides are fp32 on the CPU)."""
import math

import numpy as np
import torch

from oracle import compact_oracle as co


def T(a):
    return torch.from_numpy(np.asarray(a))


def test_union_and_block_table(golden):
    g = golden("union_table")
    Hq, Qb, Kb, G, bs, Hq7, Qb7, Kb7 = [int(x) for x in g["meta"]]
    keep_block = T(g["mask"]).any(dim=1).unsqueeze(0)
    assert torch.equal(keep_block, T(g["keep_block"]))
    keep_kv = co.kv_head_union(keep_block, Qb * bs, Kb * bs, bs, G)
    assert torch.equal(keep_kv, T(g["keep_kv"]))
    idx, counts = co.block_union_table(keep_block, Qb * bs, Kb * bs, bs, G)
    assert torch.equal(idx, T(g["idx"])) and idx.dtype == torch.int32
    assert torch.equal(counts, T(g["counts"]))
    # G = 7, batch 2, with an empty and a full row
    kb7 = T(g["keep_block_g7"])
    assert torch.equal(co.kv_head_union(kb7, Qb7 * bs, Kb7 * bs, bs, 7), T(g["keep_kv_g7"]))
    idx7, counts7 = co.block_union_table(kb7, Qb7 * bs, Kb7 * bs, bs, 7)
    assert torch.equal(idx7, T(g["idx_g7"])) and torch.equal(counts7, T(g["counts_g7"]))
    assert int(counts7.min()) == 0 and int(counts7.max()) == Kb7 - Qb7
    # CSR metadata
    pages, indptr, indices = co.flashinfer_index_metadata(keep_kv)
    assert torch.equal(pages, T(g["fi_pages"])) and torch.equal(indptr, T(g["fi_indptr"]))
    assert torch.equal(indices, T(g["fi_indices"]))


def test_seer_keep_rules(golden):
    g = golden("seer_keep")
    B, H, Qb, Kb, bs = [int(x) for x in g["meta"]]
    score, valid = T(g["score"]), T(g["valid"])
    for ti, thr in enumerate(g["thresholds"]):
        for kr in (0, 2):
            generic = co.seer_keep_block(score, valid, float(thr), kr)
            fast = co.seer_keep_block_fast(score, float(thr), kr, Qb * bs, Kb * bs, bs)
            assert torch.equal(generic, T(g[f"generic_t{ti}_r{kr}"]))
            assert torch.equal(fast, T(g[f"fast_t{ti}_r{kr}"]))
            # the row formulation used by the CUDA kernels: OR over rows of (score > thr)
            rows = co.threshold_rows(score, valid.expand_as(score), float(thr)).any(dim=2)
            if kr > 0:
                rows[..., Kb - kr:] = True
            assert torch.equal(rows, fast)


def test_attn_gate(golden):
    g = golden("attn_gate")
    B, Q, K, Hq, Hkv, D, bs = [int(x) for x in g["meta"]]
    q, k = T(g["q"]).float(), T(g["k"]).float()
    cos, sin, mask = T(g["cos"]), T(g["sin"]), T(g["mask"])
    Qb, Kb = Q // bs, K // bs
    for name, qk, kk in (("Qavg_Kmaxminavg", ("avg",), ("max", "min", "avg")), ("Qavg_Kavg", ("avg",), ("avg",))):
        qb = co.pool_blocks(q, bs, qk)
        if f"{name}_wq" in g.files:
            qb = co.multi_head_linear(qb, T(g[f"{name}_wq"]).float())
        kb = co.multi_head_linear(co.pool_blocks(k, bs, kk), T(g[f"{name}_wk"]).float())
        assert torch.allclose(qb, T(g[f"{name}_qb"]), atol=1e-5, rtol=1e-5)
        assert torch.allclose(kb, T(g[f"{name}_kb"]), atol=1e-5, rtol=1e-5)
        qb_r = co.apply_block_rope(qb, cos[:, Kb - Qb:], sin[:, Kb - Qb:])
        kb_r = co.apply_block_rope(kb, cos, sin)
        assert torch.allclose(qb_r, T(g[f"{name}_qb_rope"]), atol=1e-5, rtol=1e-5)
        assert torch.allclose(kb_r, T(g[f"{name}_kb_rope"]), atol=1e-5, rtol=1e-5)
        soft = co.gate_score(qb_r, kb_r, mask, use_softmax=True)
        raw = co.gate_score(qb_r, kb_r, mask, use_softmax=False)
        assert torch.allclose(soft, T(g[f"{name}_score_softmax"]), atol=1e-6, rtol=1e-5)
        assert torch.allclose(raw, T(g[f"{name}_score_raw"]), atol=1e-5, rtol=1e-5)


def test_flashprefill_scores_and_rules(golden):
    g = golden("flashprefill")
    B, Q, K, Hq, Hkv, D, bs = [int(x) for x in g["meta"]]
    q, k = T(g["q"]).float(), T(g["k"]).float()
    mean_k = co.mean_pool_blocks(k, bs)
    assert torch.allclose(mean_k, T(g["mean_k"]), atol=1e-6, rtol=1e-6)
    assert torch.allclose(co.mean_pool_blocks(k[:, :674], bs), T(g["mean_k_ragged"]), atol=1e-6, rtol=1e-6)
    score, mx = co.flashprefill_block_score_raw(q, mean_k, K, bs)
    ref_mx, ref_sc = T(g["max_raw"]), T(g["score_raw"])
    fin = torch.isfinite(ref_mx)
    assert torch.equal(torch.isfinite(mx), fin)
    assert torch.allclose(mx[fin], ref_mx[fin], atol=1e-5, rtol=1e-5)
    assert torch.allclose(score[fin], ref_sc[fin], atol=1e-5, rtol=1e-5)
    norm = co.flashprefill_normalize_scores(score, mx)
    ref_norm = T(g["score_norm"])
    assert torch.allclose(norm, ref_norm, atol=1e-7, rtol=1e-4)
    G = Hq // Hkv
    for tag in ("a", "b", "c"):
        sink, window, alpha, last_n, budget = g[f"params_{tag}"]
        keep_row, keep_q, keep_kv = co.flashprefill_keep_rowwise(
            ref_norm, Q, K, bs, G, int(sink), int(window), float(alpha), int(last_n), int(budget))
        assert torch.equal(keep_q, T(g[f"keep_q_{tag}"]))
        assert torch.equal(keep_kv, T(g[f"keep_kv_{tag}"]))
        if int(budget) == 0:
            assert torch.equal(keep_kv, T(g[f"keep_kv_fused_{tag}"]))


def test_topk_rows(golden):
    g = golden("topk")
    x = T(g["x"])
    n = x.shape[-1]
    for ti, nz in enumerate(g["nz"]):
        k = max(1, int((1 - math.sqrt(1 - float(nz))) * n))
        valid = torch.ones_like(x, dtype=torch.bool)
        mask = co.topk_rows(x, valid, torch.full((n,), k)).tril()
        assert torch.equal(mask, T(g[f"mask_{ti}"]))
    # ties go to the lower index
    tied = torch.tensor([[[[1.0, 3.0, 3.0, 3.0, 0.5]]]])
    keep = co.topk_rows(tied, torch.ones_like(tied, dtype=torch.bool), torch.tensor([2]))
    assert keep.flatten().tolist() == [False, True, True, False, False]


def test_block_causal_mask(golden):
    g = golden("block_mask")
    for ci, (Q, K, bs) in enumerate(g["cases"]):
        assert torch.equal(co.gate_block_causal_mask(int(Q), int(K), int(bs)), T(g[f"mask_{ci}"]))


def test_gather_and_attention(golden):
    g = golden("gather_attention")
    B, Q, K, Hq, Hkv, D, bs = [int(x) for x in g["meta"]]
    q, k, v = T(g["q"]).float(), T(g["k"]).float(), T(g["v"]).float()
    G = Hq // Hkv
    keep_block = T(g["keep_block"])
    keep_kv = co.kv_head_union(keep_block, Q, K, bs, G)
    assert torch.equal(keep_kv, T(g["keep_kv"]))
    idx, counts = co.block_union_table(keep_block, Q, K, bs, G)
    assert torch.equal(idx, T(g["idx"])) and torch.equal(counts, T(g["counts"]))
    kc, vc, table, seqlens = co.gather_compact_kv(k, v, idx, counts, Q, bs, page_size=256)
    assert torch.equal(table, T(g["block_table"])) and torch.equal(seqlens, T(g["sel_lens"]))
    assert torch.equal(kc, T(g["k_cache"]).float()) and torch.equal(vc, T(g["v_cache"]).float())
    out = co.compact_attention(q, k, v, idx, counts, bs)
    assert torch.allclose(out, T(g["out_compact"]), atol=2e-6, rtol=1e-5)
    dense = co.compact_attention(q, k, v, None, None, bs)
    assert torch.allclose(dense, T(g["out_dense"]), atol=2e-6, rtol=1e-5)
    assert torch.allclose(co.dense_causal_attention(q, k, v), T(g["out_dense"]), atol=2e-6, rtol=1e-5)


def test_cummass_rule_definition():
    p = torch.tensor([[[[0.05, 0.4, 0.1, 0.4, 0.05]]]])
    valid = torch.ones_like(p, dtype=torch.bool)
    # 0.4 (idx1) + 0.4 (idx3) = 0.8 >= 0.8 -> exactly those two
    assert co.cummass_rows(p, valid, 0.8).flatten().tolist() == [False, True, False, True, False]
    # tau 0.85 needs one more: 0.1 (idx 2)
    assert co.cummass_rows(p, valid, 0.85).flatten().tolist() == [False, True, True, True, False]
    # ties: equal masses enter in index order
    q = torch.full((1, 1, 1, 4), 0.25)
    assert co.cummass_rows(q, torch.ones_like(q, dtype=torch.bool), 0.5).flatten().tolist() == [True, True, False, False]
    # invalid entries never enter; an unreachable tau keeps every valid entry
    valid2 = torch.tensor([[[[True, True, False, True, True]]]])
    assert co.cummass_rows(p, valid2, 2.0).flatten().tolist() == [True, True, False, True, True]


def test_rope_matches_reference(golden):
    """apply_rope against the reference's apply_rotary_pos_emb, bit for bit, for 16-bit and fp32 tables."""
    f = golden("rope")
    q = torch.from_numpy(f["q"]).to(torch.bfloat16)
    k = torch.from_numpy(f["k"]).to(torch.bfloat16)
    cos, sin = torch.from_numpy(f["cos"]), torch.from_numpy(f["sin"])
    c16, s16 = cos.to(torch.bfloat16), sin.to(torch.bfloat16)
    assert torch.equal(co.apply_rope(q, c16, s16).float(), torch.from_numpy(f["q_rot_bf16_tables"]))
    assert torch.equal(co.apply_rope(k, c16, s16).float(), torch.from_numpy(f["k_rot_bf16_tables"]))
    # fp32 tables: the reference returns fp32; the cache stores it rounded to the tensors' type
    assert torch.equal(co.apply_rope(q, cos, sin), torch.from_numpy(f["q_rot_f32_tables"]).to(torch.bfloat16))
    assert torch.equal(co.apply_rope(k, cos, sin), torch.from_numpy(f["k_rot_f32_tables"]).to(torch.bfloat16))
