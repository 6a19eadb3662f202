"""Generates the golden fixtures in this directory by executing the reference project's own
functions for the path on seeded CPU inputs.  Needs a checkout of the reference
(``COMPACTATTN_REFERENCE_ROOT``, default: a ``reference`` directory next to this repository); the fixtures it writes are committed
so the tests run without it.

    python tests/golden/make_golden.py

The reference's Triton kernels (mean-K pooling, block score, fused KV union) are executed through
Triton's CPU interpreter (``TRITON_INTERPRET=1``) on fp32 inputs, launching the kernel body directly
(the autotuner wrapper needs a GPU driver for its benchmarking).
Each ``.npz`` holds the inputs and the reference outputs of one group of functions.
"""
from __future__ import annotations

import math
import os
import sys
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from oracle import reference_loader  # noqa: E402

SEED = 1234  # the reference's default seed (eval/chunked_prefill/test_unified_latency_sweep.py:73)


def gen(seed_offset: int) -> torch.Generator:
    return torch.Generator().manual_seed(SEED + seed_offset)


def h16(x: torch.Tensor) -> torch.Tensor:
    """Rounds to the fp16 grid (kept in fp32) so an input can be stored in half the bytes exactly."""
    return x.to(torch.float16).to(torch.float32)


def save(name: str, half=(), **arrays) -> None:
    """Writes one fixture; arrays named in `half` hold fp16-representable values and are stored as fp16."""
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().cpu()
            if k in half:
                assert torch.equal(v.to(torch.float16).to(torch.float32), v.to(torch.float32)), k
                v = v.to(torch.float16)
            v = v.to(torch.float32).numpy() if v.dtype == torch.bfloat16 else v.numpy()
        out[k] = np.asarray(v)
    path = HERE / f"{name}.npz"
    np.savez_compressed(path, **out)
    print(f"wrote {path.name}: {path.stat().st_size / 1024:.1f} KiB")


def config1_block_mask(g: torch.Generator, Hq=32, Qb=4, Kb=128, density=0.2):
    """Bernoulli(density) per (head, q-block, k-block); sink block and the 2 diagonal/local blocks
    forced on, acausal blocks forced off (the CPU configuration of the benchmark definition)."""
    Pb = Kb - Qb
    m = torch.rand((Hq, Qb, Kb), generator=g) < density
    j = torch.arange(Kb).view(1, 1, Kb)
    i = torch.arange(Qb).view(1, Qb, 1)
    d = (Pb + i) - j
    m = m | (j == 0) | ((d >= 0) & (d < 2))
    return m & (d >= 0)


def group_union_table(ref) -> None:
    cd = ref.chunked_dense
    g = gen(1)
    Hq, Qb, Kb, G, bs = 32, 4, 128, 4, 64
    q_len, kv_len = Qb * bs, Kb * bs
    mask = config1_block_mask(g, Hq, Qb, Kb)  # [Hq, Qb, Kb]
    keep_block = mask.any(dim=1).unsqueeze(0)  # Q-block union -> [1, Hq, Kb]
    keep_kv = cd._build_kv_head_union_keep_block_mask(keep_block.clone(), q_len, kv_len, bs, G)
    idx, counts = cd._build_kv_head_union_past_block_indices(keep_block.clone(), q_len, kv_len, bs, G)
    idx2, counts2 = cd._build_kv_head_past_block_indices_from_kv_keep_block(keep_kv.clone(), q_len, kv_len, bs)
    assert torch.equal(idx, idx2) and torch.equal(counts, counts2)
    # G = 7 (28 q heads / 4 kv heads), batch 2, ragged selections incl. an empty and a full row
    g2 = gen(2)
    Hq7, Kb7, Qb7 = 28, 40, 4
    kb7 = torch.rand((2, Hq7, Kb7), generator=g2) < 0.15
    kb7[0, 0:7, : Kb7 - Qb7] = False
    kb7[1, 7:14, :] = True
    keep_kv7 = cd._build_kv_head_union_keep_block_mask(kb7.clone(), Qb7 * bs, Kb7 * bs, bs, 7)
    idx7, counts7 = cd._build_kv_head_union_past_block_indices(kb7.clone(), Qb7 * bs, Kb7 * bs, bs, 7)
    # short-width projection helper
    short = torch.rand((1, 8, 5), generator=g2) < 0.5
    proj = cd._project_short_qhead_keep_block_to_kv_full_width(short.clone(), 12, 4)
    # FlashInfer-style CSR metadata
    zc = ref.zero_copy
    pages, indptr, indices, _, _, _ = zc._build_index_metadata_reference_from_keep_block_kv(
        keep_block_kv=keep_kv.clone(), q_len=q_len, block_size=bs)
    save("union_table", mask=mask, keep_block=keep_block, keep_kv=keep_kv, idx=idx, counts=counts,
         keep_block_g7=kb7, keep_kv_g7=keep_kv7, idx_g7=idx7, counts_g7=counts7,
         short=short, short_proj=proj, fi_pages=pages, fi_indptr=indptr, fi_indices=indices,
         meta=np.array([Hq, Qb, Kb, G, bs, Hq7, Qb7, Kb7]))


def group_seer_keep(ref) -> None:
    cd = ref.chunked_dense
    g = gen(3)
    B, H, Qb, Kb, bs = 2, 8, 4, 36, 64
    q_len, kv_len = Qb * bs, Kb * bs
    Pb = Kb - Qb
    valid = (torch.arange(Kb).view(1, Kb) <= (Pb + torch.arange(Qb)).view(Qb, 1)).view(1, 1, Qb, Kb).expand(B, 1, Qb, Kb)
    logits = torch.randn((B, H, Qb, Kb), generator=g) * 2.0
    score = torch.softmax(logits.masked_fill(~valid, torch.finfo(torch.float32).min), dim=-1)
    outs = {}
    for ti, thr in enumerate((5e-4, 0.02, 0.05)):
        for kr in (0, 2):
            kb_generic, _, _, _ = cd._build_keep_block_mask(score.clone(), valid.clone(), thr, kr)
            kb_fast, _, _, _ = cd._build_keep_block_mask_chunked_fast_path(
                score.clone(), valid.clone(), thr, kr, q_len, kv_len, bs)
            outs[f"generic_t{ti}_r{kr}"] = kb_generic
            outs[f"fast_t{ti}_r{kr}"] = kb_fast
    save("seer_keep", score=score, valid=valid, thresholds=np.array([5e-4, 0.02, 0.05], dtype=np.float64),
         meta=np.array([B, H, Qb, Kb, bs]), **outs)


def group_attn_gate(ref) -> None:
    ag = ref.attn_gate
    g = gen(4)
    B, Q, K, Hq, Hkv, D, bs = 1, 128, 320, 2, 1, 128, 64
    Qb, Kb = Q // bs, K // bs
    q = h16(torch.randn((B, K, Hq, D), generator=g))  # full-sequence tensors; the chunk is the tail
    k = h16(torch.randn((B, K, Hkv, D), generator=g))
    # block positions: every bs-th position, half-rotation RoPE tables (theta 500000)
    inv = 1.0 / (500000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    pos = torch.arange(0, K, bs, dtype=torch.float32)
    ang = torch.cat([pos.view(-1, 1) * inv.view(1, -1)] * 2, dim=-1)
    cos, sin = ang.cos().unsqueeze(0), ang.sin().unsqueeze(0)  # [1, Kb, D]
    mask = (torch.arange(Kb).view(1, Kb) <= (Kb - Qb + torch.arange(Qb)).view(Qb, 1)).view(1, 1, Qb, Kb)
    out = {}
    for name, kwargs in (("Qavg_Kmaxminavg", {}), ("Qavg_Kavg", {"force_double": True})):
        gate = ag.ATTNGATE_CLASSES[name](bs, D, 128, Hkv, Hq, **kwargs)
        with torch.no_grad():
            for p in gate.parameters():
                p.copy_(h16(torch.randn(p.shape, generator=g) * 0.02))
            q_chunk = q[:, K - Q :]
            qb = gate.compress_query_blocks(q_chunk)
            kb = gate.compress_key_blocks(k)
            qb_r, _ = gate.apply_block_position_embeddings(q=qb, k=None, position_embeddings=(cos[:, Kb - Qb :], sin[:, Kb - Qb :]))
            _, kb_r = gate.apply_block_position_embeddings(q=None, k=kb, position_embeddings=(cos, sin))
            sc_soft = gate.score_compressed_blocks(qb_r, kb_r, mask, use_softmax=True)
            sc_raw = gate.score_compressed_blocks(qb_r, kb_r, mask, use_softmax=False)
        out[f"{name}_wk"] = gate.mask_linear_k.weight.detach()
        if gate.mask_linear_q is not None:
            out[f"{name}_wq"] = gate.mask_linear_q.weight.detach()
        out[f"{name}_qb"] = qb
        out[f"{name}_kb"] = kb
        out[f"{name}_qb_rope"] = qb_r
        out[f"{name}_kb_rope"] = kb_r
        out[f"{name}_score_softmax"] = sc_soft
        out[f"{name}_score_raw"] = sc_raw
    half = ("q", "k") + tuple(n for n in out if n.endswith("_wk") or n.endswith("_wq"))
    save("attn_gate", half=half, q=q[:, K - Q :], k=k, cos=cos, sin=sin, mask=mask, meta=np.array([B, Q, K, Hq, Hkv, D, bs]), **out)


def group_flashprefill(ref) -> None:
    fv = ref.flashprefill_vendor
    fp = ref.flashprefill_prefill
    g = gen(5)
    B, Q, K, Hq, Hkv, D, bs = 1, 192, 704, 4, 2, 128, 64
    Qb, Kb = Q // bs, K // bs
    G = Hq // Hkv
    q = torch.randn((B, Q, Hq, D), generator=g)
    k = torch.randn((B, K, Hkv, D), generator=g)
    # per-head low-rank bias so the pooled scores are peaked
    u = torch.randn((Hkv, D), generator=g)
    a = torch.randn((K, Hkv), generator=g).clamp_min(0) * (torch.rand((K, Hkv), generator=g) < 0.1)
    k = k + 2.0 * a.unsqueeze(-1) * u.unsqueeze(0)
    q = h16(q + 0.5 * u.repeat_interleave(G, dim=0).unsqueeze(0).unsqueeze(0))
    k = h16(k)
    mean_k = torch.empty((B, Kb, Hkv, D), dtype=k.dtype)
    fv.compute_mean_vector.fn[(Kb, B * Hkv, 1)](k, mean_k, *k.stride(), *mean_k.stride(), Hkv, K, bs, D)
    # ragged length: 674 tokens -> last block has 34 tokens
    k_ragged = k[:, :674].contiguous()
    mean_k_ragged = torch.empty((B, 11, Hkv, D), dtype=k.dtype)
    fv.compute_mean_vector.fn[(11, B * Hkv, 1)](k_ragged, mean_k_ragged, *k_ragged.stride(), *mean_k_ragged.stride(), Hkv, 674, bs, D)
    score = torch.full((B, Qb, Kb, Hq), float("-inf"), dtype=torch.float32)
    mx = torch.full_like(score, float("-inf"))
    fv.compute_block_score_chunked.fn[(Qb, B * Hq, 1)](
        q, mean_k, 1 / math.sqrt(D), score, mx, *q.stride(), *mean_k.stride(), *score.stride(), *mx.stride(),
        Hq, Hkv, Q, Kb, K - Q, bs, K_TILE_SIZE=64, K_STRIDE=bs, D_HEAD=D)
    norm = fv.normalize_scores(score.clone(), mx.clone())
    out = {}
    for tag, (sink, window, alpha, last_n, budget) in {
        "a": (2, 4, 0.06, 0, 0),
        "b": (1, 2, 0.3, 1, 0),
        "c": (2, 4, 0.5, 0, 3),
    }.items():
        kb_q, kb_kv = fp._flashprefill_keep_block_from_scores_rowwise(
            norm.clone(), q_len=Q, kv_len=K, block_size=bs, num_key_value_groups=G, attention_sink=sink,
            window_size=window, alpha=alpha, last_n_block=last_n, min_budget=budget)
        out[f"keep_q_{tag}"] = kb_q
        out[f"keep_kv_{tag}"] = kb_kv
        if budget == 0:
            fused = torch.empty((B, Hkv, Kb), dtype=torch.bool)
            tail = min(max(last_n, 0), Qb - 1) if Qb > 1 else 0
            fp._flashprefill_kv_union_from_scores_kernel[(math.ceil(Kb / 64), B * Hkv)](
                norm, fused, *norm.stride(), *fused.stride(), Hq, Kb, (K - Q) // bs, max(Qb - tail, 1),
                sink, window, float(alpha), G, BLOCK_K=64)
            out[f"keep_kv_fused_{tag}"] = fused
        out[f"params_{tag}"] = np.array([sink, window, alpha, last_n, budget], dtype=np.float64)
    save("flashprefill", half=("q", "k"), q=q, k=k, mean_k=mean_k, mean_k_ragged=mean_k_ragged, score_raw=score, max_raw=mx,
         score_norm=norm, meta=np.array([B, Q, K, Hq, Hkv, D, bs]), **out)


def group_topk(ref) -> None:
    cm = ref.common
    g = gen(6)
    n = 24
    x = torch.randn((1, 4, n, n), generator=g)  # distinct values: no ties
    out = {}
    for ti, nz in enumerate((0.2, 0.5, 0.9)):
        out[f"mask_{ti}"] = cm.get_sparse_attn_mask_from_nz_ratio(x.clone(), nz)
    save("topk", x=x, nz=np.array([0.2, 0.5, 0.9]), **out)


def group_block_mask(ref) -> None:
    # the block-causal mask builder lives on a model class that cannot be imported with current
    # transformers; its stand-alone twin is in the evaluation runtime, whose source is executed here
    import ast
    import torch.nn.functional as F
    src_path = Path(reference_loader.DEFAULT_ROOT) / "eval" / "chunked_prefill" / "chunked_prefill_runtime.py"
    tree = ast.parse(src_path.read_text())
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "_build_replacement_block_attention_mask")
    ns = {"torch": torch, "F": F}
    mod = ast.fix_missing_locations(ast.Module(body=[fn], type_ignores=[]))
    fn.returns = None
    for a in fn.args.kwonlyargs + fn.args.args:
        a.annotation = None
    exec(compile(mod, str(src_path), "exec"), ns)
    build = ns["_build_replacement_block_attention_mask"]
    out = {}
    cases = [(256, 8192, 64), (1024, 4096, 64), (100, 1000, 64), (512, 512, 128), (64, 640, 64)]
    for ci, (Q, K, bs) in enumerate(cases):
        out[f"mask_{ci}"] = build(attention_mask=None, batch_size=1, query_len=Q, kv_len=K, block_size=bs, device=torch.device("cpu"))
    save("block_mask", cases=np.array(cases), **out)


def group_gather_attention(ref) -> None:
    cd = ref.chunked_dense
    vl = ref.varlen
    fp = ref.flashprefill_prefill
    g = gen(7)
    B, Q, K, Hq, Hkv, D, bs = 1, 128, 640, 4, 2, 128, 64
    G = Hq // Hkv
    Kb, Qb = K // bs, Q // bs
    q = h16(torch.randn((B, Q, Hq, D), generator=g))
    k = h16(torch.randn((B, K, Hkv, D), generator=g))
    v = h16(torch.randn((B, K, Hkv, D), generator=g))
    keep_block = torch.rand((B, Hq, Kb), generator=g) < 0.2
    keep_kv = cd._build_kv_head_union_keep_block_mask(keep_block.clone(), Q, K, bs, G)
    idx, counts = cd._build_kv_head_union_past_block_indices(keep_block.clone(), Q, K, bs, G)
    keep_tok = cd._expand_blocks_to_tokens(keep_kv, bs, K)
    kc, vc, table, sel_lens = vl.build_paged_kv_cache_from_token_mask(k, v, keep_tok.clone(), page_block_size=256)
    # compact attention through the reference's own CPU attention (explicit mask + SDPA): one call per
    # KV head with that head's kept tokens as the padding mask
    out = torch.empty((B, Q, Hq, D))
    for h in range(Hkv):
        o, _ = fp._flashprefill_dense_fallback(
            q[:, :, h * G : (h + 1) * G], k[:, :, h : h + 1], v[:, :, h : h + 1], keep_tok[:, h],
            softmax_scale=1 / math.sqrt(D), num_key_value_groups=G, measure_timing=False, attn_module=None)
        out[:, :, h * G : (h + 1) * G] = o
    dense, _ = fp._flashprefill_dense_fallback(q, k, v, None, softmax_scale=1 / math.sqrt(D), num_key_value_groups=G,
                                               measure_timing=False, attn_module=None)
    save("gather_attention", half=("q", "k", "v", "k_cache", "v_cache"), q=q, k=k, v=v, keep_block=keep_block, keep_kv=keep_kv, idx=idx, counts=counts,
         k_cache=kc, v_cache=vc, block_table=table, sel_lens=sel_lens, out_compact=out, out_dense=dense,
         meta=np.array([B, Q, K, Hq, Hkv, D, bs]))


def group_rope(ref) -> None:
    """apply_rotary_pos_emb (compact_attn/modules/common.py:49-75) on [B, L, H, D] bf16 tensors with
    bf16 tables (the dtype the model passes) and with fp32 tables (type promotion to fp32)."""
    g = gen(8)
    B, L, Hq, Hkv, D = 1, 96, 4, 2, 64
    q = torch.randn((B, L, Hq, D), generator=g).to(torch.bfloat16)
    k = torch.randn((B, L, Hkv, D), generator=g).to(torch.bfloat16)
    inv = 1.0 / (500000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = torch.arange(1000, 1000 + L, dtype=torch.float32)[:, None] * inv[None]
    emb = torch.cat((ang, ang), dim=-1)
    cos, sin = emb.cos()[None], emb.sin()[None]
    q16, k16 = ref.common.apply_rotary_pos_emb(q, k, cos.to(torch.bfloat16), sin.to(torch.bfloat16), unsqueeze_dim=2)
    q32, k32 = ref.common.apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim=2)
    assert q16.dtype == torch.bfloat16 and q32.dtype == torch.float32
    save("rope", q=q, k=k, cos=cos, sin=sin, q_rot_bf16_tables=q16, k_rot_bf16_tables=k16,
         q_rot_f32_tables=q32, k_rot_f32_tables=k32)


def main() -> None:
    ref = reference_loader.load()
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    group_union_table(ref)
    group_seer_keep(ref)
    group_attn_gate(ref)
    group_flashprefill(ref)
    group_topk(ref)
    group_block_mask(ref)
    group_gather_attention(ref)
    group_rope(ref)


if __name__ == "__main__":
    main()
