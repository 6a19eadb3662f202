"""Shape / density sweep of the attention and gather kernels on one GPU (single layer):

    python -m compactattention_b200.sweep [--quick] [--positions | --append]

For every point: latency of ``ca_attn_compact`` over a synthetic block table with the exact density,
effective TFLOP/s (algorithmic FLOPs / time) and its fraction of the cuBLAS bf16 peak, latency of the
dense kernel of the same shape (speed-up), and the compact KV gather's HBM throughput (read + write
bytes / time).  ``--positions`` walks all chunk positions of a 128K-token prefill (chunk 1024) at
10 / 20 / 30 % density.  ``--append`` times the chunk append (RoPE + paged write + mean-K pooling,
``ca_rope_append``) against the three torch steps it replaces.  Prints one JSON line per point.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from . import ops

D, BS = 128, 64


def timed(fn, iters):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3  # us


def peaks():
    p = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if p.exists():
        j = json.loads(p.read_text())
        return j["bf16_tflops"], j["hbm_gbs"], "measured"
    return 1590.0, 6650.0, "fallback"


def make_table(hkv, pb, density, dev, g):
    n = max(0, min(pb, int(round(pb * density))))
    idx = torch.full((hkv, max(pb, 1)), -1, dtype=torch.int32, device=dev)
    for r in range(hkv):
        idx[r, :n] = torch.randperm(pb, device=dev, generator=g)[:n].sort().values.int()
    return idx, torch.full((hkv,), n, dtype=torch.int32, device=dev), n


def point(hq, hkv, q_len, kv_len, density, dev, g, kv_cache, iters, with_dense, with_gather):
    k, v = kv_cache
    q = torch.randn((1, q_len, hq, D), device=dev, dtype=torch.bfloat16, generator=g)
    out = torch.empty_like(q)
    kv = ops.KvCacheView.from_seq_first(k[:, :kv_len], v[:, :kv_len])
    pb = (kv_len - q_len) // BS
    idx, counts, n = make_table(hkv, pb, density, dev, g)
    us = timed(lambda: ops.attn_compact(q, kv, kv_len, hkv, idx, counts, out=out), iters)
    G = hq // hkv
    flops = 4.0 * D * G * (q_len * hkv * n * BS + hkv * q_len * (q_len + 1) / 2.0)
    peak_tf, peak_bw, src = peaks()
    rec = {"hq": hq, "hkv": hkv, "chunk": q_len, "kv_len": kv_len, "density": density, "selected_blocks_per_head": n,
           "attn_us": round(us, 1), "attn_tflops": round(flops / us / 1e6, 1), "frac_of_bf16_peak": round(flops / us / 1e6 / peak_tf, 3),
           "peak_source": src}
    if with_dense:
        dus = timed(lambda: ops.attn_compact(q, kv, kv_len, hkv, None, None, out=out), max(2, iters // 3))
        rec["dense_us"] = round(dus, 1)
        rec["speedup_vs_dense"] = round(dus / us, 2)
    if with_gather:
        tokens = (n + q_len // BS) * BS
        kd = torch.empty((hkv * tokens, D), dtype=torch.bfloat16, device=dev)
        vd = torch.empty_like(kd)
        gus = timed(lambda: ops.gather_kv(kv, hkv, 1, q_len, kv_len, idx, counts, kd, vd, block_size=BS,
                                          dst_row_stride_tokens=tokens), iters)
        moved = 2.0 * 2 * hkv * tokens * D * 2  # K and V, read + write
        rec["gather_us"] = round(gus, 1)
        rec["gather_gbs"] = round(moved / gus / 1e3, 1)
        rec["gather_frac_of_hbm_peak"] = round(moved / gus / 1e3 / peak_bw, 3)
    return rec


def append_points(dev, g, iters):
    """ca_rope_append: HBM bytes = q, k, v read once and written once (+ tables, + mean-K).  The
    inputs rotate over enough chunk-sized sets to exceed L2, and the destination walks through the
    cache, so no launch finds its data in L2."""
    from .paged_cache import PagedKVCache
    from .prefill_sparse.llama.modeling_llama_compactattn import apply_rotary_pos_emb
    hbm = peaks()[1]
    for hq, hkv in ((32, 8), (28, 4)):
        for q_len in (256, 1024, 2048, 8192):
            max_tokens = 131072
            set_bytes = 2 * q_len * (hq + 2 * hkv) * D
            n_sets = max(2, -(-300 * 2 ** 20 // set_bytes))
            cache = PagedKVCache(1, max_tokens, hkv, D, dev)
            qs = torch.randn((n_sets, q_len, hq, D), device=dev, dtype=torch.bfloat16, generator=g)
            ks = torch.randn((n_sets, q_len, hkv, D), device=dev, dtype=torch.bfloat16, generator=g)
            vs = torch.randn((n_sets, q_len, hkv, D), device=dev, dtype=torch.bfloat16, generator=g)
            cos = torch.rand((1, q_len, D), device=dev, generator=g).to(torch.bfloat16)
            sin = torch.rand((1, q_len, D), device=dev, generator=g).to(torch.bfloat16)
            mean_k = torch.empty((1, max_tokens // BS, hkv, D), device=dev, dtype=torch.bfloat16)
            q_out = torch.empty_like(qs)
            state = {"i": 0}

            def step(fused):
                i = state["i"]
                state["i"] = i + 1
                s_, pos = i % n_sets, (i * q_len) % (max_tokens - q_len + 1) // BS * BS
                q, k, v = qs[s_: s_ + 1], ks[s_: s_ + 1], vs[s_: s_ + 1]
                if fused:
                    ops.rope_append(q, k, v, cos, sin, cache.view(), pos, mean_k=mean_k, block_size=BS, q_out=q_out[s_: s_ + 1])
                else:
                    _, kr = apply_rotary_pos_emb(q, k, cos, sin)
                    cache.append(kr, v, position=pos)
                    ops.pool_blocks(kr, BS, ("avg",), out=mean_k, out_block_offset=pos // BS)

            n_it = max(iters, 2 * n_sets)
            us = timed(lambda: step(True), n_it)
            us_torch = timed(lambda: step(False), n_it)
            nbytes = 2 * set_bytes + 2 * 2 * q_len * D + 2 * (q_len // BS) * hkv * D
            rec = {"op": "rope_append", "hq": hq, "hkv": hkv, "chunk": q_len, "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1),
                   "frac_of_hbm_peak": round(nbytes / us / 1e3 / hbm, 3), "algorithmic_bytes": nbytes,
                   "torch_rope_plus_append_plus_pool_us": round(us_torch, 2)}
            print(json.dumps(rec), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="a small subset of the grid")
    ap.add_argument("--positions", action="store_true", help="all chunk positions of a 128K prefill, chunk 1024")
    ap.add_argument("--append", action="store_true", help="the chunk append kernel against its torch equivalent")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1234 + 5)
    if args.append:
        append_points(dev, g, args.iters)
        return
    max_kv = 131072 if (args.positions or args.quick) else 262144
    caches = {}
    for hkv in (8, 4):
        caches[hkv] = (torch.randn((1, max_kv, hkv, D), device=dev, dtype=torch.bfloat16, generator=g),
                       torch.randn((1, max_kv, hkv, D), device=dev, dtype=torch.bfloat16, generator=g))
    if args.positions:
        for density in (0.1, 0.2, 0.3):
            for i in range(1, 128):
                if args.quick and i % 16 != 15:
                    continue
                rec = point(32, 8, 1024, 1024 * (i + 1), density, dev, g, caches[8], args.iters, with_dense=True, with_gather=False)
                rec["position"] = i
                print(json.dumps(rec), flush=True)
        return
    heads = [(32, 8), (28, 4)]
    chunks = [1024] if args.quick else [256, 512, 1024, 2048, 4096, 8192]
    kv_lens = [16384, 131072] if args.quick else [16384, 65536, 131072, 262144]
    densities = [0.05, 0.2, 0.5] if args.quick else [0.05, 0.1, 0.2, 0.3, 0.5]
    for hq, hkv in heads:
        for q_len in chunks:
            for kv_len in kv_lens:
                if kv_len <= q_len:
                    continue
                for density in densities:
                    rec = point(hq, hkv, q_len, kv_len, density, dev, g, caches[hkv], args.iters,
                                with_dense=(density == densities[0]), with_gather=(q_len == 1024))
                    print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
