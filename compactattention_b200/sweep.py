"""Shape / density sweep of the attention and gather kernels on one GPU (single layer):

    python -m compactattention_b200.sweep [--quick] [--positions]

For every point: latency of ``ca_attn_compact`` over a synthetic block table with the exact density,
effective TFLOP/s (algorithmic FLOPs / time) and its fraction of the cuBLAS bf16 peak, latency of the
dense kernel of the same shape (speed-up), and the compact KV gather's HBM throughput (read + write
bytes / time).  ``--positions`` walks all chunk positions of a 128K-token prefill (chunk 1024) at
10 / 20 / 30 % density.  Prints one JSON line per point.
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="a small subset of the grid")
    ap.add_argument("--positions", action="store_true", help="all chunk positions of a 128K prefill, chunk 1024")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1234 + 5)
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
