"""Runs ONE kernel of the path a few times on seeded synthetic inputs — the program that the ncu
captures summarised under ``profiles/`` wrap.  Each case holds well under a few GB on the device and
its inputs exceed L2, so DRAM counters mean something and a capture ends by itself.

    python -m compactattention_b200.kernel_case attn    [--kv-len 131072] [--density 0.2] [--launches 4]
    python -m compactattention_b200.kernel_case gather  [--kv-len 131072] [--density 0.2]
    python -m compactattention_b200.kernel_case append  [--chunk 8192]
    python -m compactattention_b200.kernel_case fpscore [--kv-len 131072]
    python -m compactattention_b200.kernel_case select  [--kv-len 131072]      # select_rows + union_table (stand-alone)
    python -m compactattention_b200.kernel_case gate    [--kv-len 131072]      # gate_prepare + gate_scores_tc + select_rows with the fused union

Shapes: 32 query / 8 KV heads, d = 128, block 64, chunk 1024 (unless ``--chunk``), bf16.  Prints the
average time per launch from CUDA events (never quote it from a run under a profiler).
"""
from __future__ import annotations

import argparse

import torch

from . import ops

HQ, HKV, D, BS = 32, 8, 128, 64


def _table(pb: int, density: float, dev, g):
    n = max(1, int(pb * density))
    idx = torch.stack([torch.randperm(pb, device=dev, generator=g)[:n].sort().values for _ in range(HKV)]).int().contiguous()
    return idx, torch.full((HKV,), n, dtype=torch.int32, device=dev), n


def _time(fn, launches: int) -> float:
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / launches * 1e3


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=["attn", "gather", "append", "fpscore", "select", "gate"])
    ap.add_argument("--kv-len", type=int, default=131072)
    ap.add_argument("--chunk", type=int, default=1024)
    ap.add_argument("--density", type=float, default=0.2)
    ap.add_argument("--launches", type=int, default=4)
    ap.add_argument("--kv-heads", type=int, default=8, help="KV heads with 4 query heads each (1 = one rank of TP8)")
    args = ap.parse_args()
    global HQ, HKV
    HKV, HQ = args.kv_heads, 4 * args.kv_heads
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1234)
    K, Q = args.kv_len, args.chunk
    pb = (K - Q) // BS

    def rnd(*shape):
        return torch.randn(shape, device=dev, dtype=torch.bfloat16, generator=g)

    if args.case in ("attn", "gather"):
        q, k, v = rnd(1, Q, HQ, D), rnd(1, K, HKV, D), rnd(1, K, HKV, D)
        kv = ops.KvCacheView.from_seq_first(k, v)
        idx, counts, n = _table(pb, args.density, dev, g)
        if args.case == "attn":
            out = torch.empty_like(q)
            us = _time(lambda: ops.attn_compact(q, kv, K, HKV, idx, counts, out=out), args.launches)
            flops = 4.0 * D * (HQ // HKV) * (Q * HKV * n * BS + HKV * Q * (Q + 1) / 2)
            print(f"attn_compact_kernel: {n} of {pb} past blocks per KV head, {us:.1f} us/launch, {flops / us / 1e6:.0f} TFLOP/s")
        else:
            cap = (n + Q // BS) * BS
            kd = torch.empty((HKV * cap, D), device=dev, dtype=torch.bfloat16)
            vd = torch.empty_like(kd)
            us = _time(lambda: ops.gather_kv(kv, HKV, 1, Q, K, idx, counts, kd, vd, block_size=BS, dst_row_stride_tokens=cap), args.launches)
            nbytes = 2 * 2 * HKV * cap * D * 2
            print(f"gather_kv_kernel: {n} blocks + chunk per KV head, {nbytes / 1e6:.1f} MB read+written, {us:.1f} us/launch, {nbytes / us / 1e3:.0f} GB/s")
    elif args.case == "append":
        from .paged_cache import PagedKVCache
        cache = PagedKVCache(1, max(2 * Q, 16384), HKV, D, dev)
        q, k, v = rnd(1, Q, HQ, D), rnd(1, Q, HKV, D), rnd(1, Q, HKV, D)
        cos, sin = rnd(1, Q, D), rnd(1, Q, D)
        mean_k = torch.empty((1, cache.pages_per_seq * cache.page_size // BS, HKV, D), device=dev, dtype=torch.bfloat16)
        q_out = torch.empty_like(q)
        us = _time(lambda: ops.rope_append(q, k, v, cos, sin, cache.view(), 0, mean_k=mean_k, block_size=BS, q_out=q_out), args.launches)
        nbytes = 2 * 2 * Q * (HQ + 2 * HKV) * D
        print(f"rope_append_kernel: chunk {Q}, {nbytes / 1e6:.1f} MB read+written, {us:.1f} us/launch, {nbytes / us / 1e3:.0f} GB/s")
    elif args.case == "fpscore":
        q, mean_k = rnd(1, Q, HQ, D), rnd(1, K // BS, HKV, D)
        us = _time(lambda: ops.flashprefill_score(q, mean_k, K, BS), args.launches)
        print(f"fp_score_kernel + normalize: {K // BS} key blocks, {us:.1f} us per call")
    elif args.case == "select":
        score = torch.randn((1, HQ, Q // BS, K // BS), device=dev, generator=g)
        bits = ops.select_rows(score, pb, "topk", topk_ratio=(1, 5), sink=1, local=2)
        table = ops.union_table(bits=bits, num_kv_heads=HKV, kv_blocks=K // BS, past_blocks=pb, block_size=BS)

        def run():
            ops.select_rows(score, pb, "topk", topk_ratio=(1, 5), sink=1, local=2, bits=bits)
            ops.union_table(bits=bits, num_kv_heads=HKV, kv_blocks=K // BS, past_blocks=pb, block_size=BS, out=table)

        us = _time(run, args.launches)
        print(f"select_rows_kernel + union_table_kernel: {K // BS} key blocks, {us:.1f} us per pair")
    else:
        from .chunk_driver import GateSelectorState
        from .prefill_sparse.attn_gate import ATTNGATE_CLASSES
        gate = ATTNGATE_CLASSES["Qavg_Kavg"](BS, D, 128, HKV, HQ, force_double=True).to(dev).to(torch.bfloat16)
        st = GateSelectorState(gate, 1, dev, cache_dtype=torch.bfloat16)
        st.cache.reserve(K // BS)
        st.cache.blocks_view().normal_(generator=g)   # stands in for the blocks of earlier chunks
        q, k = rnd(1, Q, HQ, D), rnd(1, Q, HKV, D)

        from .chunk_driver import SelectionRule
        rule = SelectionRule(rule="topk", softmax=False, topk_ratio=(1, 5), sink=1, local=2)

        def run():
            st.cache.length = pb   # the chunk's blocks are (re)appended after the past blocks
            st.append(q, k, None, None)
            st.score_select(rule, HKV, BS)   # tensor-core scores, then rule + Block-Union + table

        us = _time(run, args.launches)
        print(f"gate_prepare_kernel + gate_scores_tc_kernel + select_rows_kernel (fused union): {K // BS} key blocks, "
              f"{us:.1f} us per chain")


if __name__ == "__main__":
    main()
