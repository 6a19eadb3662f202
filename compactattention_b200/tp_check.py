"""Checks and times the fused output projection + tensor-parallel sum on the GPUs of one node:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29551 \
        -m compactattention_b200.tp_check [--rows 1024] [--hidden 4096] [--iters 50]

Every rank holds K = hidden / N input columns (the attention output of its heads).  The fused route
(``tp.FusedOutputProjection``: this library's three kernels over symmetric memory) is compared with a library
GEMM followed by an NCCL all-reduce on the same operands, then both are timed with CUDA events (max over
ranks).  Prints one JSON line on rank 0.  NCCL's in-switch reduction is left as the environment sets it.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from . import tp


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=1024)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--switch", action="store_true", help="also time the form that reduces through the NVLink switch (multimem)")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group(backend="nccl", device_id=dev)
    M, N, K = args.rows, args.hidden, args.hidden // world
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn((1, M, K), device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn((N, K), device=dev, generator=g) * 0.02).to(torch.bfloat16)
    # the default form (two ranks: one exchange; more: through the NVLink switch where it offers multicast) and the
    # reduce-scatter + all-gather form over plain peer stores
    routes = {"auto": tp.FusedOutputProjection(M, N, dev, torch.bfloat16)}
    routes["two_shot"] = tp.FusedOutputProjection(M, N, dev, torch.bfloat16, mode=1)   # reduce-scatter + all-gather over peer stores
    if 2 < world <= 4:
        routes["one_shot"] = tp.FusedOutputProjection(M, N, dev, torch.bfloat16, mode=2)      # every partial tile to every rank
    if world > 2 and args.switch and routes["auto"]._mc is not None:
        routes["switch"] = tp.FusedOutputProjection(M, N, dev, torch.bfloat16, mode=3)        # additions done by the NVLink switch
    # correctness: three calls in a row (buffers reused), against GEMM + all-reduce in fp32
    worst = 0.0
    for _ in range(3):
        ref = x.float() @ w.float().T
        dist.all_reduce(ref)
        for fused in routes.values():
            got = fused(x, w).float()
            worst = max(worst, ((got - ref).abs() / (ref.abs() + 1.0)).max().item())
        x = (x.float() * 0.5 + 0.1).to(torch.bfloat16)
    for fused in routes.values():
        fused.check()

    def timed(fn):
        for _ in range(5):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(int(4e6))   # ~2 ms of device spin: the host queues the whole loop behind it, so the
        e0.record()                   # events time the device, not the enqueue rate of this script
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return tp.max_over_ranks([e0.elapsed_time(e1) / args.iters * 1e3], dev)[0]

    def library_route():
        y = torch.nn.functional.linear(x, w)
        dist.all_reduce(y)
        return y

    # The launches one by one.  Each loop replays the same calls with one phase enabled: the pushes of the first
    # loop leave every counter ahead of what the later loops wait for, so those measure the kernels themselves,
    # not the waiting (and, launched back to back without a dependency, they overlap: a rate, not a latency).
    results = {}
    for name, fused in routes.items():
        phase_us = {}
        start = fused.ledger.snapshot()
        for pname, mask in (("gemm_and_push", 1), ("reduce", 2), ("final_wait", 4)):
            fused.ledger.restore(start)
            fused.phases = mask
            phase_us[pname] = round(timed(lambda: fused(x, w)), 1)
        fused.phases = 7
        total = timed(lambda: fused(x, w))
        fused.check()
        results[name] = {"fused_us": round(total, 1), "phase_us": phase_us}
    # the exchange alone (no GEMM) against NCCL's all-reduce of the same [rows, hidden] tensor
    y_part = torch.nn.functional.linear(x, w)
    fused0 = routes["auto"]
    got = fused0.all_reduce(y_part).float().clone()
    ref = y_part.float().clone()
    dist.all_reduce(ref)
    ar_err = ((got - ref).abs() / (ref.abs() + 1.0)).max().item()
    own_ar_us = timed(lambda: fused0.all_reduce(y_part))
    fused0.check()
    two_shot_ar_us = timed(lambda: routes["two_shot"].all_reduce(y_part))
    routes["two_shot"].check()
    one_shot_ar_us = None
    if "one_shot" in routes:
        one_shot_ar_us = round(timed(lambda: routes["one_shot"].all_reduce(y_part)), 1)
        routes["one_shot"].check()
    y_nccl = y_part.clone()
    nccl_ar_us = timed(lambda: dist.all_reduce(y_nccl))
    lib_us = timed(library_route)
    gemm_us = timed(lambda: torch.nn.functional.linear(x, w))
    if rank == 0:
        print(json.dumps({"world": world, "rows": M, "hidden": N, "k_per_rank": K, "max_rel_err_vs_gemm_plus_allreduce": round(worst, 5),
                          "fused": results, "library_gemm_plus_nccl_allreduce_us": round(lib_us, 1),
                          "library_gemm_alone_us": round(gemm_us, 1),
                          "auto_form": "one exchange" if world == 2 else "reduce-scatter + all-gather",
                          "all_reduce_alone": {"own_exchange_us": round(own_ar_us, 1), "own_two_shot_us": round(two_shot_ar_us, 1), "own_one_shot_us": one_shot_ar_us, "nccl_us": round(nccl_ar_us, 1),
                                               "max_rel_err": round(ar_err, 5)}}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
