"""Chunked prefill of a long random prompt through the Llama-3.1-8B-shaped stack (random-init bf16
weights), optionally tensor-parallel over the GPUs of one node:

    python -m compactattention_b200.prefill_sparse.llama.run_prefill --layers 32 --prompt 131072 --chunk 2048
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29531 \
        -m compactattention_b200.prefill_sparse.llama.run_prefill --layers 32 --prompt 131072 --chunk 2048

Prints one JSON line (rank 0): total prefill time, per-chunk time of the last chunks, and the time
spent inside the attention modules (CUDA events around every ``self_attn`` call, max over ranks) -
the same quantity the reference's profiler reports as ``attn_per_chunk_ms``
(``eval/chunked_prefill/profile_attention_latency.py:105-168, 902-907``).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ... import tp
from .harness import LlamaCompactAttnStack
from .modeling_llama_compactattn import CompactAttnLlamaConfig


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=131072)
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--selector", choices=["gate", "flashprefill"], default="gate")
    ap.add_argument("--topk", type=float, default=0.2, help="per-row top-k fraction of the gate selector")
    ap.add_argument("--rule", choices=["topk", "synthetic_topk", "threshold"], default="synthetic_topk",
                    help="synthetic_topk imposes the union density exactly (random-init gates do not agree across heads)")
    ap.add_argument("--dense", action="store_true", help="force dense attention in every chunk (comparator)")
    ap.add_argument("--graph-mlp", action="store_true",
                    help="replay the local part of the residual + norm + MLP half of every layer from a CUDA graph")
    ap.add_argument("--fused-projections", action="store_true",
                    help="tensor parallel: o_proj and the MLP's down projection with their sums over the ranks as the "
                         "library's fused kernels over peer memory instead of library GEMMs + NCCL all-reduces")
    ap.add_argument("--seed", type=int, default=1234 + 4)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        torch.distributed.init_process_group(backend="nccl", device_id=dev)
    cfg = CompactAttnLlamaConfig(num_hidden_layers=args.layers, seerattn_gate_type="Qavg_Kavg", seerattn_gate_force_double=True,
                                 seerattn_sparsity_method=args.rule, seerattn_topk_ratio=(int(round(args.topk * 1000)), 1000),
                                 seerattn_chunked_prefill_force_dense=args.dense, max_position_embeddings=args.prompt,
                                 compactattn_fused_oproj_rows=args.chunk if args.fused_projections else 0)
    shard = tp.HeadShard(world, rank, cfg.num_attention_heads, cfg.num_key_value_heads)
    model = LlamaCompactAttnStack(cfg, args.selector, shard).to(torch.bfloat16).to(dev)
    model.init_weights(seed=args.seed)
    for layer in model.layers:
        layer.graph_mlp = args.graph_mlp
    # token ids seeded like the reference's synthetic prompts (seed + seq_len * 104729)
    g = torch.Generator().manual_seed(args.seed + args.prompt * 104729)
    ids = torch.randint(0, cfg.vocab_size, (1, args.prompt), generator=g).to(dev)
    # CUDA events around every attention module call
    events = []
    host_s = [0.0]
    import time
    for layer in model.layers:
        orig = layer.self_attn.forward

        def timed(*a, _orig=orig, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            w0 = time.perf_counter()
            out = _orig(*a, **kw)
            host_s[0] += time.perf_counter() - w0   # host time to enqueue the module's work (nothing waits inside)
            e1.record()
            events.append((e0, e1))
            return out

        layer.self_attn.forward = timed
    # warm-up outside the timed region: two chunks on a throw-away cache bring up the NCCL communicator
    # (its first collective takes seconds), cuBLAS workspaces and the library's scratch buffers
    warm = model.new_cache(1, 2 * args.chunk)
    model.prefill(ids[:, : 2 * args.chunk], args.chunk, warm)
    del warm
    events.clear()
    host_s[0] = 0.0
    cache = model.new_cache(1, args.prompt)
    for i in range(args.layers):   # the paged caches are allocated (and zero-filled) before the clock starts
        cache.layer(i, len(shard.kv_heads), cfg.head_dim)
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    w_all = time.perf_counter()
    hidden, cache = model.prefill(ids, args.chunk, cache)
    host_total_s = time.perf_counter() - w_all      # host time to enqueue the whole prefill
    t1.record()
    torch.cuda.synchronize()
    total_ms = t0.elapsed_time(t1)
    n_chunks = args.prompt // args.chunk
    per_call = [a.elapsed_time(b) for a, b in events]
    attn_ms_total = sum(per_call)
    last = per_call[-args.layers:]
    vals = tp.max_over_ranks([total_ms, attn_ms_total, sum(last)], dev)
    if rank == 0:
        print(json.dumps({
            "workload": f"{args.layers}-layer Llama-3.1-8B-shaped stack, prompt {args.prompt}, chunk {args.chunk}, "
                        f"selector {args.selector}/{args.rule} {args.topk:.0%}{' (dense forced)' if args.dense else ''}"
                        f"{', MLP half from CUDA graphs' if args.graph_mlp else ''}"
                        f"{', fused projections' if args.fused_projections and world > 1 else ''}, tp{world}",
            "prefill_ms": round(vals[0], 2), "chunks": n_chunks,
            "attn_per_chunk_ms": round(vals[1] / n_chunks, 3),
            "attn_last_chunk_ms": round(vals[2], 3),
            "attn_last_chunk_per_layer_us": round(vals[2] / args.layers * 1e3, 1),
            "host_enqueue_ms": round(host_total_s * 1e3, 1),
            "host_attn_module_us_per_layer_call": round(host_s[0] / max(len(events), 1) * 1e6, 1),
            "host_us_per_layer_call": round(host_total_s / max(len(events), 1) * 1e6, 1),
            "finite": bool(torch.isfinite(hidden.float()).all()),
            "hidden_checksum": round(float(hidden.float().abs().mean()), 5),
        }))
    for proj in tp._SHARED_PROJECTIONS.values():
        proj.check()   # a device-side wait that ran out would have left invalid outputs
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
