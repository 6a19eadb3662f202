#!/usr/bin/env python
"""Benchmark of the CompactAttention chunked-prefill hot path on B200.

Workload (N = 1): one Llama-3.1-8B-shaped attention layer (32 q heads / 8 KV heads, d = 128, bf16),
a 1024-token chunk appended at the end of a 128K-token paged KV cache (64-token pages, randomly
permuted page ids), block size 64.  Selection = learned-gate-style selector with random-init weights
(pooled Q and pooled K, 128 -> 128 projections per head, block RoPE) and per-row block top-k at 20 %
density plus sink and local blocks.  A step is one pass of the path for one chunk:
pool Q/K blocks, project + RoPE + append to the gate's K-block cache (one launch), gate logits on the tensor
core (one launch), top-k rows + Block-Union table (one launch), block-table attention (the kernel and, when it
cuts work units over the SMs, its merge kernel).  The steps of the timed loop re-issue the library calls from
parameter blocks kept per layer state.  Data is synthetic (seeded N(0,1)); steps rotate over
several independent layer states so consecutive steps read different HBM (total > L2).

At N > 1 the KV heads are sharded over the ranks (tensor parallel): every rank selects and attends
its own heads, then the layer output partial sums are summed over the ranks - by the library's own exchange over
peer memory (`ca_oproj_allreduce` without the GEMM) or, with `--nccl-all-reduce`, by NCCL; total work is fixed
("strong" scaling) and the value is the max-over-ranks latency.

`--impl reference` times the CPU restatement of the reference's path (oracle port, torch on all host
cores) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HQ, HKV, D, BS = 32, 8, 128, 64
METRIC = "per-chunk attn latency @128K ctx, chunk 1024"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
    ap.add_argument("--kv-len", type=int, default=131072)
    ap.add_argument("--chunk", type=int, default=1024)
    ap.add_argument("--density", type=float, default=0.2)
    ap.add_argument("--layers", type=int, default=4, help="independent layer states the steps rotate over")
    ap.add_argument("--seed", type=int, default=1234 + 3)
    ap.add_argument("--no-dense", action="store_true", help="skip the dense comparator")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="skip the CUDA-graph replay of the step")
    ap.add_argument("--no-sustained", action="store_true", help="skip the seconds-long repeat of the timed loop")
    ap.add_argument("--sustained-seconds", type=float, default=1.0)
    ap.add_argument("--dependent-launch", action="store_true",
                    help="enqueue programmatic dependent launches instead of plain ones (for A/B timing)")
    ap.add_argument("--no-call-lists", action="store_true",
                    help="fill the parameter blocks of every library call afresh in every step (the tensor-level wrappers) "
                         "instead of re-issuing the calls recorded once per layer state")
    ap.add_argument("--own-all-reduce", action="store_true",
                    help="N > 1: the library's own exchange for the layer-output all-reduce even where NCCL is the default")
    ap.add_argument("--nccl-all-reduce", action="store_true",
                    help="N > 1: NCCL for the layer-output all-reduce of the step even where the library's own exchange is the default")
    ap.add_argument("--two-launch-selection", action="store_true",
                    help="gate scores and rule + table as two launches (the form before ca_gate_score_select; for A/B timing)")
    return ap.parse_args()


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples the SM clock, power and the throttle reasons while the benchmark's timed regions run.
    The samples come from NVML inside this process (read only), one every millisecond or two from a
    thread that polls without sleeping long; ``nvidia-smi -lms`` (one sample per 100 ms at best) is the
    fallback when NVML cannot be loaded.  ``mark(name)`` timestamps the region boundaries so the report
    can say how many samples fell inside each region."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.rows, self.proc = [], None
        self.device_index = device_index
        self.nvml, self.handle, self.samples, self.stop_flag = None, None, [], False
        self.marks = {}
        self.started = False

    def mark(self, name: str) -> None:
        self.marks[name] = time.perf_counter()

    def _open_nvml(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = None
            try:
                uuid = str(torch.cuda.get_device_properties(self.device_index).uuid)
                handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                handle = pynvml.nvmlDeviceGetHandleByIndex(self.device_index)
            self.nvml, self.handle = pynvml, handle
            return True
        except Exception:
            self.nvml = None
            return False

    def _poll_nvml(self):
        nv, h = self.nvml, self.handle
        power, n = 0.0, 0
        while not self.stop_flag:
            try:
                sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                stamp = time.perf_counter()   # the clock is what the regions are judged by: stamped right after its read
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                if n % 8 == 0:               # the power query is the slow one: every eighth sample
                    power = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                n += 1
                self.samples.append((sm, reasons, power, stamp))
            except Exception:
                break
            time.sleep(0.0002)

    def start(self):
        self.started = True
        if self._open_nvml():
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.device_index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def _inside(self, begin: str, end: str):
        t0, t1 = self.marks.get(begin), self.marks.get(end)
        if t0 is None or t1 is None:
            return []
        return [x for x in self.samples if t0 <= x[3] <= t1]

    def stop(self):
        if self.nvml is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)
            nv = self.nvml
            try:
                mx = float(nv.nvmlDeviceGetMaxClockInfo(self.handle, nv.NVML_CLOCK_SM))
            except Exception:
                mx = None
            names = (("hw_slowdown", nv.nvmlClocksEventReasonHwSlowdown), ("hw_thermal_slowdown", nv.nvmlClocksEventReasonHwThermalSlowdown),
                     ("sw_thermal_slowdown", nv.nvmlClocksEventReasonSwThermalSlowdown), ("sw_power_cap", nv.nvmlClocksEventReasonSwPowerCap),
                     ("hw_power_brake_slowdown", nv.nvmlClocksEventReasonHwPowerBrakeSlowdown))
            timed = self._inside("timed_begin", "timed_end")
            sus = self._inside("sustained_begin", "sustained_end")
            load = timed + sus  # every sample taken while one of the two timed loops was running
            sm = [float(x[0]) for x in load]
            reasons = sorted({n for x in load for n, bit in names if x[1] & bit})
            out = {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "samples": len(sm),
                   "samples_in_timed_region": len(timed), "samples_in_sustained_loop": len(sus),
                   "power_w_max": round(max((x[2] for x in load), default=0.0), 1),
                   "power_w_median": round(statistics.median([x[2] for x in load]), 1) if load else None,
                   "source": "nvml (in-process, while the timed loops ran)", "reasons": reasons}
            out["note"] = ("sm_mhz is the median over both timed loops and is dominated by the seconds-long sustained loop at the "
                           "board's power cap; `value` comes from the short region whose median is sm_mhz_timed_region")
            if timed:
                out["sm_mhz_timed_region"] = statistics.median(float(x[0]) for x in timed)
            if sus:
                out["sm_mhz_sustained_loop"] = statistics.median(float(x[0]) for x in sus)
                out["sm_mhz_sustained_last_quarter"] = statistics.median(float(x[0]) for x in sus[-max(1, len(sus) // 4):])
            return out
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, idx in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > idx and r[idx].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "source": "nvidia-smi", "reasons": sorted(reasons)}


def make_layer_inputs(seed, kv_len, chunk, hq, hkv, device):
    """Seeded synthetic tensors of one layer: logical K/V [1,K,hkv,D], the chunk's Q, gate weights."""
    device = torch.device(device)
    g = torch.Generator(device=device).manual_seed(seed)
    past = kv_len - chunk
    k = torch.randn((1, kv_len, hkv, D), generator=g, dtype=torch.float32, device=device).to(torch.bfloat16)
    v = torch.randn((1, kv_len, hkv, D), generator=g, dtype=torch.float32, device=device).to(torch.bfloat16)
    q = torch.randn((1, chunk, hq, D), generator=g, dtype=torch.float32, device=device).to(torch.bfloat16)
    wq = (torch.randn((hq, D, 128), generator=g, device=device) * 0.02).to(torch.bfloat16)
    wk = (torch.randn((hkv, D, 128), generator=g, device=device) * 0.02).to(torch.bfloat16)
    perm = torch.randperm(kv_len // 64, generator=g, device=device).to(torch.int32).view(1, -1)
    # Per-head rank-1 bias so that the query heads of a group and the Q-blocks of a chunk agree on
    # which key blocks matter (the premise of Block-Union selection).  For each KV-head group a unit
    # direction g is chosen in the gate's slowly rotating RoPE channels (so it survives the block
    # RoPE for every Q-block of the chunk) such that the inputs that the random projections map onto
    # g are as small as possible; key block j carries importance a_j along that input direction and
    # every query token leans the same way.  Without it, independent per-row top-k selections of
    # random data union to ~100 % of the blocks.
    G = hq // hkv
    slow = torch.cat([torch.arange(45, 64), torch.arange(109, 128)]).to(device)
    inv_k = torch.linalg.inv(wk.double())  # input = g @ inv(W)
    inv_q = torch.linalg.inv(wq.double())
    x = torch.empty((hkv, 128), dtype=torch.float64, device=device)
    y = torch.empty((hq, 128), dtype=torch.float64, device=device)
    for h in range(hkv):
        mats = [inv_k[h]] + [inv_q[h * G + gi] for gi in range(G)]
        m = sum(a_[slow] @ a_[slow].T for a_ in mats)
        g_dir = torch.zeros(128, dtype=torch.float64, device=device)
        g_dir[slow] = torch.linalg.eigh(m).eigenvectors[:, 0]
        x[h] = g_dir @ inv_k[h]
        for gi in range(G):
            y[h * G + gi] = g_dir @ inv_q[h * G + gi]
    a = torch.rand((kv_len // BS, hkv), generator=g, device=device) ** 3
    k = (k.float() + a.repeat_interleave(BS, dim=0).view(1, kv_len, hkv, 1) * x.float().view(1, 1, hkv, 128)).to(torch.bfloat16)
    q = (q.float() + 1.5 * y.float().view(1, 1, hq, 128)).to(torch.bfloat16)
    return {"k": k, "v": v, "q": q, "wq": wq, "wk": wk, "perm": perm, "past": past, "q_lean": (1.5 * y.float()).to(torch.bfloat16)}


def block_rope_tables(n_blocks, block_size, device):
    inv = 1.0 / (500000.0 ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))
    pos = torch.arange(0, n_blocks * block_size, block_size, dtype=torch.float32)
    ang = torch.cat([pos.view(-1, 1) * inv.view(1, -1)] * 2, dim=-1)
    return ang.cos().unsqueeze(0).to(device), ang.sin().unsqueeze(0).to(device)


def percentile(values, q):
    """Nearest-rank percentile of a small sample (q in [0, 1])."""
    v = sorted(values)
    return v[min(len(v) - 1, max(0, int(math.ceil(q * len(v))) - 1))]


def run_native(args):
    from compactattention_b200 import _lib, ops, tp
    _lib.set_programmatic_launch(args.dependent_launch)
    from compactattention_b200.chunk_driver import GateSelectorState, SelectionRule
    from compactattention_b200.prefill_sparse.llama.modeling_llama_compactattn import (
        CompactAttnCache, CompactAttnLlamaConfig, LlamaSeerAttentionChunkedDense)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU path); use --impl reference for the CPU baseline")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group(backend="nccl", device_id=dev)
    try:
        shard = tp.HeadShard(world, rank, HQ, HKV)
    except ValueError as exc:
        raise SystemExit(str(exc))
    hkv, hq = len(shard.kv_heads), len(shard.q_heads)
    K, Q = args.kv_len, args.chunk
    Kb, Qb = K // BS, Q // BS
    Pb = Kb - Qb
    num, den = int(round(args.density * 1000)), 1000
    rule = SelectionRule(rule="topk", softmax=False, topk_ratio=(num, den), sink=1, local=2)
    cos, sin = block_rope_tables(Kb, BS, dev)
    hidden_size = HQ * D

    # The reference-facing plugin call of this workload is the attention module's forward (top-k
    # method): hidden states in, layer output out, projections included.  Its q projection carries
    # the per-head lean of the queries as a bias, so the module selects like the operator-level step.
    cfg = CompactAttnLlamaConfig(hidden_size=hidden_size, num_attention_heads=HQ, num_key_value_heads=HKV, head_dim=D,
                                 seerattn_gate_type="Qavg_Kavg", seerattn_gate_force_double=True, seerattn_gate_block_size=BS,
                                 seerattn_sparsity_method="topk", seerattn_topk_ratio=(num, den),
                                 seerattn_compactattn_keep_recent_blocks=2, max_position_embeddings=K, attention_bias=True,
                                 # e2e at N > 1: o_proj and its sum over the ranks through the fused kernels
                                 compactattn_fused_oproj_rows=Q if world in FUSED_PROJECTION_WORLDS else 0)
    inv = 1.0 / (500000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = torch.arange(K - Q, K, dtype=torch.float32).view(-1, 1) * inv.view(1, -1)
    ang = torch.cat([ang, ang], dim=-1)
    tok_rope = (ang.cos().unsqueeze(0).to(dev).to(torch.bfloat16), ang.sin().unsqueeze(0).to(dev).to(torch.bfloat16))

    # ---- resident state of `layers` independent layers (each rank: its own heads) ----
    layers = []
    for li in range(args.layers):
        t = make_layer_inputs(args.seed + 1000 * li + 17 * rank, K, Q, hq, hkv, dev)
        module = LlamaSeerAttentionChunkedDense(cfg, li, shard).to(dev).to(torch.bfloat16).eval()
        g = torch.Generator(device=dev).manual_seed(args.seed + 1000 * li + 17 * rank + 7)
        with torch.no_grad():
            module.attn_gate.mask_linear_q.weight.copy_(t["wq"])
            module.attn_gate.mask_linear_k.weight.copy_(t["wk"])
            for lin in (module.q_proj, module.k_proj, module.v_proj, module.o_proj):
                lin.weight.copy_(torch.randn(lin.weight.shape, generator=g, device=dev) * 0.02)
                if lin.bias is not None:
                    lin.bias.zero_()
            module.q_proj.bias.copy_(t["q_lean"].reshape(-1))
        pkv = CompactAttnCache(1, K, dev, torch.bfloat16, page_table=t["perm"])
        st = pkv.layer(li, hkv, D)
        st.kv.append(t["k"][:, : K - Q], t["v"][:, : K - Q], position=0)
        st.gate = GateSelectorState(module.attn_gate, 1, dev)
        st.gate.cache.reserve(Kb)
        module.attn_gate.append_key_blocks(st.gate.cache, t["k"][:, : K - Q], (cos[:, :Pb], sin[:, :Pb]))  # past blocks
        hidden = torch.randn((1, Q, hidden_size), generator=g, device=dev).to(torch.bfloat16)
        layers.append({
            "module": module, "pkv": pkv, "state": st, "cache": st.kv, "kv": st.kv.view(), "sel": st.gate,
            "q": t["q"], "k_chunk": t["k"][:, K - Q:].contiguous(), "v_chunk": t["v"][:, K - Q:].contiguous(),
            "hidden": hidden, "hidden_host": hidden.cpu().pin_memory(),
            "out": torch.empty((1, Q, hq, D), dtype=torch.bfloat16, device=dev),
            "table": ops.BlockTable(torch.empty((1, hkv, Pb), dtype=torch.int32, device=dev),
                                    torch.empty((1, hkv), dtype=torch.int32, device=dev),
                                    torch.empty((1, hkv), dtype=torch.int32, device=dev),
                                    torch.empty((1, hkv), dtype=torch.int32, device=dev)),
            "bits": torch.empty((1, hq, Qb, ops.words_for(Kb)), dtype=torch.int32, device=dev),
            "status": torch.zeros(1, dtype=torch.int32, device=dev),
        })
        st.kv.append(layers[-1]["k_chunk"], layers[-1]["v_chunk"], position=K - Q)
        del t
    reduce_buf = torch.zeros((1, Q, HQ * D), dtype=torch.bfloat16, device=dev) if world > 1 else None
    own_exchange, own_exchange_note = None, None
    if (world in OWN_ALL_REDUCE_WORLDS or (args.own_all_reduce and world > 1)) and not args.nccl_all_reduce:
        # Symmetric (peer-mapped) buffers are a collective allocation: every rank either gets them or none does.
        try:
            own_exchange = tp.shared_fused_projection(Q, HQ * D, dev, torch.bfloat16)   # the module's e2e path shares it
            ok = 1.0
        except Exception as exc:   # no peer access / no symmetric memory on this box: NCCL carries the collective
            own_exchange_note = f"symmetric memory unavailable ({type(exc).__name__}): NCCL used"
            ok = 0.0
        if tp.max_over_ranks([1.0 - ok], dev)[0] > 0.0:
            own_exchange = None
            own_exchange_note = own_exchange_note or "symmetric memory unavailable on another rank: NCCL used"
            cfg.compactattn_fused_oproj_rows = 0
    rope_chunk = (cos[:, Pb:], sin[:, Pb:])

    # ---- one step = one pass of the path for one chunk, as a list of stages (one or two launches each, the
    # attention stage two when it cuts work units) so the same code runs timed as a whole and stage by stage
    def stages(L):
        sel = L["sel"]

        def prepare():
            sel.cache.length = Pb  # the chunk's blocks are (re)appended at the end of the past blocks
            sel.append(L["q"], L["k_chunk"], rope_chunk, rope_chunk)

        def select():
            return ops.select_union_table(sel.logits, Pb, rule.rule, num_kv_heads=hkv, block_size=BS, softmax=rule.softmax,
                                          topk_ratio=rule.topk_ratio, sink=rule.sink, local=rule.local, out=L["table"])

        def attention():
            ops.attn_compact(L["q"], L["kv"], K, hkv, L["table"].block_idx, L["table"].counts, block_size=BS, out=L["out"],
                             status=L["status"])

        def score_select():
            return sel.score_select(rule, hkv, BS, table=L["table"])

        if args.two_launch_selection:
            out = [("gate_prepare", prepare), ("gate_scores", sel.score), ("select_union_table", select), ("attention", attention)]
        else:   # scores, row rule, Block-Union and table behind one library call (two launches)
            out = [("gate_prepare", prepare), ("gate_score_select", score_select), ("attention", attention)]
        if world > 1:
            if own_exchange is not None:   # the library's own all-reduce over peer memory (ca_oproj_allreduce without the GEMM)
                out.append(("all_reduce", lambda: own_exchange.all_reduce(reduce_buf)))
            else:
                out.append(("all_reduce", lambda: tp.reduce_layer_output(reduce_buf)))
        return out

    def step(L, attn_events=None, fresh=False):
        """One step.  The library calls of a stage are re-issued from the call list recorded for this layer state
        (same entry points, same parameter blocks: a host that keeps its parameter blocks between chunks, as
        `GateLayerStep` does); the collective is issued afresh."""
        recorded = None if fresh else L.get("calls")   # the kept blocks carry the stream they were recorded on
        for name, fn in (recorded if recorded is not None else stages(L)):
            run = fn.run if isinstance(fn, _lib.CallList) else fn
            if name == "attention" and attn_events is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                run()
                e1.record()
                attn_events.append((e0, e1))
            else:
                run()

    def record_calls(L):
        """Runs every stage of `L` once and keeps its library calls; the collective stays a Python call."""
        kept = []
        for name, fn in stages(L):
            if name == "all_reduce":
                kept.append((name, fn))
                continue
            with _lib.record() as calls:
                fn()
            kept.append((name, calls))
        L["calls"] = kept

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max_ranks(vals):
        return tp.max_over_ranks(vals, dev)

    if not args.no_call_lists:
        for L in layers:
            record_calls(L)
    for i in range(max(args.warmup, 3)):
        step(layers[i % len(layers)])
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # ---- the timed region: exactly `steps` steps, an event after every step ----
    attn_events = []
    launches0 = _lib.launch_count()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    sampler.mark("timed_begin")
    marks[0].record()
    for i in range(args.steps):
        step(layers[i % len(layers)], attn_events)
        marks[i + 1].record()
    barrier()
    sampler.mark("timed_end")
    launches = _lib.launch_count() - launches0
    ms_total = marks[0].elapsed_time(marks[-1])
    per_step_us = [marks[i].elapsed_time(marks[i + 1]) * 1e3 for i in range(args.steps)]
    attn_us = [a.elapsed_time(b) * 1e3 for a, b in attn_events]
    ms_total, attn_ms = max_ranks([ms_total, statistics.mean(attn_us) * 1e-3])
    ms_per_step = ms_total / args.steps
    step_stats = {"mean": ms_per_step * 1e3, "median": statistics.median(per_step_us), "p10": percentile(per_step_us, 0.1),
                  "p90": percentile(per_step_us, 0.9), "min": min(per_step_us), "max": max(per_step_us)}
    attn_stats = {"mean": attn_ms * 1e3, "median": statistics.median(attn_us), "p10": percentile(attn_us, 0.1),
                  "p90": percentile(attn_us, 0.9)}

    # ---- dense comparator: same shape, same kernel, every past block ----
    dense_us = None
    if not args.no_dense:
        L = layers[0]
        for _ in range(2):
            ops.attn_compact(L["q"], L["kv"], K, hkv, None, None, block_size=BS, out=L["out"])
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        d0.record()
        for i in range(5):
            LL = layers[i % len(layers)]
            ops.attn_compact(LL["q"], LL["kv"], K, hkv, None, None, block_size=BS, out=LL["out"])
        d1.record()
        barrier()
        dense_us = max_ranks([d0.elapsed_time(d1) / 5 * 1e3])[0]

    # ---- the reference's own GPU routes on the same GPU (library calls, timing only, rank 0) ----
    ref_gpu = {}
    if not args.no_dense and rank == 0:
        ref_gpu = time_reference_gpu_routes(layers[0], K, Q, hq, hkv, dev)
    # ---- the path's other selectors at the same shape (informational; the headline is the learned gate with top-k):
    # the learned gate with the reference's default rule (softmax + threshold), and the training-free selector
    # (mean-K block score at block 128 + alpha * row-max rule with sink and window), selector launches only ----
    other_selectors = {}
    if not args.no_dense and rank == 0:
        other_selectors = time_other_selectors(layers[0], K, Q, hq, hkv, dev)
    if world > 1:
        barrier()

    # ---- per-stage split: events between the launches of a step (a separate loop; the events cost a
    # little, so its sum is not the value) ----
    names = [n for n, _ in stages(layers[0])]
    acc = {n: [] for n in names}
    barrier()
    rounds = []
    for i in range(max(8, min(args.steps, 40))):
        # no synchronisation inside the loop: while one step's attention runs, the host enqueues the next
        # step's launches and events, so a stage's time is its time on the device, not the host's
        evs = [torch.cuda.Event(enable_timing=True)]
        evs[0].record()
        for name, fn in stages(layers[i % len(layers)]):
            fn()
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            evs.append(e)
        rounds.append(evs)
    torch.cuda.current_stream().synchronize()
    for evs in rounds[2:]:
        for j, name in enumerate(names):
            acc[name].append(evs[j].elapsed_time(evs[j + 1]) * 1e3)
    stage_vals = max_ranks([statistics.median(acc[n]) for n in names])
    stage_us = {n: round(v, 1) for n, v in zip(names, stage_vals)}
    launches_attention = _lib.launch_count()
    dict(stages(layers[0]))["attention"]()
    launches_attention = _lib.launch_count() - launches_attention
    stage_us["attention_launches"] = launches_attention  # 2: the merge of cut work units ran inside the attention stage

    # ---- sustained phase: the same loop repeated until >= 1 s has elapsed (the board reaches its
    # power cap and the SM clock settles), clocks sampled throughout ----
    sustained = None
    if not args.no_sustained:
        s_attn, n_sus = [], 0
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        sampler.mark("sustained_begin")
        w0 = time.perf_counter()
        s0.record()
        while True:
            for i in range(args.steps):
                step(layers[i % len(layers)], s_attn)
            n_sus += args.steps
            torch.cuda.current_stream().synchronize()
            go = 1.0 if time.perf_counter() - w0 < args.sustained_seconds else 0.0
            if max_ranks([go])[0] == 0.0 or n_sus >= 100000:  # every rank leaves the loop in the same round
                break
        s1.record()
        barrier()
        sampler.mark("sustained_end")
        sus_ms, sus_attn = max_ranks([s0.elapsed_time(s1) / n_sus, statistics.mean(a.elapsed_time(b) for a, b in s_attn[-200:])])
        sustained = {"steps": n_sus, "step_us": round(sus_ms * 1e3, 1), "attention_us": round(sus_attn * 1e3, 1)}
    clocks = sampler.stop() if rank == 0 else None
    status = max(int(L["status"].item()) for L in layers)

    # ---- algorithmic work of one attention launch (this rank) ----
    G = hq // hkv
    counts = torch.stack([L["table"].counts.reshape(-1) for L in layers]).float().mean(0).cpu()
    sel_blocks = float(counts.sum())
    flops = 4.0 * D * G * (Q * sel_blocks * BS + hkv * Q * (Q + 1) / 2.0)
    kv_bytes = 2.0 * D * 2 * (sel_blocks * BS + hkv * Q) + 2.0 * Q * hq * D * 2
    peaks = load_peaks()
    capture = load_attention_capture()
    achieved = flops / (attn_ms * 1e-3) / 1e12
    # the slower of tensor time and HBM time bounds the launch; here it is the tensor pipe
    t_tensor = flops / (peaks["bf16_tflops"] * 1e12)
    t_hbm = kv_bytes / (peaks["hbm_gbs"] * 1e9)
    roofline = {
        "bound": "tensor" if t_tensor >= t_hbm else "hbm",
        "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
        "frac": round(achieved / peaks["bf16_tflops"], 4), "peak_source": f"{peaks['source']} (cuBLAS bf16 burst; the timed region is short)",
        "traffic": None if capture is None else round(capture["dram_bytes"] * kv_bytes / capture["algorithmic_bytes"]),
        "kernel": "attn_compact_kernel", "kernel_us": round(attn_ms * 1e3, 1),
        "algorithmic_flops": flops, "algorithmic_bytes": kv_bytes,
        "roofline_us": round(max(t_tensor, t_hbm) * 1e6, 1),
        "path_frac_of_roofline": round(max(t_tensor, t_hbm) * 1e3 / ms_per_step, 4),
    }
    if sustained is not None and peaks.get("bf16_tflops_sustained"):
        # the seconds-long loop against the seconds-long cuBLAS figure
        sus_tf = flops / (sustained["attention_us"] * 1e-6) / 1e12
        sustained["attention_tflops"] = round(sus_tf, 1)
        sustained["frac_of_sustained_peak"] = round(sus_tf / peaks["bf16_tflops_sustained"], 4)
        roofline["sustained"] = sustained

    # ---- end to end through the plugin call (the attention module's forward) with host buffers:
    # hidden states from pinned host memory, layer output back to pinned host memory, every step ----
    host_out = torch.empty((1, Q, hidden_size), dtype=torch.bfloat16).pin_memory()

    def e2e_step(L):
        st = L["state"]
        st.kv.length = K - Q        # the chunk is appended again at the end of the past tokens
        st.gate.cache.length = Pb
        x = L["hidden"].copy_(L["hidden_host"], non_blocking=True)
        with torch.no_grad():
            y = L["module"](x, tok_rope, None, past_key_value=L["pkv"], block_position_embeddings=rope_chunk)[0]
        host_out.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(3):
        e2e_step(layers[i % len(layers)])
    barrier()
    n_e2e = max(5, min(args.steps, 40))
    e2e_each = []
    w_all = time.perf_counter()
    for i in range(n_e2e):
        w0 = time.perf_counter()
        e2e_step(layers[i % len(layers)])
        e2e_each.append((time.perf_counter() - w0) * 1e6)
    e2e_mean_local = (time.perf_counter() - w_all) / n_e2e * 1e6
    barrier()
    e2e_us, e2e_med = max_ranks([e2e_mean_local, statistics.median(e2e_each)])
    # the module's device time alone (CUDA events, inputs resident): what the plugin call costs on the GPU
    m0, m1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    m0.record()
    for i in range(n_e2e):
        L = layers[i % len(layers)]
        L["state"].kv.length, L["state"].gate.cache.length = K - Q, Pb
        with torch.no_grad():
            L["module"](L["hidden"], tok_rope, None, past_key_value=L["pkv"], block_position_embeddings=rope_chunk)
    m1.record()
    barrier()
    module_us = max_ranks([m0.elapsed_time(m1) / n_e2e * 1e3])[0]

    # ---- the same step replayed from CUDA graphs (informational, last of all so that a failed
    # capture cannot touch a required number; `value` stays the eager loop) ----
    graph_us = None
    if world == 1 and not args.no_graph:
        try:
            from compactattention_b200.chunk_driver import capture_step
            graphs = [capture_step(lambda L=L: step(L, fresh=True)) for L in layers]
            for i in range(4):
                graphs[i % len(graphs)].replay()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            g0.record()
            for i in range(args.steps):
                graphs[i % len(graphs)].replay()
            g1.record()
            torch.cuda.synchronize()
            graph_us = g0.elapsed_time(g1) / args.steps * 1e3
            del graphs
        except Exception as exc:  # graph capture is optional evidence, never the measured path
            graph_us = None
            print(f"[bench] graph replay not timed: {exc!r}", file=sys.stderr)

    h2d = Q * hidden_size * 2
    d2h = Q * hidden_size * 2

    if rank != 0:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()
        return
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(args, sample_heads=1)
    value_us = ms_per_step * 1e3
    sm_mhz = (clocks or {}).get("sm_mhz")
    line = {
        "metric": METRIC, "value": round(value_us, 1), "unit": "us", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4), "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "workload": f"config 3: 1 layer, {HQ}q/{HKV}kv heads d{D}, chunk {Q} at the end of a {K}-token paged KV cache "
                        f"(page 64, permuted), block {BS}, learned-gate selector (128->128, random init) + per-row top-k "
                        f"{args.density:.0%} + sink 1 + local 2",
            "kv_len": K, "chunk": Q, "density_target": args.density,
            "selected_past_blocks_per_kv_head": round(sel_blocks / hkv, 1), "past_blocks": Pb,
            "parallelism": f"tp{world} (KV-head sharded)" if world > 1 else "single GPU",
            "layer_output_all_reduce": (None if world == 1 else
                                        ("library exchange over peer memory (ca_oproj_allreduce without the GEMM)"
                                         if own_exchange is not None else (own_exchange_note or "NCCL"))),
            "l2": f"steps rotate over {len(layers)} layer states ({len(layers) * 2 * K * hkv * D * 2 / 2**30:.1f} GiB of KV), more than L2",
            "launches_per_step": launches / args.steps,
            "programmatic_dependent_launch": args.dependent_launch,
            "host_side": ("library calls re-issued from parameter blocks kept per layer state" if not args.no_call_lists
                          else "parameter blocks filled afresh every step by the tensor-level wrappers"),
            "step_us": {k: round(v, 1) for k, v in step_stats.items()},
            "attention_us": {k: round(v, 1) for k, v in attn_stats.items()},
            "stage_us": stage_us,
            "attention_kernel_cycles_at_median_clock": None if not sm_mhz else round(attn_ms * 1e3 * sm_mhz),
            "step_replayed_from_cuda_graph_us": None if graph_us is None else round(graph_us, 1),
            "dense_same_shape_us": None if dense_us is None else round(dense_us, 1),
            "speedup_vs_dense": None if dense_us is None else round(dense_us / value_us, 2),
            "reference_gpu_routes_us": ref_gpu,
            "other_selectors_us": other_selectors,
            "attention_effective_tflops": round(achieved, 1),
            "e2e_call": "LlamaSeerAttentionChunkedDense.forward (top-k method): hidden states from pinned host memory, "
                        "q/k/v projections, RoPE + paged append, gate, rule, table, attention, o_proj"
                        + (", all-reduce" if world > 1 else "") + ", output to pinned host memory",
            "e2e_median_us": round(e2e_med, 1), "module_forward_device_us": round(module_us, 1),
            "status_word": status,
        },
        "roofline": roofline,
        "cpu_baseline": cpu,
        "e2e": {"value": round(e2e_us, 1), "unit": "us", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def load_attention_capture():
    """DRAM bytes of one attention launch from the committed ncu capture (a small JSON beside the
    profile summaries: measured read + write bytes and the algorithmic bytes of the captured launch).
    K/V traffic is proportional to the selected blocks, so the benchmark's launch is scaled by its own
    algorithmic bytes.  None when the file is absent."""
    path = ROOT / "profiles" / "attn_compact_kernel_capture.json"
    if not path.exists():
        return None
    d = json.loads(path.read_text())
    return {"dram_bytes": float(d["dram_bytes"]), "algorithmic_bytes": float(d["algorithmic_bytes"])}


def time_other_selectors(L, K, Q, hq, hkv, dev, reps=10):
    """Selector launches of the two routes the benchmark's headline does not take, on the same shape: device time
    per chunk (CUDA events over `reps` chunks behind a device spin, so the host's enqueue rate is not timed).
      gate_softmax_threshold   gate scores -> softmax + threshold 5e-4 + keep_recent 2 -> union + table
                               (compact_attn/modules/attention_forward_chunked_dense.py:352-403, the reference's default)
      flashprefill_block128    mean-K block score (block 128; its normalisation is folded into the rule's row load) ->
                               alpha 0.06 * row-max, sink 2, window 4 -> union + table (compact_attn/modules/flashprefill_prefill.py:307-376, 596-666)
    """
    import torch
    from compactattention_b200 import ops
    out = {}

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(int(2e6))
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return round(e0.elapsed_time(e1) / reps * 1e3, 1)

    try:
        sel = L["sel"]
        kb = sel.cache.blocks()
        Kb, Qb = kb.shape[1], sel.q_blocks.shape[1]
        logits = torch.empty((1, hq, Qb, Kb), dtype=torch.float32, device=dev)
        out["gate_softmax_threshold"] = {
            "scores_rule_table": timed(lambda: ops.gate_score_select(sel.q_blocks, kb, Kb - Qb, "threshold", num_kv_heads=hkv, scores=logits,
                                                                     scale=sel.gate.scale, block_size=64, softmax=True, threshold=5e-4,
                                                                     keep_recent=2))}
    except Exception as exc:  # informational: never fails the benchmark
        out["gate_softmax_threshold"] = {"error": repr(exc)[:200]}
    try:
        bs = 128
        g = torch.Generator(device=dev).manual_seed(11)
        mean_k = torch.randn((1, K // bs, hkv, 128), device=dev, generator=g).to(torch.bfloat16)
        q = L["q"]
        state = {}

        def score():   # score_raw and max_raw; the rule forms score_raw * 2^(max_raw - row max) itself: no normalisation launch
            state["raw"], state["mx"], _ = ops.flashprefill_score(q, mean_k, K, bs, normalize=False)

        def rule_table():
            s = state["raw"].permute(0, 3, 1, 2)   # [B, Hq, Qb, Kb] view of [B, Qb, Kb, Hq]
            ops.select_union_table(s, (K - Q) // bs, "alpha_rowmax", num_kv_heads=hkv, block_size=bs, alpha=0.06, sink=2, local=4,
                                   score_max=state["mx"].permute(0, 3, 1, 2))

        score()
        out["flashprefill_block128"] = {"score": timed(score), "rule_table": timed(rule_table)}
    except Exception as exc:
        out["flashprefill_block128"] = {"error": repr(exc)[:200]}
    return out


def time_reference_gpu_routes(L, K, Q, hq, hkv, dev, reps=3):
    """Times, on the block table this library built, the library calls the reference's compact routes
    bottom out in, plus its dense comparator.  These libraries are parts of the image, not of this
    repository; they are only timed here (and their outputs compared with this library's at the
    path's tolerance), never used by the path.  Returns {route: {"us": .., "max_abs_vs_ours": ..} |
    {"error": text}}.
      dense_flash_attn2       flash_attn_func(causal=True)  (compact_attn/modules/dense_prefill.py:304-310)
      fa2_paged               flash_attn_with_kvcache over the compact cache this library's gather fills
                              (compact_attn/kernels/varlen/indexed_dense_prefill_varlen.py:1563-1571)
      fi_zero_copy            FlashInfer BatchPrefillWithPagedKVCacheWrapper.plan/run over the selected page ids,
                              one pseudo-batch row per KV head (.../flashinfer_zero_copy_prefill.py:1284-1320)
      cudnn_one_shot          flashinfer.cudnn_batch_prefill_with_kv_cache (same file, :1503-1540)
    """
    from compactattention_b200 import ops
    G = hq // hkv
    Kb, Qb = K // BS, Q // BS
    Pb = Kb - Qb
    q, table = L["q"], L["table"]
    cache = L["cache"]
    ours = ops.attn_compact(q, L["kv"], K, hkv, table.block_idx, table.counts, block_size=BS).float()
    results = {}

    def timed(fn):
        for _ in range(2):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            out = fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3, out

    def compare(out_bqhd):
        err = (out_bqhd.float() - ours).abs()
        return {"max_abs_vs_ours": round(err.max().item(), 5), "mean_abs_vs_ours": round(err.mean().item(), 6)}

    def attempt(name, fn):
        try:
            results[name] = fn()
        except Exception as exc:  # an absent library, an unsupported device or build: recorded, not fatal
            results[name] = {"error": f"{type(exc).__name__}: {str(exc)[:300]}"}
            print(f"[bench] reference route {name} not timed: {exc!r}", file=sys.stderr)

    # logical (un-permuted) copies of the layer's K and V, as the reference holds them
    ids = cache.page_table[0].to(torch.long)
    k_log = cache.k_pages[ids].reshape(1, K, hkv, D)
    v_log = cache.v_pages[ids].reshape(1, K, hkv, D)
    q_group = q.view(1, Q, hkv, G, D).permute(0, 2, 1, 3, 4).reshape(hkv, Q, G, D).contiguous()

    def ungroup(o):  # [R, Q, G, D] -> [1, Q, Hq, D]
        return o.view(1, hkv, Q, G, D).permute(0, 2, 1, 3, 4).reshape(1, Q, hq, D)

    def dense_fa2():
        from flash_attn import flash_attn_func
        us, _ = timed(lambda: flash_attn_func(q, k_log, v_log, causal=True))
        return {"us": round(us, 1)}

    def fa2_paged():
        from flash_attn import flash_attn_with_kvcache
        offs, block_table = ops.paged_metadata(table.pages_per_row, max_pages=(Kb * BS + 255) // 256)
        total_pages = hkv * ((Kb * BS + 255) // 256)
        kc = torch.zeros((total_pages, 256, 1, D), dtype=q.dtype, device=dev)
        vc = torch.zeros_like(kc)
        kv = L["kv"]

        def fill():
            ops.gather_kv(kv, hkv, 1, Q, K, table.block_idx, table.counts, kc, vc, block_size=BS, page_offsets=offs,
                          dst_page_size=256)

        fill_us, _ = timed(fill)
        seqlens = table.cache_seqlens.view(-1).contiguous()
        attn_us, out = timed(lambda: flash_attn_with_kvcache(q=q_group, k_cache=kc, v_cache=vc, cache_seqlens=seqlens,
                                                             block_table=block_table, softmax_scale=D ** -0.5, causal=True))
        return {"us": round(fill_us + attn_us, 1), "cache_fill_us": round(fill_us, 1), "attention_us": round(attn_us, 1),
                **compare(ungroup(out))}

    def zero_copy_metadata():
        # CSR over the selected blocks of every KV-head row followed by the chunk's own blocks; a page id
        # is row * Kb + block in the heads-first view [Hkv * Kb, 64, 1, D]
        counts = table.counts.view(-1).to(torch.long)
        n = counts + Qb
        indptr = torch.zeros(hkv + 1, dtype=torch.int32, device=dev)
        indptr[1:] = torch.cumsum(n, 0).to(torch.int32)
        rows = []
        for r in range(hkv):
            c = int(counts[r])
            rows.append(torch.cat([table.block_idx.view(hkv, -1)[r, :c].to(torch.int32),
                                   torch.arange(Pb, Kb, dtype=torch.int32, device=dev)]) + r * Kb)
        indices = torch.cat(rows).contiguous()
        last = torch.full((hkv,), BS, dtype=torch.int32, device=dev)
        qo = torch.arange(0, (hkv + 1) * Q, Q, dtype=torch.int32, device=dev)
        k_hf = k_log.permute(0, 2, 1, 3).contiguous().view(hkv * Kb, BS, 1, D)
        v_hf = v_log.permute(0, 2, 1, 3).contiguous().view(hkv * Kb, BS, 1, D)
        return indptr, indices, last, qo, k_hf, v_hf

    def fi_zero_copy():
        import flashinfer
        indptr, indices, last, qo, k_hf, v_hf = zero_copy_metadata()
        ws = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
        wrapper = flashinfer.BatchPrefillWithPagedKVCacheWrapper(ws, "NHD")
        q_fi = q_group.reshape(hkv * Q, G, D)

        def plan():
            wrapper.plan(qo_indptr=qo, paged_kv_indptr=indptr, paged_kv_indices=indices, paged_kv_last_page_len=last,
                         num_qo_heads=G, num_kv_heads=1, head_dim_qk=D, page_size=BS, causal=True, sm_scale=D ** -0.5,
                         q_data_type=q.dtype)

        plan()
        w0 = time.perf_counter()
        for _ in range(reps):
            plan()
        torch.cuda.synchronize()
        plan_us = (time.perf_counter() - w0) / reps * 1e6
        run_us, out = timed(lambda: wrapper.run(q_fi, (k_hf, v_hf)))
        return {"us": round(plan_us + run_us, 1), "plan_host_us": round(plan_us, 1), "run_us": round(run_us, 1),
                **compare(ungroup(out.view(hkv, Q, G, D)))}

    def cudnn_one_shot():
        from flashinfer.prefill import cudnn_batch_prefill_with_kv_cache as fn
        indptr, indices, last, qo, k_hf, v_hf = zero_copy_metadata()
        n = (indptr[1:] - indptr[:-1]).to(torch.int32)
        max_pages = int(n.max())
        block_tables = torch.zeros((hkv, max_pages), dtype=torch.int32, device=dev)
        for r in range(hkv):
            block_tables[r, : int(n[r])] = indices[int(indptr[r]): int(indptr[r + 1])]
        q_fi = q_group.reshape(hkv * Q, G, D)
        ws = torch.empty(128 * 1024 * 1024, dtype=torch.uint8, device=dev)
        seq_q = torch.full((hkv, 1, 1, 1), Q, dtype=torch.int32, device=dev)
        seq_kv = (n * BS).view(hkv, 1, 1, 1).to(torch.int32)
        # this entry point takes pages as [pages, 1, 64, D] (the same memory) and element offsets of each row's queries
        k_c, v_c = k_hf.view(hkv * Kb, 1, BS, D), v_hf.view(hkv * Kb, 1, BS, D)
        offs = (qo * (G * D)).contiguous()

        def run():
            return fn(q_fi, k_c, v_c, D ** -0.5, ws, max_token_per_sequence=Q, max_sequence_kv=max_pages * BS,
                      actual_seq_lens_q=seq_q, actual_seq_lens_kv=seq_kv, block_tables=block_tables, causal=True,
                      return_lse=True, batch_offsets_q=offs, batch_offsets_o=offs, is_cuda_graph_compatible=False)

        us, out = timed(run)
        out = out[0] if isinstance(out, (tuple, list)) else out
        return {"us": round(us, 1), **compare(ungroup(out.view(hkv, Q, G, D)))}

    attempt("dense_flash_attn2", dense_fa2)
    attempt("fa2_paged", fa2_paged)
    attempt("fi_zero_copy", fi_zero_copy)
    attempt("cudnn_one_shot", cudnn_one_shot)
    return results


def cpu_path_once(q, k, v, wq, wk, cos, sin, num, den, G):
    """The reference's CPU path (oracle port) for the given heads: gate scores, top-k rows, union,
    block table, gather, attention over the gathered KV."""
    from oracle import compact_oracle as co
    Q, K = q.shape[1], k.shape[1]
    Qb, Kb = Q // BS, K // BS
    Pb = Kb - Qb
    qb = co.apply_block_rope(co.multi_head_linear(co.pool_blocks(q.float(), BS, ("avg",)), wq.float()), cos[:, Pb:], sin[:, Pb:])
    kb = co.apply_block_rope(co.multi_head_linear(co.pool_blocks(k.float(), BS, ("avg",)), wk.float()), cos, sin)
    mask = co.gate_block_causal_mask(Q, K, BS)
    logits = co.gate_score(qb, kb, mask, use_softmax=False)
    valid = mask.expand_as(logits)
    n_valid = Pb + torch.arange(Qb) + 1
    kk = torch.minimum(torch.clamp((num * n_valid + den // 2) // den, min=1), n_valid)
    keep = co.topk_rows(logits, valid, kk) | (co.forced_mask(Qb, Kb, Pb, 1, 2) & valid)
    keep_block = keep.any(dim=2)
    idx, counts = co.block_union_table(keep_block, Q, K, BS, G)
    co.gather_compact_kv(k, v, idx, counts, Q, BS)
    return co.compact_attention(q, k, v, idx, counts, BS)


def cpu_baseline(args, sample_heads=1, runs=1):
    """Times the CPU path on `sample_heads` of the 8 KV heads (with their query heads) at the full
    context, all host threads, and scales to the full layer (heads are independent)."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    K, Q = args.kv_len, args.chunk
    G = HQ // HKV
    t = make_layer_inputs(args.seed, K, Q, G * sample_heads, sample_heads, "cpu")
    cos, sin = block_rope_tables(K // BS, BS, "cpu")
    num, den = int(round(args.density * 1000)), 1000
    best = None
    for _ in range(runs):
        w0 = time.perf_counter()
        cpu_path_once(t["q"], t["k"], t["v"], t["wq"], t["wk"], cos, sin, num, den, G)
        dt = time.perf_counter() - w0
        best = dt if best is None else min(best, dt)
    return {"value": round(best * (HKV / sample_heads) * 1e6, 1), "unit": "us", "cores": cores, "kind": "port",
            "sample": f"{sample_heads} of {HKV} KV heads (with their {G} query heads each) at the full {K}-token context, "
                      f"measured {best:.2f} s, scaled x{HKV // sample_heads} (heads are independent)"}


def run_reference(args):
    """Reference arm: the CPU restatement of the reference's path on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 3))
    vals = []
    cpu = None
    for _ in range(min(args.warmup, 1)):
        cpu_baseline(args, sample_heads=1)
    for _ in range(steps):
        cpu = cpu_baseline(args, sample_heads=1)
        vals.append(cpu["value"])
    value = statistics.mean(vals)
    cpu["value"] = round(value, 1)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 1), "unit": "us",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps, "warmup": min(args.warmup, 1),
        "ms_per_step": round(value / 1e3, 3), "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"config 3 on the host CPU: chunk {args.chunk} at the end of a {args.kv_len}-token cache, "
                               f"top-k {args.density:.0%}; {cpu['sample']}"},
        "cpu_baseline": cpu,
        "e2e": {"value": round(value, 1), "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# world sizes at which the fused output projection measured faster than a library GEMM + NCCL all-reduce
FUSED_PROJECTION_WORLDS = (2, 8)
# world sizes at which the library's own exchange measured faster than NCCL's all-reduce of the layer output
OWN_ALL_REDUCE_WORLDS = (2, 4, 8)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
