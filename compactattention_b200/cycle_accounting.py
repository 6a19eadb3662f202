"""Per-role cycle accounting of the attention kernel (development tool, needs a B200).

Builds the library with ``-DCA_ATTN_PROFILE=1`` into a separate ``.so``, runs the kernel on the
benchmark's attention shape (chunk 1024 at the end of a 131072-token cache, 32 query / 8 KV heads, 20 % of the past blocks, whole work units per CTA) and prints, for a
few CTAs, the clock cycles per 128-token KV step that each role spent between its marks:

* MMA issuer: issuing (which includes being held by the tensor pipe's queue), and the waits for the
  V tile, the pieces of P of tile A, the K tile, the pieces of P of tile B;
* softmax warpgroups: waiting for S, loading S from TMEM, row max + rescale decision,
  exponentials + P store, epilogue.

Each mark costs about 90 cycles of its own, so the buckets that show ~90 are empty waits.

    python -m compactattention_b200.cycle_accounting [--density 0.2]
"""
from __future__ import annotations

import argparse
import ctypes
from pathlib import Path

import numpy as np
import torch

from . import _lib, build

MMA_BUCKETS = ["issue", "wait V", "wait pA0", "wait pA1", "wait K", "wait pB0", "wait pB1", "segment end"]
SOFTMAX_BUCKETS = ["loop", "wait S", "load S", "row max", "exp + store P", "epilogue"]


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--density", type=float, default=0.2)
    ap.add_argument("--kv-len", type=int, default=131072)
    ap.add_argument("--launches", type=int, default=50)
    ap.add_argument("--kv-heads", type=int, default=8, help="KV heads (4 query heads each); 1 = one rank of TP8")
    ap.add_argument("--cut", action="store_true", help="let the launch cut work units across SMs (default: whole units)")
    args = ap.parse_args()

    defines = ["CA_ATTN_PROFILE=1"]
    lib_path = build.PKG_DIR / "libcompactattn_b200_profile.so"
    build.build_variant(defines, lib_path)
    _lib.LIB_PATH = Path(lib_path)   # must happen before the first ops call loads the library
    from . import ops

    torch.manual_seed(1)
    B, Q, Hkv, K, bs, D = 1, 1024, args.kv_heads, args.kv_len, 64, 128
    Hq = 4 * Hkv
    q = torch.randn(B, Q, Hq, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, K, Hkv, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, K, Hkv, D, device="cuda", dtype=torch.bfloat16)
    Pb = (K - Q) // bs
    n = int(Pb * args.density)
    idx = torch.stack([torch.randperm(Pb, device="cuda")[:n].sort().values for _ in range(Hkv)]).int().contiguous()
    counts = torch.full((Hkv,), n, dtype=torch.int32, device="cuda")
    kv = ops.KvCacheView.from_seq_first(k, v)
    out = torch.empty_like(q)
    for _ in range(args.launches):
        ops.attn_compact(q, kv, K, Hkv, idx, counts, out=out, use_workspace=args.cut)
    torch.cuda.synchronize()

    raw = (ctypes.c_longlong * (160 * 32))()
    rc = ctypes.CDLL(str(lib_path)).ca_debug_attn_profile(raw)
    if rc != 0:
        raise RuntimeError(f"ca_debug_attn_profile failed ({rc})")
    prof = np.frombuffer(raw, dtype=np.int64).reshape(160, 32)
    # KV steps of one work unit: selected blocks in pairs + the chunk's blocks up to the pair's diagonal
    steps = (n * bs + Q // 2 + 127) // 128
    if args.cut:
        steps = max(1, steps * Hkv * 16 // 148)   # 16 tile pairs per KV head, laid end to end over 148 CTAs
    print(f"defines: {' '.join(defines)}; {n} of {Pb} past blocks per KV head; ~{steps} KV steps per CTA")
    print(f"whole kernel per CTA (cycles): median {int(np.median(prof[:148, 31]))}, max {int(prof[:148, 31].max())}; "
          f"prologue median {int(np.median(prof[:148, 30]))}")
    for cta in (0, 1, 64, 127):
        print(f"CTA {cta}: cycles per KV step")
        mma = prof[cta, :8] / steps
        print("  MMA issuer: " + ", ".join(f"{nm} {x:.0f}" for nm, x in zip(MMA_BUCKETS, mma)) + f" | total {mma.sum():.0f}")
        for t in range(2):
            sm = prof[cta, 10 + 10 * t: 16 + 10 * t] / steps
            print(f"  softmax {'AB'[t]}: " + ", ".join(f"{nm} {x:.0f}" for nm, x in zip(SOFTMAX_BUCKETS, sm)) + f" | total {sm.sum():.0f}")


if __name__ == "__main__":
    main()
