"""Builds and runs the three tcgen05 micro-benchmarks behind the attention kernel's design notes
(development tools, need a B200; nothing in the library uses them):

    python -m compactattention_b200.microbench mma_rate    # cycles per tcgen05.mma, shapes and operand sources
    python -m compactattention_b200.microbench handoff     # MMA commit -> waiting warps -> issuer round trip
    python -m compactattention_b200.microbench chain       # S -> softmax -> P -> P.V dependency chain of one tile

* ``mma_rate.cu``: one thread of one CTA per SM issues 8192 MMAs back to back (operands are zeros):
  128x128x16 with both operands in shared memory, with A in tensor memory, alternating groups as the
  attention loop issues them, 128x256x16, and 128x64x16 / 128x32x16 (``MMA_N``).
* ``handoff.cu``: an issuer thread issues n MMAs and commits to an mbarrier, 128 worker threads wait
  on it and arrive on a second mbarrier the issuer waits on: the fixed latency of one S -> P hand-off.
* ``chain.cu``: the attention kernel's per-tile loop in isolation (S = Q.K^T, softmax of a 128-column
  row per thread, P back to tensor memory in two pieces, O += P.V, next S): cycles per KV step for the
  kernel's softmax and for variants (chunked load, two warpgroups per tile, polynomial exp2).
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
RUNS = {
    "mma_rate": [["0"], ["1"], ["2"], ["3"], ["0", "8192", "0", "16"], ("MMA_N=64", ["0"]), ("MMA_N=32", ["0"])],
    "handoff": [["0", "2000", "8"], ["1", "2000", "8"], ["2", "2000", "8"], ["0", "2000", "1"], ["0", "2000", "16"]],
    "chain": [["0"], ["1"], ["2"], ("POLY=4", ["4"]), ("POLY=6", ["4"]), ("POLY=4", ["3"])],
}


def main() -> None:
    if len(sys.argv) < 2 or sys.argv[1] not in RUNS:
        raise SystemExit(__doc__)
    name = sys.argv[1]
    exe = HERE / f"{name}.bin"
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-o", str(exe), str(HERE / f"{name}.cu"),
           str(HERE.parent / "csrc" / "ca_runtime.cu"), "-lcuda"]
    subprocess.run(cmd, check=True)
    for run in RUNS[name]:
        env = dict(os.environ)
        if isinstance(run, tuple):
            k, v = run[0].split("=")
            env[k] = v
            run = run[1]
        subprocess.run([str(exe), *run], check=True, env=env)


if __name__ == "__main__":
    main()
