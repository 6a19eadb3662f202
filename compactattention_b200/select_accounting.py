"""Where the cycles of the selection kernels go: builds the library with ``-DCA_SELECT_PROFILE=1`` into a separate
``.so`` (thread 0 of CTA 0 then stores ``clock64()`` at every phase boundary of ``gate_scores_tc_kernel`` and
``select_rows_kernel`` into a ``__device__`` array, and ``ca_debug_select_profile`` copies it out; the product
library has neither), runs the chain gate scores -> row rule + Block-Union + table once at the headline shape and
prints the stamps in cycles from each kernel's start.

    python -m compactattention_b200.select_accounting [--kv-blocks 2048] [--q-blocks 16] [--rule topk]
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import tempfile
from pathlib import Path


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kv-blocks", type=int, default=2048)
    ap.add_argument("--q-blocks", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--group", type=int, default=4)
    ap.add_argument("--rule", choices=["topk", "threshold"], default="topk")
    args = ap.parse_args()

    import torch

    from . import _lib, build

    out = Path(tempfile.gettempdir()) / "libcompactattn_b200_select_profile.so"
    build.build_variant(["CA_SELECT_PROFILE=1"], out)
    _lib.LIB_PATH = out          # before the first load(): this process uses the development build
    from . import ops
    lib = _lib.load()
    fn = lib.ca_debug_select_profile
    fn.restype, fn.argtypes = C.c_int, [C.POINTER(C.c_longlong)]

    Hkv, G, Qb, Kb = args.kv_heads, args.group, args.q_blocks, args.kv_blocks
    g = torch.Generator().manual_seed(1)
    qb = torch.randn((1, Qb, Hkv * G, 128), generator=g).cuda()
    kb = torch.randn((1, Kb, Hkv, 128), generator=g).to(torch.bfloat16).cuda()
    kw = dict(topk_ratio=(1, 5), sink=1, local=2) if args.rule == "topk" else dict(softmax=True, threshold=5e-4, keep_recent=2)
    for _ in range(3):
        ops.gate_score_select(qb, kb, Kb - Qb, args.rule, num_kv_heads=Hkv, block_size=64, **kw)
    torch.cuda.synchronize()
    buf = (C.c_longlong * 32)()
    if fn(buf) != 0:
        raise RuntimeError("ca_debug_select_profile failed")
    t = list(buf)
    names = {0: "select_rows: CTA start", 4: "select_rows: row start", 5: "select_rows: row loaded (+softmax)", 6: "select_rows: rule done",
             7: "select_rows: bits stored", 9: "select_rows: ticket taken",
             16: "gate_scores_tc: CTA start", 17: "gate_scores_tc: Q tile built", 18: "gate_scores_tc: MMAs done",
             19: "gate_scores_tc: logits stored"}
    print(json.dumps({"shape": {"kv_heads": Hkv, "group": G, "q_blocks": Qb, "kv_blocks": Kb, "rule": args.rule},
                      "cycles_from_kernel_start": {names[k]: t[k] - (t[16] if k >= 16 else t[0]) for k in sorted(names)}}))


if __name__ == "__main__":
    main()
