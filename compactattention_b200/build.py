"""Builds ``libcompactattn_b200.so`` in-tree with nvcc for sm_100a.

The library is plain CUDA C++ behind a C ABI (``include/compactattn_b200.h``); it links only the
static CUDA runtime, so it loads on a machine without a GPU driver (symbols can be inspected
there) and runs on a B200.

Usage: ``python -m compactattention_b200.build [--force] [--verbose]``

Development builds (cycle accounting, timing experiments) go to a separate file and never replace
the product library: ``python -m compactattention_b200.build --define CA_ATTN_PROFILE=1 --output
compactattention_b200/libcompactattn_b200_profile.so``.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libcompactattn_b200.so"
STAMP_PATH = PKG_DIR / "libcompactattn_b200.so.stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-cudart", "static",
    "-shared",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _fingerprint() -> str:
    h = hashlib.sha256()
    files = sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "compactattn_b200.h"])
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build libcompactattn_b200.so")
    return nvcc


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` into one shared library; skip when sources are unchanged."""
    fp = _fingerprint()
    if not force and LIB_PATH.exists() and STAMP_PATH.exists() and STAMP_PATH.read_text().strip() == fp:
        return LIB_PATH
    cmd = [find_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB_PATH), *[str(s) for s in sources()]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {proc.returncode}")
    STAMP_PATH.write_text(fp + "\n")
    return LIB_PATH


def build_variant(defines: list[str], output: Path, verbose: bool = False) -> Path:
    """Compile the same sources with extra ``-D`` macros into ``output`` (a development build)."""
    output = Path(output).resolve()
    if output == LIB_PATH:
        raise ValueError("a development build must not overwrite the product library")
    cmd = [find_nvcc(), *NVCC_FLAGS, *[f"-D{d}" for d in defines]]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(output), *[str(s) for s in sources()]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {proc.returncode}")
    return output


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--define", action="append", default=[], help="extra macro NAME=VALUE (development build; needs --output)")
    ap.add_argument("--output", default=None, help="where a development build is written")
    args = ap.parse_args()
    if args.define or args.output:
        if not (args.define and args.output):
            ap.error("--define and --output go together")
        print(build_variant(args.define, Path(args.output), verbose=args.verbose))
    else:
        print(build(force=args.force, verbose=args.verbose))


if __name__ == "__main__":
    main()
