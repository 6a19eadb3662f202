"""Imports the reference project's own Python modules for this path on the CPU.  TEST
INFRASTRUCTURE ONLY, and only usable where a checkout of the reference exists (it does not travel
with this repository): it is used to generate the golden fixtures and to cross-check the oracle.

``compact_attn/__init__.py`` imports every model class and fails on current transformers releases,
so the package is stubbed: empty parent packages are pre-seeded in ``sys.modules`` and the leaf
modules of the path are then imported normally from the checkout.
"""
from __future__ import annotations

import importlib
import os
import sys
import types
from pathlib import Path

# A checkout of the reference project: COMPACTATTN_REFERENCE_ROOT, else a `reference` directory next
# to this repository.
DEFAULT_ROOT = os.environ.get("COMPACTATTN_REFERENCE_ROOT", str(Path(__file__).resolve().parent.parent.parent / "reference"))

_STUB_PACKAGES = [
    "compact_attn",
    "compact_attn.modules",
    "compact_attn.kernels",
    "compact_attn.kernels.varlen",
    "compact_attn.prefill_sparse",
]


def available(root: str = DEFAULT_ROOT) -> bool:
    return (Path(root) / "compact_attn" / "modules" / "attention_forward_chunked_dense.py").exists()


def load(root: str = DEFAULT_ROOT) -> types.SimpleNamespace:
    """Returns a namespace with the reference modules of the path (CPU import)."""
    if not available(root):
        raise FileNotFoundError(f"no reference checkout at {root}")
    root_path = Path(root)
    for name in _STUB_PACKAGES:
        if name not in sys.modules:
            mod = types.ModuleType(name)
            mod.__path__ = [str(root_path / name.replace(".", "/"))]
            sys.modules[name] = mod
    if str(root_path) not in sys.path:
        sys.path.insert(0, str(root_path))
    ns = types.SimpleNamespace()
    ns.common = importlib.import_module("compact_attn.modules.common")
    ns.chunked_dense = importlib.import_module("compact_attn.modules.attention_forward_chunked_dense")
    ns.flashprefill_prefill = importlib.import_module("compact_attn.modules.flashprefill_prefill")
    ns.flashprefill_vendor = importlib.import_module("compact_attn.flashprefill_vendor.flashprefill_native_forward")
    ns.attn_gate = importlib.import_module("compact_attn.prefill_sparse.attn_gate")
    ns.varlen = importlib.import_module("compact_attn.kernels.varlen.indexed_dense_prefill_varlen")
    ns.zero_copy = importlib.import_module("compact_attn.kernels.varlen.flashinfer_zero_copy_prefill")
    return ns
