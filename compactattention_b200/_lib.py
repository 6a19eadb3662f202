"""ctypes binding of ``libcompactattn_b200.so`` (the C ABI declared in ``include/compactattn_b200.h``).

The library is the product: there is no Python or CPU fallback. ``load()`` raises when the shared
object is missing, and every call that returns a negative status raises ``RuntimeError`` carrying
``ca_last_error()``.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libcompactattn_b200.so"

CA_OK = 0
CA_DTYPE_BF16, CA_DTYPE_F16, CA_DTYPE_F32 = 0, 1, 2
CA_STATUS_TIMEOUT, CA_STATUS_BAD_INDEX = 1, 2


class KvLayout(C.Structure):
    _fields_ = [
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("page_stride", C.c_int64),
        ("token_stride", C.c_int64),
        ("head_stride", C.c_int64),
        ("page_size", C.c_int32),
        ("num_pages", C.c_int32),
        ("pages_per_seq", C.c_int32),
        ("reserved", C.c_int32),
        ("page_table", C.c_void_p),
    ]


class AttnParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("q_stride_b", C.c_int64), ("q_stride_t", C.c_int64), ("q_stride_h", C.c_int64),
        ("out", C.c_void_p),
        ("o_stride_b", C.c_int64), ("o_stride_t", C.c_int64), ("o_stride_h", C.c_int64),
        ("kv", KvLayout),
        ("block_idx", C.c_void_p),
        ("counts", C.c_void_p),
        ("block_idx_stride", C.c_int32),
        ("B", C.c_int32), ("Q", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32),
        ("kv_len", C.c_int32),
        ("block_size", C.c_int32),
        ("dtype", C.c_int32),
        ("softmax_scale", C.c_float),
        ("lse", C.c_void_p),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p),
    ]


# name -> (restype, argtypes); filled in below and applied by load().
_SIGNATURES = {
    "ca_last_error": (C.c_char_p, []),
    "ca_abi_version": (C.c_int, []),
    "ca_launch_count": (C.c_int64, []),
    "ca_attn_workspace_bytes": (C.c_int, [C.POINTER(AttnParams), C.POINTER(C.c_size_t)]),
    "ca_attn_compact": (C.c_int, [C.POINTER(AttnParams), C.c_void_p]),
}

_lib = None


class MissingLibraryError(RuntimeError):
    pass


def load() -> C.CDLL:
    """Load the shared library once. Fails loudly: nothing in this package computes without it."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise MissingLibraryError(
            f"{LIB_PATH} is missing. Build it with `python -m compactattention_b200.build` "
            "(needs nvcc); this package has no fallback implementation."
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def exported_names() -> list[str]:
    return sorted(_SIGNATURES)


def check(rc: int, what: str) -> None:
    if rc != CA_OK:
        msg = load().ca_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")


def launch_count() -> int:
    return int(load().ca_launch_count())
