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
        ("head_div", C.c_int32),
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


class SelectParams(C.Structure):
    _fields_ = [
        ("score", C.c_void_p),
        ("score_stride_b", C.c_int64), ("score_stride_h", C.c_int64), ("score_stride_q", C.c_int64), ("score_stride_k", C.c_int64),
        ("score_dtype", C.c_int32),
        ("rule", C.c_int32),
        ("valid", C.c_void_p),
        ("valid_stride_b", C.c_int64), ("valid_stride_h", C.c_int64), ("valid_stride_q", C.c_int64), ("valid_stride_k", C.c_int64),
        ("bits", C.c_void_p),
        ("prob_out", C.c_void_p),
        ("B", C.c_int32), ("H", C.c_int32), ("Qb", C.c_int32), ("Kb", C.c_int32), ("Pb", C.c_int32),
        ("softmax", C.c_int32),
        ("threshold", C.c_float),
        ("alpha", C.c_float),
        ("topk_k", C.c_int32), ("topk_num", C.c_int32), ("topk_den", C.c_int32),
        ("min_budget", C.c_int32),
        ("sink", C.c_int32), ("local", C.c_int32),
        ("rows_voting", C.c_int32),
        ("threshold_ptr", C.c_void_p),
        ("threshold_stride_b", C.c_int64),
        ("score_max", C.c_void_p),
    ]


class UnionParams(C.Structure):
    _fields_ = [
        ("bits", C.c_void_p),
        ("mask", C.c_void_p),
        ("mask_stride_b", C.c_int64), ("mask_stride_h", C.c_int64), ("mask_stride_q", C.c_int64), ("mask_stride_k", C.c_int64),
        ("B", C.c_int32), ("Hkv", C.c_int32), ("G", C.c_int32), ("Qin", C.c_int32), ("Kb", C.c_int32), ("Pb", C.c_int32),
        ("keep_recent", C.c_int32),
        ("block_size", C.c_int32), ("page_size", C.c_int32),
        ("block_idx", C.c_void_p),
        ("idx_stride", C.c_int32),
        ("counts", C.c_void_p),
        ("cache_seqlens", C.c_void_p),
        ("pages_per_row", C.c_void_p),
        ("keep_kv", C.c_void_p),
    ]


class PoolParams(C.Structure):
    _fields_ = [
        ("x", C.c_void_p),
        ("x_stride_b", C.c_int64), ("x_stride_t", C.c_int64), ("x_stride_h", C.c_int64),
        ("x_dtype", C.c_int32),
        ("out_dtype", C.c_int32),
        ("out", C.c_void_p),
        ("out_stride_b", C.c_int64), ("out_stride_blk", C.c_int64), ("out_stride_h", C.c_int64),
        ("out_block_offset", C.c_int32),
        ("B", C.c_int32), ("L", C.c_int32), ("H", C.c_int32), ("D", C.c_int32), ("block_size", C.c_int32),
        ("kinds", C.c_int32),
    ]


class ProjectParams(C.Structure):
    _fields_ = [
        ("x", C.c_void_p),
        ("w", C.c_void_p),
        ("w_dtype", C.c_int32),
        ("out_dtype", C.c_int32),
        ("cos", C.c_void_p),
        ("sin", C.c_void_p),
        ("rope_batch", C.c_int32),
        ("out_block_offset", C.c_int32),
        ("out", C.c_void_p),
        ("out_stride_b", C.c_int64), ("out_stride_blk", C.c_int64), ("out_stride_h", C.c_int64),
        ("B", C.c_int32), ("nb", C.c_int32), ("Hin", C.c_int32), ("Hout", C.c_int32), ("Cin", C.c_int32), ("Cout", C.c_int32),
    ]


class GateSide(C.Structure):
    _fields_ = [
        ("x", C.c_void_p),
        ("x_stride_b", C.c_int64), ("x_stride_t", C.c_int64), ("x_stride_h", C.c_int64),
        ("x_dtype", C.c_int32),
        ("H", C.c_int32),
        ("kinds", C.c_int32),
        ("w_dtype", C.c_int32),
        ("w", C.c_void_p),
        ("Hw", C.c_int32),
        ("rope_batch", C.c_int32),
        ("cos", C.c_void_p),
        ("sin", C.c_void_p),
        ("out", C.c_void_p),
        ("out_stride_b", C.c_int64), ("out_stride_blk", C.c_int64), ("out_stride_h", C.c_int64),
        ("out_dtype", C.c_int32),
        ("out_block_offset", C.c_int32),
    ]


class GatePrepareParams(C.Structure):
    _fields_ = [
        ("q", GateSide), ("k", GateSide),
        ("B", C.c_int32), ("L", C.c_int32), ("D", C.c_int32), ("C", C.c_int32), ("block_size", C.c_int32),
    ]


class GateScoreParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("q_stride_b", C.c_int64), ("q_stride_blk", C.c_int64), ("q_stride_h", C.c_int64),
        ("k", C.c_void_p),
        ("k_stride_b", C.c_int64), ("k_stride_blk", C.c_int64), ("k_stride_h", C.c_int64),
        ("q_dtype", C.c_int32), ("k_dtype", C.c_int32),
        ("out", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hk", C.c_int32), ("Qb", C.c_int32), ("Kb", C.c_int32), ("Pb", C.c_int32), ("C", C.c_int32),
        ("scale", C.c_float),
        ("masked_value", C.c_float),
    ]


class FlashPrefillScoreParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("q_stride_b", C.c_int64), ("q_stride_t", C.c_int64), ("q_stride_h", C.c_int64),
        ("mean_k", C.c_void_p),
        ("k_stride_b", C.c_int64), ("k_stride_blk", C.c_int64), ("k_stride_h", C.c_int64),
        ("q_dtype", C.c_int32), ("k_dtype", C.c_int32),
        ("score_raw", C.c_void_p),
        ("max_raw", C.c_void_p),
        ("score_norm", C.c_void_p),
        ("B", C.c_int32), ("Q", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32), ("Kb", C.c_int32),
        ("block_size", C.c_int32), ("kv_len", C.c_int32),
    ]


class GatherParams(C.Structure):
    _fields_ = [
        ("kv", KvLayout),
        ("block_idx", C.c_void_p),
        ("counts", C.c_void_p),
        ("block_idx_stride", C.c_int32),
        ("dtype", C.c_int32),
        ("page_offsets", C.c_void_p),
        ("dst_row_stride_tokens", C.c_int64),
        ("k_dst", C.c_void_p),
        ("v_dst", C.c_void_p),
        ("dst_page_size", C.c_int32),
        ("B", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32), ("Q", C.c_int32), ("kv_len", C.c_int32), ("block_size", C.c_int32),
        ("status", C.c_void_p),
    ]


class RopeAppendParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("q_out", C.c_void_p),
        ("q_stride_b", C.c_int64), ("q_stride_t", C.c_int64), ("q_stride_h", C.c_int64),
        ("qo_stride_b", C.c_int64), ("qo_stride_t", C.c_int64), ("qo_stride_h", C.c_int64),
        ("k", C.c_void_p),
        ("k_stride_b", C.c_int64), ("k_stride_t", C.c_int64), ("k_stride_h", C.c_int64),
        ("v", C.c_void_p),
        ("v_stride_b", C.c_int64), ("v_stride_t", C.c_int64), ("v_stride_h", C.c_int64),
        ("cos", C.c_void_p), ("sin", C.c_void_p),
        ("cs_stride_b", C.c_int64), ("cs_stride_t", C.c_int64),
        ("rope_dtype", C.c_int32), ("dtype", C.c_int32),
        ("cache", KvLayout),
        ("mean_k", C.c_void_p),
        ("mk_stride_b", C.c_int64), ("mk_stride_blk", C.c_int64), ("mk_stride_h", C.c_int64),
        ("B", C.c_int32), ("Q", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32),
        ("position", C.c_int32), ("block_size", C.c_int32), ("reserved", C.c_int32),
        ("status", C.c_void_p),
    ]


class OprojParams(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("a_stride_m", C.c_int64),
        ("w", C.c_void_p), ("w_stride_n", C.c_int64),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
        ("dtype", C.c_int32),
        ("world", C.c_int32), ("rank", C.c_int32),
        ("stage", C.POINTER(C.c_void_p)),
        ("tile_counters", C.POINTER(C.c_void_p)),
        ("done_counters", C.POINTER(C.c_void_p)),
        ("out", C.POINTER(C.c_void_p)),
        ("out_stride_m", C.c_int64),
        ("epoch", C.c_uint32), ("phases", C.c_uint32),
        ("wait_limit_ns", C.c_uint64),
        ("status", C.c_void_p),
        ("mode", C.c_int32),
        ("stage_bytes", C.c_size_t),
        ("row_epochs", C.POINTER(C.c_uint32)),
        ("stage_mc", C.c_void_p), ("out_mc", C.c_void_p),
        ("done_tiles_total", C.c_uint32),
    ]


class ChunkStepParams(C.Structure):
    _fields_ = [
        ("append", RopeAppendParams),
        ("prepare", GatePrepareParams),
        ("score", GateScoreParams),
        ("fp_score", FlashPrefillScoreParams),
        ("select", SelectParams),
        ("table", UnionParams),
        ("union_scratch", C.c_void_p),
        ("union_scratch_bytes", C.c_size_t),
        ("attn", AttnParams),
        ("write_scores", C.c_int32),
    ]


CA_RULE_THRESHOLD, CA_RULE_ALPHA_ROWMAX, CA_RULE_TOPK, CA_RULE_CUMMASS, CA_RULE_MASK = 0, 1, 2, 3, 4
CA_POOL_MAX, CA_POOL_MIN, CA_POOL_AVG = 1, 2, 4

# name -> (restype, argtypes); filled in below and applied by load().
_SIGNATURES = {
    "ca_last_error": (C.c_char_p, []),
    "ca_abi_version": (C.c_int, []),
    "ca_launch_count": (C.c_int64, []),
    "ca_set_programmatic_launch": (C.c_int, [C.c_int]),
    "ca_attn_workspace_bytes": (C.c_int, [C.POINTER(AttnParams), C.POINTER(C.c_size_t)]),
    "ca_attn_compact": (C.c_int, [C.POINTER(AttnParams), C.c_void_p]),
    "ca_attn_compact_static_scratch": (C.c_int, [C.POINTER(AttnParams), C.c_void_p]),
    "ca_select_rows": (C.c_int, [C.POINTER(SelectParams), C.c_void_p]),
    "ca_union_table": (C.c_int, [C.POINTER(UnionParams), C.c_void_p]),
    "ca_select_union_scratch_bytes": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_size_t)]),
    "ca_select_union_table": (C.c_int, [C.POINTER(SelectParams), C.POINTER(UnionParams), C.c_void_p, C.c_size_t, C.c_void_p]),
    "ca_paged_metadata": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "ca_pool_blocks": (C.c_int, [C.POINTER(PoolParams), C.c_void_p]),
    "ca_gate_project": (C.c_int, [C.POINTER(ProjectParams), C.c_void_p]),
    "ca_gate_prepare": (C.c_int, [C.POINTER(GatePrepareParams), C.c_void_p]),
    "ca_gate_scores": (C.c_int, [C.POINTER(GateScoreParams), C.c_void_p]),
    "ca_flashprefill_score": (C.c_int, [C.POINTER(FlashPrefillScoreParams), C.c_void_p]),
    "ca_gather_kv": (C.c_int, [C.POINTER(GatherParams), C.c_void_p]),
    "ca_rope_append": (C.c_int, [C.POINTER(RopeAppendParams), C.c_void_p]),
    "ca_chunk_step": (C.c_int, [C.POINTER(ChunkStepParams), C.c_void_p]),
    "ca_oproj_scratch_bytes": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "ca_oproj_allreduce": (C.c_int, [C.POINTER(OprojParams), C.c_void_p]),
    "ca_oproj_tile_count": (C.c_int, [C.c_int, C.c_int]),
    "ca_selftest_bounded_wait": (C.c_int, [C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "ca_gate_score_select": (C.c_int, [C.POINTER(GateScoreParams), C.POINTER(SelectParams), C.POINTER(UnionParams), C.c_void_p,
                                       C.c_size_t, C.c_int, C.c_void_p]),
}

_lib = None


class MissingLibraryError(RuntimeError):
    pass


class CallList:
    """Library calls recorded once (see ``record``) and re-issued as they were: the same entry points with the
    same parameter blocks, pointers and stream.  What a host keeps between chunks when shapes and buffers do
    not change (a benchmark loop, a layer at a fixed chunk position): replaying costs one foreign call per
    entry, not the Python that filled the structs.  The blocks hold raw device pointers: the tensors they came
    from must stay alive, and calls whose parameters change per call (epochs, positions) must not be replayed."""

    def __init__(self):
        self.calls = []

    def run(self) -> None:
        for name, fn, args in self.calls:
            rc = fn(*args)
            if rc != CA_OK:
                check(rc, name)


# Entry points that enqueue work take the stream as their last argument; only these are recorded - except the
# ones whose parameters must change from call to call (the exchange's epochs).
_NEVER_RECORDED = {"ca_oproj_allreduce", "ca_selftest_bounded_wait"}
_recording: "CallList | None" = None


class _Recording:
    def __enter__(self) -> CallList:
        global _recording
        if _recording is not None:
            raise RuntimeError("library calls are already being recorded")
        _recording = CallList()
        return _recording

    def __exit__(self, *exc) -> None:
        global _recording
        _recording = None


def record() -> _Recording:
    """``with record() as calls:`` runs the body normally and also keeps every enqueuing library call it makes
    in ``calls`` (a ``CallList``)."""
    return _Recording()


class _Library:
    """The loaded library.  Attribute access gives the foreign functions; while ``record()`` is active the
    enqueuing ones are also appended to the recording."""

    def __init__(self, cdll: C.CDLL):
        self._cdll = cdll
        self._wrapped = {}

    def __getattr__(self, name):
        fn = getattr(self._cdll, name)   # AttributeError for names the library does not export
        if name not in _SIGNATURES or _SIGNATURES[name][1][-1:] != [C.c_void_p] or name in _NEVER_RECORDED:
            return fn
        w = self._wrapped.get(name)
        if w is None:
            def w(*args, _fn=fn, _name=name):
                if _recording is not None:
                    _recording.calls.append((_name, _fn, args))
                return _fn(*args)
            self._wrapped[name] = w
        return w


def load() -> "_Library":
    """Load the shared library once. Fails loudly: nothing in this package computes without it."""
    global _lib
    if _lib is not None:
        return _lib
    path = LIB_PATH
    if not path.exists():
        raise MissingLibraryError(
            f"{path} is missing. Build it with `python -m compactattention_b200.build` "
            "(needs nvcc); this package has no fallback implementation."
        )
    lib = C.CDLL(str(path))
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = _Library(lib)
    return _lib


def exported_names() -> list[str]:
    return sorted(_SIGNATURES)


def check(rc: int, what: str) -> None:
    if rc != CA_OK:
        msg = load().ca_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")


def set_programmatic_launch(enabled: bool) -> bool:
    """Turns programmatic dependent launch of the library's kernels on or off (off by default);
    returns the previous setting."""
    return bool(load().ca_set_programmatic_launch(1 if enabled else 0))


def launch_count() -> int:
    return int(load().ca_launch_count())
