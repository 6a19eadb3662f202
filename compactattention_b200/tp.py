"""KV-head tensor parallelism for the path: which heads a rank owns, how the selector weights are
sliced, and the one collective that follows the path (the sum of the row-parallel output projection).

Mirrors the reference's use of the HuggingFace tensor-parallel plan (q/k/v projections column-wise,
o_proj row-wise: ``compact_attn/prefill_sparse/llama/modeling_llama_seerattn.py:111-120``) and its
per-rank slicing of the gate (``_localize_seer_gate_for_tp``,
``eval/chunked_prefill/chunked_prefill_runtime.py:1929-1980``).  Scoring, selection, the block table,
the gather and the attention of a rank touch only its own KV heads, so nothing is exchanged until the
layer output: one all-reduce over NCCL (NVLink) per layer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class HeadShard:
    """The contiguous KV heads (and their query heads) owned by one rank."""

    world: int
    rank: int
    num_q_heads: int
    num_kv_heads: int

    def __post_init__(self):
        if self.num_q_heads % self.num_kv_heads:
            raise ValueError("query heads must be a multiple of KV heads")
        if self.num_kv_heads % self.world:
            raise ValueError(f"{self.world} ranks do not divide {self.num_kv_heads} KV heads")
        if not 0 <= self.rank < self.world:
            raise ValueError("rank out of range")

    @property
    def group(self) -> int:
        return self.num_q_heads // self.num_kv_heads

    @property
    def kv_heads(self) -> range:
        n = self.num_kv_heads // self.world
        return range(self.rank * n, (self.rank + 1) * n)

    @property
    def q_heads(self) -> range:
        return range(self.kv_heads.start * self.group, self.kv_heads.stop * self.group)

    def slice_q(self, x: torch.Tensor, head_dim: int = 2) -> torch.Tensor:
        """Slice a tensor with a query-head dimension to this rank's heads."""
        return x.narrow(head_dim, self.q_heads.start, len(self.q_heads))

    def slice_kv(self, x: torch.Tensor, head_dim: int = 2) -> torch.Tensor:
        return x.narrow(head_dim, self.kv_heads.start, len(self.kv_heads))

    def slice_gate_weight(self, w: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Per-head gate weights ``[H, Cin, C]`` with H = query heads or KV heads."""
        if w is None:
            return None
        if w.shape[0] == self.num_q_heads:
            return self.slice_q(w, 0).contiguous()
        if w.shape[0] == self.num_kv_heads:
            return self.slice_kv(w, 0).contiguous()
        raise ValueError(f"gate weight has {w.shape[0]} heads, expected {self.num_q_heads} or {self.num_kv_heads}")

    def slice_o_proj(self, w: torch.Tensor, head_size: int) -> torch.Tensor:
        """Row-parallel slice of an output projection ``[hidden, Hq*D]`` (input columns of this rank's heads)."""
        return w[:, self.q_heads.start * head_size : self.q_heads.stop * head_size].contiguous()


def reduce_layer_output(partial: torch.Tensor, group=None, async_op: bool = False):
    """Sum of the ranks' partial layer outputs (row-parallel o_proj): the path's only collective.
    Returns the work handle when ``async_op`` (the reference may defer this wait,
    ``modeling_llama_flashprefill_compactattn.py:37-41, 321-322``)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return None
    return dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group, async_op=async_op)


class ProjectionCallLedger:
    """What the counters of ``ca_oproj_allreduce`` expect after each call on one set of buffers: the call number
    (``epoch``), per block of 128 rows the number of calls that covered it (``row_epochs``), and the running
    number of output tiles (``done_tiles_total``).  Every rank keeps the same ledger because every rank issues
    the same calls; counters only grow, so a call with fewer rows (a ragged last chunk, a decode step) leaves
    the targets of the uncovered row blocks where they were."""

    TILE_ROWS, TILE_COLS = 128, 256

    def __init__(self, max_rows: int, out_features: int):
        self.max_rows, self.out_features = int(max_rows), int(out_features)
        self.epoch = 0
        self.row_calls = [0] * ((self.max_rows + self.TILE_ROWS - 1) // self.TILE_ROWS)
        self.tiles_total = 0

    def next_call(self, rows: int):
        """Advances the ledger by one call of ``rows`` rows; returns ``(epoch, row_epochs, done_tiles_total)``."""
        if not 0 < rows <= self.max_rows:
            raise ValueError(f"{rows} rows exceed the buffers of this projection ({self.max_rows})")
        self.epoch += 1
        blocks = (rows + self.TILE_ROWS - 1) // self.TILE_ROWS
        for tm in range(blocks):
            self.row_calls[tm] += 1
        self.tiles_total = (self.tiles_total + blocks * ((self.out_features + self.TILE_COLS - 1) // self.TILE_COLS)) & 0xFFFFFFFF
        return self.epoch, [c & 0xFFFFFFFF for c in self.row_calls[:blocks]], self.tiles_total

    def snapshot(self):
        return self.epoch, list(self.row_calls), self.tiles_total

    def restore(self, snap) -> None:
        self.epoch, self.row_calls, self.tiles_total = snap[0], list(snap[1]), snap[2]


class FusedOutputProjection:
    """Row-parallel output projection whose tensor-parallel sum travels inside the library's kernels
    (``ca_oproj_allreduce``: a tcgen05 GEMM that stores partial tiles into the owning rank's memory, a
    reduction that stores finished tiles into every rank's output, a bounded wait) instead of a library GEMM
    followed by an NCCL all-reduce.  Buffers live in symmetric memory (``torch.distributed._symmetric_memory``),
    allocated and exchanged once; every call reuses them, so a call's output is valid until the next call.

    All ranks must construct it with the same sizes and call it in the same order.  ``check()`` reads the
    status word (a device-to-host read) and raises if a wait ran out - e.g. a rank that died."""

    def __init__(self, max_rows: int, out_features: int, device, dtype=torch.bfloat16, group=None, wait_limit_s: float = 2.0,
                 mode: int = 0):
        import ctypes as C

        from . import _lib
        self._lib, self._C = _lib, C
        self.group = group if group is not None else (dist.group.WORLD if dist.is_initialized() else None)
        self.world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        self.max_rows, self.N, self.dtype, self.device = int(max_rows), int(out_features), dtype, torch.device(device)
        self.ledger = ProjectionCallLedger(self.max_rows, self.N)
        self.phases = 7   # all three launches; a subset only for tests and timing (see ca_oproj_params.phases)
        self.mode = int(mode)   # 0: one exchange on two ranks, reduce-scatter + all-gather over peer stores beyond;
                                # 1 / 2 force either; 3: through the NVLink switch (multimem), where it offers multicast
        self._mc = None
        self._stage_bytes = 0
        self.wait_limit_ns = int(wait_limit_s * 1e9)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        stage_b, cnt_b = C.c_size_t(0), C.c_size_t(0)
        _lib.check(_lib.load().ca_oproj_scratch_bytes(self.max_rows, self.N, self.world, C.byref(stage_b), C.byref(cnt_b)),
                   "ca_oproj_scratch_bytes")
        esize = torch.empty((), dtype=dtype).element_size()
        if self.world == 1:
            self.out = torch.empty((self.max_rows, self.N), dtype=dtype, device=device)
            self._ptrs = {"out": [self.out.data_ptr()], "stage": None, "tiles": None, "done": None}
            return
        import torch.distributed._symmetric_memory as symm
        name = self.group.group_name
        self.out = symm.empty((self.max_rows, self.N), dtype=dtype, device=self.device)
        self.stage = symm.empty(max(int(stage_b.value) // esize, 8), dtype=dtype, device=self.device)
        self.counters = symm.empty(int(cnt_b.value) // 4, dtype=torch.int32, device=self.device)
        self.counters.zero_()
        self._stage_bytes = self.stage.numel() * esize
        handles = [symm.rendezvous(t, name) for t in (self.out, self.stage, self.counters)]
        n_tile_counters = int(cnt_b.value) // 4 - 1
        self._ptrs = {
            "out": list(handles[0].buffer_ptrs), "stage": list(handles[1].buffer_ptrs),
            "tiles": list(handles[2].buffer_ptrs), "done": [p + 4 * n_tile_counters for p in handles[2].buffer_ptrs],
        }
        self._handles = handles
        # NVLink-switch multicast addresses of the outputs and the staging buffers (0 where the fabric has none):
        # mode 3 lets the switch do the additions (multimem.ld_reduce / multimem.st)
        out_mc = int(getattr(handles[0], "multicast_ptr", 0) or 0)
        stage_mc = int(getattr(handles[1], "multicast_ptr", 0) or 0)
        self._mc = (stage_mc, out_mc) if (out_mc and stage_mc) else None
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)   # every rank's counters are zero before anyone's first call

    def _array(self, ptrs):
        C = self._C
        return None if ptrs is None else (C.c_void_p * len(ptrs))(*ptrs)

    def __call__(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """``x [..., K]`` (this rank's attention output, K contiguous) times ``weight [N, K]`` (this rank's input
        columns of the projection), summed over the ranks.  Returns a view ``[..., N]`` of the shared output
        buffer."""
        from . import ops
        C = self._C
        lead = x.shape[:-1]
        K = x.shape[-1]
        a = x.reshape(-1, K)
        M = a.shape[0]
        if a.stride(1) != 1 or weight.stride(1) != 1 or weight.shape != (self.N, K) or a.dtype != self.dtype or weight.dtype != self.dtype:
            raise ValueError("x must be [..., K] and weight [N, K], both K-contiguous and of the projection's dtype")
        epoch, row_calls, tiles_total = self.ledger.next_call(M)
        row_epochs = (C.c_uint32 * len(row_calls))(*row_calls)
        p = self._lib.OprojParams()
        p.mode, p.stage_bytes, p.done_tiles_total = self.mode, self._stage_bytes, tiles_total
        p.row_epochs = C.cast(row_epochs, C.POINTER(C.c_uint32))
        if self._mc is not None:
            p.stage_mc, p.out_mc = self._mc
        p.a, p.a_stride_m, p.w, p.w_stride_n = a.data_ptr(), a.stride(0), weight.data_ptr(), weight.stride(0)
        p.M, p.N, p.K, p.dtype = M, self.N, K, ops._DTYPES[self.dtype]
        p.world, p.rank = self.world, self.rank
        arrays = {k: self._array(v) for k, v in self._ptrs.items()}
        p.out = C.cast(arrays["out"], C.POINTER(C.c_void_p))
        if self.world > 1:
            p.stage = C.cast(arrays["stage"], C.POINTER(C.c_void_p))
            p.tile_counters = C.cast(arrays["tiles"], C.POINTER(C.c_void_p))
            p.done_counters = C.cast(arrays["done"], C.POINTER(C.c_void_p))
        p.out_stride_m, p.epoch, p.wait_limit_ns, p.status = self.N, epoch, self.wait_limit_ns, self.status.data_ptr()
        p.phases = self.phases
        self._lib.check(self._lib.load().ca_oproj_allreduce(C.byref(p), ops._stream()), "ca_oproj_allreduce")
        return self.out[:M].view(*lead, self.N)

    def all_reduce(self, partial: torch.Tensor) -> torch.Tensor:
        """Sum over the ranks of ``partial [..., N]`` (this rank's already projected output) through the same
        exchange, without the GEMM: the library's own all-reduce over peer memory.  Returns a view of the shared
        output buffer, valid until the next call."""
        from . import ops
        C = self._C
        lead = partial.shape[:-1]
        a = partial.reshape(-1, partial.shape[-1])
        M = a.shape[0]
        if a.shape[1] != self.N or a.stride(1) != 1 or a.dtype != self.dtype or self.world == 1:
            raise ValueError("partial must be [..., N] of the projection's dtype, N contiguous, on more than one rank")
        epoch, row_calls, tiles_total = self.ledger.next_call(M)
        row_epochs = (C.c_uint32 * len(row_calls))(*row_calls)
        p = self._lib.OprojParams()
        p.mode, p.stage_bytes, p.done_tiles_total = self.mode, self._stage_bytes, tiles_total
        p.row_epochs = C.cast(row_epochs, C.POINTER(C.c_uint32))
        if self._mc is not None:
            p.stage_mc, p.out_mc = self._mc
        p.a, p.a_stride_m, p.w, p.w_stride_n = a.data_ptr(), a.stride(0), None, 0
        p.M, p.N, p.K, p.dtype = M, self.N, 0, ops._DTYPES[self.dtype]
        p.world, p.rank = self.world, self.rank
        arrays = {k: self._array(v) for k, v in self._ptrs.items()}
        p.out = C.cast(arrays["out"], C.POINTER(C.c_void_p))
        p.stage = C.cast(arrays["stage"], C.POINTER(C.c_void_p))
        p.tile_counters = C.cast(arrays["tiles"], C.POINTER(C.c_void_p))
        p.done_counters = C.cast(arrays["done"], C.POINTER(C.c_void_p))
        p.out_stride_m, p.epoch, p.wait_limit_ns, p.status = self.N, epoch, self.wait_limit_ns, self.status.data_ptr()
        p.phases = self.phases
        self._lib.check(self._lib.load().ca_oproj_allreduce(C.byref(p), ops._stream()), "ca_oproj_allreduce")
        return self.out[:M].view(*lead, self.N)

    def check(self) -> None:
        """Raises if a device-side wait of an earlier call ran out (reads the status word: synchronises)."""
        if int(self.status.item()) & self._lib.CA_STATUS_TIMEOUT:
            raise RuntimeError("the fused output projection timed out waiting for another rank's tiles; its output is invalid")


_SHARED_PROJECTIONS: dict = {}


def shared_fused_projection(max_rows: int, out_features: int, device, dtype=torch.bfloat16, group=None) -> FusedOutputProjection:
    """One ``FusedOutputProjection`` per (sizes, device, dtype, group) for all layers of a stack: every layer's
    projection reuses the same symmetric buffers, so a layer's output must be consumed (the residual add)
    before the next layer's projection is enqueued - which stream order gives for free.  All ranks must ask in
    the same order (the first request allocates and exchanges the buffers, a collective step)."""
    key = (int(max_rows), int(out_features), str(torch.device(device)), dtype, id(group))
    proj = _SHARED_PROJECTIONS.get(key)
    if proj is None:
        proj = _SHARED_PROJECTIONS[key] = FusedOutputProjection(max_rows, out_features, device, dtype, group)
    return proj


def fused_projection_applies(x: torch.Tensor, weight: torch.Tensor, bias, max_rows: int) -> bool:
    """Whether ``linear(x, weight)`` + sum over ranks can go through the fused kernels: more than one rank,
    no bias, 16-bit operands, K a multiple of 64, N a multiple of 256, rows within the buffers."""
    if not (dist.is_initialized() and dist.get_world_size() > 1) or bias is not None or not x.is_cuda:
        return False
    if x.dtype not in (torch.bfloat16, torch.float16) or weight.dtype != x.dtype or weight.stride(1) != 1 or x.stride(-1) != 1:
        return False
    rows = x.numel() // x.shape[-1]
    return 0 < rows <= max_rows and x.shape[-1] % 64 == 0 and weight.shape[0] % 256 == 0


def project_and_reduce(x: torch.Tensor, weight: torch.Tensor, max_rows: int) -> torch.Tensor:
    """``linear(x, weight)`` summed over the ranks through the shared fused projection."""
    proj = shared_fused_projection(max_rows, weight.shape[0], x.device, x.dtype)
    return proj(x, weight)


def max_over_ranks(values, device, group=None):
    """Element-wise max of a list of floats over the ranks (multi-GPU timings are max over ranks)."""
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return [float(x) for x in t]
