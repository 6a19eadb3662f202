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


def max_over_ranks(values, device, group=None):
    """Element-wise max of a list of floats over the ranks (multi-GPU timings are max over ranks)."""
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return [float(x) for x in t]
