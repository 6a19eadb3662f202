"""Tensor-level wrappers over the C ABI: each function checks its torch arguments, fills the C
struct with raw device pointers / element strides and enqueues the kernels on the current CUDA
stream. Nothing here computes on the host and nothing falls back to torch ops.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

_DTYPES = {torch.bfloat16: _lib.CA_DTYPE_BF16, torch.float16: _lib.CA_DTYPE_F16, torch.float32: _lib.CA_DTYPE_F32}


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("compactattention_b200 runs on CUDA tensors only (no CPU path)")


@dataclass
class KvCacheView:
    """Addressing of a source KV cache (see ``ca_kv_layout`` in the C header).

    ``k``/``v`` are the tensors that own the memory; strides are in elements.
    """

    k: torch.Tensor
    v: torch.Tensor
    page_stride: int
    token_stride: int
    head_stride: int
    page_size: int
    num_pages: int
    pages_per_seq: int
    page_table: Optional[torch.Tensor] = None  # int32 [B, pages_per_seq]

    @staticmethod
    def from_seq_first(k: torch.Tensor, v: torch.Tensor) -> "KvCacheView":
        """``[B, K, Hkv, D]`` tensors (the reference's ``key_states`` layout); K % 64 == 0."""
        B, K, Hkv, D = k.shape
        if K % 64 != 0:
            raise ValueError(f"kv_len {K} must be a multiple of 64")
        if k.stride() != v.stride() or k.stride(3) != 1:
            raise ValueError("k and v must share strides and have a contiguous head dim")
        if B > 1 and k.stride(0) != K * k.stride(1):
            raise ValueError("batch stride must equal K * token stride")
        return KvCacheView(k, v, 64 * k.stride(1), k.stride(1), k.stride(2), 64, B * (K // 64), K // 64)

    @staticmethod
    def from_heads_first(k: torch.Tensor, v: torch.Tensor) -> "KvCacheView":
        """``[B, Hkv, K, D]`` tensors (the reference's ``k_hf`` layout); K % 64 == 0."""
        B, Hkv, K, D = k.shape
        if K % 64 != 0:
            raise ValueError(f"kv_len {K} must be a multiple of 64")
        if k.stride() != v.stride() or k.stride(3) != 1:
            raise ValueError("k and v must share strides and have a contiguous head dim")
        if B > 1:
            raise ValueError("heads-first views are supported for B == 1; use a paged cache for batches")
        return KvCacheView(k, v, 64 * k.stride(2), k.stride(2), k.stride(1), 64, K // 64, K // 64)

    @staticmethod
    def from_paged(k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor) -> "KvCacheView":
        """``[num_pages, page_size, Hkv, D]`` physical pages and an int32 ``[B, pages_per_seq]`` table."""
        num_pages, page_size, Hkv, D = k_pages.shape
        if k_pages.stride() != v_pages.stride() or k_pages.stride(3) != 1:
            raise ValueError("k_pages and v_pages must share strides and have a contiguous head dim")
        if page_table.dtype != torch.int32 or page_table.dim() != 2 or not page_table.is_contiguous():
            raise ValueError("page_table must be a contiguous int32 [B, pages_per_seq] tensor")
        return KvCacheView(k_pages, v_pages, k_pages.stride(0), k_pages.stride(1), k_pages.stride(2), page_size,
                           num_pages, page_table.shape[1], page_table)

    def to_c(self) -> _lib.KvLayout:
        return _lib.KvLayout(self.k.data_ptr(), self.v.data_ptr(), self.page_stride, self.token_stride,
                             self.head_stride, self.page_size, self.num_pages, self.pages_per_seq, 0,
                             _ptr(self.page_table))


def attn_compact(
    q: torch.Tensor,  # [B, Q, Hq, D]
    kv: KvCacheView,
    kv_len: int,
    num_kv_heads: int,
    block_idx: Optional[torch.Tensor],  # int32 [B*Hkv, cap] or [B, Hkv, cap]; None = every past block
    counts: Optional[torch.Tensor],  # int32 [B*Hkv] / [B, Hkv]
    block_size: int = 64,
    softmax_scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Dense causal attention over the selected KV blocks, read in place through the block table."""
    _require_cuda(q, kv.k, kv.v, block_idx, counts, out, lse, status)
    B, Q, Hq, D = q.shape
    if q.dtype not in (torch.bfloat16, torch.float16) or kv.k.dtype != q.dtype or kv.v.dtype != q.dtype:
        raise ValueError("q, k, v must share dtype bfloat16 or float16")
    if q.stride(3) != 1:
        raise ValueError("q must have a contiguous head dim")
    if out is None:
        out = torch.empty((B, Q, Hq, D), dtype=q.dtype, device=q.device)
    if out.stride(3) != 1 or out.dtype != q.dtype:
        raise ValueError("out must match q's dtype and have a contiguous head dim")
    if block_idx is not None:
        if block_idx.dtype != torch.int32 or counts is None or counts.dtype != torch.int32:
            raise ValueError("block_idx and counts must be int32")
        if not block_idx.is_contiguous() or not counts.is_contiguous():
            raise ValueError("block_idx and counts must be contiguous")
        if block_idx.numel() // max(block_idx.shape[-1], 1) != B * num_kv_heads or counts.numel() != B * num_kv_heads:
            raise ValueError("block_idx/counts must have one row per (batch, kv head)")
    if lse is not None and (lse.dtype != torch.float32 or lse.shape != (B, Hq, Q) or not lse.is_contiguous()):
        raise ValueError("lse must be a contiguous float32 [B, Hq, Q] tensor")
    p = _lib.AttnParams()
    p.q, p.q_stride_b, p.q_stride_t, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
    p.out, p.o_stride_b, p.o_stride_t, p.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
    p.kv = kv.to_c()
    p.block_idx = _ptr(block_idx)
    p.counts = _ptr(counts)
    p.block_idx_stride = 0 if block_idx is None else block_idx.shape[-1]
    p.B, p.Q, p.Hq, p.Hkv, p.D = B, Q, Hq, num_kv_heads, D
    p.kv_len = kv_len
    p.block_size = block_size
    p.dtype = _DTYPES[q.dtype]
    p.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    p.lse = _ptr(lse)
    p.workspace = None
    p.workspace_bytes = 0
    p.status = _ptr(status)
    lib = _lib.load()
    _lib.check(lib.ca_attn_compact(C.byref(p), _stream()), "ca_attn_compact")
    return out
