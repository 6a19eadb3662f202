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


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Handle of torch's current stream on the current device.  The raw accessor costs well under a
    microsecond; ``torch.cuda.current_stream()`` builds a Stream object and costs ~12 us per call,
    which was a third of a wrapper's host time."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
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
    head_div: int = 0  # > 1: block-table row r reads KV head r // head_div (see ``with_head_div``)

    def with_head_div(self, rows_per_kv_head: int) -> "KvCacheView":
        """The same cache addressed by ``rows_per_kv_head`` block-table rows per KV head: per-query-head
        tables (``rows_per_kv_head = G``) or query-sub-group tables (``G // sub-group size``), the
        reference's ``fi_zero_copy_per_query`` / ``fi_zero_copy_subgroup`` routes.  Only
        ``attn_compact`` accepts such a view."""
        if rows_per_kv_head < 1:
            raise ValueError("rows_per_kv_head must be positive")
        import dataclasses
        return dataclasses.replace(self, head_div=int(rows_per_kv_head))

    @staticmethod
    def from_seq_first(k: torch.Tensor, v: torch.Tensor) -> "KvCacheView":
        """``[B, K, Hkv, D]`` tensors (the reference's ``key_states`` layout).  A length that is a
        multiple of 64 is viewed as 64-token pages; any other length as one page per sequence, whose
        ragged end the attention kernel's loads fill with zeros (only ``attn_compact`` takes such a view)."""
        B, K, Hkv, D = k.shape
        if k.stride() != v.stride() or k.stride(3) != 1:
            raise ValueError("k and v must share strides and have a contiguous head dim")
        if K % 64 != 0:
            return KvCacheView(k, v, k.stride(0), k.stride(1), k.stride(2), K, B, 1)
        if B > 1 and k.stride(0) != K * k.stride(1):
            raise ValueError("batch stride must equal K * token stride")
        return KvCacheView(k, v, 64 * k.stride(1), k.stride(1), k.stride(2), 64, B * (K // 64), K // 64)

    @staticmethod
    def from_heads_first(k: torch.Tensor, v: torch.Tensor) -> "KvCacheView":
        """``[B, Hkv, K, D]`` tensors (the reference's ``k_hf`` layout), B == 1; a ragged K is one page."""
        B, Hkv, K, D = k.shape
        if k.stride() != v.stride() or k.stride(3) != 1:
            raise ValueError("k and v must share strides and have a contiguous head dim")
        if B > 1:
            raise ValueError("heads-first views are supported for B == 1; use a paged cache for batches")
        if K % 64 != 0:
            return KvCacheView(k, v, k.stride(0), k.stride(2), k.stride(1), K, 1, 1)
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
                             self.head_stride, self.page_size, self.num_pages, self.pages_per_seq, self.head_div,
                             _ptr(self.page_table))


_ATTN_WORKSPACES: dict = {}


def attn_workspace(device: torch.device, params: "_lib.AttnParams") -> torch.Tensor:
    """Scratch for the attention kernel's split units (partial accumulators of the segments that the
    combine kernel merges).  One buffer per (device, stream): launches on one stream run in order, so
    they can share it; launches on different streams must not."""
    key = (device.index, _stream())
    ws = _ATTN_WORKSPACES.get(key)
    if ws is None:
        need = C.c_size_t(0)
        _lib.check(_lib.load().ca_attn_workspace_bytes(C.byref(params), C.byref(need)), "ca_attn_workspace_bytes")
        ws = torch.empty(max(int(need.value), 256), dtype=torch.uint8, device=device)
        _ATTN_WORKSPACES[key] = ws
    return ws


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
    workspace: Optional[torch.Tensor] = None,
    use_workspace: bool = True,
) -> torch.Tensor:
    """Dense causal attention over the selected KV blocks, read in place through the block table.

    With a workspace (default: a cached per-stream buffer) the kernel may cut work units across SMs
    and merge the pieces; ``use_workspace=False`` keeps every unit on one SM."""
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
    if use_workspace:
        ws = attn_workspace(q.device, p) if workspace is None else workspace
        p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel() * ws.element_size()
    lib = _lib.load()
    _lib.check(lib.ca_attn_compact(C.byref(p), _stream()), "ca_attn_compact")
    return out


def attn_compact_static_scratch(
    q: torch.Tensor,  # [B, Q, Hq, D]
    kv: KvCacheView,
    kv_len: int,
    num_kv_heads: int,
    block_idx: Optional[torch.Tensor],
    counts: Optional[torch.Tensor],
    out: torch.Tensor,  # [B, Q, Hq, D], required: this route allocates nothing, here or in the library
    block_size: int = 64,
    softmax_scale: Optional[float] = None,
    lse: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``attn_compact`` for hosts that may not allocate device memory (an engine that has given all
    of HBM to its own pool, a loop in which allocation is banned).  The kernel's scratch is a buffer
    built into the library (41.6 MiB per GPU, devices of up to 160 SMs) instead of a workspace
    tensor.  Every call on a device shares that buffer, so calls must be ordered on one stream, and
    the first call on a device (which looks the buffer's address up) belongs outside any stream
    capture."""
    _require_cuda(q, kv.k, kv.v, block_idx, counts, out, lse, status)
    B, Q, Hq, D = q.shape
    if q.dtype not in (torch.bfloat16, torch.float16) or kv.k.dtype != q.dtype or out.dtype != q.dtype:
        raise ValueError("q, k, v, out must share dtype bfloat16 or float16")
    if q.stride(3) != 1 or out.stride(3) != 1:
        raise ValueError("q and out must have a contiguous head dim")
    if block_idx is not None and (block_idx.dtype != torch.int32 or counts is None or counts.dtype != torch.int32
                                  or not block_idx.is_contiguous() or not counts.is_contiguous()):
        raise ValueError("block_idx and counts must be contiguous int32")
    p = _lib.AttnParams()
    p.q, p.q_stride_b, p.q_stride_t, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
    p.out, p.o_stride_b, p.o_stride_t, p.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
    p.kv = kv.to_c()
    p.block_idx, p.counts = _ptr(block_idx), _ptr(counts)
    p.block_idx_stride = 0 if block_idx is None else block_idx.shape[-1]
    p.B, p.Q, p.Hq, p.Hkv, p.D = B, Q, Hq, num_kv_heads, D
    p.kv_len, p.block_size, p.dtype = kv_len, block_size, _DTYPES[q.dtype]
    p.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    p.lse, p.status = _ptr(lse), _ptr(status)
    _lib.check(_lib.load().ca_attn_compact_static_scratch(C.byref(p), _stream()), "ca_attn_compact_static_scratch")
    return out


# ---------------------------------------------------------------------------------------------
# Block selection
# ---------------------------------------------------------------------------------------------
RULES = {
    "threshold": _lib.CA_RULE_THRESHOLD,
    "alpha_rowmax": _lib.CA_RULE_ALPHA_ROWMAX,
    "topk": _lib.CA_RULE_TOPK,
    "cummass": _lib.CA_RULE_CUMMASS,
    "mask": _lib.CA_RULE_MASK,
}


def words_for(kv_blocks: int) -> int:
    return (kv_blocks + 31) // 32


def _select_params(score, past_blocks, rule, valid, softmax, threshold, alpha, topk_k, topk_ratio, min_budget, sink, local,
                   rows_voting, bits, prob_out, bits_required=True, score_max=None):
    """Fills ``ca_select_params`` from torch arguments; returns (params, bits, tensors to keep alive)."""
    _require_cuda(score, valid, bits, prob_out)
    B, H, Qb, Kb = score.shape
    p = _lib.SelectParams()
    if rule == "mask":
        if score.dtype not in (torch.bool, torch.uint8):
            raise ValueError("rule 'mask' needs a bool/uint8 tensor")
        p.score_dtype = 0
    else:
        if score.dtype not in _DTYPES:
            raise ValueError(f"unsupported score dtype {score.dtype}")
        p.score_dtype = _DTYPES[score.dtype]
    if bits is None and bits_required:
        bits = torch.empty((B, H, Qb, words_for(Kb)), dtype=torch.int32, device=score.device)
    if bits is not None and (bits.dtype != torch.int32 or not bits.is_contiguous() or bits.shape != (B, H, Qb, words_for(Kb))):
        raise ValueError("bits must be a contiguous int32 [B,H,Qb,ceil(Kb/32)] tensor")
    if prob_out is not None and (prob_out.dtype != torch.float32 or not prob_out.is_contiguous() or prob_out.shape != (B, H, Qb, Kb)):
        raise ValueError("prob_out must be a contiguous float32 [B,H,Qb,Kb] tensor")
    p.score = score.data_ptr()
    p.score_stride_b, p.score_stride_h, p.score_stride_q, p.score_stride_k = score.stride()
    p.rule = RULES[rule]
    if valid is not None:
        if valid.dtype not in (torch.bool, torch.uint8) or valid.dim() != 4:
            raise ValueError("valid must be a bool [B,1|H,Qb,Kb] tensor")
        valid = valid.expand(B, valid.shape[1], Qb, Kb)
        p.valid = valid.data_ptr()
        sb, sh, sq, sk = valid.stride()
        p.valid_stride_b, p.valid_stride_h, p.valid_stride_q, p.valid_stride_k = sb, (sh if valid.shape[1] > 1 else 0), sq, sk
    p.bits = _ptr(bits)
    p.prob_out = _ptr(prob_out)
    p.B, p.H, p.Qb, p.Kb, p.Pb = B, H, Qb, Kb, past_blocks
    p.softmax = int(softmax)
    keep_thr = None
    if isinstance(threshold, torch.Tensor):
        # a scalar or per-batch threshold tensor stays on the device: the kernel reads it (no .item() sync)
        if threshold.numel() not in (1, B) or threshold.dim() > 1:
            raise ValueError(f"Expected scalar or 1D batch threshold tensor, got shape={tuple(threshold.shape)}")
        keep_thr = threshold.detach().to(device=score.device, dtype=torch.float32).reshape(-1).contiguous()
        p.threshold_ptr, p.threshold_stride_b = keep_thr.data_ptr(), (1 if keep_thr.numel() > 1 else 0)
        threshold = 0.0
    p.threshold, p.alpha = float(threshold), float(alpha)
    p.topk_k = int(topk_k)
    p.topk_num, p.topk_den = (topk_ratio if topk_ratio is not None else (0, 1))
    p.min_budget, p.sink, p.local, p.rows_voting = int(min_budget), int(sink), int(local), int(rows_voting)
    if score_max is not None:
        # per-entry exponents with the score's shape and strides: the rule sees score * 2^(score_max - row max)
        if score_max.dtype != torch.float32 or score.dtype != torch.float32 or score_max.shape != score.shape or \
                score_max.stride() != score.stride() or not score_max.is_cuda:
            raise ValueError("score_max must be a float32 CUDA tensor with the score's shape and strides (and the score float32)")
        p.score_max = score_max.data_ptr()
    return p, bits, (valid, keep_thr, score_max)


def select_rows(
    score: torch.Tensor,  # [B, H, Qb, Kb] (any strides); bool/uint8 for rule "mask"
    past_blocks: int,
    rule: str,
    *,
    valid: Optional[torch.Tensor] = None,  # bool [B, 1|H, Qb, Kb]; None = block-causal
    softmax: bool = False,
    threshold=0.0,  # float, or a scalar / per-batch tensor read on the device
    alpha: float = 0.0,
    topk_k: int = 0,
    topk_ratio: Optional[tuple[int, int]] = None,  # (num, den): k = max(1, round_half_up(num*n_valid/den))
    min_budget: int = 0,
    sink: int = 0,
    local: int = 0,
    rows_voting: int = 0,
    bits: Optional[torch.Tensor] = None,
    prob_out: Optional[torch.Tensor] = None,
    score_max: Optional[torch.Tensor] = None,  # f32, the score's shape and strides: the rule sees score * 2^(score_max - row max)
) -> torch.Tensor:
    """Per-row selection rule -> packed keep bits int32 [B, H, Qb, ceil(Kb/32)]."""
    p, bits, keep = _select_params(score, past_blocks, rule, valid, softmax, threshold, alpha, topk_k, topk_ratio, min_budget,
                                   sink, local, rows_voting, bits, prob_out, score_max=score_max)
    _lib.check(_lib.load().ca_select_rows(C.byref(p), _stream()), "ca_select_rows")
    del keep
    return bits


_UNION_SCRATCH: dict = {}


def union_scratch(device: torch.device, batch: int, heads: int, num_kv_heads: int, q_blocks: int, kv_blocks: int) -> torch.Tensor:
    """Scratch of the fused selection + table launch: a ticket per KV-head row (zero on entry, left zero by the
    kernel) followed by room for the rows' packed bits.  One buffer per (device, stream) serves every call on
    that stream and ticket count (the ticket words must never have held anything else); it only grows."""
    key = (device.index, _stream(), batch * num_kv_heads)
    need = C.c_size_t(0)
    _lib.check(_lib.load().ca_select_union_scratch_bytes(batch, heads, num_kv_heads, q_blocks, kv_blocks, C.byref(need)),
               "ca_select_union_scratch_bytes")
    buf = _UNION_SCRATCH.get(key)
    if buf is None or buf.numel() * 4 < need.value:
        buf = torch.zeros((int(need.value) + 3) // 4, dtype=torch.int32, device=device)
        _UNION_SCRATCH[key] = buf
    return buf


def select_union_table(
    score: torch.Tensor,  # [B, Hkv*G, Qb, Kb]
    past_blocks: int,
    rule: str,
    *,
    num_kv_heads: int,
    block_size: int = 64,
    page_size: int = 256,
    keep_recent: int = 0,
    valid: Optional[torch.Tensor] = None,
    softmax: bool = False,
    threshold: float = 0.0,
    alpha: float = 0.0,
    topk_k: int = 0,
    topk_ratio: Optional[tuple[int, int]] = None,
    min_budget: int = 0,
    sink: int = 0,
    local: int = 0,
    rows_voting: int = 0,
    bits: Optional[torch.Tensor] = None,  # optional: the per-row bits are written only when given
    prob_out: Optional[torch.Tensor] = None,
    out: Optional["BlockTable"] = None,
    scratch: Optional[torch.Tensor] = None,
    score_max: Optional[torch.Tensor] = None,  # as in select_rows
    _gate=None,  # (GateScoreParams writing `score`, write_scores): set by gate_score_select
) -> "BlockTable":
    """``select_rows`` followed by ``union_table`` in ONE launch (see ``ca_select_union_table``): row rule,
    Q-block union, GQA union and the per-KV-head block table.  ``scratch`` must be zero on first use and
    must not be shared by calls that can overlap on the device (default: a cached per-stream buffer)."""
    B, H, Qb, Kb = score.shape
    if H % num_kv_heads != 0:
        raise ValueError(f"{H} score heads is not a multiple of {num_kv_heads} kv heads")
    if Kb - past_blocks != Qb:
        raise ValueError("the score must cover the chunk's own key blocks: Kb - past_blocks must equal Qb")
    p, bits, keep = _select_params(score, past_blocks, rule, valid, softmax, threshold, alpha, topk_k, topk_ratio, min_budget,
                                   sink, local, rows_voting, bits, prob_out, bits_required=False, score_max=score_max)
    dev = score.device
    if out is None:
        cap = max(past_blocks, 1)
        out = BlockTable(
            torch.empty((B, num_kv_heads, cap), dtype=torch.int32, device=dev),
            torch.empty((B, num_kv_heads), dtype=torch.int32, device=dev),
            torch.empty((B, num_kv_heads), dtype=torch.int32, device=dev),
            torch.empty((B, num_kv_heads), dtype=torch.int32, device=dev),
        )
    u = _lib.UnionParams()
    u.B, u.Hkv, u.G, u.Qin, u.Kb, u.Pb = B, num_kv_heads, H // num_kv_heads, Qb, Kb, past_blocks
    u.keep_recent = int(keep_recent)
    u.block_size, u.page_size = block_size, page_size
    u.block_idx, u.idx_stride = out.block_idx.data_ptr(), out.block_idx.shape[-1]
    u.counts = out.counts.data_ptr()
    u.cache_seqlens = out.cache_seqlens.data_ptr()
    u.pages_per_row = out.pages_per_row.data_ptr()
    if scratch is None:
        scratch = union_scratch(dev, B, H, num_kv_heads, Qb, Kb)
    if scratch.dtype != torch.int32 or not scratch.is_contiguous():
        raise ValueError("scratch must be a contiguous int32 tensor (zero on first use)")
    if _gate is not None:
        _lib.check(_lib.load().ca_gate_score_select(C.byref(_gate[0]), C.byref(p), C.byref(u), scratch.data_ptr(), scratch.numel() * 4,
                                                    1 if _gate[1] else 0, _stream()), "ca_gate_score_select")
    else:
        _lib.check(_lib.load().ca_select_union_table(C.byref(p), C.byref(u), scratch.data_ptr(), scratch.numel() * 4, _stream()),
                   "ca_select_union_table")
    del keep
    return out


@dataclass
class BlockTable:
    """Per-KV-head block table: ascending selected past block ids (-1 padded) and their counts."""

    block_idx: torch.Tensor  # int32 [B, Hkv, cap]
    counts: torch.Tensor  # int32 [B, Hkv]
    cache_seqlens: torch.Tensor  # int32 [B, Hkv] = (count + Qb) * bs
    pages_per_row: torch.Tensor  # int32 [B, Hkv]
    keep_kv: Optional[torch.Tensor] = None  # bool [B, Hkv, Kb]


def union_table(
    *,
    bits: Optional[torch.Tensor] = None,  # int32 [B, Hkv*G, Qin, W]
    mask: Optional[torch.Tensor] = None,  # bool [B, Hkv*G, Qin, Kb] or [B, Hkv*G, Kb]
    num_kv_heads: int,
    kv_blocks: int,
    past_blocks: int,
    block_size: int = 64,
    page_size: int = 256,
    keep_recent: int = 0,
    want_keep_kv: bool = False,
    out: Optional[BlockTable] = None,
) -> BlockTable:
    """Block-Union KV selection (Q-block union, GQA union) and compaction into the block table."""
    src = bits if bits is not None else mask
    if src is None or (bits is not None and mask is not None):
        raise ValueError("give exactly one of bits and mask")
    _require_cuda(src)
    p = _lib.UnionParams()
    if mask is not None:
        if mask.dtype not in (torch.bool, torch.uint8):
            raise ValueError("mask must be bool/uint8")
        if mask.dim() == 3:
            mask = mask.unsqueeze(2)
        B, Hin, Qin, Kb = mask.shape
        if Kb != kv_blocks:
            raise ValueError(f"mask has {Kb} key blocks, expected {kv_blocks}")
        p.mask = mask.data_ptr()
        p.mask_stride_b, p.mask_stride_h, p.mask_stride_q, p.mask_stride_k = mask.stride()
    else:
        if bits.dtype != torch.int32 or not bits.is_contiguous() or bits.shape[-1] != words_for(kv_blocks):
            raise ValueError("bits must be a contiguous int32 [B,H,Qin,ceil(Kb/32)] tensor")
        B, Hin, Qin, _ = bits.shape
        p.bits = bits.data_ptr()
    if Hin % num_kv_heads != 0:
        raise ValueError(f"{Hin} input heads is not a multiple of {num_kv_heads} kv heads")
    dev = src.device
    cap = max(past_blocks, 1)
    if out is None:
        out = BlockTable(
            torch.empty((B, num_kv_heads, cap), dtype=torch.int32, device=dev),
            torch.empty((B, num_kv_heads), dtype=torch.int32, device=dev),
            torch.empty((B, num_kv_heads), dtype=torch.int32, device=dev),
            torch.empty((B, num_kv_heads), dtype=torch.int32, device=dev),
            torch.empty((B, num_kv_heads, kv_blocks), dtype=torch.bool, device=dev) if want_keep_kv else None,
        )
    p.B, p.Hkv, p.G, p.Qin, p.Kb, p.Pb = B, num_kv_heads, Hin // num_kv_heads, Qin, kv_blocks, past_blocks
    p.keep_recent = int(keep_recent)
    p.block_size, p.page_size = block_size, page_size
    p.block_idx, p.idx_stride = out.block_idx.data_ptr(), out.block_idx.shape[-1]
    p.counts = out.counts.data_ptr()
    p.cache_seqlens = out.cache_seqlens.data_ptr()
    p.pages_per_row = out.pages_per_row.data_ptr()
    p.keep_kv = _ptr(out.keep_kv)
    _lib.check(_lib.load().ca_union_table(C.byref(p), _stream()), "ca_union_table")
    return out


def paged_metadata(pages_per_row: torch.Tensor, max_pages: int = 0):
    """Exclusive prefix of pages_per_row -> page_offsets [R+1]; optional block_table [R, max_pages]."""
    _require_cuda(pages_per_row)
    flat = pages_per_row.reshape(-1)
    R = flat.numel()
    offsets = torch.empty(R + 1, dtype=torch.int32, device=flat.device)
    table = torch.empty((R, max_pages), dtype=torch.int32, device=flat.device) if max_pages > 0 else None
    _lib.check(_lib.load().ca_paged_metadata(flat.data_ptr(), R, offsets.data_ptr(), _ptr(table), max_pages, _stream()),
               "ca_paged_metadata")
    return offsets, table


# ---------------------------------------------------------------------------------------------
# Block scoring
# ---------------------------------------------------------------------------------------------
_POOL_BITS = {"max": _lib.CA_POOL_MAX, "min": _lib.CA_POOL_MIN, "avg": _lib.CA_POOL_AVG}


def pool_blocks(
    x: torch.Tensor,  # [B, L, H, D]
    block_size: int,
    kinds: tuple[str, ...] = ("avg",),
    out: Optional[torch.Tensor] = None,  # [B, >= off + nb, H, nk*D] (any batch/block/head strides)
    out_block_offset: int = 0,
    out_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """max/min/avg pooling of token blocks, channels ordered max|min|avg; can append into a cache."""
    _require_cuda(x, out)
    B, L, H, D = x.shape
    if x.stride(3) != 1:
        raise ValueError("x must have a contiguous last dim")
    nb = (L + block_size - 1) // block_size
    bitsel = 0
    for k in kinds:
        bitsel |= _POOL_BITS[k]
    nk = bin(bitsel).count("1")
    if out is None:
        out = torch.empty((B, nb, H, nk * D), dtype=out_dtype or torch.float32, device=x.device)
    if out.stride(3) != 1 or out.shape[3] != nk * D or out.shape[1] < out_block_offset + nb:
        raise ValueError("out has the wrong shape for this pooling")
    p = _lib.PoolParams()
    p.x, p.x_stride_b, p.x_stride_t, p.x_stride_h = x.data_ptr(), x.stride(0), x.stride(1), x.stride(2)
    p.x_dtype, p.out_dtype = _DTYPES[x.dtype], _DTYPES[out.dtype]
    p.out, p.out_stride_b, p.out_stride_blk, p.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
    p.out_block_offset = out_block_offset
    p.B, p.L, p.H, p.D, p.block_size, p.kinds = B, L, H, D, block_size, bitsel
    _lib.check(_lib.load().ca_pool_blocks(C.byref(p), _stream()), "ca_pool_blocks")
    return out


def gate_project(
    x: torch.Tensor,  # f32 contiguous [B, nb, Hin, Cin]
    weight: Optional[torch.Tensor],  # [Hout, Cin, Cout] or None (identity)
    cos: Optional[torch.Tensor] = None,  # f32 [1|B, nb, Cout]
    sin: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,  # [B, >= off + nb, Hout, Cout]
    out_block_offset: int = 0,
    out_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """Per-head linear + block RoPE, written at a block offset of ``out`` (cache append)."""
    _require_cuda(x, weight, cos, sin, out)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise ValueError("x must be contiguous float32")
    B, nb, Hin, Cin = x.shape
    if weight is not None:
        if not weight.is_contiguous() or weight.shape[1] != Cin:
            raise ValueError("weight must be contiguous [Hout, Cin, Cout]")
        Hout, _, Cout = weight.shape
    else:
        Hout, Cout = Hin, Cin
    if cos is not None:
        cos, sin = cos.to(torch.float32).contiguous(), sin.to(torch.float32).contiguous()
        if cos.shape[-2:] != (nb, Cout) or sin.shape != cos.shape:
            raise ValueError("cos/sin must be [1|B, nb, Cout]")
    if out is None:
        out = torch.empty((B, nb, Hout, Cout), dtype=out_dtype or torch.float32, device=x.device)
    if out.stride(3) != 1 or out.shape[2] != Hout or out.shape[3] != Cout or out.shape[1] < out_block_offset + nb:
        raise ValueError("out has the wrong shape for this projection")
    p = _lib.ProjectParams()
    p.x, p.w = x.data_ptr(), _ptr(weight)
    p.w_dtype = _DTYPES[weight.dtype] if weight is not None else 0
    p.out_dtype = _DTYPES[out.dtype]
    p.cos, p.sin = _ptr(cos), _ptr(sin)
    p.rope_batch = cos.shape[0] if cos is not None else 1
    p.out_block_offset = out_block_offset
    p.out, p.out_stride_b, p.out_stride_blk, p.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
    p.B, p.nb, p.Hin, p.Hout, p.Cin, p.Cout = B, nb, Hin, Hout, Cin, Cout
    _lib.check(_lib.load().ca_gate_project(C.byref(p), _stream()), "ca_gate_project")
    return out


def _gate_side(x, kinds, weight, rope, out, out_block_offset):
    sd = _lib.GateSide()
    if x.stride(3) != 1:
        raise ValueError("token tensors must have a contiguous last dim")
    sd.x, sd.x_stride_b, sd.x_stride_t, sd.x_stride_h = x.data_ptr(), x.stride(0), x.stride(1), x.stride(2)
    sd.x_dtype, sd.H = _DTYPES[x.dtype], x.shape[2]
    bitsel = 0
    for k in kinds:
        bitsel |= _POOL_BITS[k]
    sd.kinds = bitsel
    if weight is not None:
        if not weight.is_contiguous():
            raise ValueError("gate weights must be contiguous [H, Cin, C]")
        sd.w, sd.w_dtype, sd.Hw = weight.data_ptr(), _DTYPES[weight.dtype], weight.shape[0]
    else:
        sd.Hw = x.shape[2]
    keep = []
    if rope is not None:
        cos, sin = rope
        cos, sin = cos.to(torch.float32).contiguous(), sin.to(torch.float32).contiguous()
        keep = [cos, sin]
        sd.cos, sd.sin, sd.rope_batch = cos.data_ptr(), sin.data_ptr(), cos.shape[0]
    else:
        sd.rope_batch = 1
    if out.stride(3) != 1 or out.shape[2] != sd.Hw:
        raise ValueError("gate block output has the wrong head count or a strided channel dim")
    sd.out, sd.out_stride_b, sd.out_stride_blk, sd.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
    sd.out_dtype, sd.out_block_offset = _DTYPES[out.dtype], out_block_offset
    return sd, keep


def gate_prepare(
    q: torch.Tensor,  # [B, L, Hq, D] chunk queries (pre-RoPE)
    k: torch.Tensor,  # [B, L, Hkv, D] chunk keys (pre-RoPE)
    block_size: int,
    q_kinds: tuple[str, ...],
    k_kinds: tuple[str, ...],
    wq: Optional[torch.Tensor],  # [Hq, nq*D, C] or None
    wk: torch.Tensor,  # [Hk, nk*D, C]
    rope_q: Optional[tuple[torch.Tensor, torch.Tensor]],  # f32 [1|B, nb, C] each, the chunk's block positions
    rope_k: Optional[tuple[torch.Tensor, torch.Tensor]],
    q_out: torch.Tensor,  # [B, >= nb, Hq, C]
    k_out: torch.Tensor,  # [B, >= off + nb, Hk, C] (block-major view of the K-block cache)
    k_out_block_offset: int = 0,
) -> None:
    """Pool + project + RoPE the chunk's Q and K blocks and append the K blocks, in one launch."""
    _require_cuda(q, k, wq, wk, q_out, k_out)
    B, L, _, D = q.shape
    if k.shape[0] != B or k.shape[1] != L or k.shape[3] != D:
        raise ValueError("q and k chunks must share batch, length and head dim")
    p = _lib.GatePrepareParams()
    p.q, keep_q = _gate_side(q, q_kinds, wq, rope_q, q_out, 0)
    p.k, keep_k = _gate_side(k, k_kinds, wk, rope_k, k_out, k_out_block_offset)
    p.B, p.L, p.D, p.C, p.block_size = B, L, D, q_out.shape[3], block_size
    if k_out.shape[3] != p.C:
        raise ValueError("q and k gate blocks must share the channel count")
    _lib.check(_lib.load().ca_gate_prepare(C.byref(p), _stream()), "ca_gate_prepare")
    del keep_q, keep_k


def gate_scores(
    q_blocks: torch.Tensor,  # [B, Qb, Hq, C]
    k_blocks: torch.Tensor,  # [B, Kb, Hk, C] (a view of the K-block cache)
    past_blocks: int,
    scale: Optional[float] = None,
    masked_value: float = float(torch.finfo(torch.float32).min),
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Gate logits [B, Hq, Qb, Kb] float32; entries above the block diagonal get masked_value."""
    p, out = _gate_score_params(q_blocks, k_blocks, past_blocks, scale, masked_value, out)
    _lib.check(_lib.load().ca_gate_scores(C.byref(p), _stream()), "ca_gate_scores")
    return out


def _gate_score_params(q_blocks, k_blocks, past_blocks, scale, masked_value, out):
    _require_cuda(q_blocks, k_blocks, out)
    B, Qb, Hq, Cc = q_blocks.shape
    Kb, Hk = k_blocks.shape[1], k_blocks.shape[2]
    if q_blocks.stride(3) != 1 or k_blocks.stride(3) != 1:
        raise ValueError("block tensors must have a contiguous channel dim")
    if out is None:
        out = torch.empty((B, Hq, Qb, Kb), dtype=torch.float32, device=q_blocks.device)
    if out.dtype != torch.float32 or not out.is_contiguous() or out.shape != (B, Hq, Qb, Kb):
        raise ValueError("out must be a contiguous float32 [B,Hq,Qb,Kb] tensor")
    p = _lib.GateScoreParams()
    p.q, p.q_stride_b, p.q_stride_blk, p.q_stride_h = q_blocks.data_ptr(), q_blocks.stride(0), q_blocks.stride(1), q_blocks.stride(2)
    p.k, p.k_stride_b, p.k_stride_blk, p.k_stride_h = k_blocks.data_ptr(), k_blocks.stride(0), k_blocks.stride(1), k_blocks.stride(2)
    p.q_dtype, p.k_dtype = _DTYPES[q_blocks.dtype], _DTYPES[k_blocks.dtype]
    p.out = out.data_ptr()
    p.B, p.Hq, p.Hk, p.Qb, p.Kb, p.Pb, p.C = B, Hq, Hk, Qb, Kb, past_blocks, Cc
    p.scale = float(scale) if scale is not None else Cc ** -0.5
    p.masked_value = masked_value
    return p, out


def gate_score_select(
    q_blocks: torch.Tensor,  # [B, Qb, Hq, C]
    k_blocks: torch.Tensor,  # [B, Kb, Hk, C] (a view of the K-block cache)
    past_blocks: int,
    rule: str,
    *,
    num_kv_heads: int,
    scores: Optional[torch.Tensor] = None,  # [B, Hq, Qb, Kb] f32 buffer of the logits (allocated when missing)
    write_scores: bool = False,
    scale: Optional[float] = None,
    masked_value: float = float(torch.finfo(torch.float32).min),
    **select_kwargs,
) -> "BlockTable":
    """``gate_scores`` + ``select_union_table`` behind ONE library call (``ca_gate_score_select``): the tensor-core
    score kernel, then the rule + Block-Union + table kernel.  ``scores`` always receives the logits
    (``write_scores`` is kept for callers of an earlier single-launch form and ignored).  ``select_kwargs`` are
    those of ``select_union_table``."""
    g, scores = _gate_score_params(q_blocks, k_blocks, past_blocks, scale, masked_value, scores)
    return select_union_table(scores, past_blocks, rule, num_kv_heads=num_kv_heads, _gate=(g, bool(write_scores)), **select_kwargs)


def flashprefill_score(
    q: torch.Tensor,  # [B, Q, Hq, D]
    mean_k: torch.Tensor,  # [B, Kb, Hkv, D]
    kv_len: int,
    block_size: int,
    normalize: bool = True,
):
    """Training-free block score -> (score_raw, max_raw, score_norm|None), each [B, Qb, Kb, Hq] f32."""
    _require_cuda(q, mean_k)
    B, Q, Hq, D = q.shape
    Kb, Hkv = mean_k.shape[1], mean_k.shape[2]
    Qb = (Q + block_size - 1) // block_size
    if q.stride(3) != 1 or mean_k.stride(3) != 1:
        raise ValueError("q and mean_k must have a contiguous head dim")
    raw = torch.empty((B, Qb, Kb, Hq), dtype=torch.float32, device=q.device)
    mx = torch.empty_like(raw)
    norm = torch.empty_like(raw) if normalize else None
    p = _lib.FlashPrefillScoreParams()
    p.q, p.q_stride_b, p.q_stride_t, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
    p.mean_k, p.k_stride_b, p.k_stride_blk, p.k_stride_h = mean_k.data_ptr(), mean_k.stride(0), mean_k.stride(1), mean_k.stride(2)
    p.q_dtype, p.k_dtype = _DTYPES[q.dtype], _DTYPES[mean_k.dtype]
    p.score_raw, p.max_raw, p.score_norm = raw.data_ptr(), mx.data_ptr(), _ptr(norm)
    p.B, p.Q, p.Hq, p.Hkv, p.D, p.Kb, p.block_size, p.kv_len = B, Q, Hq, Hkv, D, Kb, block_size, kv_len
    _lib.check(_lib.load().ca_flashprefill_score(C.byref(p), _stream()), "ca_flashprefill_score")
    return raw, mx, norm


# ---------------------------------------------------------------------------------------------
# Compact KV gather
# ---------------------------------------------------------------------------------------------
def gather_kv(
    kv: KvCacheView,
    num_kv_heads: int,
    batch: int,
    q_len: int,
    kv_len: int,
    block_idx: torch.Tensor,
    counts: torch.Tensor,
    k_dst: torch.Tensor,  # contiguous [tokens, D] (or [pages, page, 1, D])
    v_dst: torch.Tensor,
    *,
    block_size: int = 64,
    page_offsets: Optional[torch.Tensor] = None,
    dst_page_size: int = 256,
    dst_row_stride_tokens: int = 0,
    status: Optional[torch.Tensor] = None,
) -> None:
    """Copies the selected past blocks and the chunk of every (b, kv head) row into the compact cache."""
    _require_cuda(kv.k, kv.v, block_idx, counts, k_dst, v_dst, page_offsets, status)
    if not (k_dst.is_contiguous() and v_dst.is_contiguous()) or k_dst.dtype != kv.k.dtype:
        raise ValueError("destination caches must be contiguous and match the source dtype")
    if block_idx.dtype != torch.int32 or counts.dtype != torch.int32 or not block_idx.is_contiguous():
        raise ValueError("block_idx/counts must be contiguous int32")
    p = _lib.GatherParams()
    p.kv = kv.to_c()
    p.block_idx, p.counts, p.block_idx_stride = block_idx.data_ptr(), counts.data_ptr(), block_idx.shape[-1]
    p.dtype = _DTYPES[kv.k.dtype]
    p.page_offsets = _ptr(page_offsets)
    p.dst_row_stride_tokens = dst_row_stride_tokens
    p.k_dst, p.v_dst = k_dst.data_ptr(), v_dst.data_ptr()
    p.dst_page_size = dst_page_size
    p.B, p.Hkv, p.D, p.Q, p.kv_len, p.block_size = batch, num_kv_heads, kv.k.shape[-1], q_len, kv_len, block_size
    p.status = _ptr(status)
    _lib.check(_lib.load().ca_gather_kv(C.byref(p), _stream()), "ca_gather_kv")


def rope_append(
    q: Optional[torch.Tensor],  # [B, Q, Hq, D] pre-RoPE queries (or None)
    k: torch.Tensor,            # [B, Q, Hkv, D] pre-RoPE keys
    v: torch.Tensor,            # [B, Q, Hkv, D]
    cos: torch.Tensor,          # [B or 1, Q, D], the tensors' dtype or fp32
    sin: torch.Tensor,
    cache: KvCacheView,         # destination pages (written)
    position: int,
    *,
    mean_k: Optional[torch.Tensor] = None,  # [B, blocks, Hkv, D], block position/block_size + i is written
    block_size: int = 64,
    q_out: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
) -> Optional[torch.Tensor]:
    """One launch for a chunk: RoPE(q) -> q_out, RoPE(k) -> cache pages (+ per-block mean -> mean_k),
    v -> cache pages.  Returns q_out (allocated when q is given and q_out is not)."""
    _require_cuda(q, k, v, cos, sin, cache.k, cache.v, mean_k, q_out, status)
    if k.dim() != 4 or v.shape != k.shape or k.dtype != v.dtype or k.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("k and v must be [B, Q, Hkv, D] of one 16-bit dtype")
    B, Q, Hkv, D = k.shape
    if cache.k.dtype != k.dtype or cache.k.shape[-1] != D:
        raise ValueError("the cache must have the chunk's dtype and head dimension")
    if cos.shape != sin.shape or cos.dim() != 3 or cos.shape[1] != Q or cos.shape[2] != D or cos.shape[0] not in (1, B):
        raise ValueError("cos/sin must be [B or 1, Q, D] (the full head dimension is rotated)")
    if cos.dtype != sin.dtype or cos.dtype not in (k.dtype, torch.float32):
        raise ValueError("cos/sin must be fp32 or the tensors' dtype")
    for t in (q, k, v, cos, sin, mean_k, q_out):
        if t is not None and t.stride(-1) != 1:
            raise ValueError("the last dimension must be contiguous")
    p = _lib.RopeAppendParams()
    Hq = 0
    if q is not None:
        if q.dim() != 4 or q.shape[0] != B or q.shape[1] != Q or q.shape[3] != D or q.dtype != k.dtype:
            raise ValueError("q must be [B, Q, Hq, D] of the keys' dtype")
        Hq = q.shape[2]
        if q_out is None:
            q_out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        if q_out.shape != q.shape or q_out.dtype != q.dtype:
            raise ValueError("q_out must match q")
        p.q, p.q_out = q.data_ptr(), q_out.data_ptr()
        p.q_stride_b, p.q_stride_t, p.q_stride_h = q.stride(0), q.stride(1), q.stride(2)
        p.qo_stride_b, p.qo_stride_t, p.qo_stride_h = q_out.stride(0), q_out.stride(1), q_out.stride(2)
    p.k, p.v = k.data_ptr(), v.data_ptr()
    p.k_stride_b, p.k_stride_t, p.k_stride_h = k.stride(0), k.stride(1), k.stride(2)
    p.v_stride_b, p.v_stride_t, p.v_stride_h = v.stride(0), v.stride(1), v.stride(2)
    p.cos, p.sin = cos.data_ptr(), sin.data_ptr()
    if cos.stride() != sin.stride():
        raise ValueError("cos and sin must share their strides")
    p.cs_stride_b = 0 if cos.shape[0] == 1 else cos.stride(0)
    p.cs_stride_t = cos.stride(1)
    p.rope_dtype, p.dtype = _DTYPES[cos.dtype], _DTYPES[k.dtype]
    p.cache = cache.to_c()
    if mean_k is not None:
        if mean_k.dim() != 4 or mean_k.shape[0] != B or mean_k.shape[2] != Hkv or mean_k.shape[3] != D or mean_k.dtype != k.dtype:
            raise ValueError("mean_k must be [B, blocks, Hkv, D] of the keys' dtype")
        if position % block_size or position // block_size + -(-Q // block_size) > mean_k.shape[1]:
            raise ValueError("the chunk's blocks do not fit in mean_k at this position")
        p.mean_k = mean_k.data_ptr()
        p.mk_stride_b, p.mk_stride_blk, p.mk_stride_h = mean_k.stride(0), mean_k.stride(1), mean_k.stride(2)
    p.B, p.Q, p.Hq, p.Hkv, p.D = B, Q, Hq, Hkv, D
    p.position, p.block_size = int(position), block_size
    p.status = _ptr(status)
    _lib.check(_lib.load().ca_rope_append(C.byref(p), _stream()), "ca_rope_append")
    return q_out


def unpack_bits(bits: torch.Tensor, kv_blocks: int) -> torch.Tensor:
    """Packed keep bits [..., W] -> bool [..., Kb] (host-side helper for tests and statistics)."""
    shifts = torch.arange(32, device=bits.device, dtype=torch.int64)
    expanded = ((bits.to(torch.int64).unsqueeze(-1) & 0xFFFFFFFF) >> shifts) & 1
    return expanded.reshape(*bits.shape[:-1], -1)[..., :kv_blocks].to(torch.bool)
