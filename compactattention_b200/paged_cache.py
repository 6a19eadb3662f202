"""Paged KV cache in HBM: physical pages ``[num_pages, page_size, Hkv, D]`` plus an int32 page table
``[B, pages_per_seq]`` (logical page -> physical page).  Appending a chunk writes only the chunk's
pages; nothing is re-copied as the sequence grows (the reference's ``DynamicCache.update``
concatenates the whole layer cache every chunk,
compact_attn/prefill_sparse/llama/modeling_llama_seerattn_chunked_dense.py:518-536).
The attention and gather kernels address it through ``ops.KvCacheView``.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


class PagedKVCache:
    def __init__(self, batch: int, max_tokens: int, num_kv_heads: int, head_dim: int, device, dtype=torch.bfloat16,
                 page_size: int = 64, page_table: Optional[torch.Tensor] = None):
        if page_size % 64 or max_tokens % page_size:
            raise ValueError("page_size must be a multiple of 64 and divide max_tokens")
        self.batch, self.page_size = batch, page_size
        self.pages_per_seq = max_tokens // page_size
        n = batch * self.pages_per_seq
        # zero-filled: a chunk that ends inside a page leaves the page's tail unwritten, and the attention
        # kernel multiplies those value rows by exact zeros, which must not meet NaN or Inf bit patterns
        self.k_pages = torch.zeros((n, page_size, num_kv_heads, head_dim), dtype=dtype, device=device)
        self.v_pages = torch.zeros_like(self.k_pages)
        if page_table is None:
            page_table = torch.arange(n, dtype=torch.int32, device=device).view(batch, self.pages_per_seq)
        if page_table.shape != (batch, self.pages_per_seq) or page_table.dtype != torch.int32:
            raise ValueError("page_table must be int32 [batch, max_tokens // page_size]")
        self.page_table = page_table.contiguous()
        self.length = 0  # tokens held per sequence

    def append(self, k_chunk: torch.Tensor, v_chunk: torch.Tensor, position: Optional[int] = None) -> int:
        """Writes ``[B, Q, Hkv, D]`` at token ``position`` (default: the current length); Q and the
        position must be page multiples.  Returns the new length."""
        pos = self.length if position is None else int(position)
        B, Q = k_chunk.shape[0], k_chunk.shape[1]
        if pos % self.page_size or Q % self.page_size:
            raise ValueError("chunks must start and end on page boundaries")
        p0, n = pos // self.page_size, Q // self.page_size
        if p0 + n > self.pages_per_seq:
            raise ValueError("chunk does not fit in the cache")
        ids = self.page_table[:, p0 : p0 + n].reshape(-1).to(torch.long)
        self.k_pages.index_copy_(0, ids, k_chunk.reshape(B * n, self.page_size, *k_chunk.shape[2:]))
        self.v_pages.index_copy_(0, ids, v_chunk.reshape(B * n, self.page_size, *v_chunk.shape[2:]))
        self.length = max(self.length, pos + Q)
        return self.length

    def append_rope(self, q: Optional[torch.Tensor], k_chunk: torch.Tensor, v_chunk: torch.Tensor, cos: torch.Tensor,
                    sin: torch.Tensor, position: Optional[int] = None, mean_k: Optional[torch.Tensor] = None,
                    block_size: int = 64, q_out: Optional[torch.Tensor] = None):
        """Fused form of ``apply_rotary_pos_emb`` + ``append`` (+ mean-K pooling): pre-RoPE
        ``q/k_chunk`` in, rotated queries out, rotated keys and the values written to the chunk's
        pages in one launch.  Any token position is accepted (no page-boundary rule).  Returns
        ``(q_rotated, new_length)``."""
        pos = self.length if position is None else int(position)
        Q = k_chunk.shape[1]
        if pos + Q > self.pages_per_seq * self.page_size:
            raise ValueError("chunk does not fit in the cache")
        q_rot = ops.rope_append(q, k_chunk, v_chunk, cos, sin, self.view(), pos, mean_k=mean_k, block_size=block_size, q_out=q_out)
        self.length = max(self.length, pos + Q)
        return q_rot, self.length

    def view(self) -> ops.KvCacheView:
        v = getattr(self, "_view", None)
        if v is None:  # pages and table never move: build the addressing once
            v = self._view = ops.KvCacheView.from_paged(self.k_pages, self.v_pages, self.page_table)
        return v
