"""Paged KV cache with FP8 pages.

Pool layout per layer (what the CUDA kernels index), chosen so that the decode-attention kernel can fetch a
page with one bulk copy and read tensor-core fragments with single shared-memory loads:

* ``k : [pages, kv_heads, head_dim/64, page_size, 64]`` E4M3 (64-dim chunks, token-major inside a chunk);
* ``v : [pages, kv_heads, head_dim, page_size]`` E4M3, transposed, the 16 token slots of a page stored in the
  order ``0,1,8,9, 2,3,10,11, 4,5,12,13, 6,7,14,15`` (:data:`V_TOKEN_ORDER`);
* ``k_scale, v_scale : [pages, kv_heads, page_size]`` fp32 (one multiplier per token and head).

:func:`k_logical` / :func:`v_logical` give the plain ``[pages, kv_heads, page_size, head_dim]`` views.
Pages are 16 tokens, like the reference's paged cache (``cpp_runtime/backends/cuda/models/qwen35/paged_kv.h:25-26``),
whose pages hold fp16/bf16 or TurboQuant codes; FP8 pages halve the decode-attention traffic.  The host
side keeps a free list and per-sequence page lists; a sequence's block-table row is written to a device
tensor that the kernels (and the captured decode graph) read.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

PAGE_SIZE = 16
V_TOKEN_ORDER = (0, 1, 8, 9, 2, 3, 10, 11, 4, 5, 12, 13, 6, 7, 14, 15)  # slot p holds token V_TOKEN_ORDER[p]
V_SLOT_OF_TOKEN = tuple(V_TOKEN_ORDER.index(t) for t in range(16))


def k_logical(k: torch.Tensor) -> torch.Tensor:
    """``[..., D/64, page, 64]`` physical -> ``[..., page, D]`` logical (a copy)."""
    return k.transpose(-3, -2).reshape(*k.shape[:-3], k.shape[-2], k.shape[-3] * k.shape[-1])


def v_logical(v: torch.Tensor) -> torch.Tensor:
    """``[..., D, page(slot order)]`` physical -> ``[..., page, D]`` logical (a copy)."""
    slots = torch.tensor(V_SLOT_OF_TOKEN, device=v.device)
    return v.index_select(-1, slots).transpose(-1, -2)


@dataclass
class LayerKV:
    k: torch.Tensor
    v: torch.Tensor
    k_scale: torch.Tensor
    v_scale: torch.Tensor
    page_size: int


class PageAllocator:
    """Host-side free list of physical pages (page 0 is reserved as the null page)."""

    def __init__(self, num_pages: int) -> None:
        self.num_pages = num_pages
        self.free = list(range(num_pages - 1, 0, -1))
        self.owned: dict[int, list[int]] = {}

    @property
    def free_pages(self) -> int:
        return len(self.free)

    def pages_for(self, tokens: int, page_size: int = PAGE_SIZE) -> int:
        return (tokens + page_size - 1) // page_size

    def ensure(self, seq_id: int, tokens: int, page_size: int = PAGE_SIZE) -> list[int]:
        """Grow ``seq_id`` to hold ``tokens`` tokens; raises ``MemoryError`` when the pool is exhausted."""
        pages = self.owned.setdefault(seq_id, [])
        need = self.pages_for(tokens, page_size) - len(pages)
        if need > len(self.free):
            raise MemoryError(f"KV pool exhausted: need {need} pages, {len(self.free)} free")
        for _ in range(max(0, need)):
            pages.append(self.free.pop())
        return pages

    def release(self, seq_id: int) -> None:
        for p in self.owned.pop(seq_id, []):
            self.free.append(p)


class PagedKVCache:
    def __init__(self, *, layers: int, kv_heads: int, head_dim: int, num_pages: int, max_seqs: int,
                 max_pages_per_seq: int, device: torch.device | str, page_size: int = PAGE_SIZE) -> None:
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_pages_per_seq = max_pages_per_seq
        dev = torch.device(device)
        if page_size != 16 or head_dim % 64:
            raise ValueError("the FP8 page layout needs 16-token pages and a head dim that is a multiple of 64")
        self.head_dim, self.kv_heads, self.layers = head_dim, kv_heads, layers
        self.k = torch.zeros((layers, num_pages, kv_heads, head_dim // 64, page_size, 64), dtype=torch.float8_e4m3fn, device=dev)
        self.v = torch.zeros((layers, num_pages, kv_heads, head_dim, page_size), dtype=torch.float8_e4m3fn, device=dev)
        self.k_scale = torch.zeros((layers, num_pages, kv_heads, page_size), dtype=torch.float32, device=dev)
        self.v_scale = torch.zeros((layers, num_pages, kv_heads, page_size), dtype=torch.float32, device=dev)
        self.block_table = torch.zeros((max_seqs, max_pages_per_seq), dtype=torch.int32, device=dev)
        self.allocator = PageAllocator(num_pages)

    def layer(self, i: int) -> LayerKV:
        return LayerKV(self.k[i], self.v[i], self.k_scale[i], self.v_scale[i], self.page_size)

    # -- page export / import (prefix cache, session snapshots) ------------------------------------------------------
    def export_pages(self, page_ids: list[int]):
        """All layers' K, V and multipliers of the given pages as one contiguous uint8 numpy array (host)."""
        import numpy as np
        idx = torch.tensor(page_ids, dtype=torch.long, device=self.k.device)
        parts = [(t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t).index_select(1, idx).contiguous().view(torch.uint8).reshape(-1)
                 for t in (self.k, self.v, self.k_scale, self.v_scale)]
        return np.ascontiguousarray(torch.cat(parts).cpu().numpy())

    def page_blob_bytes(self, pages: int) -> int:
        per = self.kv_heads * self.page_size * (2 * self.head_dim + 8)
        return self.layers * pages * per

    def import_pages(self, page_ids: list[int], blob) -> None:
        """Inverse of :meth:`export_pages` into (possibly different) physical pages."""
        idx = torch.tensor(page_ids, dtype=torch.long, device=self.k.device)
        raw = torch.from_numpy(blob).to(self.k.device)
        off = 0
        for t in (self.k, self.v, self.k_scale, self.v_scale):
            shape = (t.shape[0], len(page_ids)) + tuple(t.shape[2:])
            n = 1
            for d in shape:
                n *= d
            nbytes = n * t.element_size()
            src = raw[off : off + nbytes]
            if t.dtype == torch.float8_e4m3fn:  # index ops go through the byte view (no fp8 index kernels on every device)
                t.view(torch.uint8).index_copy_(1, idx, src.view(shape))
            else:
                t.index_copy_(1, idx, src.view(t.dtype).view(shape))
            off += nbytes

    def bytes_per_token(self) -> int:
        return self.layers * self.kv_heads * (2 * self.head_dim + 8)

    def assign(self, row: int, seq_id: int, tokens: int) -> None:
        """Make block-table ``row`` cover ``tokens`` tokens of ``seq_id`` (allocating pages as needed)."""
        pages = self.allocator.ensure(seq_id, tokens, self.page_size)
        if len(pages) > self.max_pages_per_seq:
            raise MemoryError("sequence exceeds max_pages_per_seq")
        self.block_table[row, : len(pages)] = torch.tensor(pages, dtype=torch.int32)

    def slots(self, seq_id: int, start: int, count: int) -> torch.Tensor:
        pages = self.allocator.owned[seq_id]
        pos = torch.arange(start, start + count)
        page_ids = torch.tensor(pages, dtype=torch.int64)[pos // self.page_size]
        return (page_ids * self.page_size + pos % self.page_size).to(torch.int32)

    def release(self, seq_id: int) -> None:
        self.allocator.release(seq_id)
