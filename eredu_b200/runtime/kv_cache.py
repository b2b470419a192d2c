"""Paged KV pool on the device: 16-token pages, one pool per layer, block tables per sequence.

The pool replaces the reference's per-request growing caches and its block store
(eredu/src/backend/mlx/runtime/cache/kv.rs:2781-2860 chunked growth, :1535-1627 paged truncate):
pages are fixed [n_kv, 16, head_dim] slabs inside two large tensors (K and V) per model shard, so a
sequence's cache is a list of page ids and truncation (speculative rollback) is a length change.
Page 0 is never handed out: padded block-table entries point at it.
"""
from __future__ import annotations

import torch

PAGE = 16


class PageAllocator:
    """Free-list page allocator (host side). The C++ block manager (``_eredu_host.BlockManager``) has the
    same interface and is used when the native module is built; this is the portable fallback."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, 0, -1))

    def free_pages(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> list[int]:
        if n > len(self._free):
            raise MemoryError(f"KV pool exhausted: need {n} pages, {len(self._free)} free")
        out = self._free[-n:][::-1] if n else []
        del self._free[len(self._free) - n:]
        return out

    def release(self, pages) -> None:
        self._free.extend(reversed(list(pages)))


class PagedKVCache:
    def __init__(self, n_layers: int, n_kv_heads: int, head_dim: int, num_pages: int, dtype, device,
                 first_layer: int = 0):
        self.n_layers, self.n_kv_heads, self.head_dim = n_layers, n_kv_heads, head_dim
        self.num_pages = num_pages
        self.first_layer = first_layer
        self.k = torch.zeros((n_layers, num_pages, n_kv_heads, PAGE, head_dim), dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)
        try:
            from ..lib import _eredu_host  # type: ignore

            self.allocator = _eredu_host.BlockManager(num_pages)
        except Exception:
            self.allocator = PageAllocator(num_pages)

    def layer(self, li: int):
        i = li - self.first_layer
        return self.k[i], self.v[i]

    def bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()

    @staticmethod
    def pages_for(tokens: int) -> int:
        return (tokens + PAGE - 1) // PAGE
