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
                 first_layer: int = 0, attention_layers=None, conv_layers=None, conv_channels: int = 0, conv_hist: int = 0):
        """``attention_layers`` / ``conv_layers``: global indices of the layers that keep K/V pages respectively a
        short-convolution state (hybrid models); by default every one of the ``n_layers`` layers keeps K/V.
        The convolution state pool [layer, page, conv_hist, channels] is indexed by a sequence's first page."""
        self.n_kv_heads, self.head_dim = n_kv_heads, head_dim
        self.num_pages = num_pages
        self.first_layer = first_layer
        if attention_layers is None:
            attention_layers = list(range(first_layer, first_layer + n_layers))
        self._kv_index = {li: i for i, li in enumerate(attention_layers)}
        self.n_layers = len(attention_layers)
        self.k = torch.zeros((self.n_layers, num_pages, n_kv_heads, PAGE, head_dim), dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)
        self._conv_index = {li: i for i, li in enumerate(conv_layers or [])}
        self.conv_state = None
        if self._conv_index:
            self.conv_state = torch.zeros((len(self._conv_index), num_pages, conv_hist, conv_channels), dtype=dtype,
                                          device=device)
        try:
            from ..lib import _eredu_host  # type: ignore

            self.allocator = _eredu_host.BlockManager(num_pages)
        except Exception:
            self.allocator = PageAllocator(num_pages)

    def layer(self, li: int):
        i = self._kv_index[li]
        return self.k[i], self.v[i]

    def conv_layer(self, li: int):
        return self.conv_state[self._conv_index[li]]

    def bytes(self) -> int:
        extra = self.conv_state.numel() * self.conv_state.element_size() if self.conv_state is not None else 0
        return 2 * self.k.numel() * self.k.element_size() + extra

    @staticmethod
    def pages_for(tokens: int) -> int:
        return (tokens + PAGE - 1) // PAGE
