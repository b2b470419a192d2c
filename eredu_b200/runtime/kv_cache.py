"""Paged KV pool on the device: 16-token pages, one pool per layer, block tables per sequence.

The pool replaces the reference's per-request growing caches and its block store
(eredu/src/backend/mlx/runtime/cache/kv.rs:2781-2860 chunked growth, :1535-1627 paged truncate):
pages are fixed [n_kv, 16, head_dim] slabs inside two large tensors (K and V) per model shard, so a
sequence's cache is a list of page ids and truncation (speculative rollback) is a length change.
Page 0 is never handed out: padded block-table entries point at it.
"""
from __future__ import annotations

from typing import Optional

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
                 first_layer: int = 0, attention_layers=None, conv_layers=None, conv_channels: int = 0, conv_hist: int = 0,
                 value_dim: Optional[int] = None):
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
        # latent-attention models cache one row per token in ``k`` and nothing in ``v`` (value_dim 1 keeps the plumbing)
        self.v = torch.zeros_like(self.k) if value_dim in (None, head_dim) else \
            torch.zeros((self.n_layers, num_pages, n_kv_heads, PAGE, value_dim), dtype=dtype, device=device)
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
        # Recurrent state of gated-delta layers: too large to keep per page, so sequences get a compact state slot and
        # `page_to_slot` (indexed by a sequence's first page, read on the device) finds it.
        self.la_conv_state = self.la_rec_state = self.page_to_slot = None
        self._la_index: dict = {}
        self._free_state_slots: list[int] = []

    def alloc(self, n: int) -> list:
        """Pages from the allocator. When lower tiers are attached (``block_tiers``), published pages that this
        allocation evicted are copied out at once - their contents are intact only until the new owner's first write."""
        pages = list(self.allocator.alloc(n))
        tiers = getattr(self, "block_tiers", None)
        if tiers is not None:
            tiers.demote(self.allocator.take_evicted())
        return pages

    def enable_linear_attention_state(self, layers, slots: int, conv_hist: int, conv_channels: int, heads: int, dk: int, dv: int):
        dev, dt = self.k.device, self.k.dtype
        self._la_index = {li: i for i, li in enumerate(layers)}
        n = len(self._la_index)
        self.la_conv_state = torch.zeros((n, slots, conv_hist, conv_channels), dtype=dt, device=dev)
        self.la_rec_state = torch.zeros((n, slots, heads, dk, dv), dtype=torch.float32, device=dev)
        self.page_to_slot = torch.zeros(self.num_pages, dtype=torch.int32, device=dev)
        self._free_state_slots = list(range(slots - 1, -1, -1))
        self._slot_of_page: dict = {}

    def bind_state(self, first_page: int) -> int:
        """Give the sequence that starts at ``first_page`` a zeroed state slot."""
        if self.page_to_slot is None:
            return -1
        if not self._free_state_slots:
            raise RuntimeError("KV pool exhausted (no free recurrent-state slot)")
        slot = self._free_state_slots.pop()
        self._slot_of_page[int(first_page)] = slot
        self.page_to_slot[int(first_page)] = slot
        self.la_conv_state[:, slot].zero_()
        self.la_rec_state[:, slot].zero_()
        return slot

    def unbind_state(self, first_page: int) -> None:
        if self.page_to_slot is None:
            return
        slot = self._slot_of_page.pop(int(first_page), None)
        if slot is not None:
            self._free_state_slots.append(slot)

    def detach_state(self, first_page: int) -> int:
        """The sequence gives its pages up but keeps its state slot (parked in a host tier). Returns the slot or -1."""
        if self.page_to_slot is None:
            return -1
        return self._slot_of_page.pop(int(first_page), -1)

    def attach_state(self, slot: int, first_page: int) -> None:
        """A detached slot follows the sequence's new first page."""
        if self.page_to_slot is None or slot < 0:
            return
        self._slot_of_page[int(first_page)] = slot
        self.page_to_slot[int(first_page)] = slot

    def free_state_slot(self, slot: int) -> None:
        if self.page_to_slot is not None and slot >= 0:
            self._free_state_slots.append(slot)

    # ---- recurrent-state snapshots: K/V pages roll back by a length change, the fixed-size states of hybrid layers
    # (short-convolution history, gated-delta / Mamba matrices) have to be copied out and put back.
    def has_recurrent_state(self) -> bool:
        return self.conv_state is not None or self.page_to_slot is not None

    def recurrent_tensors(self) -> list:
        """Every fixed-size state tensor a forward pass mutates in place (empty for attention-only models). A step that
        is run twice on the same inputs - a warm-up before graph capture - must put these back in between: unlike a
        K/V append, advancing a recurrent state is not idempotent."""
        return [t for t in (self.conv_state, self.la_conv_state, self.la_rec_state) if t is not None]

    def snapshot_state(self, first_page: int):
        """Copies of this sequence's recurrent states (None for attention-only models)."""
        if not self.has_recurrent_state():
            return None
        conv = self.conv_state[:, int(first_page)].clone() if self.conv_state is not None else None
        la = None
        if self.page_to_slot is not None:
            slot = self._slot_of_page[int(first_page)]
            la = (self.la_conv_state[:, slot].clone(), self.la_rec_state[:, slot].clone())
        return conv, la

    def restore_state(self, first_page: int, snap) -> None:
        if snap is None:
            return
        conv, la = snap
        if conv is not None:
            self.conv_state[:, int(first_page)].copy_(conv)
        if la is not None:
            slot = self._slot_of_page[int(first_page)]
            self.la_conv_state[:, slot].copy_(la[0])
            self.la_rec_state[:, slot].copy_(la[1])

    def linear_attention_state(self, li: int):
        i = self._la_index[li]
        return self.la_conv_state[i], self.la_rec_state[i]

    def layer(self, li: int):
        i = self._kv_index[li]
        return self.k[i], self.v[i]

    def conv_layer(self, li: int):
        return self.conv_state[self._conv_index[li]]

    def bytes(self) -> int:
        extra = self.conv_state.numel() * self.conv_state.element_size() if self.conv_state is not None else 0
        if self.la_rec_state is not None:
            extra += self.la_rec_state.numel() * 4 + self.la_conv_state.numel() * self.la_conv_state.element_size()
        return (self.k.numel() + self.v.numel()) * self.k.element_size() + extra

    @staticmethod
    def pages_for(tokens: int) -> int:
        return (tokens + PAGE - 1) // PAGE
