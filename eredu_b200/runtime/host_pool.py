"""Pinned host-transfer buffers with accounting.

Counterpart of the host transfer-buffer service of the reference backend (buffers by purpose with active / peak byte
counters, eredu-core/src/cache.rs transfer reservations; eredu/src/backend/mlx/runtime/transfer.rs): weight windows, KV
parking, expert banks and prompt-cache I/O all stage through page-locked memory. Pinning is expensive (it is a driver
call that can take milliseconds per buffer), so released buffers are kept by size class and handed out again; every
acquisition is booked under its purpose so that telemetry can say which subsystem holds how much pinned memory.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, field

import torch

KINDS = ("weights", "kv", "experts", "prompt_cache", "tokens", "other")


@dataclass
class KindStats:
    active_bytes: int = 0
    peak_bytes: int = 0
    acquisitions: int = 0
    reuses: int = 0


@dataclass
class HostTransferPool:
    """``acquire(nbytes, kind)`` -> uint8 tensor of at least that size in pinned memory (plain memory without CUDA);
    ``release(tensor)`` returns it. ``cached_limit_bytes`` bounds what released buffers may keep pinned."""
    cached_limit_bytes: int = 1 << 30
    pin: bool = field(default_factory=torch.cuda.is_available)

    def __post_init__(self):
        self._free: dict[int, list[torch.Tensor]] = {}
        self._owner: dict[int, tuple[str, int]] = {}      # data_ptr -> (kind, class bytes)
        self._stats = {k: KindStats() for k in KINDS}
        self._cached_bytes = 0
        self._lock = threading.Lock()

    @staticmethod
    def _size_class(nbytes: int) -> int:
        n = max(4096, int(nbytes))
        return 1 << (n - 1).bit_length() if n < (1 << 20) else (n + (1 << 20) - 1) // (1 << 20) * (1 << 20)

    def acquire(self, nbytes: int, kind: str = "other") -> torch.Tensor:
        if kind not in self._stats:
            raise ValueError(f"unknown transfer-buffer kind {kind!r} (one of {KINDS})")
        cls = self._size_class(nbytes)
        with self._lock:
            bucket = self._free.get(cls)
            st = self._stats[kind]
            if bucket:
                t = bucket.pop()
                self._cached_bytes -= cls
                st.reuses += 1
            else:
                t = None
            st.acquisitions += 1
            st.active_bytes += cls
            st.peak_bytes = max(st.peak_bytes, st.active_bytes)
        if t is None:
            t = torch.empty(cls, dtype=torch.uint8)
            if self.pin:
                t = t.pin_memory()
        with self._lock:
            self._owner[t.data_ptr()] = (kind, cls)
        return t

    def release(self, t: torch.Tensor) -> None:
        with self._lock:
            kind, cls = self._owner.pop(t.data_ptr(), (None, 0))
            if kind is None:
                raise ValueError("buffer was not handed out by this pool (or was released twice)")
            self._stats[kind].active_bytes -= cls
            if self._cached_bytes + cls <= self.cached_limit_bytes:
                self._free.setdefault(cls, []).append(t)
                self._cached_bytes += cls

    def view(self, t: torch.Tensor, shape, dtype) -> torch.Tensor:
        """A typed view over the front of a pool buffer."""
        n = 1
        for d in shape:
            n *= int(d)
        return t[:n * torch.empty((), dtype=dtype).element_size()].view(dtype).view(*shape)

    def trim(self) -> int:
        """Drop every cached buffer; returns the bytes unpinned."""
        with self._lock:
            freed, self._cached_bytes = self._cached_bytes, 0
            self._free.clear()
        return freed

    def stats(self) -> dict:
        with self._lock:
            out = {k: vars(v).copy() for k, v in self._stats.items() if v.acquisitions}
            out["cached_bytes"] = self._cached_bytes
            out["active_bytes"] = sum(v.active_bytes for v in self._stats.values())
            out["peak_bytes"] = sum(v.peak_bytes for v in self._stats.values())
        return out


_default = None


def default_pool() -> HostTransferPool:
    global _default
    if _default is None:
        _default = HostTransferPool()
    return _default
