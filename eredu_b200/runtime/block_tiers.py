"""Host and disk tiers under the published KV pages.

Sealed pages (full, immutable 16-token blocks published under the chained hash of their tokens) live in the device pool
while some sequence leases them or until the pool needs the room. Without lower tiers an evicted page is simply gone.
With a :class:`BlockTierStore` an evicted page is demoted instead: its K and V slabs of every layer are copied to pinned
host memory (copy stream, device -> host, before the page's new owner writes it), the host tier spills its least
recently used blocks to files when it is over budget, and a later request whose prompt continues through such a block
gets it promoted back into a fresh device page (host -> device on the copy stream, disk blocks through host) and
published again. The counterpart of the reference's residency tiers for sealed blocks (device / host / disk with leases
and LRU, eredu/src/backend/mlx/runtime/cache/residency.rs:60-135; blocks are immutable once sealed, kv.rs:2018-2128).

What this is not: attention over blocks that are not on the device. A live sequence's pages are all device pages; the
tiers extend the lifetime of REUSABLE prefixes beyond the device pool, they do not extend a single context beyond it.
"""
from __future__ import annotations

import os
from collections import OrderedDict
from pathlib import Path
from typing import Optional

import numpy as np
import torch


class BlockTierStore:
    def __init__(self, kv, host_bytes: int, disk_dir=None, disk_bytes: int = 0, copy_stream=None):
        self.kv = kv
        L, _, nkv, page, D = kv.k.shape
        self.k_elems = L * nkv * page * D
        self.v_elems = L * kv.v.shape[2] * kv.v.shape[3] * kv.v.shape[4]
        self.dtype = kv.k.dtype
        self.block_bytes = (self.k_elems + self.v_elems) * kv.k.element_size()
        self.host_blocks = max(0, int(host_bytes) // self.block_bytes)
        self.disk_dir = Path(disk_dir) if disk_dir else None
        self.disk_blocks = max(0, int(disk_bytes) // self.block_bytes) if self.disk_dir else 0
        if self.disk_dir:
            self.disk_dir.mkdir(parents=True, exist_ok=True)
        self.cuda = kv.k.is_cuda
        self.stream = copy_stream if copy_stream is not None else (torch.cuda.Stream(kv.k.device) if self.cuda else None)
        self.host: OrderedDict = OrderedDict()      # hash -> (tensor [k_elems + v_elems], event or None), least recent first
        self.disk: OrderedDict = OrderedDict()      # hash -> path
        self.stats = {"demoted": 0, "spilled": 0, "dropped": 0, "promoted_host": 0, "promoted_disk": 0,
                      "host_blocks": 0, "disk_blocks": 0}

    # ------------------------------------------------------------------ queries
    def where(self, h: int) -> Optional[str]:
        return "host" if h in self.host else "disk" if h in self.disk else None

    def _path(self, h: int) -> Path:
        return self.disk_dir / f"{h:016x}.kvb"

    def _host_buffer(self):
        t = torch.empty(self.k_elems + self.v_elems, dtype=self.dtype)
        return t.pin_memory() if self.cuda else t

    # ------------------------------------------------------------------ demotion
    def demote(self, evicted) -> None:
        """``evicted``: (page, hash) pairs whose device contents are still intact. Enqueues the copies on the copy stream
        behind the compute stream's work so far; the compute stream then waits for them before it may write the pages."""
        evicted = [(int(p), int(h)) for p, h in evicted if int(h) not in self.host and int(h) not in self.disk]
        if not evicted or self.host_blocks + self.disk_blocks == 0:
            self.stats["dropped"] += len(evicted)
            return
        kv = self.kv
        pages = torch.tensor([p for p, _ in evicted], dtype=torch.long, device=kv.k.device)
        if self.cuda:
            compute = torch.cuda.current_stream(kv.k.device)
            self.stream.wait_stream(compute)
            ctx = torch.cuda.stream(self.stream)
        else:
            ctx = _Null()
        with ctx:
            # [n, L * ...] staging on the device: one gather per pool, then one copy per block into its own pinned buffer
            ks = kv.k.index_select(1, pages).transpose(0, 1).reshape(len(evicted), self.k_elems)
            vs = kv.v.index_select(1, pages).transpose(0, 1).reshape(len(evicted), self.v_elems)
            for i, (_, h) in enumerate(evicted):
                buf = self._host_buffer()
                buf[:self.k_elems].copy_(ks[i], non_blocking=True)
                buf[self.k_elems:].copy_(vs[i], non_blocking=True)
                ev = None
                if self.cuda:
                    ev = torch.cuda.Event()
                    ev.record(self.stream)
                    ks.record_stream(self.stream)
                    vs.record_stream(self.stream)
                self.host[h] = (buf, ev)
                self.stats["demoted"] += 1
        if self.cuda:
            compute.wait_stream(self.stream)          # the new owners' kernels come after the copies out
        self._trim_host()

    def _trim_host(self) -> None:
        while len(self.host) > self.host_blocks:
            h, (buf, ev) = self.host.popitem(last=False)
            if self.disk_blocks > 0:
                if ev is not None:
                    ev.synchronize()
                buf.view(torch.uint8).numpy().tofile(self._path(h))
                self.disk[h] = self._path(h)
                self.stats["spilled"] += 1
                while len(self.disk) > self.disk_blocks:
                    _, path = self.disk.popitem(last=False)
                    try:
                        os.unlink(path)
                    except OSError:
                        pass
                    self.stats["dropped"] += 1
            else:
                self.stats["dropped"] += 1
        self.stats["host_blocks"], self.stats["disk_blocks"] = len(self.host), len(self.disk)

    # ------------------------------------------------------------------ promotion
    def promote(self, items) -> None:
        """``items``: (hash, device page) pairs; every hash is in a tier. Call after :meth:`demote` of the same step."""
        if not items:
            return
        kv = self.kv
        L = kv.k.shape[0]
        bufs = []
        for h, _ in items:
            h = int(h)
            if h in self.host:
                buf, ev = self.host.pop(h)
                if ev is not None:
                    ev.synchronize()
                self.stats["promoted_host"] += 1
            else:
                path = self.disk.pop(h)
                raw = torch.from_numpy(np.fromfile(path, dtype=np.uint8)).view(self.dtype)
                buf = self._host_buffer()
                buf.copy_(raw)
                try:
                    os.unlink(path)
                except OSError:
                    pass
                self.stats["promoted_disk"] += 1
            bufs.append(buf)
        pages = torch.tensor([int(p) for _, p in items], dtype=torch.long, device=kv.k.device)
        if self.cuda:
            compute = torch.cuda.current_stream(kv.k.device)
            self.stream.wait_stream(compute)
            ctx = torch.cuda.stream(self.stream)
        else:
            ctx = _Null()
        with ctx:
            stage = torch.empty((len(items), self.k_elems + self.v_elems), dtype=self.dtype, device=kv.k.device)
            for i, buf in enumerate(bufs):
                stage[i].copy_(buf, non_blocking=True)
            ks = stage[:, :self.k_elems].reshape(len(items), L, *kv.k.shape[2:]).transpose(0, 1)
            vs = stage[:, self.k_elems:].reshape(len(items), L, *kv.v.shape[2:]).transpose(0, 1)
            kv.k.index_copy_(1, pages, ks)
            kv.v.index_copy_(1, pages, vs)
            if self.cuda:
                stage.record_stream(self.stream)
        if self.cuda:
            compute.wait_stream(self.stream)
            self._keep = bufs                         # pinned sources stay alive until the next call's copies are enqueued
        self.stats["host_blocks"], self.stats["disk_blocks"] = len(self.host), len(self.disk)

    def clear(self) -> None:
        self.host.clear()
        for path in self.disk.values():
            try:
                os.unlink(path)
            except OSError:
                pass
        self.disk.clear()


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
