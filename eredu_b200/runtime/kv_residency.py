"""KV-cache residency: a pinned host tier behind the device page pool.

Counterpart of ``CacheResidencyPolicy::Paged(PagedCacheOptions{block_size_tokens, device_budget_bytes,
host_budget_bytes, recent_device_blocks, eviction, ...})`` and the ``CacheResidencyManager`` (eredu/src/backend/mlx/
runtime/cache/residency.rs:60-135 options; block store, tiers, transfer stream, leases) together with the portable
accounting of eredu-core/src/cache.rs:48-450 (device / host / transfer byte reservations) and cache/storage.rs (the
device <-> host phase machine).

With ``live_disk`` set, a third tier sits behind the host tier: when a park would exceed the host budget, the parked
sequences that have waited longest are written to files in that directory (their host copies are dropped) and read back
on resume (eredu-core/src/cache/storage.rs: device <-> host <-> disk phases).

Unit of transfer: all pages of one sequence ("park" / "resume"). Parking gathers the sequence's pages of every layer
into one contiguous staging tensor on the device (a single gather kernel per pool), copies it to pinned host memory
on a transfer stream and returns the device pages to the pool; resuming allocates fresh device pages and scatters
the data back. The page ids change, the contents do not: a resumed sequence continues bit-identically.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .kv_cache import PAGE


@dataclass
class PagedCacheOptions:
    block_size_tokens: int = PAGE
    device_budget_bytes: Optional[int] = None
    host_budget_bytes: Optional[int] = None
    recent_device_blocks: int = 0        # newest blocks of a parked sequence that stay on the device (0 = none)
    eviction: str = "lru"                # which running sequence is parked first under pressure: lru | largest
    live_disk: Optional[str] = None      # directory of the disk tier behind the host tier (None: no disk tier)
    disk_budget_bytes: Optional[int] = None


@dataclass
class ParkedSequence:
    k_host: torch.Tensor                 # [layers, pages, n_kv, PAGE, D] pinned
    v_host: torch.Tensor
    pages: int
    reserved_pages: int                  # pages the sequence had reserved (prompt + budget), restored on resume
    event: object = None                 # transfer completion (CUDA event) or None
    conv_state: object = None            # hybrid models: the short-convolution state of every conv layer [layers, hist, C]
    state_slot: int = -1                 # gated-delta models: the recurrent-state slot the sequence keeps while parked
    disk_path: Optional[str] = None      # set while the pages live in the disk tier (k_host / v_host are None then)
    order: int = 0                       # park order: the disk tier takes the longest-parked sequences first
    buffers: tuple = ()                  # the pool buffers behind k_host / v_host (returned to the pool when done)


class KVHostTier:
    def __init__(self, engine, options: Optional[PagedCacheOptions] = None):
        self.engine = engine
        self.kv = engine.kv
        self.opt = options or PagedCacheOptions()
        if self.opt.block_size_tokens != PAGE:
            raise ValueError(f"the device pool uses {PAGE}-token pages")
        self.cuda = engine.cuda
        self.stream = torch.cuda.Stream(device=engine.device) if self.cuda else None
        self.parked: dict[int, ParkedSequence] = {}
        self.host_bytes = 0
        self.disk_bytes = 0
        self.stats = {"parked": 0, "resumed": 0, "bytes_to_host": 0, "bytes_to_device": 0, "refused": 0,
                      "spilled": 0, "bytes_to_disk": 0, "bytes_from_disk": 0}
        if self.opt.live_disk:
            import os

            os.makedirs(self.opt.live_disk, exist_ok=True)
        self._clock = 0
        self._last_use: dict[int, int] = {}
        from .host_pool import HostTransferPool, default_pool

        self.pool = default_pool() if self.cuda else HostTransferPool(pin=False)
        self._retired: list = []

    # ------------------------------------------------------------------------------------------ accounting
    def page_bytes(self) -> int:
        k = self.kv.k
        v = self.kv.v
        return (k.shape[0] * k.shape[2] * k.shape[3] * k.shape[4] + v.shape[0] * v.shape[2] * v.shape[3] * v.shape[4]) * k.element_size()

    def touch(self, seq) -> None:
        self._clock += 1
        self._last_use[seq.seq_id] = self._clock

    def victim(self, candidates):
        """The sequence to park first among ``candidates`` under the configured policy."""
        cands = [s for s in candidates if s.pages and s.seq_id not in self.parked]
        if not cands:
            return None
        if self.opt.eviction == "largest":
            return max(cands, key=lambda s: s.kv_len)
        return min(cands, key=lambda s: self._last_use.get(s.seq_id, 0))

    # ------------------------------------------------------------------------------------------ park / resume
    @torch.no_grad()
    def park(self, seq) -> bool:
        """Move the sequence's cached pages to the host tier and free its device pages. False when the host budget
        would be exceeded (nothing changes)."""
        if seq.seq_id in self.parked:
            return True
        used = (seq.kv_len + PAGE - 1) // PAGE
        nbytes = used * self.page_bytes()
        if self.opt.host_budget_bytes is not None and self.host_bytes + nbytes > self.opt.host_budget_bytes:
            if not self._spill(self.host_bytes + nbytes - self.opt.host_budget_bytes):
                self.stats["refused"] += 1
                return False
        dev = self.engine.device
        idx = torch.as_tensor(seq.pages[:used], dtype=torch.long, device=dev)
        shape = (self.kv.k.shape[0], used) + tuple(self.kv.k.shape[2:])
        # staging memory comes from the pinned transfer pool (booked under "kv"): a buffer released by a resume is pinned
        # already, so steady park / resume traffic costs no page-locking calls
        self._reap()
        v_shape = (self.kv.v.shape[0], used) + tuple(self.kv.v.shape[2:])
        k_buf, k_host = self._host_tensor(shape, self.kv.k.dtype)
        v_buf, v_host = self._host_tensor(v_shape, self.kv.v.dtype)
        event = None
        if used:
            k_stage = self.kv.k.index_select(1, idx)     # gather on the compute stream: ordered after the last step
            v_stage = self.kv.v.index_select(1, idx)
            if self.cuda:
                ready = torch.cuda.Event()
                ready.record(torch.cuda.current_stream(dev))
                with torch.cuda.stream(self.stream):
                    self.stream.wait_event(ready)
                    k_host.copy_(k_stage, non_blocking=True)
                    v_host.copy_(v_stage, non_blocking=True)
                    k_stage.record_stream(self.stream)
                    v_stage.record_stream(self.stream)
                    event = torch.cuda.Event()
                    event.record(self.stream)
            else:
                k_host.copy_(k_stage)
                v_host.copy_(v_stage)
        conv = None
        if self.kv.conv_state is not None and seq.pages:
            conv = self.kv.conv_state[:, seq.pages[0]].to("cpu")   # the state is named by the sequence's first page
        self._clock += 1
        self.parked[seq.seq_id] = ParkedSequence(k_host, v_host, used, len(seq.pages), event, conv,
                                                 self.kv.detach_state(seq.pages[0]) if seq.pages else -1, order=self._clock,
                                                 buffers=(k_buf, v_buf))
        self.engine.kv.allocator.release(seq.pages)
        seq.pages = []
        self.host_bytes += nbytes
        self.stats["parked"] += 1
        self.stats["bytes_to_host"] += nbytes
        return True

    @torch.no_grad()
    def resume(self, seq) -> bool:
        """Bring a parked sequence back. False when the device pool has too few free pages (it stays parked)."""
        p = self.parked.get(seq.seq_id)
        if p is None:
            return True
        if self.kv.allocator.free_pages() < p.reserved_pages:
            self.stats["refused"] += 1
            return False
        if p.disk_path is not None and not self._unspill(p):
            self.stats["refused"] += 1
            return False
        pages = self.kv.alloc(p.reserved_pages)
        dev = self.engine.device
        if p.pages:
            idx = torch.as_tensor(pages[:p.pages], dtype=torch.long, device=dev)
            if self.cuda:
                with torch.cuda.stream(self.stream):
                    if p.event is not None:
                        self.stream.wait_event(p.event)
                    k_dev = p.k_host.to(dev, non_blocking=True)
                    v_dev = p.v_host.to(dev, non_blocking=True)
                    done = torch.cuda.Event()
                    done.record(self.stream)
                torch.cuda.current_stream(dev).wait_event(done)
                k_dev.record_stream(torch.cuda.current_stream(dev))
                v_dev.record_stream(torch.cuda.current_stream(dev))
            else:
                k_dev, v_dev = p.k_host, p.v_host
            self.kv.k.index_copy_(1, idx, k_dev)
            self.kv.v.index_copy_(1, idx, v_dev)
            self._retire(p.buffers, done if self.cuda else None)
        else:
            self._retire(p.buffers, None)
        if p.conv_state is not None:
            self.kv.conv_state[:, pages[0]] = p.conv_state.to(dev)
        self.kv.attach_state(p.state_slot, pages[0])         # gated-delta state stayed in its slot while parked
        seq.pages = pages
        nbytes = p.pages * self.page_bytes()
        self.host_bytes -= nbytes
        self.stats["resumed"] += 1
        self.stats["bytes_to_device"] += nbytes
        del self.parked[seq.seq_id]
        self.touch(seq)
        return True

    def drop(self, seq) -> None:
        """Forget a parked sequence (cancelled while parked)."""
        p = self.parked.pop(seq.seq_id, None)
        if p is not None:
            if p.disk_path is not None:
                self.disk_bytes -= p.pages * self.page_bytes()
                self._remove(p.disk_path)
            else:
                self.host_bytes -= p.pages * self.page_bytes()
                self._retire(p.buffers, p.event)
            self.kv.free_state_slot(p.state_slot)

    # ------------------------------------------------------------------------------------------ pinned staging
    def _host_tensor(self, shape, dtype):
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        buf = self.pool.acquire(max(1, nbytes), "kv")
        return buf, self.pool.view(buf, shape, dtype)

    def _retire(self, buffers, event) -> None:
        """Give staging buffers back to the pool once the copy that reads them (``event``) has completed."""
        if buffers:
            self._retired.append((tuple(buffers), event))
            self._reap()

    def _reap(self) -> None:
        keep = []
        for bufs, ev in self._retired:
            if ev is None or ev.query():
                for b in bufs:
                    self.pool.release(b)
            else:
                keep.append((bufs, ev))
        self._retired = keep

    # ------------------------------------------------------------------------------------------ disk tier
    @staticmethod
    def _remove(path: str) -> None:
        import os

        try:
            os.remove(path)
        except OSError:
            pass

    def _spill(self, need: int) -> bool:
        """Move host copies to the disk tier, longest-parked first, until ``need`` bytes are free. False when there is no
        disk tier, its budget is too small, or the host tier holds too little to spill (nothing is left half-moved)."""
        if not self.opt.live_disk:
            return False
        import os

        order = sorted((p for p in self.parked.values() if p.disk_path is None and p.pages), key=lambda p: p.order)
        plan, freed = [], 0
        for p in order:
            if freed >= need:
                break
            plan.append(p)
            freed += p.pages * self.page_bytes()
        if freed < need:
            return False
        if self.opt.disk_budget_bytes is not None and self.disk_bytes + freed > self.opt.disk_budget_bytes:
            return False
        for p in plan:
            if p.event is not None:
                p.event.synchronize()                     # the device-to-host copy must have landed before it is written out
            sid = next(k for k, v in self.parked.items() if v is p)
            path = os.path.join(self.opt.live_disk, f"sequence-{sid}-{p.order}.kv")
            tmp = path + ".partial"
            torch.save({"k": p.k_host, "v": p.v_host}, tmp)
            os.replace(tmp, path)
            nbytes = p.pages * self.page_bytes()
            p.k_host = p.v_host = None
            self._retire(p.buffers, None)
            p.buffers = ()
            p.event = None
            p.disk_path = path
            self.host_bytes -= nbytes
            self.disk_bytes += nbytes
            self.stats["spilled"] += 1
            self.stats["bytes_to_disk"] += nbytes
        return True

    def _unspill(self, p: ParkedSequence) -> bool:
        """Read a spilled sequence back into (pinned) host memory; other host copies make room through the disk tier."""
        nbytes = p.pages * self.page_bytes()
        if self.opt.host_budget_bytes is not None and self.host_bytes + nbytes > self.opt.host_budget_bytes:
            if not self._spill(self.host_bytes + nbytes - self.opt.host_budget_bytes):
                return False
        blob = torch.load(p.disk_path, map_location="cpu")
        k_buf, p.k_host = self._host_tensor(tuple(blob["k"].shape), blob["k"].dtype)
        v_buf, p.v_host = self._host_tensor(tuple(blob["v"].shape), blob["v"].dtype)
        p.k_host.copy_(blob["k"])
        p.v_host.copy_(blob["v"])
        p.buffers = (k_buf, v_buf)
        self._remove(p.disk_path)
        p.disk_path = None
        self.disk_bytes -= nbytes
        self.host_bytes += nbytes
        self.stats["bytes_from_disk"] += nbytes
        return True

    def report(self) -> dict:
        return dict(self.stats, parked_now=len(self.parked), host_bytes=self.host_bytes, disk_bytes=self.disk_bytes,
                    on_disk_now=sum(1 for p in self.parked.values() if p.disk_path is not None),
                    device_free_pages=self.kv.allocator.free_pages())
