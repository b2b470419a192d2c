"""Layerwise host residency: a model whose repeated layers live in pinned host memory and pass through a bounded
window of device slots, prefetched on a copy stream while earlier layers compute.

Counterpart of the reference's ``WeightResidency::LayerwiseHost`` execution (eredu/src/backend/mlx/runtime/
execution/layerwise.rs:177-300 options, runtime/residency/manager.rs: immutable host-pinned weight units and device
window leases; eredu-core/src/residency.rs ledger: reserve / publish / evict accounting). Embedding, final norm and
the output head stay resident; every decoder layer (dense, quantised or sparse) is a unit.

Slots: ``device_layer_window + 1`` sets of device buffers. While layer i computes out of its slot the copy stream
fills the slot of layer i + window; a slot is only overwritten after the compute stream recorded that its last user
finished (event per slot), and a layer only runs after its slot's copy completed (event per slot).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass
class ResidencyStats:
    loads: int = 0                # layer units copied host -> device
    bytes_loaded: int = 0
    hits: int = 0                 # acquire() found the layer already in its slot
    stalls: int = 0               # acquire() had to issue the copy itself (prefetch had not covered it)
    host_bytes: int = 0
    device_slot_bytes: int = 0
    events: list = field(default_factory=list)


class LayerwiseHostResidency:
    def __init__(self, model, device_layer_window: int = 1, defer: bool = False):
        """``defer``: layers are handed over one at a time with :meth:`adopt_layer` while the model is being built
        (the device never holds more than one freshly built layer), then :meth:`finalize` sets up the window."""
        if device_layer_window < 1:
            raise ValueError("device_layer_window must be at least 1")
        self.model = model
        self.device = model.device
        self.cuda = self.device.type == "cuda"
        self.requested_window = device_layer_window
        self.stats = ResidencyStats()
        self.units: list[list[tuple]] = []   # per layer: (owner object, attribute name, host tensor)
        if not defer:
            for lw in model.layers:
                self.adopt_layer(lw)
            self.finalize()

    def adopt_layer(self, lw) -> None:
        """Move one layer's tensors to (pinned) host memory and remember where they belong."""
        owners = [lw] + list(lw.qlin.values()) + ([lw.moe] if lw.moe is not None else [])
        ents = []
        for obj in owners:
            for attr, val in list(vars(obj).items()):
                if isinstance(val, torch.Tensor) and val.device == self.device and val.numel() > 0:
                    host = val.detach().to("cpu")
                    host = host.pin_memory() if self.cuda else host.clone()
                    ents.append((obj, attr, host))
                    setattr(obj, attr, None)
                    self.stats.host_bytes += host.numel() * host.element_size()
                elif isinstance(val, tuple) and val and all(isinstance(t, torch.Tensor) for t in val):
                    raise NotImplementedError("tuple-valued weights (shared experts) are not windowed yet")
        self.units.append(ents)

    def finalize(self) -> None:
        self.window = min(self.requested_window, max(1, len(self.units)))
        self.n_slots = self.window + 1
        if self.cuda:
            torch.cuda.empty_cache()
            self.copy_stream = torch.cuda.Stream(device=self.device)
            self.ready = [torch.cuda.Event() for _ in range(self.n_slots)]
            self.free = [torch.cuda.Event() for _ in range(self.n_slots)]
            for e in self.free:
                e.record(torch.cuda.current_stream(self.device))
        self.slots: list[dict] = [{} for _ in range(self.n_slots)]
        self.loaded = [-1] * self.n_slots
        self.in_use = [False] * self.n_slots
        for li in range(min(self.window, len(self.units))):
            self._load(li)
        self.model.residency = self

    # ------------------------------------------------------------------------------------------ internals
    def _slot_of(self, li: int) -> int:
        return li % self.n_slots

    def _load(self, li: int) -> None:
        slot = self._slot_of(li)
        bufs = self.slots[slot]
        nbytes = 0

        def copy_all():
            nonlocal nbytes
            for j, (_, _, host) in enumerate(self.units[li]):
                buf = bufs.get(j)
                if buf is None or buf.shape != host.shape or buf.dtype != host.dtype:
                    buf = torch.empty(host.shape, dtype=host.dtype, device=self.device)
                    bufs[j] = buf
                    self.stats.device_slot_bytes += buf.numel() * buf.element_size()
                buf.copy_(host, non_blocking=True)
                nbytes += host.numel() * host.element_size()

        if self.cuda:
            with torch.cuda.stream(self.copy_stream):
                self.copy_stream.wait_event(self.free[slot])   # the slot's previous user has finished computing
                copy_all()
                self.ready[slot].record(self.copy_stream)
        else:
            copy_all()
        self.loaded[slot] = li
        self.stats.loads += 1
        self.stats.bytes_loaded += nbytes

    # ------------------------------------------------------------------------------------------ model hooks
    def acquire(self, i: int) -> None:
        """Called before local layer ``i`` runs: binds its tensors to the slot that holds them."""
        slot = self._slot_of(i)
        if self.loaded[slot] != i:
            self.stats.stalls += 1
            self._load(i)
        else:
            self.stats.hits += 1
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_event(self.ready[slot])
        for j, (obj, attr, _) in enumerate(self.units[i]):
            setattr(obj, attr, self.slots[slot][j])
        self.in_use[slot] = True
        # prefetch the layer `window` ahead (wrapping to the next step's first layers) into a slot nobody is using
        n = len(self.units)
        nxt = (i + self.window) % n
        ns = self._slot_of(nxt)
        if nxt != i and not self.in_use[ns] and self.loaded[ns] != nxt:
            self._load(nxt)

    def release(self, i: int) -> None:
        """Called after local layer ``i`` ran: its slot may be refilled once the compute stream gets here."""
        slot = self._slot_of(i)
        if self.cuda:
            self.free[slot].record(torch.cuda.current_stream(self.device))
        for obj, attr, _ in self.units[i]:
            setattr(obj, attr, None)
        self.in_use[slot] = False

    def report(self) -> dict:
        s = self.stats
        return {"loads": s.loads, "bytes_loaded": s.bytes_loaded, "hits": s.hits, "stalls": s.stalls,
                "host_bytes": s.host_bytes, "device_slot_bytes": s.device_slot_bytes, "device_layer_window": self.window}


class DiskStreamResidency(LayerwiseHostResidency):
    """Dense disk streaming: the layers live in a spill file on disk, a bounded set of them is materialised in
    (pinned) host memory by background reader threads, and a fixed current-plus-next window sits on the device.

    Counterpart of the reference's ``ResidencyPlan::DenseDiskStream`` (eredu/src/backend/mlx/runtime/residency/
    dense_stream.rs:24-120: finite device and host budgets, ``host_lookahead`` protected host copies,
    ``background_queue_capacity`` pending materialisations, demand reads when the background work has not covered a
    layer; ``--dense-disk-stream``, ``--dense-host-lookahead``, ``--dense-background-queue``). The reference streams
    tensors straight from the checkpoint; here the units are the load-time prepared layers (fused projections, folded
    norms, compute dtype), so they are written once to a spill directory and streamed from there."""

    def __init__(self, model, host_lookahead: int = 2, background_queue: int = 2, spill_dir=None,
                 host_budget_bytes: Optional[int] = None, defer: bool = False):
        import tempfile
        import threading

        if host_lookahead < 1 or background_queue < 1:
            raise ValueError("host_lookahead and background_queue must be at least 1")
        self.host_lookahead = host_lookahead
        self.background_queue = background_queue
        self.host_budget_bytes = host_budget_bytes
        self._tmp = None
        if spill_dir is None:
            self._tmp = tempfile.TemporaryDirectory(prefix="eredu-dense-stream-")
            spill_dir = self._tmp.name
        self.spill_dir = str(spill_dir)
        import os

        os.makedirs(self.spill_dir, exist_ok=True)
        self.files: list[str] = []
        self.layouts: list[list[tuple]] = []   # per layer: (shape, dtype, byte offset, byte length)
        self.host: dict[int, list] = {}        # layer -> materialised host tensors
        self.host_order: list[int] = []        # least recently used first
        self.pending: dict[int, object] = {}   # layer -> threading.Event of an in-flight materialisation
        self.lock = threading.Lock()
        self.disk = {"background_reads": 0, "demand_reads": 0, "bytes_read": 0, "evictions": 0, "refused": 0,
                     "max_host_layers": 0}
        super().__init__(model, device_layer_window=1, defer=True)   # window 1 => two device slots: current + next
        if not defer:
            for lw in model.layers:
                self.adopt_layer(lw)
            self.finalize()

    # ------------------------------------------------------------------------------------------ load time
    def adopt_layer(self, lw) -> None:
        """Write one prepared layer to the spill file and drop it from memory."""
        import numpy as np

        owners = [lw] + list(lw.qlin.values()) + ([lw.moe] if lw.moe is not None else [])
        li = len(self.units)
        path = f"{self.spill_dir}/layer-{li:05d}.bin"
        ents, layout, off = [], [], 0
        with open(path, "wb") as f:
            for obj in owners:
                for attr, val in list(vars(obj).items()):
                    if isinstance(val, torch.Tensor) and val.device == self.device and val.numel() > 0:
                        host = val.detach().to("cpu").contiguous()
                        raw = host.view(torch.uint8).numpy() if host.dtype != torch.uint8 else host.numpy()
                        f.write(np.ascontiguousarray(raw).tobytes())
                        n = host.numel() * host.element_size()
                        ents.append((obj, attr, None))
                        layout.append((tuple(host.shape), host.dtype, off, n))
                        off += n
                        setattr(obj, attr, None)
                    elif isinstance(val, tuple) and val and all(isinstance(t, torch.Tensor) for t in val):
                        raise NotImplementedError("tuple-valued weights (shared experts) are not streamed yet")
        self.units.append(ents)
        self.files.append(path)
        self.layouts.append(layout)
        self.stats.host_bytes = 0

    def finalize(self) -> None:
        import queue
        import threading

        from ..lib import _eredu_host as H

        # tier accounting lives in the C++ ledger: every layer is a windowed unit whose home copy is the spill file
        self.ledger = H.ResidencyLedger(-1, -1 if self.host_budget_bytes is None else int(self.host_budget_bytes), -1, "lru")
        for li in range(len(self.units)):
            self.ledger.add_unit(f"layer.{li}", self._layer_bytes(li), "windowed", "disk")
        self.jobs: "queue.Queue" = queue.Queue(maxsize=self.background_queue)
        self.workers = [threading.Thread(target=self._worker, daemon=True) for _ in range(min(2, self.background_queue))]
        for w in self.workers:
            w.start()
        super().finalize()

    # ------------------------------------------------------------------------------------------ disk -> host
    def _layer_bytes(self, li: int) -> int:
        return sum(n for _, _, _, n in self.layouts[li])

    def _read(self, li: int) -> list:
        out = []
        with open(self.files[li], "rb", buffering=0) as f:
            for shape, dtype, off, n in self.layouts[li]:
                t = torch.empty(shape, dtype=dtype, pin_memory=self.cuda)
                f.seek(off)
                view = t.view(torch.uint8).reshape(-1).numpy() if dtype != torch.uint8 else t.reshape(-1).numpy()
                got = f.readinto(memoryview(view))
                if got != n:
                    raise IOError(f"short read from {self.files[li]}: {got} of {n} bytes")
                out.append(t)
        return out

    def _publish(self, li: int, tensors: list, background: bool) -> None:
        with self.lock:
            name = f"layer.{li}"
            if not self.ledger.is_resident(name, "host"):
                self.ledger.reserve(name, "host")
                self.ledger.resolve_transfer(name, "host", self.ledger.begin_transfer(name, "host"), "disk")
            self.ledger.record_prefetch("host", "hit" if background else "miss")
            self.host[li] = tensors
            if li in self.host_order:
                self.host_order.remove(li)
            self.host_order.append(li)
            self.disk["background_reads" if background else "demand_reads"] += 1
            self.disk["bytes_read"] += self._layer_bytes(li)
            self.disk["max_host_layers"] = max(self.disk["max_host_layers"], len(self.host))

    def _worker(self) -> None:
        while True:
            li = self.jobs.get()
            if li is None:
                return
            try:
                self._publish(li, self._read(li), background=True)
            finally:
                with self.lock:
                    ev = self.pending.pop(li, None)
                if ev is not None:
                    ev.set()

    def _protected(self, i: int) -> set:
        n = len(self.units)
        return {(i + d) % n for d in range(self.host_lookahead + 1)}

    def _evict_for(self, i: int) -> None:
        """Keep at most the current layer plus ``host_lookahead`` imminent ones (and the byte budget) on the host."""
        keep = self._protected(i)
        with self.lock:
            def over():
                # counted with the protected layers that are still on their way in
                want = set(self.host) | keep
                if self.host_budget_bytes is not None:
                    return sum(self._layer_bytes(l) for l in want) > self.host_budget_bytes
                return len(want) > self.host_lookahead + 1
            for li in list(self.host_order):
                if not over():
                    break
                if li in keep:
                    continue
                slot = self._slot_of(li)
                if self.cuda and self.loaded[slot] == li:
                    self.ready[slot].synchronize()   # its host->device copy may still be reading the buffers
                del self.host[li]
                self.host_order.remove(li)
                self.ledger.evict(f"layer.{li}", "host")
                self.units[li] = [(obj, attr, None) for obj, attr, _ in self.units[li]]
                self.disk["evictions"] += 1

    def _submit(self, li: int) -> None:
        import queue
        import threading

        with self.lock:
            if li in self.host or li in self.pending:
                return
            ev = threading.Event()
            self.pending[li] = ev
        try:
            self.jobs.put_nowait(li)
        except queue.Full:
            with self.lock:
                self.pending.pop(li, None)
            self.disk["refused"] += 1

    def _host_tensors(self, li: int) -> list:
        with self.lock:
            got = self.host.get(li)
            ev = self.pending.get(li)
        if got is not None:
            return got
        if ev is not None:
            ev.wait()
            with self.lock:
                got = self.host.get(li)
            if got is not None:
                return got
        tensors = self._read(li)                  # demand read: the background work had not covered this layer
        self._publish(li, tensors, background=False)
        return tensors

    # ------------------------------------------------------------------------------------------ host -> device
    def _load(self, li: int) -> None:
        host = self._host_tensors(li)
        self.units[li] = [(obj, attr, h) for (obj, attr, _), h in zip(self.units[li], host)]
        prev = self.loaded[self._slot_of(li)]
        with self.lock:
            if prev >= 0 and prev != li and self.ledger.is_resident(f"layer.{prev}", "device"):
                self.ledger.evict(f"layer.{prev}", "device")
            if not self.ledger.is_resident(f"layer.{li}", "device"):
                self.ledger.reserve(f"layer.{li}", "device")
                self.ledger.resolve_transfer(f"layer.{li}", "device", self.ledger.begin_transfer(f"layer.{li}", "device"), "host")
        super()._load(li)

    def acquire(self, i: int) -> None:
        n = len(self.units)
        self._evict_for(i)                 # make room first: the copies behind the current layer go
        for d in range(1, self.host_lookahead + 1):
            self._submit((i + d) % n)
        super().acquire(i)
        self._evict_for(i)

    def report(self) -> dict:
        return dict(super().report(), mode="dense_disk_stream", host_lookahead=self.host_lookahead,
                    background_queue=self.background_queue, host_layers_now=len(self.host), ledger=self.ledger.report(),
                    **self.disk)

    def close(self) -> None:
        for _ in getattr(self, "workers", []):
            self.jobs.put(None)
        if self._tmp is not None:
            self._tmp.cleanup()
            self._tmp = None
