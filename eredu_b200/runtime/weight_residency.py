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
