"""Routed-expert cache: the experts of a sparse layer live in pinned host memory, a bounded bank of device slots
holds the ones in use.

Counterpart of the reference's independent rank-owned ``ExpertCache`` (eredu/src/backend/mlx/runtime/residency/
expert_cache.rs: demand histogram -> acquire -> compact bank; ``--expert-cache``, ``--expert-cache-device-budget-bytes``,
``--expert-cache-eviction lru|lfu``, ``--expert-cache-benchmark``; plan schema ``ExpertCachePlan``
eredu-core/src/execution.rs). It composes with expert parallelism: every rank caches only the experts it owns.

Per call the router's ids are read on the host (this mode trades a synchronisation per sparse layer for fitting a
model whose experts exceed device memory), the missing experts are copied into victim slots chosen by LRU or LFU,
the ids are rewritten to slot numbers and the ordinary grouped expert kernels run over the slot bank. A step that
needs more distinct experts than there are slots runs in several passes over disjoint expert subsets.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import moe as moe_ops


@dataclass
class ExpertCacheStats:
    hits: int = 0
    misses: int = 0
    evictions: int = 0
    bytes_loaded: int = 0
    passes: int = 0
    calls: int = 0


class ExpertCache:
    def __init__(self, w_gate_up: torch.Tensor, w_down: torch.Tensor, slots: int, eviction: str = "lru", e0: int = 0):
        """w_gate_up [E_local, 2I, H], w_down [E_local, H, I] on the compute device: moved to pinned host memory;
        ``slots`` device-resident experts."""
        if eviction not in ("lru", "lfu"):
            raise ValueError("eviction must be lru or lfu")
        self.device = w_gate_up.device
        self.cuda = self.device.type == "cuda"
        self.e0 = e0
        self.n_experts = w_gate_up.shape[0]
        self.slots = max(1, min(int(slots), self.n_experts))
        self.eviction = eviction
        host = lambda t: (t.detach().to("cpu").pin_memory() if self.cuda else t.detach().to("cpu").clone())  # noqa: E731
        self.host_gu, self.host_dn = host(w_gate_up), host(w_down)
        self.bank_gu = torch.empty((self.slots,) + tuple(w_gate_up.shape[1:]), dtype=w_gate_up.dtype, device=self.device)
        self.bank_dn = torch.empty((self.slots,) + tuple(w_down.shape[1:]), dtype=w_down.dtype, device=self.device)
        self.slot_of: dict[int, int] = {}          # local expert -> slot
        self.expert_in = [-1] * self.slots          # slot -> local expert
        self.last_use = [0] * self.slots
        self.use_count = [0] * self.slots
        self.clock = 0
        self.stats = ExpertCacheStats()
        self.expert_bytes = (self.host_gu[0].numel() * self.host_gu.element_size()
                             + self.host_dn[0].numel() * self.host_dn.element_size())

    @classmethod
    def slots_for_budget(cls, w_gate_up, w_down, device_budget_bytes: int) -> int:
        per = w_gate_up[0].numel() * w_gate_up.element_size() + w_down[0].numel() * w_down.element_size()
        return max(1, int(device_budget_bytes // per))

    # ------------------------------------------------------------------------------------------ residency
    def _victim(self, protected: set) -> int:
        free = [s for s in range(self.slots) if self.expert_in[s] < 0]
        if free:
            return free[0]
        cands = [s for s in range(self.slots) if self.expert_in[s] not in protected]
        key = (lambda s: (self.use_count[s], self.last_use[s])) if self.eviction == "lfu" else (lambda s: self.last_use[s])
        return min(cands, key=key)

    def acquire(self, experts: list[int]) -> dict[int, int]:
        """Make the given local experts resident (at most ``slots`` of them); returns expert -> slot."""
        assert len(experts) <= self.slots
        self.clock += 1
        need = set(experts)
        for e in experts:
            s = self.slot_of.get(e)
            if s is not None:
                self.stats.hits += 1
            else:
                self.stats.misses += 1
                s = self._victim(need)
                old = self.expert_in[s]
                if old >= 0:
                    del self.slot_of[old]
                    self.stats.evictions += 1
                    self.use_count[s] = 0
                self.bank_gu[s].copy_(self.host_gu[e], non_blocking=True)
                self.bank_dn[s].copy_(self.host_dn[e], non_blocking=True)
                self.expert_in[s] = e
                self.slot_of[e] = s
                self.stats.bytes_loaded += self.expert_bytes
            self.last_use[s] = self.clock
            self.use_count[s] += 1
        return {e: self.slot_of[e] for e in experts}

    # ------------------------------------------------------------------------------------------ forward
    def forward(self, x, ids, weights, residual=None, extra=None, limit: float = 0.0, act: str = "swiglu"):
        """Same contract as :func:`ops.moe.experts_forward` for the local experts [e0, e0 + E_local)."""
        self.stats.calls += 1
        local = ids.long() - self.e0
        is_local = (local >= 0) & (local < self.n_experts)
        demand = torch.unique(local[is_local]).tolist()                # host synchronisation: the demand set
        out = None
        passes = [demand[i:i + self.slots] for i in range(0, len(demand), self.slots)] or [[]]
        for pi, group in enumerate(passes):
            self.stats.passes += 1
            mapping = self.acquire(group)
            # ids of this pass: resident experts -> slot number; everything else -> an id no slot owns
            remap = torch.full((self.n_experts,), self.slots, dtype=torch.int32, device=ids.device)
            for e, s in mapping.items():
                remap[e] = s
            pass_ids = torch.where(is_local, remap[local.clamp(0, self.n_experts - 1)], torch.full_like(ids, self.slots)).to(torch.int32)
            part = moe_ops.experts_forward(x, pass_ids, weights, self.bank_gu, self.bank_dn, 0,
                                           residual=residual if pi == 0 else None, extra=extra if pi == 0 else None,
                                           limit=limit, act=act)
            out = part if out is None else out + part
        return out

    def report(self) -> dict:
        s = self.stats
        total = max(1, s.hits + s.misses)
        return {"hits": s.hits, "misses": s.misses, "hit_rate": s.hits / total, "evictions": s.evictions,
                "bytes_loaded": s.bytes_loaded, "passes": s.passes, "calls": s.calls, "slots": self.slots,
                "eviction": self.eviction}


def attach_expert_cache(model, slots: int = 0, device_budget_bytes: int = 0, eviction: str = "lru") -> list:
    """Replace every sparse block's resident expert banks by an :class:`ExpertCache`. Returns the caches."""
    caches = []
    for lw in model.layers:
        blk = lw.moe
        if blk is None:
            continue
        if blk.gu_bias is not None or blk.down_bias is not None:
            raise NotImplementedError("expert cache: per-expert biases are not carried through the slot bank yet")
        n = slots or ExpertCache.slots_for_budget(blk.w_gate_up, blk.w_down, device_budget_bytes)
        cache = ExpertCache(blk.w_gate_up, blk.w_down, n, eviction, blk.e0)
        blk.expert_cache = cache
        blk.w_gate_up = blk.w_gate_up[:0]   # the banks now live in the cache (host) - keep shape metadata only
        blk.w_down = blk.w_down[:0]
        caches.append(cache)
    if model.device.type == "cuda":
        torch.cuda.empty_cache()
    return caches
