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
    def __init__(self, w_gate_up: torch.Tensor, w_down: torch.Tensor, slots: int, eviction: str = "lru", e0: int = 0,
                 gu_bias: torch.Tensor = None, down_bias: torch.Tensor = None, scratch_bytes: int = 0,
                 prefill_bank_bytes: int = 0):
        """w_gate_up [E_local, 2I, H], w_down [E_local, H, I] on the compute device: moved to pinned host memory;
        ``slots`` device-resident experts. Per-expert biases (``gu_bias`` [E_local, 2I], ``down_bias`` [E_local, H])
        travel with their expert. ``scratch_bytes`` bounds the permuted activations of one pass (longer inputs run in
        token slices, ``--expert-cache-scratch-bytes``); ``prefill_bank_bytes`` sizes a second, transient bank that
        prompt-sized calls use instead of the decode bank, so that a prefill does not evict the decode working set
        (``--expert-cache-prefill-bank-bytes``)."""
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
        self.host_gub = host(gu_bias) if gu_bias is not None else None
        self.host_dnb = host(down_bias) if down_bias is not None else None
        self.bank_gub = (torch.zeros((self.slots, gu_bias.shape[1]), dtype=gu_bias.dtype, device=self.device)
                         if gu_bias is not None else None)
        self.bank_dnb = (torch.zeros((self.slots, down_bias.shape[1]), dtype=down_bias.dtype, device=self.device)
                         if down_bias is not None else None)
        self.scratch_bytes = int(scratch_bytes)
        self.prefill_slots = min(self.n_experts, int(prefill_bank_bytes // max(1, self.expert_bytes))) if prefill_bank_bytes else 0
        self._prefill_bank = None      # allocated at the first prompt-sized call

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
                if self.bank_gub is not None:
                    self.bank_gub[s].copy_(self.host_gub[e], non_blocking=True)
                if self.bank_dnb is not None:
                    self.bank_dnb[s].copy_(self.host_dnb[e], non_blocking=True)
                self.expert_in[s] = e
                self.slot_of[e] = s
                self.stats.bytes_loaded += self.expert_bytes
            self.last_use[s] = self.clock
            self.use_count[s] += 1
        return {e: self.slot_of[e] for e in experts}

    # ------------------------------------------------------------------------------------------ forward
    PREFILL_TOKENS = 64      # calls with more tokens than this count as prompt-sized

    def _fill_prefill_bank(self, group):
        """Load ``group`` into the transient bank (device copies for experts the decode bank holds, host copies for the
        rest); returns (gate_up bank, down bank, gate_up bias bank, down bias bank, expert -> slot)."""
        if self._prefill_bank is None:
            n = self.prefill_slots
            self._prefill_bank = (torch.empty((n,) + tuple(self.bank_gu.shape[1:]), dtype=self.bank_gu.dtype, device=self.device),
                                  torch.empty((n,) + tuple(self.bank_dn.shape[1:]), dtype=self.bank_dn.dtype, device=self.device),
                                  torch.zeros((n, self.bank_gub.shape[1]), dtype=self.bank_gub.dtype, device=self.device)
                                  if self.bank_gub is not None else None,
                                  torch.zeros((n, self.bank_dnb.shape[1]), dtype=self.bank_dnb.dtype, device=self.device)
                                  if self.bank_dnb is not None else None)
        gu, dn, gub, dnb = self._prefill_bank
        mapping = {}
        for s_, e in enumerate(group):
            res = self.slot_of.get(e)
            if res is not None:
                self.stats.hits += 1
            else:
                self.stats.misses += 1
                self.stats.bytes_loaded += self.expert_bytes
            gu[s_].copy_(self.bank_gu[res] if res is not None else self.host_gu[e], non_blocking=True)
            dn[s_].copy_(self.bank_dn[res] if res is not None else self.host_dn[e], non_blocking=True)
            if gub is not None:
                gub[s_].copy_(self.bank_gub[res] if res is not None else self.host_gub[e], non_blocking=True)
            if dnb is not None:
                dnb[s_].copy_(self.bank_dnb[res] if res is not None else self.host_dnb[e], non_blocking=True)
            mapping[e] = s_
        return gu, dn, gub, dnb, mapping

    def forward(self, x, ids, weights, residual=None, extra=None, limit: float = 0.0, act: str = "swiglu"):
        """Same contract as :func:`ops.moe.experts_forward` for the local experts [e0, e0 + E_local)."""
        T, H = x.shape
        if self.scratch_bytes > 0:
            # permuted inputs, gated activations and expert outputs of one pass: (2 H + I) elements per route
            inter = self.bank_dn.shape[2]
            per_token = ids.shape[1] * (2 * H + inter) * x.element_size()
            chunk = max(1, self.scratch_bytes // max(1, per_token))
            if T > chunk:
                parts = [self.forward(x[a:a + chunk], ids[a:a + chunk], weights[a:a + chunk],
                                      None if residual is None else residual[a:a + chunk],
                                      None if extra is None else extra[a:a + chunk], limit, act) for a in range(0, T, chunk)]
                return torch.cat(parts, 0)
        self.stats.calls += 1
        local = ids.long() - self.e0
        is_local = (local >= 0) & (local < self.n_experts)
        demand = torch.unique(local[is_local]).tolist()                # host synchronisation: the demand set
        out = None
        transient = T > self.PREFILL_TOKENS and self.prefill_slots > self.slots
        width = self.prefill_slots if transient else self.slots
        passes = [demand[i:i + width] for i in range(0, len(demand), width)] or [[]]
        for pi, group in enumerate(passes):
            self.stats.passes += 1
            if transient:
                gu, dn, gub, dnb, mapping = self._fill_prefill_bank(group)
            else:
                mapping = self.acquire(group)
                gu, dn, gub, dnb = self.bank_gu, self.bank_dn, self.bank_gub, self.bank_dnb
            # ids of this pass: resident experts -> slot number; everything else -> an id no slot owns
            remap = torch.full((self.n_experts,), width, dtype=torch.int32, device=ids.device)
            for e, s in mapping.items():
                remap[e] = s
            pass_ids = torch.where(is_local, remap[local.clamp(0, self.n_experts - 1)], torch.full_like(ids, width)).to(torch.int32)
            part = moe_ops.experts_forward(x, pass_ids, weights, gu, dn, 0,
                                           residual=residual if pi == 0 else None, extra=extra if pi == 0 else None,
                                           limit=limit, gu_bias=gub, down_bias=dnb, act=act)
            out = part if out is None else out + part
        return out

    def report(self) -> dict:
        s = self.stats
        total = max(1, s.hits + s.misses)
        return {"hits": s.hits, "misses": s.misses, "hit_rate": s.hits / total, "evictions": s.evictions,
                "bytes_loaded": s.bytes_loaded, "passes": s.passes, "calls": s.calls, "slots": self.slots,
                "eviction": self.eviction}


def attach_expert_cache(model, slots: int = 0, device_budget_bytes: int = 0, eviction: str = "lru", scratch_bytes: int = 0,
                        prefill_bank_bytes: int = 0) -> list:
    """Replace every sparse block's resident expert banks by an :class:`ExpertCache`. Returns the caches."""
    caches = []
    for lw in model.layers:
        blk = lw.moe
        if blk is None:
            continue
        n = slots or ExpertCache.slots_for_budget(blk.w_gate_up, blk.w_down, device_budget_bytes)
        cache = ExpertCache(blk.w_gate_up, blk.w_down, n, eviction, blk.e0, gu_bias=blk.gu_bias, down_bias=blk.down_bias,
                            scratch_bytes=scratch_bytes, prefill_bank_bytes=prefill_bank_bytes)
        blk.gu_bias = blk.down_bias = None      # the biases now travel with their expert through the bank
        blk.expert_cache = cache
        blk.w_gate_up = blk.w_gate_up[:0]   # the banks now live in the cache (host) - keep shape metadata only
        blk.w_down = blk.w_down[:0]
        caches.append(cache)
    if model.device.type == "cuda":
        torch.cuda.empty_cache()
    return caches
