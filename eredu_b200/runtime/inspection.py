"""Activation inspection hooks: named tensors of a forward pass handed to an observer, optional interventions at
block outputs, and normalised MoE routing records.

Counterpart of eredu/src/backend/mlx/runtime/execution/inspection.rs (``ActivationObserver::{observe, intervene,
observe_moe_routing}``, ``MoeRoutingObservation``). An observed pass runs eagerly (no CUDA graph) and, for sparse
blocks, through the unfused routing path so that the intermediate tensors exist; unobserved passes pay one attribute
test per layer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class MoeRoutingObservation:
    prefix: str                        # path-like name of the block, e.g. "model.layers.3.mlp"
    selected_experts: torch.Tensor     # [tokens, top_k] int32
    selected_scores: torch.Tensor      # [tokens, top_k] scores of the selected experts before renormalisation
    routing_weights: torch.Tensor      # [tokens, top_k] weights applied to the expert outputs
    routed_output: torch.Tensor        # [tokens, hidden] summed routed contribution (this rank's experts)
    num_experts: int
    local_routed_output: Optional[torch.Tensor] = None    # before the expert-parallel reduction
    reduced_routed_output: Optional[torch.Tensor] = None  # after it
    shared_output: Optional[torch.Tensor] = None
    combined_output: Optional[torch.Tensor] = None


class ActivationObserver:
    """Base class: override what you need. ``intervene`` may return a replacement for the named activation."""

    def observe(self, name: str, value: torch.Tensor) -> None:
        pass

    def intervene(self, name: str, value: torch.Tensor) -> Optional[torch.Tensor]:
        return None

    def observe_moe_routing(self, routing: MoeRoutingObservation) -> None:
        pass


class RecordingObserver(ActivationObserver):
    """Keeps detached CPU copies of everything it sees (small models, tests, debugging sessions)."""

    def __init__(self, names=None):
        self.names = set(names) if names is not None else None
        self.tensors: dict[str, torch.Tensor] = {}
        self.routing: list[MoeRoutingObservation] = []

    def observe(self, name, value):
        if self.names is None or name in self.names:
            self.tensors[name] = value.detach().float().cpu()

    def observe_moe_routing(self, routing):
        self.routing.append(routing)


class observed:
    """Context manager that installs an observer on a model for the passes run inside it."""

    def __init__(self, model, observer: ActivationObserver):
        self.model, self.observer = getattr(model, "inner", model), observer

    def __enter__(self):
        self.prev = getattr(self.model, "observer", None)
        self.model.observer = self.observer
        return self.observer

    def __exit__(self, *exc):
        self.model.observer = self.prev


class ComponentProfiler(ActivationObserver):
    """Wall time between consecutive observation points of an observed pass: embedding, every block, and (via
    :meth:`finish`) the output head. CUDA work is synchronised at each point, so the figures are per-component device
    times of an eager pass, not of the graph-replayed decode step (``--profile-components``)."""

    def __init__(self, device=None):
        import time

        self._now = time.perf_counter
        self.device = device
        self.stages: list[tuple[str, float]] = []
        self._t = None

    def _sync(self):
        if self.device is not None and torch.device(self.device).type == "cuda":
            torch.cuda.synchronize(self.device)

    def start(self):
        self._sync()
        self._t = self._now()

    def observe(self, name, value):
        self._sync()
        t = self._now()
        if self._t is not None:
            self.stages.append((name, t - self._t))
        self._t = t

    def finish(self, name="lm_head"):
        self.observe(name, None)

    def summary(self) -> dict:
        total = sum(d for _, d in self.stages) or 1e-12
        return {"total_seconds": total,
                "stages": [{"name": n, "seconds": d, "share": d / total} for n, d in self.stages]}
