"""NVTX ranges for external profilers (Nsight Systems / Compute range filters).

The device-side timeline of ``utils/trace.py`` needs no tool; these ranges are for the tools: with ``EREDU_NVTX=1`` (or
``enable()``) the engine marks prefill groups, decode steps, graph captures, speculative phases and - when the model
runs eagerly - every decoder layer. Disabled, ``annotate`` returns a shared no-op context, so the hot path pays one
attribute lookup. The reference tags its device work through MLX's own trace hooks
(eredu/src/backend/mlx/runtime/execution/inspection.rs); this is the CUDA-tool counterpart."""
from __future__ import annotations

import contextlib
import os

import torch

_enabled = os.environ.get("EREDU_NVTX", "0") not in ("", "0")
_null = contextlib.nullcontext()
ranges_opened = 0          # counted so that tests can see the instrumentation fire without a profiler attached


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


class _Range:
    __slots__ = ("name", "pushed")

    def __init__(self, name: str):
        self.name = name
        self.pushed = False

    def __enter__(self):
        global ranges_opened
        ranges_opened += 1
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)
            self.pushed = True
        return self

    def __exit__(self, *exc):
        if self.pushed:
            torch.cuda.nvtx.range_pop()
        return False


def annotate(name: str):
    """``with annotate("decode_step"):`` - an NVTX range when enabled, nothing otherwise."""
    return _Range(name) if _enabled else _null


def mark(name: str) -> None:
    if _enabled and torch.cuda.is_available():
        torch.cuda.nvtx.mark(name)
