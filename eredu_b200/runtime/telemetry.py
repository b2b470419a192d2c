"""Execution telemetry: the structured record of one run (plan, hardware, byte and time accounting).

Counterpart of eredu/src/runtime/telemetry.rs:29-400 (``ExecutionTelemetry`` with the frozen plan, per-stage
timing, residency and cache counters, written by ``--telemetry-json``) and of the hardware survey in
eredu/src/runtime/plan/inspection.rs (device name, memory, interconnect).
"""
from __future__ import annotations

import json
import os
import platform
import time
from dataclasses import asdict, dataclass, field
from typing import Optional

SCHEMA_VERSION = 1


def hardware_profile(device: str = "cpu") -> dict:
    """What the planner knows about the machine: host memory and cores, and for CUDA devices name, memory,
    SM count and peer reachability."""
    prof = {"host": {"platform": platform.platform(), "cpus": os.cpu_count()}}
    try:
        import psutil

        vm = psutil.virtual_memory()
        prof["host"]["memory_bytes"] = int(vm.total)
        prof["host"]["available_bytes"] = int(vm.available)
    except Exception:
        pass
    import torch

    if device.startswith("cuda") and torch.cuda.is_available():
        idx = int(device.split(":")[1]) if ":" in device else torch.cuda.current_device()
        p = torch.cuda.get_device_properties(idx)
        free, total = torch.cuda.mem_get_info(idx)
        prof["device"] = {"index": idx, "name": p.name, "sm_count": p.multi_processor_count, "memory_bytes": int(total),
                          "free_bytes": int(free), "compute_capability": f"{p.major}.{p.minor}",
                          "device_count": torch.cuda.device_count()}
    else:
        prof["device"] = {"name": "cpu"}
    return prof


def allocator_metrics(device: str = "cpu") -> dict:
    """Device allocator and process memory figures after a run (the allocator / process sections of the reference's
    execution telemetry, eredu-core/src/automatic.rs:360-368; residency.rs:681-760)."""
    out: dict = {}
    import torch

    if device.startswith("cuda") and torch.cuda.is_available():
        st = torch.cuda.memory_stats(device)
        out["device"] = {"active_bytes": int(st.get("active_bytes.all.current", 0)),
                         "peak_active_bytes": int(st.get("active_bytes.all.peak", 0)),
                         "reserved_bytes": int(st.get("reserved_bytes.all.current", 0)),
                         "peak_reserved_bytes": int(st.get("reserved_bytes.all.peak", 0)),
                         "allocation_retries": int(st.get("num_alloc_retries", 0))}
    from .host_pool import _default as pool

    if pool is not None:
        out["host_transfer_buffers"] = pool.stats()     # pinned staging memory by purpose: active / peak / reuse counts
    try:
        import psutil

        m = psutil.Process().memory_info()
        out["process"] = {"rss_bytes": int(m.rss), "vms_bytes": int(m.vms)}
        try:
            import resource

            ru = resource.getrusage(resource.RUSAGE_SELF)
            out["process"].update(max_rss_kib=int(ru.ru_maxrss), minor_faults=int(ru.ru_minflt), major_faults=int(ru.ru_majflt))
        except Exception:
            pass
    except Exception:
        pass
    return out


@dataclass
class StageTiming:
    name: str
    seconds: float = 0.0
    calls: int = 0


@dataclass
class ExecutionTelemetry:
    plan: dict = field(default_factory=dict)
    hardware: dict = field(default_factory=dict)
    prompt_tokens: int = 0
    generated_tokens: int = 0
    stop_reason: Optional[str] = None
    timing: dict = field(default_factory=dict)
    weights_bytes: int = 0
    kv_bytes: int = 0
    stages: list = field(default_factory=list)
    counters: dict = field(default_factory=dict)
    schema_version: int = SCHEMA_VERSION
    created_unix: float = field(default_factory=time.time)

    def stage(self, name: str):
        """Context manager that accumulates wall time for a named stage (--profile-components)."""
        tel = self

        class _Ctx:
            def __enter__(self):
                self.t0 = time.perf_counter()

            def __exit__(self, *exc):
                dt = time.perf_counter() - self.t0
                for s in tel.stages:
                    if s.name == name:
                        s.seconds += dt
                        s.calls += 1
                        return False
                tel.stages.append(StageTiming(name, dt, 1))
                return False

        return _Ctx()

    def count(self, key: str, n: int = 1):
        self.counters[key] = self.counters.get(key, 0) + n

    def to_dict(self) -> dict:
        return asdict(self)

    def write(self, path: str):
        tmp = f"{path}.tmp"
        with open(tmp, "w") as f:
            json.dump(self.to_dict(), f, indent=2, default=str)
        os.replace(tmp, path)
