"""Device-side kernel timeline: which kernel started when, when its stream dependency resolved, when it ended.

The kernels of this library carry ``trace_mark`` points (csrc/common/trace.cuh) that record the GPU's global
nanosecond timer from thread 0 of block 0. They also fire inside CUDA graphs, so this shows the overlap that
programmatic dependent launch buys (or fails to buy) in the captured decode step - something neither CUDA events
nor a serialising profiler can show. Counterpart of the reference's device timing notes (doc/device-timing.md).

    python -m eredu_b200.utils.trace --tp-shape 8 --batch 32          # timeline summary of one decode step
"""
from __future__ import annotations

import argparse
import ctypes
import dataclasses
import json

import torch

from ..ops import native

KERNELS = {1: "gemm", 2: "gemm_persistent", 3: "qgemm", 4: "attn_decode", 5: "attn_prefill", 6: "rope_kv", 7: "rmsnorm",
           8: "embedding", 9: "sampler", 10: "decode_advance", 11: "moe", 12: "silu_mul", 13: "comm"}
PHASES = {0: "start", 1: "after_wait", 2: "end"}
_UNITS = ("gemm", "gemm_persistent", "attention", "norm_rope", "sampler")


class DeviceTrace:
    def __init__(self, device, capacity: int = 1 << 16):
        self.device = torch.device(device)
        self.cap = capacity
        self.buf = torch.zeros((capacity, 2), dtype=torch.int64, device=self.device)
        self.count = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._install(self.buf.data_ptr(), self.count.data_ptr(), capacity)

    def _install(self, buf, count, cap):
        lib = native.lib()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for unit in _UNITS:
                fn = getattr(lib, f"eredu_trace_install_{unit}")
                fn.restype = ctypes.c_int
                fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint]
                code = fn(buf, count, cap)
                if code != 0:
                    raise RuntimeError(f"trace install ({unit}) failed with CUDA error {code}")

    def reset(self):
        torch.cuda.synchronize(self.device)
        self.count.zero_()

    def close(self):
        self._install(None, None, 0)

    def records(self):
        """[(time ns relative to the first record, kernel name, phase name)] in time order."""
        torch.cuda.synchronize(self.device)
        n = min(int(self.count.item()), self.cap)
        rows = self.buf[:n].cpu().tolist()
        rows.sort(key=lambda r: r[0])
        t0 = rows[0][0] if rows else 0
        return [(t - t0, KERNELS.get(tag >> 8, str(tag >> 8)), PHASES.get(tag & 0xFF, str(tag & 0xFF))) for t, tag in rows]


def summarise(records) -> dict:
    """Pair the marks of block 0 of every launch (start -> after_wait -> end in time order per kernel kind) and
    report per kind: launches, mean time blocked on the dependency, mean run time after it, and the mean gap
    from the previous kernel's end to this kernel's dependency release."""
    launches = []
    open_by_kind: dict[str, list] = {}
    for t, k, ph in records:
        if ph == "start":
            open_by_kind.setdefault(k, []).append({"kernel": k, "start": t})
        elif ph == "after_wait":
            for rec in open_by_kind.get(k, []):
                if "after_wait" not in rec:
                    rec["after_wait"] = t
                    break
        elif ph == "end":
            lst = open_by_kind.get(k, [])
            for i, rec in enumerate(lst):
                if "after_wait" in rec and "end" not in rec:
                    rec["end"] = t
                    launches.append(lst.pop(i))
                    break
    for lst in open_by_kind.values():
        launches.extend(lst)
    launches.sort(key=lambda r: r["start"])
    per: dict[str, dict] = {}
    for r in launches:
        d = per.setdefault(r["kernel"], {"launches": 0, "wait_ns": 0, "run_ns": 0, "runs": 0})
        d["launches"] += 1
        if "after_wait" in r:
            d["wait_ns"] += r["after_wait"] - r["start"]
            if "end" in r:
                d["run_ns"] += r["end"] - r["after_wait"]
                d["runs"] += 1
    out = {}
    for k, d in per.items():
        out[k] = {"launches": d["launches"], "mean_wait_us": round(d["wait_ns"] / max(1, d["launches"]) / 1e3, 2),
                  "mean_run_after_wait_us": round(d["run_ns"] / d["runs"] / 1e3, 2) if d["runs"] else None}
    span = (records[-1][0] - records[0][0]) / 1e3 if records else 0.0
    return {"span_us": round(span, 1), "launches": len(launches), "per_kernel": out, "timeline": launches}


def main():
    import numpy as np

    from ..models import config as C
    from ..models.llama import build_random
    from ..ops import SamplingParams
    from ..runtime.engine import Engine

    ap = argparse.ArgumentParser()
    ap.add_argument("--tp-shape", type=int, default=1, help="shape the model like one rank's shard at this TP degree")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--timeline", type=int, default=0, help="print the first N launches of the traced step")
    a = ap.parse_args()
    base = C.llama3_8b()
    tp = a.tp_shape
    cfg = dataclasses.replace(base, num_hidden_layers=a.layers, num_attention_heads=base.num_attention_heads // tp,
                              num_key_value_heads=max(1, base.num_key_value_heads // tp),
                              intermediate_size=base.intermediate_size // tp, vocab_size=base.vocab_size // tp)
    dev = torch.device("cuda:0")
    model = build_random(cfg, dev, torch.bfloat16, seed=0)
    eng = Engine(model, max_batch=a.batch, max_seq_len=a.ctx + 128, prefill_chunk=8192)
    rng = np.random.default_rng(0)
    seqs = [eng.new_sequence(rng.integers(0, cfg.vocab_size, a.ctx).tolist(), SamplingParams(temperature=0.0), 64)
            for _ in range(a.batch)]
    eng.start_decode(seqs, eng.prefill(seqs))
    for _ in range(8):
        eng.decode_step(sync=False)
    tr = DeviceTrace(dev)
    tr.reset()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    eng.decode_step(sync=False)
    e1.record()
    recs = tr.records()
    tr.close()
    s = summarise(recs)
    tl = s.pop("timeline")
    s["event_ms"] = round(e0.elapsed_time(e1), 4)
    print(json.dumps(s))
    if a.timeline:
        for t, k, ph in recs[:a.timeline * 6]:
            print(f"{t / 1e3:10.2f} us  {k:14s} {ph}")
    for r in tl[:0]:
        print(f"{r['kernel']:16s} start {r['start'] / 1e3:9.2f}  wait_done {r.get('after_wait', 0) / 1e3:9.2f}  "
              f"end {r.get('end', 0) / 1e3:9.2f} us")


if __name__ == "__main__":
    main()
