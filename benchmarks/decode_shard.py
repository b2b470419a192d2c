"""Decode step of ONE tensor-parallel shard on one GPU, without the collectives: what a rank of a TP=N group spends on
its own kernels (weights, KV pages, launches) per CUDA-graph step. The difference to the multi-GPU step time is the cost
of the fused collectives.

    python -m benchmarks.decode_shard --tp-shape 8 --batch 32 --steps 50          # device-timed mean step
    python -m benchmarks.decode_shard --tp-shape 8 --batch 1 --ctx 2048 --trace   # + per-kernel device timeline summary
"""
from __future__ import annotations

import argparse
import dataclasses
import json

import numpy as np
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_random
from eredu_b200.ops import SamplingParams, native
from eredu_b200.runtime.engine import Engine


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp-shape", type=int, default=8, help="shape the model like one rank's shard at this TP degree")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--trace", action="store_true")
    ap.add_argument("--timeline", type=int, default=0, help="with --trace: print the first N marks of the traced step")
    a = ap.parse_args()
    base = C.llama3_8b()
    tp = a.tp_shape
    cfg = dataclasses.replace(base, num_hidden_layers=a.layers, num_attention_heads=base.num_attention_heads // tp,
                              num_key_value_heads=max(1, base.num_key_value_heads // tp),
                              intermediate_size=base.intermediate_size // tp, vocab_size=base.vocab_size // tp)
    dev = torch.device("cuda:0")
    model = build_random(cfg, dev, torch.bfloat16, seed=0)
    eng = Engine(model, max_batch=a.batch, max_seq_len=a.ctx + a.steps + 64, prefill_chunk=8192)
    rng = np.random.default_rng(0)
    seqs = [eng.new_sequence(rng.integers(0, cfg.vocab_size, a.ctx).tolist(), SamplingParams(temperature=0.0), a.steps + 32)
            for _ in range(a.batch)]
    eng.start_decode(seqs, eng.prefill(seqs))
    for _ in range(8):
        eng.decode_step(sync=False)
    torch.cuda.synchronize()
    n0 = native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        eng.decode_step(sync=False)
    e1.record()
    torch.cuda.synchronize()
    native.check_status(dev)
    ms = e0.elapsed_time(e1) / a.steps
    out = {"tp_shape": tp, "batch": a.batch, "ctx": a.ctx, "layers": a.layers, "steps": a.steps, "ms_per_step": round(ms, 4),
           "tokens_per_s_shard": round(a.batch / ms * 1e3, 1), "eager_launches_in_loop": native.launch_count() - n0}
    if a.trace:
        from eredu_b200.utils.trace import DeviceTrace, summarise

        tr = DeviceTrace(dev)
        tr.reset()
        eng.decode_step(sync=False)
        recs = tr.records()
        s = summarise(recs)
        tr.close()
        for t, k, ph in recs[:a.timeline]:
            print(f"{t / 1e3:10.2f} us  {k:14s} {ph}")
        s.pop("timeline")
        out["trace"] = s
    print(json.dumps(out))


if __name__ == "__main__":
    main()
