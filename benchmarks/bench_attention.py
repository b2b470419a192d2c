"""Prefill attention on one GPU: the tcgen05 kernel (csrc/kernels/attention_tc.cu) against the mma.sync kernel
(csrc/kernels/attention.cu) on Llama-3-8B head geometry (32 query heads, 8 key / value heads, head size 128).

    python -m benchmarks.bench_attention [--tokens 2048 8192] [--launches N]

CUDA events around 10 launches after 3 warm-ups; causal FLOPs = 4 * S^2 * heads * 128 / 2 for one sequence of S tokens with
an empty cache (the prefill of a prompt). ``--launches N``: profiling aid, launch the tcgen05 kernel N times and exit.
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from eredu_b200 import ops
from eredu_b200.ops import core

DEV = torch.device("cuda:0")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, nargs="*", default=[2048, 8192])
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--launches", type=int, default=0)
    args = ap.parse_args()
    D = 128
    for S in args.tokens:
        pages = (S + 15) // 16
        g = torch.Generator(device=DEV).manual_seed(0)
        kc = torch.randn(pages + 1, args.kv_heads, 16, D, device=DEV, generator=g).bfloat16()
        vc = torch.randn(pages + 1, args.kv_heads, 16, D, device=DEV, generator=g).bfloat16()
        bt = (torch.randperm(pages, device=DEV, generator=g).int() + 1).view(1, pages).contiguous()
        q = torch.randn(S, args.heads, D, device=DEV, generator=g).bfloat16()
        cu = torch.tensor([0, S], device=DEV, dtype=torch.int32)
        sl = torch.tensor([S], device=DEV, dtype=torch.int32)
        scale = 1 / math.sqrt(D)
        if args.launches:
            for _ in range(args.launches):
                ops.attention_prefill(q, kc, vc, bt, sl, cu, S, scale)
            torch.cuda.synchronize()
            print(json.dumps({"tokens": S, "launched": args.launches}))
            continue
        flops = 4.0 * S * S * args.heads * D / 2
        row = {"tokens": S, "heads": args.heads, "kv_heads": args.kv_heads}
        outs = {}
        for name, on in (("tcgen05", True), ("mma_sync", False)):
            core.TC_PREFILL = on
            for _ in range(3):
                outs[name] = ops.attention_prefill(q, kc, vc, bt, sl, cu, S, scale)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                ops.attention_prefill(q, kc, vc, bt, sl, cu, S, scale)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 100.0
            row[name + "_us"] = round(us, 1)
            row[name + "_tflops"] = round(flops / us / 1e6, 1)
        core.TC_PREFILL = True
        row["speedup"] = round(row["mma_sync_us"] / row["tcgen05_us"], 2)
        row["rel_diff"] = float((outs["tcgen05"].float() - outs["mma_sync"].float()).norm() / outs["mma_sync"].float().norm())
        ops.native.check_status(DEV)
        print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
