"""4-bit weight-only linear layers at decode sizes on one GPU: the register-resident kernel (csrc/kernels/qgemv_mma.cu)
against the tcgen05 dequantise-in-pipeline kernel (csrc/kernels/qgemm_tcgen05.cu) on the Llama-3-70B projections and
their tensor-parallel slices.

    python -m benchmarks.bench_qgemm [--peak-gbs 6650]

Each shape is timed as a CUDA graph that walks a set of distinct weight matrices larger than the L2 cache, so every
launch streams its packed weights from HBM. Reported: microseconds per launch, GB/s over the bytes the format stores
(codes + scales + biases = 4.5 bit per weight at group 64) and that as a fraction of ``--peak-gbs`` (the measured copy
bandwidth); the relative error is against the fp32 product with the dequantised weights.
"""
from __future__ import annotations

import argparse
import json

import torch

from eredu_b200.ops.quant import QuantLinear

DEV = torch.device("cuda:0")
L2_BYTES = 126 << 20


def timed_graph(fns, reps=3):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for f in fns:
            f()
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            for f in fns:
                f()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * len(fns))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--peak-gbs", type=float, default=6548.5, help="copy bandwidth the fractions are quoted against")
    ap.add_argument("--group", type=int, default=64)
    ap.add_argument("--only", default=None, help="run one shape by name (e.g. o, down/tp8)")
    ap.add_argument("--tokens", type=int, nargs="*", default=[1, 8])
    ap.add_argument("--plain-launches", type=int, default=0,
                    help="profiling aid: instead of timing, launch the register kernel this many times outside a graph")
    args = ap.parse_args()
    H, I, QKV = 8192, 28672, 8192 + 2 * 1024
    shapes = [("qkv", QKV, H, False), ("o", H, H, False), ("gate_up", 2 * I, H, True), ("down", H, I, False),
              ("qkv/tp8", QKV // 8, H, False), ("o/tp8", H, H // 8, False), ("gate_up/tp8", 2 * I // 8, H, True),
              ("down/tp8", H, I // 8, False)]
    for name, N, K, gated in shapes:
        if args.only is not None and name != args.only:
            continue
        per = N * K // 2 + 2 * 2 * N * (K // args.group)
        copies = max(2, min(16, (2 * L2_BYTES + per - 1) // per))
        torch.manual_seed(0)
        base = QuantLinear.from_dense((torch.randn(N, K, device=DEV) * 0.02).bfloat16(), 4, args.group)
        lins = [base]
        for _ in range(copies - 1):
            q = object.__new__(QuantLinear)
            q.__dict__.update(base.__dict__)
            q.__dict__.pop("_dq_t", None)
            q.wq, q.scales_t, q.biases_t = base.wq.clone(), base.scales_t.clone(), base.biases_t.clone()
            lins.append(q)
        deq = base.dequantize(torch.float32)
        for M in args.tokens:
            x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
            if args.plain_launches:
                for i in range(args.plain_launches):
                    q = lins[i % len(lins)]
                    _ = q.gated(x) if gated else q(x)
                torch.cuda.synchronize()
                print(json.dumps({"shape": name, "M": M, "launched": args.plain_launches}))
                continue
            lin = x.float() @ deq.t()
            ref = torch.nn.functional.silu(lin[:, :N // 2]) * lin[:, N // 2:] if gated else lin
            row = {"shape": name, "N": N, "K": K, "M": M, "swiglu": gated, "weight_sets": copies}
            for arm, cap in (("register_mma", 8), ("tcgen05", 0)):
                QuantLinear.GEMV_MAX_TOKENS = cap
                fns = [(lambda q=q: q.gated(x)) if gated else (lambda q=q: q(x)) for q in lins]
                y = fns[0]()
                us = timed_graph(fns)
                row[arm + "_us"] = round(us, 2)
                row[arm + "_gbs"] = round(per / us / 1e3, 0)
                row[arm + "_of_peak"] = round(per / us / 1e3 / args.peak_gbs, 3)
                row[arm + "_rel"] = float((y.float() - ref).norm() / ref.norm())
            QuantLinear.GEMV_MAX_TOKENS = 8
            row["speedup"] = round(row["tcgen05_us"] / row["register_mma_us"], 2)
            print(json.dumps(row), flush=True)
        del lins, base, deq
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
