"""Recurrent scans at prefill length on one GPU: the chunk-parallel GEMM forms (ops/recurrent.py) against the
token-by-token kernels (csrc/kernels/gated_delta.cu, mamba2_scan.cu).

    python -m benchmarks.bench_scans [--tokens 2048 8192]

Shapes: a gated-delta layer of a Qwen3-Next-class model (32 value heads, key / value width 128) and a Mamba-2 layer of a
Nemotron-H-class model (64 heads of width 64, state 128, 8 groups). CUDA events, 5 launches after 2 warm-ups.
"""
from __future__ import annotations

import argparse
import json

import torch

from eredu_b200.ops import recurrent as R

DEV = torch.device("cuda:0")


def _time(fn, n=5, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, nargs="*", default=[2048, 8192])
    args = ap.parse_args()
    g = torch.Generator(device=DEV).manual_seed(0)
    for T in args.tokens:
        H, Dk, Dv = 32, 128, 128
        q = (torch.randn(1, T, H, Dk, device=DEV, generator=g) * 0.3).bfloat16()
        k = torch.nn.functional.normalize(torch.randn(1, T, H, Dk, device=DEV, generator=g), dim=-1).bfloat16()
        v = torch.randn(1, T, H, Dv, device=DEV, generator=g).bfloat16()
        ld = -torch.rand(1, T, H, device=DEV, generator=g) * 0.2
        beta = torch.rand(1, T, H, device=DEV, generator=g)
        keep = R.CHUNKED_SCAN_MIN_TOKENS
        R.CHUNKED_SCAN_MIN_TOKENS = 1 << 30
        Sk, ok = R.gated_delta_scan(q, k, v, ld, beta)
        us_kernel = _time(lambda: R.gated_delta_scan(q, k, v, ld, beta))
        R.CHUNKED_SCAN_MIN_TOKENS = keep
        Sc, oc = R.gated_delta_scan_chunked(q, k, v, ld, beta)
        us_chunk = _time(lambda: R.gated_delta_scan_chunked(q, k, v, ld, beta))
        print(json.dumps({"op": "gated_delta", "tokens": T, "heads": H, "kernel_us": round(us_kernel, 1), "chunked_us": round(us_chunk, 1),
                          "speedup": round(us_kernel / us_chunk, 2),
                          "rel_diff": float((ok.float() - oc.float()).norm() / ok.float().norm())}), flush=True)
        H, P, N, G = 64, 64, 128, 8
        x = (torch.randn(1, T, H, P, device=DEV, generator=g) * 0.5).bfloat16()
        Bm, Cm = (torch.randn(1, T, G, N, device=DEV, generator=g) * 0.3).bfloat16(), (torch.randn(1, T, G, N, device=DEV, generator=g) * 0.3).bfloat16()
        dt = torch.rand(1, T, H, device=DEV, generator=g) * 0.1 + 0.001
        A, D = -torch.rand(H, device=DEV, generator=g) * 4 - 0.5, torch.randn(H, device=DEV, generator=g)
        R.CHUNKED_SCAN_MIN_TOKENS = 1 << 30
        Sk, yk = R.mamba2_scan(x, Bm, Cm, dt, A, D)
        us_kernel = _time(lambda: R.mamba2_scan(x, Bm, Cm, dt, A, D))
        R.CHUNKED_SCAN_MIN_TOKENS = keep
        Sc, yc = R.mamba2_scan_chunked(x, Bm, Cm, dt, A, D)
        us_chunk = _time(lambda: R.mamba2_scan_chunked(x, Bm, Cm, dt, A, D))
        print(json.dumps({"op": "mamba2", "tokens": T, "heads": H, "kernel_us": round(us_kernel, 1), "chunked_us": round(us_chunk, 1),
                          "speedup": round(us_kernel / us_chunk, 2),
                          "rel_diff": float((yk.float() - yc.float()).norm() / yk.float().norm())}), flush=True)


if __name__ == "__main__":
    main()
