"""GEMM micro-benchmarks on one GPU (CUDA events, warm-up, numerics checked against an fp32 product).

    python -m benchmarks.bench_gemm prefill     # prefill-sized shapes against cuBLAS (torch.matmul / addmm)
    python -m benchmarks.bench_gemm chain       # decode-sized GEMMs as a dependent chain inside a CUDA graph
    python -m benchmarks.bench_gemm decode      # the four projections of a decoder layer, TP=1 and TP=8 slices
    python -m benchmarks.bench_gemm fp8         # block-scaled FP8 weights: FP8 tensor-core kernel against the bf16 kernel
    python -m benchmarks.bench_gemm fp8 M N K n # profiling aid: n launches of the FP8 kernel on one shape

``prefill`` covers the dense projections of a Llama-3-8B layer at 2048 and 8192 tokens (and their TP=8 slices):
plain, + residual, and fused SwiGLU (cuBLAS arm: one GEMM plus ``silu(g) * u`` as PyTorch element-wise ops).
``chain`` shows what one decode-step GEMM costs when it depends on the previous kernel, with and without the
residual, the sum-of-squares output and cluster split-K.
"""
from __future__ import annotations

import json
import sys

import torch

from eredu_b200 import ops

DEV = torch.device("cuda:0")


def _time(fn, n=10, warm=3):
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


def prefill():
    g = torch.Generator(device=DEV).manual_seed(0)
    shapes = [(8192, 6144, 4096, 0), (8192, 4096, 4096, 1), (8192, 14336, 4096, 2), (8192, 4096, 14336, 1),
              (8192, 4096, 512, 1), (8192, 4096, 1792, 1), (2048, 4096, 4096, 1), (2048, 14336, 4096, 2),
              (2048, 4096, 14336, 1), (128, 4096, 4096, 1), (64, 4096, 4096, 1)]
    for M, N, K, kind in shapes:
        x = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
        w = (torch.randn(N * 2 if kind == 2 else N, K, device=DEV, generator=g) * 0.03).bfloat16()
        r = torch.randn(M, N, device=DEV, generator=g).bfloat16() if kind == 1 else None
        if kind == 2:
            fn = lambda: ops.gated_linear(x, w, N)  # noqa: E731
            gu = x.float() @ w.float().t()
            ref = torch.nn.functional.silu(gu[:, :N]) * gu[:, N:]
            lib = lambda: (lambda z: torch.nn.functional.silu(z[:, :N]) * z[:, N:])(x @ w.t())  # noqa: E731
            flops = 2 * M * 2 * N * K
        else:
            fn = lambda: ops.linear(x, w, residual=r)  # noqa: E731
            ref = x.float() @ w.float().t() + (r.float() if r is not None else 0)
            lib = (lambda: torch.addmm(r, x, w.t())) if r is not None else (lambda: x @ w.t())  # noqa: E731
            flops = 2 * M * N * K
        err = float((fn().float() - ref).norm() / ref.norm())
        us, us_lib = _time(fn), _time(lib)
        print(json.dumps({"M": M, "N": N, "K": K, "epilogue": ["none", "residual", "swiglu"][kind], "us": round(us, 1),
                          "tflops": round(flops / us / 1e6, 1), "cublas_us": round(us_lib, 1),
                          "cublas_tflops": round(flops / us_lib / 1e6, 1), "rel_err": round(err, 5)}))


def _chain(M, N, K, res, ssq, split, n=64, dual=False):
    g = torch.Generator(device=DEV).manual_seed(0)
    x = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
    ws = [(torch.randn(2 * N if dual else N, K, device=DEV, generator=g) * 0.02).bfloat16() for _ in range(8)]
    y = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)

    def run():
        cur = y
        for i in range(n):
            if dual:
                cur = ops.gated_linear(x, ws[i % 8], N, force_split=split)
            elif ssq:
                cur, _ = ops.linear(x, ws[i % 8], residual=cur if res else None, force_split=split, want_ssq=True)
            else:
                cur = ops.linear(x, ws[i % 8], residual=cur if res else None, force_split=split)
        return cur

    run()
    torch.cuda.synchronize()
    graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(stream):
        run()
        with torch.cuda.graph(graph, stream=stream):
            run()
    torch.cuda.synchronize()
    return _time(graph.replay) / n


def chain():
    for M, N, K in [(32, 4096, 512), (32, 4096, 1792), (32, 768, 4096), (1, 4096, 512)]:
        for res, ssq, split in [(0, 0, 1), (1, 0, 1), (1, 1, 1), (0, 0, 4), (1, 0, 4), (1, 1, 4), (1, 1, 8)]:
            print(json.dumps({"M": M, "N": N, "K": K, "residual": res, "ssq_out": ssq, "split": split,
                              "us_per_gemm": round(_chain(M, N, K, res, ssq, split), 2)}))
    for split in (1, 4, 8):
        print(json.dumps({"swiglu": 1, "M": 32, "N": 1792, "K": 4096, "split": split,
                          "us_per_gemm": round(_chain(32, 1792, 4096, 0, 0, split, dual=True), 2)}))


def decode():
    """The four projections of a Llama-3-8B layer at 32 tokens and at 1 token, whole (TP=1) and as a TP=8 rank's slice,
    each as a dependent chain inside a CUDA graph with the launcher's own split choice: us per GEMM and the weight
    stream rate it amounts to."""
    for tp in (1, 8):
        for M in (32, 1):
            for name, N, K, res, ssq, dual in [("qkv", 6144 // tp, 4096, 0, 0, False), ("o_proj", 4096, 4096 // tp, 1, 1, False),
                                               ("gate_up", 14336 // tp, 4096, 0, 0, True), ("down", 4096, 14336 // tp, 1, 1, False)]:
                us = _chain(M, N, K, res, ssq, 0, n=32, dual=dual)
                wbytes = (2 if dual else 1) * N * K * 2
                print(json.dumps({"tp": tp, "M": M, "gemm": name, "N": N, "K": K, "us_per_gemm": round(us, 2),
                                  "weight_GBs": round(wbytes / us / 1e3, 1)}))


def one(M: int, N: int, K: int, kind: str = "residual", reps: int = 3):
    """A single shape, a few launches: the small case a profiler capture runs on (operands above the 126 MB L2 for
    the sizes used in profiles/)."""
    g = torch.Generator(device=DEV).manual_seed(0)
    x = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N * 2 if kind == "swiglu" else N, K, device=DEV, generator=g) * 0.03).bfloat16()
    r = torch.randn(M, N, device=DEV, generator=g).bfloat16() if kind == "residual" else None
    fn = (lambda: ops.gated_linear(x, w, N)) if kind == "swiglu" else (lambda: ops.linear(x, w, residual=r))
    us = _time(fn, n=reps, warm=2)
    flops = 2 * M * N * K * (2 if kind == "swiglu" else 1)
    print(json.dumps({"M": M, "N": N, "K": K, "epilogue": kind, "us": round(us, 1), "tflops": round(flops / us / 1e6, 1),
                      "weight_GBs": round(w.numel() * 2 / us / 1e3, 1)}))


def fp8(argv):
    """Block-FP8 weights at prefill sizes: activation quantisation + FP8 tensor-core GEMM (timed together and the GEMM
    alone) against the bf16 tcgen05 GEMM on the dequantised weight, with the error of both against the fp32 product."""
    from eredu_b200.ops.native import lib, ptr, status_word, stream_ptr
    from eredu_b200.ops.quant import Fp8Linear

    g = torch.Generator(device=DEV).manual_seed(0)
    if argv:
        M, N, K, n = (int(a) for a in argv[:4])
        q = Fp8Linear.from_dense(torch.randn(N, K, device=DEV, generator=g) * 0.03)
        x = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
        for _ in range(n):
            q.tensor_core(x)
        torch.cuda.synchronize()
        ops.native.check_status(DEV)
        print(json.dumps({"M": M, "N": N, "K": K, "launched": n}))
        return
    for M, N, K in [(8192, 4096, 4096), (8192, 14336, 4096), (8192, 4096, 14336), (8192, 7168, 2048), (2048, 4096, 4096),
                    (512, 4096, 4096)]:
        w = torch.randn(N, K, device=DEV, generator=g) * 0.03
        q = Fp8Linear.from_dense(w)
        wd = q.dequantize(torch.bfloat16)
        x = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
        ref = x.float() @ q.dequantize().t()
        y = q.tensor_core(x)
        yb = ops.linear(x, wd)
        xq = torch.empty((M, K), dtype=torch.uint8, device=DEV)
        ld = (M + 127) // 128 * 128
        sx = torch.empty((K // 128, ld), dtype=torch.float32, device=DEV)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
        lib().eredu_fp8_quant_act(ptr(x), x.stride(0), ptr(xq), ptr(sx), ld, M, K, stream_ptr(DEV))
        gemm_only = lambda: lib().eredu_gemm_fp8_tc(ptr(xq), ptr(sx), ld, ptr(q.wq), ptr(q.block_scales), ptr(out), None, None, M, N, K,  # noqa: E731
                                                    N, 0, 0, ptr(status_word(DEV)), stream_ptr(DEV))
        us_all, us_gemm, us_bf16 = _time(lambda: q.tensor_core(x)), _time(gemm_only), _time(lambda: ops.linear(x, wd))
        flops = 2 * M * N * K
        print(json.dumps({"M": M, "N": N, "K": K, "fp8_quant_plus_gemm_us": round(us_all, 1), "fp8_gemm_us": round(us_gemm, 1),
                          "fp8_gemm_tflops": round(flops / us_gemm / 1e6, 1), "bf16_gemm_us": round(us_bf16, 1),
                          "bf16_tflops": round(flops / us_bf16 / 1e6, 1), "speedup_gemm": round(us_bf16 / us_gemm, 2),
                          "speedup_with_quant": round(us_bf16 / us_all, 2),
                          "rel_err_fp8": round(float((y.float() - ref).norm() / ref.norm()), 4),
                          "rel_err_bf16": round(float((yb.float() - ref).norm() / ref.norm()), 4)}), flush=True)
    ops.native.check_status(DEV)


if __name__ == "__main__":
    mode = sys.argv[1] if len(sys.argv) > 1 else "prefill"
    if mode == "one":
        one(int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5] if len(sys.argv) > 5 else "residual")
    elif mode == "fp8":
        fp8(sys.argv[2:])
    else:
        {"prefill": prefill, "chain": chain, "decode": decode}[mode]()
