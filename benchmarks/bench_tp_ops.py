"""Micro-benchmark of the tensor-parallel row-parallel projection: the fused tcgen05 GEMM + peer-memory all-reduce
against the same GEMM followed by an NCCL all-reduce, both replayed from CUDA graphs, device-timed, max over ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29544 \\
        -m benchmarks.bench_tp_ops --hidden 4096 --inter 14336
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from eredu_b200.ops import native
from eredu_b200.parallel.context import ParallelContext
from eredu_b200.parallel.topology import ParallelTopology
from eredu_b200.parallel.tp import NcclTPOps, PeerTPOps


def timed_graph(fn, iters=50, warm=5):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(iters):
            fn()
    g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--heads_dim", type=int, default=4096)
    ap.add_argument("--plain-launches", type=int, default=0,
                    help="profiling aid: launch the fused o_proj kernel this many times for --tokens rows (no graph, no timing)")
    ap.add_argument("--tokens", type=int, default=32)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    par = ParallelContext.from_env(ParallelTopology(tensor=world))
    peer = PeerTPOps(par, dev, args.hidden, 128256, max_tokens=4096)
    nccl = NcclTPOps(par, dev)
    rows = []
    torch.manual_seed(1000 + rank)          # activations and weight shards differ per rank ...
    if args.plain_launches:
        K = args.heads_dim // world
        ws = [(torch.randn(args.hidden, K, device=dev) * 0.02).bfloat16() for _ in range(8)]     # distinct weights: cold L2
        x = (torch.randn(args.tokens, K, device=dev) * 0.5).bfloat16()
        res = torch.randn(args.tokens, args.hidden, device=dev).bfloat16()
        for i in range(args.plain_launches):
            peer.row_linear(x, ws[i % len(ws)], residual=res)
        torch.cuda.synchronize()
        native.check_status(dev)
        if rank == 0:
            print(json.dumps({"world": world, "M": args.tokens, "K_local": K, "launched": args.plain_launches}))
        dist.destroy_process_group()
        return
    res_gen = torch.Generator(device=dev).manual_seed(7)   # ... the residual is the same tensor on every rank
    for name, k_full in (("o_proj", args.heads_dim), ("down_proj", args.inter)):
        K = k_full // world
        w = (torch.randn(args.hidden, K, device=dev) * 0.02).bfloat16()
        for M in (1, 8, 32, 64, 512, 2048):
            x = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
            res = torch.randn(M, args.hidden, device=dev, generator=res_gen).bfloat16()
            t_peer = timed_graph(lambda: peer.row_linear(x, w, residual=res))
            t_nccl = timed_graph(lambda: nccl.row_linear(x, w, residual=res))
            a = peer.row_linear(x, w, residual=res).float()
            b = nccl.row_linear(x, w, residual=res).float()
            rel = float((a - b).norm() / b.norm())
            # bytes one rank sends (and receives) over NVLink: the one-shot kernel pushes its whole bf16 partial to every
            # peer; the two-shot path moves (world-1)/world of it in each of its two phases
            full = M * args.hidden * 2
            link_bytes = full * (world - 1) if M <= 64 else 2 * full * (world - 1) / world
            rows.append({"op": name, "M": M, "K_local": K, "fused_us": round(t_peer, 2), "gemm_plus_nccl_us": round(t_nccl, 2),
                         "speedup": round(t_nccl / t_peer, 2), "rel_diff": rel, "nvlink_bytes_per_rank": int(link_bytes),
                         "roofline_us": round(max(2 * M * args.hidden * K / 1.6633e15, link_bytes / 770e9) * 1e6, 2)})
    native.check_status(dev)
    if rank == 0:
        for r in rows:
            print(json.dumps({"world": world, **r}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
