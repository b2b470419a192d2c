#!/usr/bin/env python
"""Headline benchmark: decode tokens/s (batch 32 and batch 1) and p50 TTFT of a Llama-3-8B-shaped bf16
decoder, tensor-parallel over N GPUs of one node, paged KV cache with 16-token pages, prompts of 2048
uniform-random token ids, random-init weights.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched by torch.distributed.run)

A "step" is one decode step of the whole batch (32 sequences -> 32 tokens). The timed region holds
exactly K steps between CUDA events, after W warm-up steps, with the optimiser-free inference work
complete in every step (forward of all layers, logits, sampling, KV append, device-side bookkeeping).
Every step streams the full weight shard (>= 2 GB per rank, far above the 126 MB L2) and the KV pages,
so the inputs exceed L2 and no flush is needed between iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REFERENCE_UNAVAILABLE = ("reference is a Rust workspace on Apple MLX: pip install of its source tree -> 'not installable: "
                         "neither setup.py nor pyproject.toml'; no cargo/rustc here and its MLX source archive is missing")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def run_speculative(args, eng, model, cfg, prompts, dev, world, rank) -> int:
    """Speculative decoding: the target runs tensor-parallel over the ranks, the draft is replicated on every rank
    (identical proposals everywhere, no extra collective). Reports accepted tokens per round, verify / draft step
    latency and decode tokens/s over K emitted tokens per sequence."""
    import torch

    from eredu_b200.models import config as C
    from eredu_b200.models.llama import build_random
    from eredu_b200.ops import SamplingParams
    from eredu_b200.runtime.engine import Engine
    from eredu_b200.runtime.speculative import GraphSpeculativeDecoder

    K, B, P = args.steps, args.batch, args.prompt_len
    if args.spec_draft == "self":
        draft_eng = Engine(model, max_batch=B, max_seq_len=P + 2 * K + 64, prefill_chunk=8192)
    else:
        dcfg = C.draft_llama_16l()
        draft = build_random(dcfg, dev, torch.bfloat16, seed=1)
        draft_eng = Engine(draft, max_batch=B, max_seq_len=P + 2 * K + 64, prefill_chunk=8192)
    dec = GraphSpeculativeDecoder(eng, draft_eng, k=args.spec_k)

    def one(temperature, top_p):
        sp = SamplingParams(temperature=temperature, top_p=top_p, top_k=0, min_p=0.0, seed=1)
        dec.generate(prompts[:B], sp, max_new_tokens=8)  # warm-up (kernel configuration, allocator)
        dec.stats = type(dec.stats)()
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        outs = dec.generate(prompts[:B], sp, max_new_tokens=K)
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1)
        emitted = sum(len(o) for o in outs)
        st = dec.stats.summary()
        decode_ms = ms - st["prefill_ms"]   # both prefills (target and draft) are timed inside generate and taken out
        return {"temperature": temperature, "top_p": top_p, "decode_tokens_per_s": round((emitted - B) / (decode_ms / 1e3), 2),
                "total_ms": round(ms, 2), "decode_ms": round(decode_ms, 2), "verify_step_ms_p50": st["verify_ms_p50"],
                "accepted_per_round": st["accepted_per_step"], "speculative": st}

    # the preset of BASELINE configuration 5 reports the greedy and the T = 0.8 / top-p 0.95 variant side by side
    variants = [one(0.0, 1.0), one(0.8, 0.95)] if args.config == 5 else [one(args.temperature, args.top_p)]
    head = variants[0]
    result = {"metric": "speculative_decode_tokens_per_s", "value": head["decode_tokens_per_s"], "unit": "tokens/s",
              "n_gpus": world, "steps": K, "higher_is_better": True, "dtype": "bf16", "impl": "eredu_b200",
              "data": "synthetic (random-init target; the 16-layer draft shares the target's embedding, head and first "
                      "layer by seed only when built so - acceptance of a random draft is chance level)",
              "config": {"model": args.model + "-shaped", "draft": args.spec_draft, "k": args.spec_k, "global_batch": B,
                         "seq_len": P, "parallelism": f"tp{world}"},
              "includes_prefill": False, "round_ms_p50": head["verify_step_ms_p50"], "variants": variants}
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        sys.stdout.flush()
        os._exit(0)
    return 0


def run_torch_baseline(args, inline: bool = False):
    """Stand-in for the reference arm that cannot be built here: stock PyTorch operators (cuBLAS GEMMs, library
    attention, NCCL collectives) on the same shapes, batch, context and timing protocol; decode only. ``inline``: called
    from the product arm's process (process group already up); returns the result instead of printing it."""
    import torch

    from baseline.torch_llama import TorchLlamaTP
    from eredu_b200.models import config as C   # shapes only

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 and not inline:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    cfg = {"llama3-8b": C.llama3_8b, "llama3-70b": C.llama3_70b, "tiny": C.tiny_llama}[args.model]()
    K, W, B, P = args.steps, max(args.warmup, 3), args.batch, args.prompt_len
    model = TorchLlamaTP(cfg, dev, rank, world, None, max_len=P + 64, batch=B)
    model.prefill_fill(P)
    tokens = torch.randint(0, cfg.vocab_size, (B,), device=dev)
    pos = torch.full((B,), P, device=dev, dtype=torch.long)
    kv_len = P + 1   # fixed context: the timed steps all attend to P + 1 positions
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for _ in range(2):
            out = model.decode_step(tokens, pos, kv_len)
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = model.decode_step(tokens, pos, kv_len)
        tokens.copy_(out)
    for _ in range(W):
        graph.replay()
    torch.cuda.synchronize(dev)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        graph.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1)
    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    line = {"impl": "torch-baseline", "metric": "decode_tokens_per_s", "value": round(B * K / (ms / 1e3), 2),
            "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 4),
            "higher_is_better": True, "dtype": "bf16", "data": "synthetic (random weights and cache)",
            "config": {"model": args.model + "-shaped", "global_batch": B, "seq_len": P, "parallelism": f"tp{world}",
                       "stack": "F.linear (cuBLAS) + F.scaled_dot_product_attention + NCCL all-reduce / all-gather, CUDA graph",
                       "kv": "contiguous cache, fixed context of seq_len + 1"}}
    if inline:
        del graph, model
        torch.cuda.synchronize(dev)
        torch.cuda.empty_cache()
        return line
    if rank == 0:
        print(json.dumps(line))
    # The captured graph holds NCCL kernels: release it and drain the device before the communicator goes away
    # (tearing the process group down under a live graph did not return on eight ranks).
    del graph
    torch.cuda.synchronize(dev)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        torch.cuda.synchronize(dev)
        sys.stdout.flush()
        os._exit(0)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="eredu_b200", choices=["eredu_b200", "reference", "torch-baseline"],
                    help="torch-baseline: the same decode step from stock PyTorch / cuBLAS / NCCL only (baseline/torch_llama.py)")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "llama3-70b", "qwen3-30b-a3b", "tiny"])
    ap.add_argument("--quantize", type=int, default=0, help="load-time affine quantisation bits (0 = bf16 weights)")
    ap.add_argument("--group-size", type=int, default=64)
    ap.add_argument("--ttft-runs", type=int, default=5)
    ap.add_argument("--skip-b1", action="store_true")
    ap.add_argument("--spec-k", type=int, default=0, help="speculative decoding: draft tokens per round (0 = off)")
    ap.add_argument("--spec-draft", default="llama-16l", choices=["llama-16l", "self"],
                    help="draft model: a 16-layer 2048-wide Llama (random init: acceptance ~0) or the target itself "
                         "(acceptance 1 under greedy: the upper bound and the pure verify/draft step costs)")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--config", type=int, default=0, choices=[0, 2, 3, 4, 5],
                    help="preset of a benchmark configuration: 2 = Llama-3-8B bf16 (batch 32, prompt 2048; the default), "
                         "3 = Qwen3-30B-A3B (experts over the GPUs, batch 32, prompt 1024), 4 = Llama-3-70B 4-bit group 64 "
                         "(batch 8, prompt 4096), 5 = speculative decoding (8B target + 16-layer draft, k = 4, batch 1, prompt 512)")
    ap.add_argument("--ep-mode", default="replicated", choices=["replicated", "a2a"],
                    help="sparse models on several GPUs: replicated tokens + summed partial outputs, or token-sharded "
                         "all-to-all dispatch / combine")
    ap.add_argument("--ep-backend", default="peer", choices=["peer", "collective"],
                    help="collectives of the tensor / expert ranks: kernels over NVLink peer memory, or torch.distributed (NCCL)")
    ap.add_argument("--router-skew", type=float, default=0.0,
                    help="sparse models: this fraction of the tokens is biased onto 8 hot experts (0 = as routed)")
    ap.add_argument("--no-baseline", action="store_true", help="skip the in-process baseline arm that fills vs_baseline")
    args = ap.parse_args()
    if args.config == 3:
        args.model, args.batch, args.prompt_len = "qwen3-30b-a3b", 32, 1024
    elif args.config == 4:
        args.model, args.batch, args.prompt_len, args.quantize, args.group_size = "llama3-70b", 8, 4096, 4, 64
    elif args.config == 5:
        args.model, args.batch, args.prompt_len = "llama3-8b", 1, 512
        args.spec_k = args.spec_k or 4

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0

    if args.impl == "torch-baseline":
        return run_torch_baseline(args)

    import numpy as np
    import torch

    from eredu_b200.models import config as C
    from eredu_b200.models.llama import build_random
    from eredu_b200.ops import SamplingParams, native
    from eredu_b200.parallel.context import ParallelContext
    from eredu_b200.parallel.topology import ParallelTopology
    from eredu_b200.runtime.engine import Engine

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(f"bench.py --gpus {args.gpus} must be launched with torch.distributed.run", file=sys.stderr)
            return 2
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    cfg = {"llama3-8b": C.llama3_8b, "llama3-70b": C.llama3_70b, "qwen3-30b-a3b": C.qwen3_30b_a3b,
           "tiny": C.tiny_llama}[args.model]()
    is_moe = cfg.num_experts > 0
    par = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
        # sparse models: attention tensor-parallel and experts expert-parallel over the same GPUs
        topo = ParallelTopology(tensor=world, expert=world, expert_over_tensor=True) if is_moe else ParallelTopology(tensor=world)
        par = ParallelContext.from_env(topo)
    K, W, B, P = args.steps, max(args.warmup, 3), args.batch, args.prompt_len
    HOLD = 150
    budget = 2 * (W + K + HOLD) + 32
    moe_factory = quantizer = None
    if is_moe:
        from eredu_b200.models.moe import make_moe_factory

        moe_factory = make_moe_factory()
    if args.quantize:
        from types import SimpleNamespace

        from eredu_b200.ops.quant import make_quantizer

        quantizer = make_quantizer(None, SimpleNamespace(quantization=SimpleNamespace(
            bits=args.quantize, group_size=args.group_size, mode="affine"), native_gguf=False))
    model = build_random(cfg, dev, torch.bfloat16, seed=0, parallel=par, moe_factory=moe_factory, quantizer=quantizer)
    if world > 1:
        from eredu_b200.parallel import tp

        tp.attach(model, par, max_tokens=8192, backend="peer" if args.ep_backend == "peer" else "nccl",
                  ep_mode=args.ep_mode if is_moe else "replicated")
    if is_moe and args.router_skew > 0:
        period = max(1, round(1.0 / args.router_skew))
        boost = torch.zeros(cfg.num_experts, dtype=torch.float32, device=dev)
        boost[:8] = 30.0        # experts 0..7 are the hot ones (all owned by the first expert rank)
        for lw in model.layers:
            if lw.moe is not None:
                lw.moe.skew = (period, boost)
    eng = Engine(model, max_batch=B, max_seq_len=P + budget, prefill_chunk=8192)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg.vocab_size, P).tolist() for _ in range(B)]
    greedy = SamplingParams(temperature=0.0)
    if args.spec_k > 0:
        return run_speculative(args, eng, model, cfg, prompts, dev, world, rank)

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        import torch.distributed as dist

        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---------------------------------------------------------------- TTFT (batch 1, prompt P)
    ttfts = []
    for i in range(args.ttft_runs + 1):
        s = eng.new_sequence(prompts[i % B], greedy, max_new_tokens=8)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.prefill([s])
        e1.record()
        torch.cuda.synchronize(dev)
        if i > 0:
            ttfts.append(max_over_ranks(e0.elapsed_time(e1)))
        eng.release(s)
    ttft_p50 = statistics.median(ttfts)

    # ---------------------------------------------------------------- decode
    def run_decode(batch_prompts, e2e: bool):
        seqs = [eng.new_sequence(p, greedy, max_new_tokens=budget) for p in batch_prompts]
        first = eng.prefill(seqs)
        eng.start_decode(seqs, first)
        # clocks are sampled from before the warm-up (nvidia-smi needs a moment to start) until the timed region
        # ends; the GPU is under the same load during both
        sampler = ClockSampler(local_rank)
        sampler.start()
        for _ in range(W):
            eng.decode_step(sync=False)
        torch.cuda.synchronize(dev)
        for _ in range(HOLD):  # a fixed count (identical on every rank) of load-holding steps while nvidia-smi starts
            eng.decode_step(sync=False)
        torch.cuda.synchronize(dev)
        launches0 = native.launch_count()
        barrier()
        if not e2e:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(K):
                eng.decode_step(sync=False)
            e1.record()
            barrier()
            ms = e0.elapsed_time(e1)
        else:
            st = eng._decode_state
            host_in = st["host_in"]
            host_in.copy_(st["token_ids"])
            torch.cuda.synchronize(dev)
            t0 = time.perf_counter()
            for _ in range(K):
                out = eng.decode_step(host_tokens=host_in, sync=True)  # H2D of inputs + D2H of the result
                host_in.copy_(out)
            torch.cuda.synchronize(dev)
            ms = (time.perf_counter() - t0) * 1e3
            barrier()
        clocks = sampler.stop()
        per_graph = getattr(eng, "launches_per_step", None)
        for s in seqs:
            eng.release(s)
        eng._decode_state = None
        return max_over_ranks(ms), clocks, native.launch_count() - launches0

    # launches per decode step: count them on an eager (non-graph) step
    def count_launches_per_step():
        s = eng.new_sequence(prompts[0][:64], greedy, max_new_tokens=8)
        first = eng.prefill([s])
        eng.start_decode([s], first)
        was = eng.use_graph
        eng.use_graph = False
        n0 = native.launch_count()
        eng.decode_step(sync=True)
        n = native.launch_count() - n0
        eng.use_graph = was
        eng.release(s)
        eng._decode_state = None
        return n

    launches_per_step = count_launches_per_step()
    ms_b, clocks, _ = run_decode(prompts, e2e=False)
    ms_e2e, _, _ = run_decode(prompts, e2e=True)
    ms_1 = None
    if not args.skip_b1:
        ms_1, _, _ = run_decode(prompts[:1], e2e=False)
    native.check_status(dev)

    tok_s = B * K / (ms_b / 1e3)
    tok_s_e2e = B * K / (ms_e2e / 1e3)
    result = {
        "metric": "decode_tokens_per_s",
        "value": round(tok_s, 2),
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": K,
        "warmup": W,
        "ms_per_step": round(ms_b / K, 4),
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "bf16" if not args.quantize else f"bf16 activations, {args.quantize}-bit affine weights (group {args.group_size})",
        "data": "synthetic (uniform-random token prompts, random-init N(0,0.02) weights)",
        "impl": "eredu_b200",
        "config": {"model": args.model + "-shaped", "global_batch": B,
                   "seq_len": P, "decode_steps": K, "parallelism": f"tp{world}" + (f"+ep{world}" if is_moe else ""),
                   **({"ep_mode": args.ep_mode, "collectives": args.ep_backend, "router_skew": args.router_skew}
                      if is_moe else ({"collectives": args.ep_backend} if world > 1 else {})),
                   "kv_page_tokens": 16,
                   "l2": "per-step inputs (weight shard + KV pages) exceed L2; no flush needed",
                   "timing": "CUDA events around K CUDA-graph decode steps, max over ranks"},
        "decode_tokens_per_s_b1": round(K / (ms_1 / 1e3), 2) if ms_1 else None,
        "ttft_p50_ms": round(ttft_p50, 3),
        "ttft_runs_ms": [round(t, 3) for t in ttfts],
        "clocks": clocks,
        "e2e": {"value": round(tok_s_e2e, 2), "unit": "tokens/s", "h2d_bytes_per_step": 4 * B,
                "d2h_bytes_per_step": 4 * B, "ms_per_step": round(ms_e2e / K, 4),
                "api": "Engine.decode_step(host_tokens=pinned, sync=True)"},
        "gpu_launches": launches_per_step * K,
        "launches_per_step": launches_per_step,
    }
    # ---------------------------------------------------------------- baseline arm in the same process -> vs_baseline
    if not args.no_baseline:
        free_gb = torch.cuda.mem_get_info(dev)[0] / 2**30
        need_gb = (cfg.num_hidden_layers * (cfg.hidden_size * (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
                                              + cfg.hidden_size * cfg.num_attention_heads * cfg.head_dim
                                              + 3 * cfg.hidden_size * max(cfg.intermediate_size, 1)) * 2 / world
                   + 2 * cfg.vocab_size * cfg.hidden_size * 2) / 2**30 + 8
        if is_moe:
            result["baseline"] = {"unavailable": "the stock-PyTorch arm covers dense Llama-shaped models; compare --ep-backend collective"}
        elif free_gb < need_gb:
            result["baseline"] = {"unavailable": f"bf16 copy of the weights for the stock-PyTorch arm needs {need_gb:.0f} GB, {free_gb:.0f} GB free"}
        else:
            base = run_torch_baseline(args, inline=True)
            result["vs_baseline"] = round(result["value"] / base["value"], 3)
            result["baseline"] = {"impl": "torch-baseline (stock PyTorch: cuBLAS + SDPA + NCCL, CUDA graph; bf16 weights)",
                                  "value": base["value"], "ms_per_step": base["ms_per_step"], "what": "value / baseline value"}
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        import torch.distributed as dist

        barrier()
        sys.stdout.flush()
        os._exit(0)     # graphs holding NCCL kernels were captured in this process: leave without tearing the group down
    return 0


if __name__ == "__main__":
    sys.exit(main())
