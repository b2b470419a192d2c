"""Run a few eager decode steps (and optionally a prefill) of a Llama-shaped model between
``torch.cuda.profiler.start()`` / ``stop()`` so that a profiler attached with ``--profile-from-start off``
captures exactly one step.

    python -m benchmarks.profile_decode --layers 4 --batch 32 --ctx 2048
    ncu --profile-from-start off --metrics gpu__time_duration.sum --clock-control none --csv \\
        --log-file launches.csv python -m benchmarks.profile_decode --layers 4 --batch 32 --ctx 2048
"""
from __future__ import annotations

import argparse
import dataclasses

import numpy as np
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_random
from eredu_b200.ops import SamplingParams, native
from eredu_b200.runtime.engine import Engine


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "llama3-70b", "qwen3-30b-a3b"])
    ap.add_argument("--experts", type=int, default=0, help="sparse models: number of experts (0 = the model's own)")
    ap.add_argument("--topk", type=int, default=0, help="sparse models: experts per token (0 = the model's own)")
    ap.add_argument("--heads-div", type=int, default=1, help="divide the attention heads (shape of one tensor-parallel rank)")
    ap.add_argument("--phase", default="decode", choices=["decode", "prefill"])
    ap.add_argument("--steps", type=int, default=1)
    args = ap.parse_args()
    cfg = {"llama3-8b": C.llama3_8b, "llama3-70b": C.llama3_70b, "qwen3-30b-a3b": C.qwen3_30b_a3b}[args.model]()
    cfg = dataclasses.replace(cfg, num_hidden_layers=args.layers)
    if args.experts:
        cfg = dataclasses.replace(cfg, num_experts=args.experts)
    if args.topk:
        cfg = dataclasses.replace(cfg, num_experts_per_tok=args.topk)
    if args.heads_div > 1:
        cfg = dataclasses.replace(cfg, num_attention_heads=cfg.num_attention_heads // args.heads_div,
                                  num_key_value_heads=max(1, cfg.num_key_value_heads // args.heads_div))
    moe_factory = None
    if cfg.is_moe:
        from eredu_b200.models.moe import make_moe_factory

        moe_factory = make_moe_factory()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    model = build_random(cfg, dev, torch.bfloat16, seed=0, moe_factory=moe_factory)
    eng = Engine(model, max_batch=args.batch, max_seq_len=args.ctx + 64, use_cuda_graph=False)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg.vocab_size, args.ctx).tolist() for _ in range(args.batch)]
    seqs = [eng.new_sequence(p, SamplingParams(), max_new_tokens=32) for p in prompts]
    if args.phase == "prefill":
        eng.prefill(seqs[:1])
        torch.cuda.synchronize()
        for s in seqs[:1]:
            s.kv_len = 0
        torch.cuda.profiler.start()
        eng.prefill(seqs[:1])
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    else:
        first = eng.prefill(seqs)
        eng.start_decode(seqs, first)
        for _ in range(3):
            eng.decode_step(sync=True)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        for _ in range(args.steps):
            eng.decode_step(sync=True)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    native.check_status(dev)
    print("ok", args)


if __name__ == "__main__":
    main()
