"""Multi-process worker used by the distributed tests (one OS process per rank, rendezvous on 127.0.0.1).

usage: dist_worker.py <scenario> <out_json>   with RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT in the env.
"""
import dataclasses
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from eredu_b200.models import config as C  # noqa: E402
from eredu_b200.models.llama import build_from_tensors, random_state  # noqa: E402
from eredu_b200.ops import SamplingParams  # noqa: E402
from eredu_b200.parallel.context import ParallelContext  # noqa: E402
from eredu_b200.parallel.topology import ParallelTopology  # noqa: E402
from eredu_b200.runtime.engine import Engine  # noqa: E402


def tiny_cfg(gpu: bool):
    cfg = C.tiny_llama()
    if gpu:
        return dataclasses.replace(cfg, hidden_size=1024, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                                   intermediate_size=2048, vocab_size=4096, num_hidden_layers=3,
                                   tie_word_embeddings=False)
    return dataclasses.replace(cfg, vocab_size=512, num_attention_heads=4, num_key_value_heads=2)


def moe_cfg(gpu: bool):
    base = dataclasses.replace(C.tiny_llama(), model_type="qwen3_moe", qk_norm=True, vocab_size=512, num_experts=8,
                               num_experts_per_tok=2, moe_intermediate_size=64, norm_topk_prob=True,
                               tie_word_embeddings=False, rms_norm_eps=1e-6)
    if gpu:
        return dataclasses.replace(base, hidden_size=1024, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                                   moe_intermediate_size=256, vocab_size=4096, num_hidden_layers=3, num_experts=16,
                                   num_experts_per_tok=4)
    return dataclasses.replace(base, num_attention_heads=4, num_key_value_heads=2)


def probe_logits(eng, model, prompt):
    """(decode-step logits of the last prompt token after prefilling the rest) as a CPU fp32 list."""
    from eredu_b200.models.llama import ForwardBatch

    seq = eng.new_sequence(prompt[:-1], max_new_tokens=4)
    eng.prefill([seq])
    eng.start_decode([seq], torch.tensor([prompt[-1]], dtype=torch.int32))
    st = eng._decode_state
    batch = ForwardBatch(token_ids=st["token_ids"], positions=st["positions"], slots=st["slots"],
                         block_table=st["block_table"], seq_lens=st["seq_lens"], is_prefill=False, q_per_seq=1,
                         splits=st["splits"], scratch=st["scratch"])
    logits = model.forward(batch, eng.kv)[0].float().cpu()
    eng.release(seq)
    eng._decode_state = None
    return logits.tolist()


def lfm2_cfg():
    from eredu_b200.models.config import ModelConfig

    return ModelConfig.from_hf_dict({
        "model_type": "lfm2", "vocab_size": 300, "hidden_size": 64, "intermediate_size": 128, "block_auto_adjust_ff_dim": False,
        "num_hidden_layers": 4, "num_attention_heads": 4, "num_key_value_heads": 2, "max_position_embeddings": 256,
        "layer_types": ["conv", "full_attention", "conv", "full_attention"], "conv_L_cache": 3, "conv_bias": True})


def main():
    scenario, out_path = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    gpu = scenario.startswith("gpu")
    if gpu:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dev = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group("nccl", device_id=dev)
        dtype = torch.bfloat16
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        dtype = torch.float32
    result = {"rank": rank}
    cfg = tiny_cfg(gpu)
    sd = random_state(cfg, seed=0, std=0.05)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]
    sp = SamplingParams(temperature=0.0)

    if "lfm2" in scenario:      # hybrid family: short-convolution layers sharded by channel, attention by head group
        cfg = lfm2_cfg()
        sd = random_state(cfg, seed=0, std=0.08)
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]

    if "qnext" in scenario:     # Qwen3-Next style hybrid: gated-delta heads and experts spread over the same ranks
        from test_qwen_next import next_cfg, state_for

        cfg = next_cfg()
        sd = state_for(cfg)
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]

    if "nemo" in scenario:      # Nemotron-H: Mamba heads / groups, attention heads, relu^2 MLP and experts over the same ranks
        from test_nemotron_h import nh_cfg, state_for as nh_state

        cfg = nh_cfg()
        sd = nh_state(cfg)
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]

    if "kimi" in scenario:      # Kimi Linear: KDA heads, latent-attention heads and experts over the same ranks
        from test_kimi_linear import kimi_cfg, state_for as kimi_state

        cfg = kimi_cfg()
        sd = kimi_state(cfg)
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]

    if "g4" in scenario or "ckpt" in scenario:   # a checkpoint directory (EREDU_TEST_CKPT): Gemma 4, Muse-Glimmer
        from eredu_b200.formats.checkpoint import open_checkpoint

        src = open_checkpoint(os.environ["EREDU_TEST_CKPT"])
        cfg = src.cfg

        # the decoder of a vision-language checkpoint sits under model.language_model.*
        nested = src.has("model.language_model.embed_tokens.weight")
        name = (lambda n: "model.language_model." + n[len("model."):] if n.startswith("model.") else n) if nested else (lambda n: n)

        class _Tensors:
            __getitem__ = staticmethod(lambda n: src.get(name(n)))
            __contains__ = staticmethod(lambda n: src.has(name(n)))

        sd = _Tensors()
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]

    if "dsv3" in scenario:      # DeepSeek-V3 style: latent attention heads and experts spread over the same ranks
        from test_deepseek import ds_cfg, state_for as ds_state

        cfg = ds_cfg()
        sd = ds_state(cfg)
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]

    if scenario == "gpu_tpops":
        from eredu_b200.ops import native
        from eredu_b200.parallel.tp import PeerTPOps

        par = ParallelContext.from_env(ParallelTopology(tensor=world))
        H, KF, V = 1024, 2048, 4096
        ops_ = PeerTPOps(par, dev, H, V, max_tokens=1024)
        gen = torch.Generator().manual_seed(123)
        W = (torch.randn(H, KF, generator=gen) * 0.03).bfloat16()
        head = (torch.randn(V, H, generator=gen) * 0.03).bfloat16()
        errs = {}
        for M in (1, 8, 33, 64, 99, 512, 1000):
            X = (torch.randn(M, KF, generator=gen) * 0.5).bfloat16()
            R = torch.randn(M, H, generator=gen).bfloat16()
            Bv = torch.randn(H, generator=gen).bfloat16()
            ref = X.float() @ W.float().t() + R.float() + Bv.float()
            kl = KF // world
            y = ops_.row_linear(X[:, rank * kl:(rank + 1) * kl].contiguous().to(dev), W[:, rank * kl:(rank + 1) * kl].contiguous().to(dev),
                                residual=R.to(dev), bias=Bv.to(dev))
            errs[f"ar{M}"] = float((y.float().cpu() - ref).norm() / ref.norm())
            if M <= 64:
                vl = V // world
                Xh = (torch.randn(M, H, generator=gen) * 0.5).bfloat16()
                lg = ops_.gathered_logits(Xh.to(dev), head[rank * vl:(rank + 1) * vl].contiguous().to(dev), V, rank * vl)
                ref2 = Xh.float() @ head.float().t()
                errs[f"ag{M}"] = float((lg.cpu() - ref2).norm() / ref2.norm())
        # standalone all-reduce of a local partial (quantised row-parallel linears): one-shot for decode-sized
        # inputs, two-shot above
        for M in (1, 32, 64, 200):
            full = torch.randn(world, M, H, generator=gen).bfloat16()
            R = torch.randn(M, H, generator=gen).bfloat16()
            y = ops_.all_reduce(full[rank].to(dev), residual=R.to(dev))
            ref = full.float().sum(0) + R.float()
            errs[f"allreduce{M}"] = float((y.float().cpu() - ref).norm() / ref.norm())
        native.check_status(dev)
        result["errs"] = errs
    elif scenario == "cpu_server":
        # every rank serves the same request stream on its own replica; the step plans must agree word for word
        from eredu_b200.runtime.server import ConsensusError, Server, TorchTransport

        model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, dev, dtype)
        srv = Server(Engine(model, max_batch=3, max_seq_len=128), transport=TorchTransport(), prefill_chunk=16)
        ids = [srv.submit(p, sp, 6) for p in prompts]
        srv.run_until_idle(max_steps=200)
        result["tokens"] = [srv.result(i).tokens for i in ids]
        # a cancellation issued on ONE rank reaches every rank at the same step boundary
        cid = srv.submit(prompts[1], sp, 40)
        keep = srv.submit(prompts[0], sp, 8)
        for _ in range(4):
            srv.step()
        if rank == world - 1:
            srv.cancel(cid)
        srv.run_until_idle(max_steps=300)
        result["cancelled"] = [srv.result(cid).finish_reason, len(srv.result(cid).tokens), srv.result(keep).tokens]
        # now the ranks diverge: rank 1 sees a request the others do not
        srv.submit(prompts[0][: 5 + rank], sp, 3)
        try:
            srv.run_until_idle(max_steps=50)
            result["diverged"] = "none"
        except ConsensusError:
            result["diverged"] = "ConsensusError"
        result["poisoned"] = bool(srv.sched.poisoned)
    elif "ep" in scenario:
        # attention tensor-parallel and experts expert-parallel over the same ranks
        from eredu_b200.models.moe import make_moe_factory
        from eredu_b200.parallel import tp

        if "qnext" not in scenario and "dsv3" not in scenario and "nemo" not in scenario and "kimi" not in scenario:
            cfg = moe_cfg(gpu)
            sd = random_state(cfg, seed=0, std=0.08)
        par = ParallelContext.from_env(ParallelTopology(tensor=world, expert=world, expert_over_tensor=True))
        if "robin" in scenario:
            par.expert_assignment = "round_robin"
        elif "explicit" in scenario:
            # reversed blocks: the first rank owns the last experts
            per = cfg.num_experts // world
            par.expert_assignment = [world - 1 - e // per for e in range(cfg.num_experts)]
        model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, dev, dtype, par, moe_factory=make_moe_factory())
        tp.attach(model, par, max_tokens=256, backend="nccl" if "nccl" in scenario else "peer",
                  ep_mode="a2a" if "a2a" in scenario else "replicated")
        eng = Engine(model, max_batch=4, max_seq_len=128)
        result["tokens"] = eng.generate(prompts, sp, max_new_tokens=10)
        if "a2a" in scenario:
            result["a2a_calls"] = int(model.ep_a2a.stats["calls"])
        if gpu:
            from eredu_b200.ops import native

            probe = torch.randint(0, cfg.vocab_size, (100,), generator=torch.Generator().manual_seed(7)).tolist()
            result["logits"] = probe_logits(eng, model, probe)
            native.check_status(dev)
    elif "tp" in scenario and "pp" not in scenario:
        from eredu_b200.parallel import tp

        par = ParallelContext.from_env(ParallelTopology(tensor=world))
        quantizer = None
        if "quant" in scenario:  # load-time 4-bit affine quantisation of every rank's slice
            from types import SimpleNamespace

            from eredu_b200.ops.quant import make_quantizer

            quantizer = make_quantizer(None, SimpleNamespace(quantization=SimpleNamespace(bits=4, group_size=64, mode="affine"),
                                                             native_gguf=False))
        model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, dev, dtype, par, quantizer=quantizer)
        backend = "nccl" if "nccl" in scenario else "peer"
        tp.attach(model, par, max_tokens=256, backend=backend)
        eng = Engine(model, max_batch=4, max_seq_len=128)
        if "prefill" in scenario:
            long_prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (100, 70)]
            result["tokens"] = eng.generate(long_prompts, sp, max_new_tokens=4)
        else:
            result["tokens"] = eng.generate(prompts, sp, max_new_tokens=12)
        if gpu:
            from eredu_b200.ops import native

            probe = torch.randint(0, cfg.vocab_size, (100,), generator=torch.Generator().manual_seed(7)).tolist()
            result["logits"] = probe_logits(eng, model, probe)
            native.check_status(dev)
    elif "pp" in scenario:
        from eredu_b200.parallel.pipeline import PipelineRunner

        tp_size = 2 if "tp2" in scenario else 1
        axes = {}
        if "moe" in scenario:      # three axes: pipeline stages x tensor ranks, experts spread over the tensor ranks
            cfg = moe_cfg(gpu)
            sd = random_state(cfg, seed=0, std=0.08)
            if tp_size > 1:
                axes = {"expert": tp_size, "expert_over_tensor": True}
        par = ParallelContext.from_env(ParallelTopology(pipeline=world // tp_size, tensor=tp_size, **axes))
        factory = None
        if cfg.is_moe:
            from eredu_b200.models.moe import make_moe_factory

            factory = make_moe_factory()
        model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, dev, dtype, par, moe_factory=factory)
        if tp_size > 1:
            from eredu_b200.parallel import tp

            tp.attach(model, par, max_tokens=256, backend="nccl" if not gpu else "peer")
        runner = PipelineRunner(model, par, max_batch=4, max_seq_len=128, transport="peer" if "peer" in scenario else "nccl")
        result["tokens"] = runner.generate(prompts, sp, max_new_tokens=10)
        if "pcache" in scenario:
            # every stage persists the K/V of its own layers under its rank directory and resumes from them
            from eredu_b200.runtime import prompt_cache as PC

            eng = runner.engine
            long_prompt = prompts[1]
            cut = 32
            cache_dir = os.path.join(os.path.dirname(out_path), "pcache")

            def run(seq, n):
                first = eng.prefill([seq])
                eng.start_decode([seq], first)
                out = [int(first[0])]
                for _ in range(n - 1):
                    toks = eng.decode_step()
                    eng.commit(toks)
                    out.append(int(toks[0]))
                eng._decode_state = None
                return out

            s1 = eng.new_sequence(long_prompt[:cut], sp, max_new_tokens=2)
            eng.prefill([s1])
            d = PC.save_prompt_cache(eng, s1, cache_dir, "ckpt", block_tokens=16)
            eng.release(s1)
            dist.barrier()
            man = PC.open_prompt_cache(cache_dir, PC.PromptCacheTopology.of(par))
            result["pcache_layers"] = sorted({b.global_layer for b in man.blocks})
            result["pcache_dir"] = os.path.basename(str(d))
            s2 = PC.load_prompt_cache(eng, cache_dir, long_prompt, "ckpt", sp, max_new_tokens=10)
            result["pcache_cached"] = s2.kv_len
            result["pcache_tokens"] = run(s2, 10)
            eng.release(s2)
        if "peer" in scenario:
            from eredu_b200.ops import native

            native.check_status(dev)
            result["graph"] = bool(runner.engine.use_graph)
            result["hops"] = runner.stage.stats["sent"] + runner.stage.stats["received"]
    if gpu:
        # no kernel of any rank stored outside a peer-memory buffer
        for holder in (locals().get("model"), getattr(locals().get("runner"), "p2p", None)):
            pg = getattr(getattr(holder, "tp_ops", holder), "pg", None)
            if pg is not None and hasattr(pg, "check_canaries"):
                dist.barrier()
                pg.check_canaries()
                result["canaries"] = "intact"
    dist.barrier()
    with open(f"{out_path}.{rank}", "w") as f:
        json.dump(result, f)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
