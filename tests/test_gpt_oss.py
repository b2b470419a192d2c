"""GPT-OSS-shaped model: attention sinks and biases, alternating sliding / full layers, router with a linear bias and
top-k-then-softmax weights, experts with biases and the clamped (u + 1) * g * sigmoid(1.702 g) gate, interleaved
gate / up checkpoint layout (bf16 and MXFP4 block forms)."""
import dataclasses

import numpy as np
import pytest
import torch

from eredu_b200.lib import _eredu_host as H
from eredu_b200.models.config import ModelConfig
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.models.moe import make_moe_factory
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.engine import Engine

from reference_model import greedy


def oss_cfg(big=False):
    d = {"model_type": "gpt_oss", "vocab_size": 512, "hidden_size": 256, "intermediate_size": 64, "num_hidden_layers": 3,
         "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "num_local_experts": 8, "num_experts_per_tok": 2,
         "sliding_window": 8, "layer_types": ["sliding_attention", "full_attention", "sliding_attention"],
         "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "swiglu_limit": 7.0}
    if big:
        d.update(hidden_size=1024, num_attention_heads=8, head_dim=128, intermediate_size=256, vocab_size=4096,
                 num_local_experts=16, num_experts_per_tok=4)
    return ModelConfig.from_hf_dict(d)


def oss_state(cfg, seed=0, mxfp4=False, std=0.08):
    g = torch.Generator().manual_seed(seed)
    base = dataclasses.replace(cfg, num_experts=0)          # attention / norms / embeddings from the dense generator
    sd = {k: v for k, v in random_state(base, seed=seed, std=std).items() if ".mlp." not in k}
    H_, I, E = cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts
    D = cfg.head_dim
    rnd = lambda *s: torch.randn(*s, generator=g) * std                                           # noqa: E731
    for li in range(cfg.num_hidden_layers):
        p = f"model.layers.{li}."
        for n, rows in (("q", cfg.num_attention_heads * D), ("k", cfg.num_key_value_heads * D), ("v", cfg.num_key_value_heads * D)):
            sd[p + f"self_attn.{n}_proj.bias"] = rnd(rows)
        sd[p + "self_attn.o_proj.bias"] = rnd(H_)
        sd[p + "self_attn.sinks"] = torch.randn(cfg.num_attention_heads, generator=g)
        sd[p + "mlp.router.weight"] = rnd(E, H_)
        sd[p + "mlp.router.bias"] = rnd(E)
        gu = rnd(E, H_, 2 * I)            # input-major, gate / up interleaved on the last axis
        dn = rnd(E, I, H_)
        if mxfp4:
            for name, w in (("gate_up_proj", gu.transpose(1, 2)), ("down_proj", dn.transpose(1, 2))):   # rows = outputs
                E_, rows, K = w.shape
                packed, scales = H.mxfp4_quantize(np.ascontiguousarray(w.reshape(E_ * rows, K).numpy()))
                deq = torch.from_numpy(np.asarray(H.mxfp4_dequantize(packed, scales))).reshape(E_, rows, K)
                sd[p + f"mlp.experts.{name}_blocks"] = torch.from_numpy(np.asarray(packed).view(np.uint8).reshape(E_, rows, K // 32, 16).copy())
                sd[p + f"mlp.experts.{name}_scales"] = torch.from_numpy(np.asarray(scales).reshape(E_, rows, K // 32).copy())
                sd[p + f"_oracle.{name}"] = deq.transpose(1, 2).contiguous()     # what the blocks decode to, input-major
        else:
            sd[p + "mlp.experts.gate_up_proj"] = gu
            sd[p + "mlp.experts.down_proj"] = dn
        sd[p + "mlp.experts.gate_up_proj_bias"] = rnd(E, 2 * I)
        sd[p + "mlp.experts.down_proj_bias"] = rnd(E, H_)
    return sd


def oss_oracle(cfg, sd, li, x):
    p = f"model.layers.{li}.mlp."
    gu = sd.get(f"model.layers.{li}._oracle.gate_up_proj", sd.get(p + "experts.gate_up_proj")).float()
    dn = sd.get(f"model.layers.{li}._oracle.down_proj", sd.get(p + "experts.down_proj")).float()
    logits = x @ sd[p + "router.weight"].float().t() + sd[p + "router.bias"].float()
    top = torch.topk(logits, cfg.num_experts_per_tok, dim=-1)
    w = torch.softmax(top.values, -1)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for s in range(cfg.num_experts_per_tok):
            e = int(top.indices[t, s])
            y = x[t] @ gu[e] + sd[p + "experts.gate_up_proj_bias"][e].float()
            g_, u_ = y[0::2].clamp(max=cfg.swiglu_limit), y[1::2].clamp(-cfg.swiglu_limit, cfg.swiglu_limit)
            a = g_ * torch.sigmoid(1.702 * g_) * (u_ + 1.0)
            out[t] += w[t, s] * (a @ dn[e] + sd[p + "experts.down_proj_bias"][e].float())
    return out


@pytest.mark.parametrize("mxfp4", [False, True])
def test_gpt_oss_cpu_matches_oracle(mxfp4):
    cfg = oss_cfg()
    assert cfg.attention_sinks and cfg.router_scoring == "topk_softmax" and cfg.layer_window(0) == 8 and cfg.layer_window(1) == 0
    sd = oss_state(cfg, mxfp4=mxfp4)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    eng = Engine(model, max_batch=2, max_seq_len=64)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (6, 17)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=7)
    for p_, o in zip(prompts, outs):
        assert o == greedy(cfg, sd, p_, 7, moe_fn=oss_oracle)


@pytest.mark.gpu
def test_gpt_oss_gpu_logits():
    from reference_model import forward_logits

    cfg = oss_cfg(big=True)
    # weights scaled for the 1024-wide model: with the small model's 0.08 the attention logits reach a spread of several
    # units, and rounding q and k to bf16 alone then moves the output by more than the gate allows
    sd = oss_state(cfg, std=0.03)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cuda:0", torch.bfloat16, moe_factory=make_moe_factory())
    eng = Engine(model, max_batch=2, max_seq_len=128)
    prompt = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(5)).tolist()
    from eredu_b200.api.loaded import LoadedModel
    lm = LoadedModel(model, eng, None)
    got = lm.prefill_logits(prompt)
    ref = forward_logits(cfg, {k: v.float() for k, v in sd.items()}, prompt, moe_fn=oss_oracle)[-1]
    rel = float((got - ref).norm() / ref.norm())
    assert rel < 0.05 and torch.nn.functional.cosine_similarity(got, ref, dim=0) > 0.995
    out = eng.generate([prompt], SamplingParams(temperature=0.0), max_new_tokens=8)[0]
    assert len(out) == 8
