"""Qwen3-Next style hybrid: gated delta networks, gated attention output, zero-centred norms, gated shared expert."""
import dataclasses

import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.models.moe import make_moe_factory
from eredu_b200.models.qwen_next import split_fused_projections
from eredu_b200.ops import SamplingParams
from eredu_b200.ops import moe as M
from eredu_b200.runtime.engine import Engine

from reference_model import forward_logits, greedy


def next_cfg(**kw):
    d = {"model_type": "qwen3_next", "vocab_size": 300, "hidden_size": 64, "num_hidden_layers": 4, "num_attention_heads": 4,
         "num_key_value_heads": 2, "head_dim": 32, "linear_num_key_heads": 2, "linear_num_value_heads": 4,
         "linear_key_head_dim": 16, "linear_value_head_dim": 8, "linear_conv_kernel_dim": 4, "num_experts": 8,
         "num_experts_per_tok": 2, "moe_intermediate_size": 32, "shared_expert_intermediate_size": 48, "intermediate_size": 96,
         "rms_norm_eps": 1e-6, "max_position_embeddings": 256, "norm_topk_prob": True}
    d.update(kw)
    return C.ModelConfig.from_hf_dict(d)


def state_for(cfg, seed=0):
    sd = random_state(cfg, seed=seed, std=0.08)
    g = torch.Generator().manual_seed(seed)
    for k in list(sd):
        if k.endswith("norm.weight") and "linear_attn" not in k:
            sd[k] = torch.randn(sd[k].shape, generator=g) * 0.2          # zero-centred: the model applies 1 + w
        if k.endswith("A_log") or k.endswith("dt_bias"):
            sd[k] = torch.randn(sd[k].shape, generator=g) * 0.5
        if "linear_attn.norm.weight" in k:
            sd[k] = torch.rand(sd[k].shape, generator=g) + 0.5
    return sd


def moe_oracle(cfg, sd, li, x):
    p = f"model.layers.{li}.mlp."
    ids, w = M.route_ref(x @ sd[p + "gate.weight"].t(), cfg.num_experts_per_tok, "softmax", cfg.norm_topk_prob)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for s in range(ids.shape[1]):
            e = int(ids[t, s])
            gt = x[t] @ sd[p + f"experts.{e}.gate_proj.weight"].t()
            u = x[t] @ sd[p + f"experts.{e}.up_proj.weight"].t()
            out[t] += w[t, s] * ((torch.nn.functional.silu(gt) * u) @ sd[p + f"experts.{e}.down_proj.weight"].t())
    sh = torch.nn.functional.silu(x @ sd[p + "shared_expert.gate_proj.weight"].t()) * (x @ sd[p + "shared_expert.up_proj.weight"].t())
    sh = sh @ sd[p + "shared_expert.down_proj.weight"].t()
    return out + torch.sigmoid(x @ sd[p + "shared_expert_gate.weight"].t()) * sh


def test_config_schedule():
    cfg = next_cfg()
    assert cfg.layer_types == ["linear_attention"] * 3 + ["full_attention"] and cfg.is_hybrid and cfg.attn_output_gate
    assert cfg.norm_weight_offset == 1.0 and cfg.rotary_dim == 8 and cfg.shared_expert_gate and cfg.qk_norm
    assert next_cfg(num_hidden_layers=8, full_attention_interval=2).layer_types[:4] == ["linear_attention", "full_attention"] * 2
    with pytest.raises(ValueError):
        next_cfg(layer_types=["full_attention"])


@pytest.mark.parametrize("chunk", [64, 7])
def test_greedy_matches_full_recompute(chunk):
    cfg = next_cfg()
    sd = state_for(cfg)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    eng = Engine(model, max_batch=3, max_seq_len=96, prefill_chunk=chunk)
    assert eng.kv.k.shape[0] == 1 and eng.kv.la_rec_state.shape == (3, 8, 4, 16, 8) and eng.kv.la_conv_state.shape[2:] == (3, 96)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (2, 11, 23)]
    ref = forward_logits(cfg, sd, prompts[2], moe_fn=moe_oracle)[-1]
    seq = eng.new_sequence(prompts[2], max_new_tokens=2)
    got = eng.prefill_logits([seq])[0]
    eng.release(seq)
    assert torch.allclose(got, ref, atol=2e-4), float((got - ref).abs().max())
    outs = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=8)
    for p, o in zip(prompts, outs):
        assert o == greedy(cfg, sd, p, 8, moe_fn=moe_oracle)
    # a second wave reuses state slots: they start from zero again
    outs2 = eng.generate(prompts[:2], SamplingParams(temperature=0.0), max_new_tokens=3)
    assert outs2 == [o[:3] for o in outs[:2]]


def test_fused_checkpoint_layout_and_loader(tmp_path):
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats import checkpoint as ck

    cfg = next_cfg()
    sd = state_for(cfg, seed=3)
    Hk, Hv, dk, dv = 2, 4, 16, 8
    r = Hv // Hk
    fused = {}
    for k_, t in sd.items():
        if k_.endswith("linear_attn.in_proj_qkv.weight"):
            base = k_[:-len("in_proj_qkv.weight")]
            qkv, z, b, a = t, sd[base + "in_proj_z.weight"], sd[base + "in_proj_b.weight"], sd[base + "in_proj_a.weight"]
            H = t.shape[1]
            q, kk, v = qkv[:Hk * dk].view(Hk, dk, H), qkv[Hk * dk:2 * Hk * dk].view(Hk, dk, H), qkv[2 * Hk * dk:].view(Hk, r * dv, H)
            fused[base + "in_proj_qkvz.weight"] = torch.cat((q, kk, v, z.view(Hk, r * dv, H)), 1).reshape(-1, H)
            fused[base + "in_proj_ba.weight"] = torch.cat((b.view(Hk, r, H), a.view(Hk, r, H)), 1).reshape(-1, H)
        elif any(k_.endswith(f"linear_attn.in_proj_{n}.weight") for n in "zba"):
            continue
        else:
            fused[k_] = t
    name = "model.layers.0.linear_attn."
    back = split_fused_projections(cfg, fused[name + "in_proj_qkvz.weight"], fused[name + "in_proj_ba.weight"])
    for got, key in zip(back, ("qkv", "z", "b", "a")):
        assert torch.equal(got, sd[name + f"in_proj_{key}.weight"])
    ck.save_safetensors_checkpoint(tmp_path, cfg, fused, torch.float32)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    assert lm.model.layers[0].la_in is not None and lm.model.layers[3].attn_gate and lm.model.layers[3].moe.shared_gate_w is not None
    prompt = list(range(3, 21))
    ref = forward_logits(cfg, sd, prompt, moe_fn=moe_oracle)[-1]
    assert torch.allclose(lm.prefill_logits(prompt), ref, atol=2e-4)


def test_guards():
    from eredu_b200.runtime.speculative import SpeculativeDecoder

    cfg = next_cfg()
    sd = state_for(cfg)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    eng = Engine(model, max_batch=1, max_seq_len=32, num_pages=64)       # more pages than state slots (8)
    assert SpeculativeDecoder(eng, eng, 2).t_hybrid                        # hybrids speculate through state snapshots
    seqs = [eng.new_sequence([1, 2, 3], max_new_tokens=2) for _ in range(8)]
    free = eng.kv.allocator.free_pages()
    with pytest.raises(RuntimeError, match="state slot"):
        eng.new_sequence([1, 2, 3], max_new_tokens=2)
    assert eng.kv.allocator.free_pages() == free                          # the refused request left no pages behind
    for s in seqs:
        eng.release(s)
    eng.release(eng.new_sequence([1, 2, 3], max_new_tokens=2))


@pytest.mark.gpu
def test_qwen_next_on_gpu_matches_cpu_oracle():
    cfg = next_cfg(hidden_size=256, head_dim=64, linear_key_head_dim=64, linear_value_head_dim=64, vocab_size=512,
                   moe_intermediate_size=64, shared_expert_intermediate_size=64)
    sd = state_for(cfg, seed=4)
    sd = {k: v * (0.6 if v.dim() == 2 else 1.0) for k, v in sd.items()}
    model = build_from_tensors(cfg, lambda n: sd[n], sd.__contains__, "cuda", torch.bfloat16, moe_factory=make_moe_factory())
    eng = Engine(model, max_batch=4, max_seq_len=128)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 40, 21)]
    seqs = [eng.new_sequence(p, max_new_tokens=8) for p in prompts]
    logits = eng.prefill_logits(seqs)
    for p, lg in zip(prompts, logits):
        ref = forward_logits(cfg, sd, p, moe_fn=moe_oracle)[-1]
        assert torch.nn.functional.cosine_similarity(lg.float().cpu(), ref, dim=0) > 0.99
    for s in seqs:
        eng.release(s)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=6)      # CUDA-graph decode
    assert all(len(o) == 6 for o in outs)
    from eredu_b200.ops import native
    native.check_status(torch.device("cuda", torch.cuda.current_device()))
