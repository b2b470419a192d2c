"""Nemotron-H: single-mixer blocks (Mamba-2, attention without rotation, relu^2 MLP, relu^2 experts)."""
import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.models.moe import make_moe_factory
from eredu_b200.ops import SamplingParams, mamba2_scan_ref
from eredu_b200.ops import moe as M
from eredu_b200.runtime.engine import Engine

from reference_model import forward_logits, greedy


def nh_cfg(**kw):
    d = {"model_type": "nemotron_h", "hybrid_override_pattern": "M-M*-ME*", "hidden_size": 64, "num_attention_heads": 4,
         "num_key_value_heads": 2, "head_dim": 16, "mamba_num_heads": 8, "mamba_head_dim": 8, "ssm_state_size": 16,
         "n_groups": 2, "conv_kernel": 4, "intermediate_size": 96, "vocab_size": 300, "n_routed_experts": 8,
         "num_experts_per_tok": 2, "moe_intermediate_size": 32, "moe_shared_expert_intermediate_size": 48, "n_group": 2,
         "topk_group": 1, "routed_scaling_factor": 2.0, "layer_norm_epsilon": 1e-5, "max_position_embeddings": 256}
    d.update(kw)
    return C.ModelConfig.from_hf_dict(d)


def state_for(cfg, seed=0):
    sd = random_state(cfg, seed=seed, std=0.08)
    g = torch.Generator().manual_seed(seed)
    for k in list(sd):
        if k.endswith(("A_log", "dt_bias", ".D")):
            sd[k] = torch.randn(sd[k].shape, generator=g) * 0.5
        if k.endswith("mixer.norm.weight"):
            sd[k] = torch.rand(sd[k].shape, generator=g) + 0.5
        if k.endswith("e_score_correction_bias"):
            sd[k] = torch.randn(sd[k].shape, generator=g) * 0.3
    return sd


def moe_oracle(cfg, sd, li, x):
    p = f"model.layers.{li}.mixer."
    ids, w = M.route_ref(x @ sd[p + "gate.weight"].t(), cfg.num_experts_per_tok, "sigmoid", cfg.norm_topk_prob,
                         cfg.routed_scaling_factor, sd[p + "gate.e_score_correction_bias"], cfg.n_group, cfg.topk_group)
    out = torch.zeros_like(x)
    relu2 = lambda t: torch.relu(t) ** 2                                           # noqa: E731
    for t in range(x.shape[0]):
        for s in range(ids.shape[1]):
            e = int(ids[t, s])
            out[t] += w[t, s] * (relu2(x[t] @ sd[p + f"experts.{e}.up_proj.weight"].t()) @ sd[p + f"experts.{e}.down_proj.weight"].t())
    return out + relu2(x @ sd[p + "shared_experts.up_proj.weight"].t()) @ sd[p + "shared_experts.down_proj.weight"].t()


def test_config_and_scan_step():
    cfg = nh_cfg()
    assert cfg.layer_types[:4] == ["mamba", "mlp_only", "mamba", "attention_only"] and cfg.num_hidden_layers == 8
    assert cfg.is_hybrid and not cfg.use_rope and cfg.layer_is_moe(6) and not cfg.layer_is_moe(1) and cfg.layer_has_kv(3)
    assert cfg.router_scoring == "sigmoid" and cfg.n_group == 2 and cfg.routed_scaling_factor == 2.0
    with pytest.raises(ValueError):
        nh_cfg(hybrid_override_pattern="MX")
    # one step by hand: S = S exp(dt A) + x (dt B)^T ; y = S C + D x
    x = torch.tensor([[1.0, 2.0]]).view(1, 1, 1, 2)
    B = torch.tensor([0.5, -1.0, 2.0]).view(1, 1, 1, 3)
    Cm = torch.tensor([1.0, 0.0, -1.0]).view(1, 1, 1, 3)
    dt = torch.tensor([0.5]).view(1, 1, 1)
    A, D = torch.tensor([-2.0]), torch.tensor([3.0])
    S0 = torch.ones(1, 1, 2, 3)
    S, y = mamba2_scan_ref(x, B, Cm, dt, A, D, S0)
    want = S0[0, 0] * torch.exp(torch.tensor(-1.0)) + torch.outer(x.view(2), 0.5 * B.view(3))
    assert torch.allclose(S[0, 0], want) and torch.allclose(y.view(2), want @ Cm.view(3) + 3.0 * x.view(2))


@pytest.mark.parametrize("chunk", [64, 6])
def test_greedy_matches_full_recompute(chunk):
    cfg = nh_cfg()
    sd = state_for(cfg)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    eng = Engine(model, max_batch=3, max_seq_len=96, prefill_chunk=chunk)
    assert eng.kv.k.shape[0] == 2 and eng.kv.la_rec_state.shape == (3, 8, 8, 8, 16)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (3, 12, 25)]
    seq = eng.new_sequence(prompts[2], max_new_tokens=2)
    got = eng.prefill_logits([seq])[0]
    eng.release(seq)
    ref = forward_logits(cfg, sd, prompts[2], moe_fn=moe_oracle)[-1]
    assert torch.allclose(got, ref, atol=2e-4), float((got - ref).abs().max())
    outs = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=8)
    for p, o in zip(prompts, outs):
        assert o == greedy(cfg, sd, p, 8, moe_fn=moe_oracle)


def test_checkpoint_names_and_loader(tmp_path):
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models.nemotron_h import checkpoint_name, to_checkpoint_names

    assert checkpoint_name("model.embed_tokens.weight") == "backbone.embeddings.weight"
    assert checkpoint_name("model.layers.2.mixer.A_log") == "backbone.layers.2.mixer.A_log"
    assert checkpoint_name("model.norm.weight") == "backbone.norm_f.weight" and checkpoint_name("lm_head.weight") == "lm_head.weight"
    cfg = nh_cfg()
    sd = state_for(cfg, seed=2)
    ck.save_safetensors_checkpoint(tmp_path, cfg, to_checkpoint_names(sd), torch.float32)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    kinds = [lw.block_kind for lw in lm.model.layers]
    assert kinds == cfg.layer_types and lm.model.layers[6].moe.act == "relu2"
    prompt = list(range(3, 21))
    ref = forward_logits(cfg, sd, prompt, moe_fn=moe_oracle)[-1]
    assert torch.allclose(lm.prefill_logits(prompt), ref, atol=2e-4)
