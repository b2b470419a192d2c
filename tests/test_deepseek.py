"""DeepSeek-V3 style model: latent attention (absorbed form vs the decompressed oracle), dense-then-sparse schedule,
sigmoid router with correction bias and group-limited top-k, shared experts."""
import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.models.moe import make_moe_factory
from eredu_b200.ops import SamplingParams
from eredu_b200.ops import moe as M
from eredu_b200.runtime.engine import Engine

from reference_model import forward_logits, greedy


def ds_cfg(**kw):
    d = {"model_type": "deepseek_v3", "hidden_size": 64, "num_hidden_layers": 3, "num_attention_heads": 4, "q_lora_rank": 24,
         "kv_lora_rank": 16, "qk_nope_head_dim": 8, "qk_rope_head_dim": 4, "v_head_dim": 8, "intermediate_size": 96,
         "moe_intermediate_size": 32, "n_routed_experts": 8, "n_shared_experts": 1, "num_experts_per_tok": 2,
         "first_k_dense_replace": 1, "n_group": 2, "topk_group": 1, "routed_scaling_factor": 2.5, "vocab_size": 300,
         "norm_topk_prob": True, "rms_norm_eps": 1e-6, "max_position_embeddings": 256, "rope_theta": 10000.0}
    d.update(kw)
    return C.ModelConfig.from_hf_dict(d)


def state_for(cfg, seed=0):
    sd = random_state(cfg, seed=seed, std=0.1)
    g = torch.Generator().manual_seed(seed)
    for k in list(sd):
        if k.endswith("layernorm.weight") and "self_attn" in k:
            sd[k] = torch.rand(sd[k].shape, generator=g) + 0.5
        if k.endswith("e_score_correction_bias"):
            sd[k] = torch.randn(sd[k].shape, generator=g) * 0.3
    return sd


def moe_oracle(cfg, sd, li, x):
    p = f"model.layers.{li}.mlp."
    ids, w = M.route_ref(x @ sd[p + "gate.weight"].t(), cfg.num_experts_per_tok, "sigmoid", cfg.norm_topk_prob,
                         cfg.routed_scaling_factor, sd[p + "gate.e_score_correction_bias"], cfg.n_group, cfg.topk_group)
    silu = torch.nn.functional.silu
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for s in range(ids.shape[1]):
            e = int(ids[t, s])
            out[t] += w[t, s] * ((silu(x[t] @ sd[p + f"experts.{e}.gate_proj.weight"].t()) * (x[t] @ sd[p + f"experts.{e}.up_proj.weight"].t()))
                                 @ sd[p + f"experts.{e}.down_proj.weight"].t())
    sh = silu(x @ sd[p + "shared_experts.gate_proj.weight"].t()) * (x @ sd[p + "shared_experts.up_proj.weight"].t())
    return out + sh @ sd[p + "shared_experts.down_proj.weight"].t()


@pytest.mark.parametrize("variant", ["q_lora", "plain_q", "yarn", "interleaved"])
def test_greedy_matches_decompressed_oracle(variant):
    kw = {}
    if variant == "plain_q":
        kw["q_lora_rank"] = None
    if variant == "yarn":
        kw["rope_scaling"] = {"type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32, "mscale": 1.0,
                              "mscale_all_dim": 1.0, "beta_fast": 32, "beta_slow": 1}
    if variant == "interleaved":
        kw["rope_interleave"] = True
    cfg = ds_cfg(**kw)
    assert cfg.is_mla and cfg.kv_cache_dims == (1, 20, 1) and cfg.rotary_dim == 4 and cfg.mlp_only_layers == [0]
    sd = state_for(cfg)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    eng = Engine(model, max_batch=3, max_seq_len=96, prefill_chunk=16)
    assert eng.kv.k.shape[2:] == (1, 16, 20) and eng.kv.v.shape[-1] == 1         # one latent row per token, no values
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (3, 12, 37)]
    seq = eng.new_sequence(prompts[2], max_new_tokens=2)
    got = eng.prefill_logits([seq])[0]
    eng.release(seq)
    ref = forward_logits(cfg, sd, prompts[2], moe_fn=moe_oracle)[-1]
    assert torch.allclose(got, ref, atol=3e-4), float((got - ref).abs().max())
    outs = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=8)
    for p, o in zip(prompts, outs):
        assert o == greedy(cfg, sd, p, 8, moe_fn=moe_oracle)


def test_loader_and_sizing(tmp_path):
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.runtime.plan import estimate_runtime_state, inspect_artifact

    cfg = ds_cfg()
    sd = state_for(cfg, seed=2)
    ck.save_safetensors_checkpoint(tmp_path, cfg, sd, torch.float32)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    assert lm.config.is_mla and lm.model.layers[0].moe is None and lm.model.layers[1].moe.router_bias is not None
    prompt = list(range(3, 21))
    assert torch.allclose(lm.prefill_logits(prompt), forward_logits(cfg, sd, prompt, moe_fn=moe_oracle)[-1], atol=3e-4)
    prof = estimate_runtime_state(cfg)
    assert prof.kv_bytes_per_token == 3 * (16 + 4) * 2                            # latent + rotary key, every layer
    assert all(i.code != "unsupported_architecture" for i in inspect_artifact(tmp_path).issues)
