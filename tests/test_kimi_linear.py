"""Kimi Linear: KDA layers (per-channel decay delta rule) between no-rotation latent attention, DeepSeek-style MoE."""
import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.models.moe import make_moe_factory
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.engine import Engine

from reference_model import forward_logits, greedy
from test_deepseek import moe_oracle


def kimi_cfg(**kw):
    d = {"model_type": "kimi_linear", "hidden_size": 64, "num_hidden_layers": 4, "num_attention_heads": 4,
         "linear_attn_config": {"kda_layers": [1, 2, 3], "full_attn_layers": [4], "num_heads": 4, "head_dim": 8,
                                "short_conv_kernel_size": 4},
         "q_lora_rank": None, "kv_lora_rank": 16, "qk_nope_head_dim": 8, "qk_rope_head_dim": 4, "v_head_dim": 8,
         "mla_use_nope": True, "intermediate_size": 96, "moe_intermediate_size": 32, "num_experts": 8,
         "num_experts_per_token": 2, "num_shared_experts": 1, "first_k_dense_replace": 1, "moe_layer_freq": 1,
         "num_expert_group": 2, "topk_group": 1, "routed_scaling_factor": 2.5, "vocab_size": 300, "rms_norm_eps": 1e-6,
         "max_position_embeddings": 256, "moe_renormalize": True}
    d.update(kw)
    return C.ModelConfig.from_hf_dict(d)


def state_for(cfg, seed=0):
    sd = random_state(cfg, seed=seed, std=0.1)
    g = torch.Generator().manual_seed(seed)
    for k in list(sd):
        if k.endswith(("A_log", "dt_bias")):
            sd[k] = torch.randn(sd[k].shape, generator=g) * 0.5
        if k.endswith(("o_norm.weight", "kv_a_layernorm.weight")):
            sd[k] = torch.rand(sd[k].shape, generator=g) + 0.5
        if k.endswith("e_score_correction_bias"):
            sd[k] = torch.randn(sd[k].shape, generator=g) * 0.3
    return sd


def test_config_schedule():
    cfg = kimi_cfg()
    assert cfg.layer_types == ["kda", "kda", "kda", "full_attention"] and cfg.is_mla and not cfg.use_rope and cfg.is_hybrid
    assert cfg.mlp_only_layers == [0] and cfg.n_group == 2 and cfg.router_scoring == "sigmoid"
    assert C.ModelConfig.from_hf_dict(cfg.to_hf_dict()) == cfg
    with pytest.raises(ValueError):
        kimi_cfg(mla_use_nope=False)
    with pytest.raises(ValueError):
        kimi_cfg(linear_attn_config={"kda_layers": [1, 2], "full_attn_layers": [4], "num_heads": 4, "head_dim": 8})


@pytest.mark.parametrize("chunk", [64, 7])
def test_greedy_matches_full_recompute(chunk):
    cfg = kimi_cfg()
    sd = state_for(cfg)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    eng = Engine(model, max_batch=3, max_seq_len=96, prefill_chunk=chunk)
    assert eng.kv.k.shape[0] == 1 and eng.kv.k.shape[-1] == 20 and eng.kv.la_rec_state.shape == (3, 8, 4, 8, 8)
    assert eng.kv.la_conv_state.shape[2:] == (3, 96)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (2, 13, 26)]
    seq = eng.new_sequence(prompts[2], max_new_tokens=2)
    got = eng.prefill_logits([seq])[0]
    eng.release(seq)
    ref = forward_logits(cfg, sd, prompts[2], moe_fn=moe_oracle)[-1]
    assert torch.allclose(got, ref, atol=3e-4), float((got - ref).abs().max())
    outs = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=8)
    for p, o in zip(prompts, outs):
        assert o == greedy(cfg, sd, p, 8, moe_fn=moe_oracle)


def test_block_sparse_moe_names_and_loader(tmp_path):
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models.kimi_linear import checkpoint_name

    assert checkpoint_name("model.layers.2.mlp.experts.5.up_proj.weight") == "model.layers.2.block_sparse_moe.experts.5.w3.weight"
    assert checkpoint_name("model.layers.1.mlp.gate.e_score_correction_bias") == "model.layers.1.block_sparse_moe.gate.e_score_correction_bias"
    cfg = kimi_cfg()
    sd = state_for(cfg, seed=2)
    stored = {(checkpoint_name(k) if cfg.layer_is_moe(int(k.split(".")[2])) else k) if k.startswith("model.layers.") and ".mlp." in k else k: v
              for k, v in sd.items()}
    assert any("block_sparse_moe.experts.0.w1" in k for k in stored) and any(k.endswith("layers.0.mlp.gate_proj.weight") for k in stored)
    ck.save_safetensors_checkpoint(tmp_path, cfg, stored, torch.float32)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    assert lm.model.layers[0].kda_in is not None and lm.model.layers[3].mla_in is not None
    assert lm.model.layers[1].moe.shared is not None and lm.model.layers[1].moe.router_bias is not None
    prompt = list(range(3, 21))
    assert torch.allclose(lm.prefill_logits(prompt), forward_logits(cfg, sd, prompt, moe_fn=moe_oracle)[-1], atol=3e-4)
