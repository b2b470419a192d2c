"""LFM2 hybrid family: gated short convolutions with recurrent state next to q/k-normalised attention."""
import dataclasses

import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.ops import SamplingParams, short_conv, short_conv_ref
from eredu_b200.runtime.engine import Engine

from reference_model import forward_logits, greedy


def lfm2_cfg(**kw):
    d = {"model_type": "lfm2", "vocab_size": 300, "hidden_size": 64, "intermediate_size": 128,
         "block_auto_adjust_ff_dim": False, "num_hidden_layers": 5, "num_attention_heads": 4, "num_key_value_heads": 2,
         "max_position_embeddings": 256, "layer_types": ["conv", "conv", "full_attention", "conv", "full_attention"],
         "conv_L_cache": 3, "norm_eps": 1e-5}
    d.update(kw)
    return C.ModelConfig.from_hf_dict(d)


def test_config_rules():
    cfg = lfm2_cfg()
    assert cfg.is_hybrid and cfg.layer_is_conv(0) and not cfg.layer_is_conv(2) and cfg.qk_norm and cfg.rope_theta == 1e6
    assert cfg.tie_word_embeddings and cfg.rms_norm_eps == 1e-5 and cfg.head_dim == 16
    # dense width re-derived from block_ff_dim: 2/3, multiplier, rounded up to the multiple
    c2 = lfm2_cfg(block_auto_adjust_ff_dim=True, block_ff_dim=12288, block_multiple_of=256, block_ffn_dim_multiplier=1.0)
    assert c2.intermediate_size == 8192
    c3 = lfm2_cfg(layer_types=None, full_attn_idxs=[2, 4])
    assert c3.layer_types == cfg.layer_types
    with pytest.raises(ValueError):
        lfm2_cfg(layer_types=["conv"])


@pytest.mark.parametrize("conv_bias,L", [(False, 3), (True, 4), (False, 2)])
def test_greedy_matches_full_recompute(conv_bias, L):
    cfg = lfm2_cfg(conv_bias=conv_bias, conv_L_cache=L)
    sd = random_state(cfg, seed=3, std=0.08)
    for k in list(sd):
        if "q_norm" in k or "k_norm" in k:
            sd[k] = torch.rand_like(sd[k]) + 0.5
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32)
    eng = Engine(model, max_batch=4, max_seq_len=96, prefill_chunk=20)     # several prefill groups / chunks
    assert eng.kv.k.shape[0] == 2 and eng.kv.conv_state.shape[:1] == (3,) and eng.kv.conv_state.shape[2:] == (L - 1, 64)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (1, 5, 17, 33)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=10)
    for p, o in zip(prompts, outs):
        assert o == greedy(cfg, sd, p, 10)
    # a second wave reuses pages of finished sequences: stale state must not leak into position 0
    outs2 = eng.generate(prompts[::-1], SamplingParams(temperature=0.0), max_new_tokens=4)
    for p, o in zip(prompts[::-1], outs2):
        assert o == greedy(cfg, sd, p, 4)


def test_checkpoint_names_and_loader(tmp_path):
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models.lfm2 import checkpoint_name, to_checkpoint_names

    assert checkpoint_name("model.norm.weight") == "model.embedding_norm.weight"
    assert checkpoint_name("model.layers.3.mlp.up_proj.weight") == "model.layers.3.feed_forward.w3.weight"
    assert checkpoint_name("model.layers.0.self_attn.q_norm.weight") == "model.layers.0.self_attn.q_layernorm.weight"
    assert checkpoint_name("model.layers.1.conv.in_proj.weight") == "model.layers.1.conv.in_proj.weight"
    cfg = lfm2_cfg()
    sd = random_state(cfg, seed=4, std=0.08)
    ck.save_safetensors_checkpoint(tmp_path, cfg, to_checkpoint_names(sd), torch.float32)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    assert lm.config.model_type == "lfm2" and lm.model.layers[0].conv_w is not None and lm.model.layers[2].wqkv is not None
    prompt = list(range(3, 25))
    ref = forward_logits(cfg, sd, prompt)[-1]
    assert torch.allclose(lm.prefill_logits(prompt), ref, atol=2e-4)


def test_kv_tier_carries_the_convolution_state():
    from eredu_b200.runtime.kv_residency import KVHostTier

    cfg = lfm2_cfg()
    sd = random_state(cfg, seed=6, std=0.08)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32)
    eng = Engine(model, max_batch=2, max_seq_len=64)
    tier = KVHostTier(eng)
    prompt = list(range(5, 22))
    seq = eng.new_sequence(prompt, max_new_tokens=8)
    first = int(eng.prefill([seq])[0])
    assert tier.park(seq)
    blocker = eng.new_sequence(list(range(40, 50)), max_new_tokens=4)      # takes the freed pages (and their state rows)
    eng.prefill([blocker])
    assert tier.resume(seq)
    toks = [first]
    logits = eng.step_logits(seq, first)
    for _ in range(4):
        t = int(torch.argmax(logits))
        toks.append(t)
        logits = eng.step_logits(seq, t)
    assert toks == greedy(cfg, sd, prompt, 5)


@pytest.mark.gpu
@pytest.mark.parametrize("L", [2, 3, 4])
def test_short_conv_kernel_matches_reference(L):
    torch.manual_seed(L)
    dev = "cuda"
    C_, pages = 320, 12
    w = torch.randn(C_, L, device=dev)
    bias = torch.randn(C_, device=dev)
    state0 = torch.randn(pages, L - 1, C_, device=dev).bfloat16()
    # prefill: three sequences of different lengths (one starts mid-sequence, one is a single token, one is long)
    lens, starts = [200, 1, 37], [0, 9, 3]
    cu = torch.tensor([0, 200, 201, 238], dtype=torch.int32, device=dev)
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).to(dev, torch.int32)
    M = sum(lens)
    proj = torch.randn(M, 3 * C_, device=dev).bfloat16()
    bt = torch.tensor([[3, 0], [7, 1], [5, 2]], dtype=torch.int32, device=dev)
    slots = torch.zeros(M, dtype=torch.int64, device=dev)
    for b_ in (None, bias):
        s_ref, s_dev = state0.clone(), state0.clone()
        ref = short_conv_ref(proj, w, b_, s_ref, bt, cu, 1, pos, slots)
        out = short_conv(proj, w, b_, s_dev, bt, cu, 1, pos, slots, max_q_len=200)
        assert float((out.float() - ref.float()).abs().max()) <= 0.02 * float(ref.float().abs().max())
        assert torch.equal(s_dev, s_ref)
    # decode: one token per sequence, the middle row inactive
    proj_d = torch.randn(3, 3 * C_, device=dev).bfloat16()
    slots_d = torch.tensor([16, -1, 40], dtype=torch.int64, device=dev)
    pos_d = torch.tensor([200, 10, 1], dtype=torch.int32, device=dev)
    s_ref, s_dev = state0.clone(), state0.clone()
    ref = short_conv_ref(proj_d, w, bias, s_ref, bt, None, 1, pos_d, slots_d)
    out = short_conv(proj_d, w, bias, s_dev, bt, None, 1, pos_d, slots_d)
    keep = torch.tensor([0, 2], device=dev)
    assert float((out[keep].float() - ref[keep].float()).abs().max()) <= 0.02 * float(ref.float().abs().max())
    assert torch.equal(s_dev, s_ref)


@pytest.mark.gpu
def test_lfm2_engine_on_gpu_matches_cpu_oracle():
    cfg = lfm2_cfg(hidden_size=256, intermediate_size=512, num_attention_heads=4, num_key_value_heads=2, vocab_size=512)
    sd = random_state(cfg, seed=8, std=0.05)
    model = build_from_tensors(cfg, lambda n: sd[n], sd.__contains__, "cuda", torch.bfloat16)
    eng = Engine(model, max_batch=4, max_seq_len=128)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (7, 40, 19)]
    seqs = [eng.new_sequence(p, max_new_tokens=8) for p in prompts]
    logits = eng.prefill_logits(seqs)
    for p, lg in zip(prompts, logits):
        ref = forward_logits(cfg, sd, p)[-1]
        assert torch.nn.functional.cosine_similarity(lg.float().cpu(), ref, dim=0) > 0.995
    for s in seqs:
        eng.release(s)
    # decode steps against the full-recompute oracle, teacher-forced (greedy tokens of a random model flip on bf16
    # rounding alone, so the logits are compared, not the token strings): prefill n-1 tokens, decode the n-th
    from dist_worker import probe_logits

    for p in prompts:
        ref = forward_logits(cfg, sd, p)[-1]
        dec = torch.tensor(probe_logits(eng, model, p))
        assert torch.nn.functional.cosine_similarity(dec, ref, dim=0) > 0.995, p
    # the CUDA-graph decode loop and the eager one produce the same tokens (same batch composition, same kernels)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=6)
    eager = Engine(model, max_batch=4, max_seq_len=128, use_cuda_graph=False)
    assert eager.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=6) == outs
    assert all(len(o) == 6 for o in outs)


def test_lfm2_moe_matches_oracle(tmp_path):
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models.lfm2 import to_checkpoint_names
    from eredu_b200.ops import moe as M

    cfg = lfm2_cfg(model_type="lfm2_moe", num_dense_layers=2, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32,
                   norm_topk_prob=True, routed_scaling_factor=1.5, use_expert_bias=True)
    assert [cfg.layer_is_moe(i) for i in range(5)] == [False, False, True, True, True] and cfg.router_scoring == "sigmoid"
    sd = random_state(cfg, seed=9, std=0.08)
    for k in list(sd):
        if k.endswith("expert_bias"):
            sd[k] = sd[k] * 10.0          # large enough to change which experts win

    def moe_fn(cfg_, sd_, li, x):
        p = f"model.layers.{li}.mlp."
        ids, w = M.route_ref(x @ sd_[p + "gate.weight"].t(), 2, "sigmoid", True, 1.5, sd_[p + "expert_bias"])
        out = torch.zeros_like(x)
        for t in range(x.shape[0]):
            for s_ in range(2):
                e = int(ids[t, s_])
                g = x[t] @ sd_[p + f"experts.{e}.gate_proj.weight"].t()
                u = x[t] @ sd_[p + f"experts.{e}.up_proj.weight"].t()
                out[t] += w[t, s_] * ((torch.nn.functional.silu(g) * u) @ sd_[p + f"experts.{e}.down_proj.weight"].t())
        return out

    ck.save_safetensors_checkpoint(tmp_path, cfg, to_checkpoint_names(sd), torch.float32)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=2, max_seq_len=64))
    assert lm.model.layers[2].moe is not None and lm.model.layers[2].moe.router_bias is not None
    assert lm.model.layers[0].moe is None and lm.model.layers[3].conv_w is not None
    prompt = list(range(7, 30))
    out = lm.generate([prompt], SamplingParams(temperature=0.0), max_new_tokens=6)[0]
    assert out == greedy(cfg, sd, prompt, 6, moe_fn=moe_fn)
