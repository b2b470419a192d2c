"""MoE: router variants, routing plan, grouped expert GEMMs and combine against a per-expert PyTorch reference;
Qwen3-MoE-shaped model through the engine against the dense oracle."""
import dataclasses

import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.models.moe import make_moe_factory
from eredu_b200.ops import SamplingParams
from eredu_b200.ops import moe as M
from eredu_b200.runtime.engine import Engine

from reference_model import forward_logits, greedy


def moe_oracle(cfg, sd, li, x):
    p = f"model.layers.{li}.mlp."
    logits = x @ sd[p + "gate.weight"].float().t()
    ids, w = M.route_ref(logits, cfg.num_experts_per_tok, cfg.router_scoring, cfg.norm_topk_prob)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for s in range(ids.shape[1]):
            e = int(ids[t, s])
            g = x[t] @ sd[p + f"experts.{e}.gate_proj.weight"].float().t()
            u = x[t] @ sd[p + f"experts.{e}.up_proj.weight"].float().t()
            out[t] += w[t, s] * ((torch.nn.functional.silu(g) * u) @ sd[p + f"experts.{e}.down_proj.weight"].float().t())
    return out


def tiny_moe_cfg():
    return dataclasses.replace(C.tiny_llama(), model_type="qwen3_moe", qk_norm=True, vocab_size=512, num_experts=8,
                               num_experts_per_tok=2, moe_intermediate_size=64, norm_topk_prob=True,
                               tie_word_embeddings=False, rms_norm_eps=1e-6)


def test_moe_model_cpu_matches_oracle():
    cfg = tiny_moe_cfg()
    sd = random_state(cfg, seed=0, std=0.08)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32,
                               moe_factory=make_moe_factory())
    eng = Engine(model, max_batch=2, max_seq_len=64)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (7, 19)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=8)
    for p, o in zip(prompts, outs):
        assert o == greedy(cfg, sd, p, 8, moe_fn=moe_oracle)


@pytest.mark.parametrize("scoring,renorm", [("softmax", True), ("softmax", False), ("sigmoid", True),
                                            ("sqrt_softplus", True), ("topk_softmax", False)])
def test_route_ref_properties(scoring, renorm):
    logits = torch.randn(9, 16)
    ids, w = M.route_ref(logits, 4, scoring, renorm)
    assert ids.shape == (9, 4) and (w >= 0).all()
    if renorm or scoring == "topk_softmax":
        assert torch.allclose(w.sum(-1), torch.ones(9), atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("scoring,renorm", [("softmax", True), ("softmax", False), ("sigmoid", True),
                                            ("sqrt_softplus", False), ("topk_softmax", False)])
def test_route_kernel(scoring, renorm):
    torch.manual_seed(1)
    logits = torch.randn(70, 128, device="cuda")
    bias = torch.randn(128, device="cuda") * 0.1 if scoring == "sigmoid" else None
    ids, w = M.route(logits, 8, scoring, renorm, 1.0, bias)
    rids, rw = M.route_ref(logits.cpu(), 8, scoring, renorm, 1.0, None if bias is None else bias.cpu())
    assert torch.equal(ids.cpu().sort(-1).values, rids.sort(-1).values)
    order, rorder = ids.cpu().argsort(-1), rids.argsort(-1)
    assert torch.allclose(w.cpu().gather(-1, order), rw.gather(-1, rorder), atol=1e-5, rtol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("T,E,k,H,I,skew", [(1, 16, 4, 256, 128, False), (32, 16, 8, 2048, 768, False),
                                           (200, 8, 2, 512, 256, False), (64, 16, 8, 1024, 384, True),
                                           (700, 4, 2, 256, 128, False)])
def test_experts_forward_kernels(T, E, k, H, I, skew):
    torch.manual_seed(T)
    dev = "cuda"
    x = (torch.randn(T, H, device=dev) * 0.5).bfloat16()
    wgu = (torch.randn(E, 2 * I, H, device=dev) * 0.05).bfloat16()
    wd = (torch.randn(E, H, I, device=dev) * 0.05).bfloat16()
    logits = torch.randn(T, E, device=dev)
    if skew:
        logits[: T // 2, :2] += 8.0  # half of the tokens pile onto two hot experts
    ids, w = M.route(logits, k, "softmax", True)
    res = torch.randn(T, H, device=dev).bfloat16()
    out = M.experts_forward(x, ids, w, wgu, wd, 0, residual=res)
    ref = M.experts_ref(x.cpu(), ids.cpu(), w.cpu(), wgu.cpu(), wd.cpu(), 0) + res.cpu().float()
    rel = float((out.cpu().float() - ref).norm() / ref.norm())
    assert rel < 2e-2, rel
    # a rank that owns experts [E/2, E): partial sums of both halves add up to the full result
    lo = M.experts_forward(x, ids, w, wgu[: E // 2].contiguous(), wd[: E // 2].contiguous(), 0)
    hi = M.experts_forward(x, ids, w, wgu[E // 2:].contiguous(), wd[E // 2:].contiguous(), E // 2)
    both = lo.float() + hi.float() + res.float()
    assert float((both.cpu() - ref).norm() / ref.norm()) < 2e-2
    from eredu_b200.ops import native
    native.check_status(torch.device("cuda", torch.cuda.current_device()))


@pytest.mark.gpu
def test_moe_model_gpu_logits():
    cfg = dataclasses.replace(tiny_moe_cfg(), hidden_size=512, num_attention_heads=8, num_key_value_heads=2,
                              head_dim=64, moe_intermediate_size=256, num_experts=16, num_experts_per_tok=4,
                              vocab_size=2048, num_hidden_layers=2)
    sd = {k: v.bfloat16().float() for k, v in random_state(cfg, seed=3, std=0.05).items()}
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cuda", torch.bfloat16,
                               moe_factory=make_moe_factory())
    from eredu_b200.api.loaded import LoadedModel
    lm = LoadedModel(model, Engine(model, max_batch=2, max_seq_len=128), None)
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, cfg.vocab_size, (40,), generator=g).tolist()
    got = lm.prefill_logits(prompt)
    ref = forward_logits(cfg, sd, prompt, moe_fn=moe_oracle)[-1]
    rel = float((got - ref).norm() / ref.norm())
    assert rel < 0.03 and torch.nn.functional.cosine_similarity(got, ref, dim=0) > 0.999


def test_mixtral_naming_and_router_cpu():
    """Mixtral checkpoints: ``block_sparse_moe.{gate, experts.N.w1/w3/w2}``, top-k-then-softmax routing."""
    cfg = dataclasses.replace(tiny_moe_cfg(), model_type="mixtral", qk_norm=False, router_scoring="topk_softmax",
                              norm_topk_prob=False)
    sd = random_state(cfg, seed=3, std=0.08)
    mix = {}
    for k, v in sd.items():
        k2 = k.replace(".mlp.gate.weight", ".block_sparse_moe.gate.weight")
        k2 = k2.replace(".mlp.experts.", ".block_sparse_moe.experts.")
        k2 = k2.replace(".gate_proj.weight", ".w1.weight") if "block_sparse_moe.experts" in k2 else k2
        k2 = k2.replace(".up_proj.weight", ".w3.weight") if "block_sparse_moe.experts" in k2 else k2
        k2 = k2.replace(".down_proj.weight", ".w2.weight") if "block_sparse_moe.experts" in k2 else k2
        mix[k2] = v
    model = build_from_tensors(cfg, mix.__getitem__, mix.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    eng = Engine(model, max_batch=1, max_seq_len=64)
    prompt = torch.randint(0, cfg.vocab_size, (11,), generator=torch.Generator().manual_seed(5)).tolist()
    out = eng.generate([prompt], SamplingParams(temperature=0.0), max_new_tokens=6)[0]
    assert out == greedy(cfg, sd, prompt, 6, moe_fn=moe_oracle)


def test_group_limited_and_table_routing():
    torch.manual_seed(0)
    T, E, k = 16, 16, 4
    logits = torch.randn(T, E)
    bias = torch.randn(E) * 0.5
    ids, w = M.route_ref(logits, k, "sigmoid", True, 2.5, bias, n_group=4, topk_group=2, norm_eps=1e-6)
    score = torch.sigmoid(logits)
    select = score + bias
    for t in range(T):
        groups = select[t].view(4, 4)
        best = torch.topk(torch.topk(groups, 2, -1).values.sum(-1), 2).indices.tolist()
        assert all(int(e) // 4 in best for e in ids[t])                       # only the two best groups are eligible
        allowed = torch.cat([select[t, g * 4:(g + 1) * 4] for g in best])
        assert sorted(select[t, ids[t].long()].tolist()) == sorted(torch.topk(allowed, k).values.tolist())
        raw = score[t, ids[t].long()]                                          # weights come from the unbiased scores
        assert torch.allclose(w[t], raw / (raw.sum() + 1e-6) * 2.5, atol=1e-6)
    with pytest.raises(ValueError):
        M.route_ref(logits, k, "sigmoid", True, 1.0, None, n_group=3, topk_group=1)
    # table-driven routing: the ids are given, the router only weights them
    table = torch.randint(0, E, (T, k))
    ids2, w2 = M.route_ref(logits, k, "softmax", True, 1.0, None, routing_indices=table)
    assert torch.equal(ids2.long(), table)
    p = torch.softmax(logits, -1).gather(-1, table)
    assert torch.allclose(w2, p / p.sum(-1, keepdim=True), atol=1e-6)
    # configuration keys
    cfg = C.ModelConfig.from_hf_dict({"model_type": "qwen3_moe", "num_experts": 16, "num_experts_per_tok": 4, "n_group": 4,
                                      "topk_group": 2, "routed_scaling_factor": 2.5})
    assert (cfg.n_group, cfg.topk_group, cfg.routed_scaling_factor) == (4, 2, 2.5)
