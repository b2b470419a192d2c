"""DeepSeek-V4 decoder: every layer kind (local, compressed, sparse with and without index selection), hash and scored
routing, hyper-connection streams. No other implementation of this family is available to compare with, so the checks are
the invariants the reference's own tests use: a cached pass (prefill then one-token steps), a chunked prefill and one full
pass give the same logits; plus direct restatements of the pooling and visibility rules."""
import pytest
import torch

from eredu_b200.models.deepseek_v4 import DeepseekV4Config, DeepseekV4Model, PoolingState, _Compressor, _Rope
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.unpaged import UnpagedEngine


def v4_cfg(**over):
    d = dict(hidden_size=48, moe_intermediate_size=32, num_hidden_layers=4, num_attention_heads=4, head_dim=16,
             qk_rope_head_dim=8, q_lora_rank=24, o_lora_rank=12, o_groups=2, vocab_size=96, index_n_heads=2, index_head_dim=8,
             index_topk=3, n_routed_experts=6, num_experts_per_tok=2, sliding_window=6, compress_ratios=[0, 3, 4, 4], hc_mult=3,
             hc_sinkhorn_iters=6, n_shared_experts=1, num_hash_layers=1, routed_scaling_factor=1.5, swiglu_limit=4.0,
             rope_scaling={"factor": 4.0, "original_max_position_embeddings": 16, "beta_fast": 32, "beta_slow": 1},
             scoring_func="sqrtsoftplus")
    d.update(over)
    return d


def v4_state(cfg: DeepseekV4Config, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, std=0.2: torch.randn(*s, generator=g) * std          # noqa: E731
    H, n, D, Hq = cfg.hidden_size, cfg.hc_mult, cfg.head_dim, cfg.num_attention_heads
    mix = (2 + n) * n
    sd = {"embed.weight": r(cfg.vocab_size, H, std=1.0), "norm.weight": 1 + r(H, std=0.1), "head.weight": r(cfg.vocab_size, H),
          "hc_head_fn": r(n, n * H), "hc_head_base": r(n), "hc_head_scale": torch.tensor([0.7])}
    for li in range(cfg.num_hidden_layers):
        p = f"layers.{li}."
        for kind in ("attn", "ffn"):
            sd[p + f"hc_{kind}_fn"], sd[p + f"hc_{kind}_base"] = r(mix, n * H), r(mix)
            sd[p + f"hc_{kind}_scale"] = torch.tensor([0.5, 0.8, 1.1])
            sd[p + kind + "_norm.weight"] = 1 + r(H, std=0.1)
        a = p + "attn."
        sd[a + "wq_a.weight"], sd[a + "q_norm.weight"] = r(cfg.q_lora_rank, H), 1 + r(cfg.q_lora_rank, std=0.1)
        sd[a + "wq_b.weight"] = r(Hq * D, cfg.q_lora_rank)
        sd[a + "wkv.weight"], sd[a + "kv_norm.weight"] = r(D, H), 1 + r(D, std=0.1)
        sd[a + "wo_a.weight"] = r(cfg.o_groups * cfg.o_lora_rank, Hq * D // cfg.o_groups)
        sd[a + "wo_b.weight"] = r(H, cfg.o_groups * cfg.o_lora_rank)
        sd[a + "attn_sink"] = r(Hq, std=1.0)
        ratio = cfg.compress_ratios[li]
        if ratio:
            w = D * (2 if ratio == 4 else 1)
            c = a + "compressor."
            sd[c + "wkv.weight"], sd[c + "wgate.weight"], sd[c + "ape"] = r(w, H), r(w, H, std=0.5), r(ratio, w, std=0.5)
            sd[c + "norm.weight"] = 1 + r(D, std=0.1)
        if ratio == 4:
            Di = cfg.index_head_dim
            i = a + "indexer."
            sd[i + "wq_b.weight"], sd[i + "weights_proj.weight"] = r(cfg.index_n_heads * Di, cfg.q_lora_rank, std=0.5), r(cfg.index_n_heads, H, std=0.5)
            sd[i + "compressor.wkv.weight"], sd[i + "compressor.wgate.weight"] = r(2 * Di, H, std=0.5), r(2 * Di, H, std=0.5)
            sd[i + "compressor.ape"], sd[i + "compressor.norm.weight"] = r(ratio, 2 * Di, std=0.5), 1 + r(Di, std=0.1)
        f = p + "ffn."
        sd[f + "gate.weight"] = r(cfg.n_routed_experts, H, std=0.5)
        if li < cfg.num_hash_layers:
            sd[f + "gate.tid2eid"] = torch.stack([torch.randperm(cfg.n_routed_experts, generator=g)[:cfg.num_experts_per_tok]
                                                  for _ in range(cfg.vocab_size)]).to(torch.int32)
        else:
            sd[f + "gate.bias"] = r(cfg.n_routed_experts, std=0.3)
        I = cfg.moe_intermediate_size
        for e in range(cfg.n_routed_experts):
            sd[f + f"experts.{e}.w1.weight"], sd[f + f"experts.{e}.w3.weight"], sd[f + f"experts.{e}.w2.weight"] = r(I, H), r(I, H), r(H, I)
        S = I * cfg.n_shared_experts
        sd[f + "shared_experts.w1.weight"], sd[f + "shared_experts.w3.weight"], sd[f + "shared_experts.w2.weight"] = r(S, H), r(S, H), r(H, S)
    return sd


def build(**over):
    cfg = DeepseekV4Config.from_dict(v4_cfg(**over))
    sd = v4_state(cfg)
    return DeepseekV4Model(cfg, sd.__getitem__, sd.__contains__), sd


def test_cached_chunked_and_full_passes_agree():
    model, _ = build()
    tokens = torch.randint(0, 96, (29,), generator=torch.Generator().manual_seed(1)).tolist()     # 29 > window, > 4 * topk
    full = model.forward(tokens, model.new_cache(), all_rows=True)
    assert full.shape == (29, 96) and torch.isfinite(full).all()
    # prefill + one-token steps
    cache = model.new_cache()
    rows = [model.forward(tokens[:5], cache)]
    for t in tokens[5:]:
        rows.append(model.forward([t], cache))
    assert cache.length == 29
    assert torch.allclose(rows[0], full[4], atol=2e-4)
    for i, row in enumerate(rows[1:]):
        assert torch.allclose(row, full[5 + i], atol=2e-4), i
    # chunks that cut pooling windows at every phase
    cache = model.new_cache()
    last = None
    for a, b in ((0, 7), (7, 8), (8, 18), (18, 29)):
        last = model.forward(tokens[a:b], cache)
    assert torch.allclose(last, full[-1], atol=2e-4)
    # the sparse layers did select: more pooled tokens than index_topk exist at the end
    assert cache.layers[2].pool.pooled.shape[0] == 29 // 4 > model.cfg.index_topk
    assert cache.layers[1].pool.pooled.shape[0] == 29 // 3 and cache.layers[1].pool.pending_values.shape[0] == 29 % 3


def test_a_token_outside_every_window_and_pool_has_no_influence():
    """Layer kinds taken one at a time: on a local-only model, logits at position p ignore tokens before p - window + 1
    (through ONE layer); with a compressed layer the early token still reaches p through the pooled stream."""
    local, _ = build(num_hidden_layers=1, compress_ratios=[0], num_hash_layers=0)
    a = torch.randint(0, 96, (20,), generator=torch.Generator().manual_seed(2)).tolist()
    b = list(a)
    b[3] = (b[3] + 1) % 96
    la, lb = local.forward(a, local.new_cache()), local.forward(b, local.new_cache())
    assert torch.allclose(la, lb, atol=1e-5)                      # 19 - 3 >= window of 6
    pooled, _ = build(num_hidden_layers=1, compress_ratios=[3], num_hash_layers=0)
    pa, pb = pooled.forward(a, pooled.new_cache()), pooled.forward(b, pooled.new_cache())
    assert not torch.allclose(pa, pb, atol=1e-5)


def test_pooling_matches_a_direct_restatement():
    cfg = DeepseekV4Config.from_dict(v4_cfg())
    sd = v4_state(cfg)
    up = lambda t, dt=None: t.to(dt or torch.float32)               # noqa: E731
    x = torch.randn(11, cfg.hidden_size, generator=torch.Generator().manual_seed(3))
    # plain windows of 3
    comp = _Compressor(cfg, 3, cfg.head_dim, sd.__getitem__, "layers.1.attn.compressor.", up, "cpu")
    st = PoolingState()
    got = comp(x[:4], st, 0)
    got = comp(x[4:], st, 4)
    assert got.shape == (3, cfg.head_dim) and st.pending_values.shape[0] == 2
    v, g = x @ sd["layers.1.attn.compressor.wkv.weight"].t(), x @ sd["layers.1.attn.compressor.wgate.weight"].t()
    rope = _Rope(cfg, cfg.compress_rope_theta, True, "cpu")
    for i in range(3):
        w = torch.softmax(g[3 * i:3 * i + 3] + sd["layers.1.attn.compressor.ape"], 0)
        p = (v[3 * i:3 * i + 3] * w).sum(0)
        p = p * torch.rsqrt(p.square().mean() + cfg.rms_norm_eps) * sd["layers.1.attn.compressor.norm.weight"]
        p = rope(p[None, None, :], torch.tensor([3 * i]))[0, 0]
        assert torch.allclose(got[i], p, atol=1e-5)
    # overlapping windows of 4: token i pools its own window's second half with the previous window's first half
    D = cfg.head_dim
    comp4 = _Compressor(cfg, 4, D, sd.__getitem__, "layers.2.attn.compressor.", up, "cpu")
    st = PoolingState()
    got = comp4(x[:9], st, 0)
    v, g = x @ sd["layers.2.attn.compressor.wkv.weight"].t(), x @ sd["layers.2.attn.compressor.wgate.weight"].t()
    ape = sd["layers.2.attn.compressor.ape"]
    vals = torch.cat((v[0:4, :D], v[4:8, D:]))
    gates = torch.cat((g[0:4, :D] + ape[:, :D], g[4:8, D:] + ape[:, D:]))
    p = (vals * torch.softmax(gates, 0)).sum(0)
    p = p * torch.rsqrt(p.square().mean() + cfg.rms_norm_eps) * sd["layers.2.attn.compressor.norm.weight"]
    p = rope(p[None, None, :], torch.tensor([4]))[0, 0]
    assert torch.allclose(got[1], p, atol=1e-5)
    # the first window has no predecessor: only its own second half takes part
    p0 = (v[0:4, D:] * torch.softmax(g[0:4, D:] + ape[:, D:], 0)).sum(0)
    p0 = p0 * torch.rsqrt(p0.square().mean() + cfg.rms_norm_eps) * sd["layers.2.attn.compressor.norm.weight"]
    assert torch.allclose(got[0], rope(p0[None, None, :], torch.tensor([0]))[0, 0], atol=1e-5)


def test_rope_is_interleaved_on_the_trailing_channels_and_inverts():
    cfg = DeepseekV4Config.from_dict(v4_cfg())
    rope = _Rope(cfg, 10000.0, False, "cpu")
    x = torch.randn(5, 2, 16)
    pos = torch.tensor([0, 1, 7, 30, 31])
    y = rope(x, pos)
    assert torch.equal(y[..., :8], x[..., :8]) and torch.equal(y[0], x[0])
    ang = 7 * rope.inv[1]
    assert torch.allclose(y[2, 0, 10], x[2, 0, 10] * torch.cos(ang) - x[2, 0, 11] * torch.sin(ang), atol=1e-6)
    assert torch.allclose(rope(y, pos, inverse=True), x, atol=1e-5)
    # YaRN leaves the fastest pair alone and divides the slowest by the factor
    yarn = _Rope(cfg, 10000.0, True, "cpu")
    assert torch.allclose(yarn.inv[0], rope.inv[0]) and torch.allclose(yarn.inv[-1], rope.inv[-1] / 4.0)


def test_hash_layers_route_by_token_id_and_scored_layers_by_biased_score():
    model, sd = build()
    x = torch.randn(4, 48, generator=torch.Generator().manual_seed(5))
    ids = torch.tensor([3, 9, 3, 50])
    y = model._ffn(model.layers[0], x, ids)
    # the same token id with different activations still uses the table's experts: zero the others and nothing changes
    table = sd["layers.0.ffn.gate.tid2eid"].long()
    used = set(table[ids].flatten().tolist())
    w = dict(model.layers[0])
    egu = w["egu"].clone()
    for e in range(6):
        if e not in used:
            egu[e].zero_()
    w["egu"] = egu
    assert torch.allclose(model._ffn(w, x, ids), y)
    # scored layer: selection follows score + bias, weights use the score alone
    w1 = model.layers[1]
    scores = torch.sqrt(torch.nn.functional.softplus(x @ w1["gate"].t()))
    top = torch.topk(scores + w1["gate_bias"], 2).indices
    wt = torch.gather(scores, 1, top)
    wt = wt / wt.sum(-1, keepdim=True) * 1.5
    want = torch.zeros(4, 48)
    for t in range(4):
        for j in range(2):
            e = int(top[t, j])
            gu = x[t] @ w1["egu"][e].t()
            g, u = gu[:32].clamp(max=4.0), gu[32:].clamp(-4.0, 4.0)
            want[t] += (torch.nn.functional.silu(g) * u) @ w1["edn"][e].t() * wt[t, j]
    sg = x @ w1["shared_gu"].t()
    want += (torch.nn.functional.silu(sg[:, :32]) * sg[:, 32:]) @ w1["shared_dn"].t()
    assert torch.allclose(model._ffn(w1, x, ids), want, atol=1e-4)


def test_the_unpaged_engine_generates_like_a_manual_loop():
    model, _ = build()
    eng = UnpagedEngine(model, max_seq_len=64)
    prompt = list(range(5, 16))
    out = eng.generate([prompt], SamplingParams(temperature=0.0), 9)[0]
    cache = model.new_cache()
    logits = model.forward(prompt, cache)
    manual = []
    for _ in range(9):
        manual.append(int(logits.argmax()))
        logits = model.forward([manual[-1]], cache)
    assert out == manual
    seen = []
    eng.generate([prompt], SamplingParams(temperature=0.0), 9, on_token=lambda i, t: seen.append(t) or (len(seen) == 4 and "stop"))
    assert seen == manual[:4] and eng.last_finish_reasons == ["stop"]
    with pytest.raises(ValueError, match="max_seq_len"):
        eng.new_sequence(list(range(60)), max_new_tokens=10)


def test_config_validation():
    with pytest.raises(ValueError, match="lacks"):
        DeepseekV4Config.from_dict({"hidden_size": 8})
    with pytest.raises(ValueError, match="output groups"):
        DeepseekV4Config.from_dict(v4_cfg(o_groups=3))
    with pytest.raises(ValueError, match="scoring"):
        DeepseekV4Config.from_dict(v4_cfg(scoring_func="softmax"))


def test_a_checkpoint_directory_is_inspected_loaded_and_generates(tmp_path):
    import json

    from safetensors.torch import save_file

    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.runtime.plan import inspect_artifact

    raw = dict(v4_cfg(), model_type="deepseek_v4", architectures=["DeepseekV4ForCausalLM"], eos_token_id=1)
    cfg = DeepseekV4Config.from_dict(raw)
    sd = v4_state(cfg)
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(raw))
    report = inspect_artifact(tmp_path)
    assert report.is_loadable, [(i.code, i.message) for i in report.issues]
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    prompt = list(range(7, 25))
    direct = DeepseekV4Model(cfg, sd.__getitem__, sd.__contains__)
    want = direct.forward(prompt, direct.new_cache())
    assert torch.allclose(lm.prefill_logits(prompt), want, atol=1e-5)
    out = lm.generate([prompt], SamplingParams(temperature=0.0), 6)
    assert len(out[0]) <= 6 and out[0][0] == int(want.argmax())
    from eredu_b200.parallel.context import ParallelContext, ParallelTopology

    with pytest.raises(NotImplementedError, match="prefix reuse"):
        LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64, prefix_cache=True))


def test_released_low_precision_tensors_decode_at_load(tmp_path):
    """The inference-layout checkpoint keeps expert banks as microscaling FP4 (two E2M1 codes per byte + one E8M0
    exponent per 32 weights in ``<base>.scale``) and other projections as E4M3 with 128 x 128 block scales in the same
    sibling tensor: both decode when read, and the loaded model equals the one built from the decoded values."""
    import json

    import numpy as np
    from safetensors.torch import save_file

    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats.checkpoint import open_checkpoint
    from eredu_b200.lib import _eredu_host as H

    raw = dict(v4_cfg(hidden_size=128, moe_intermediate_size=64, head_dim=32, qk_rope_head_dim=16, q_lora_rank=64, o_lora_rank=32,
                      vocab_size=256, index_head_dim=16), model_type="deepseek_v4", architectures=["DeepseekV4ForCausalLM"],
               eos_token_id=1, expert_dtype="fp4")
    cfg = DeepseekV4Config.from_dict(raw)
    sd = v4_state(cfg)
    stored, dense = {}, {}
    e2m1 = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6])
    for k, v in sd.items():
        if ".ffn.experts." in k and k.endswith(".weight"):
            packed, exps = H.mxfp4_quantize(np.ascontiguousarray(v.float().numpy()))
            codes = torch.from_numpy(np.asarray(packed).view(np.uint8).copy())                 # [N, K / 2]
            exps = torch.from_numpy(np.asarray(exps).copy())                                    # [N, K / 32]
            # even experts use the 4-bit storage type (the file then counts 4-bit elements), odd ones plain bytes
            as_f4 = int(k.split(".experts.")[1].split(".")[0]) % 2 == 0
            stored[k], stored[k[:-len("weight")] + "scale"] = (codes.view(torch.float4_e2m1fn_x2) if as_f4 else codes), exps
            lo, hi = e2m1[(codes & 15).long()], e2m1[(codes >> 4).long()]
            vals = torch.stack((lo, hi), -1).flatten(1)                                         # the low nibble comes first
            dense[k] = vals * torch.pow(2.0, exps.float() - 127.0).repeat_interleave(32, 1)
        elif k.endswith("attn.wq_b.weight"):
            scale = torch.pow(2.0, torch.randint(-3, 1, ((v.shape[0] + 127) // 128, (v.shape[1] + 127) // 128)).float())
            full = scale.repeat_interleave(128, 0)[:v.shape[0]].repeat_interleave(128, 1)[:, :v.shape[1]]
            q = (v / full).to(torch.float8_e4m3fn)
            stored[k], stored[k[:-len("weight")] + "scale"] = q, scale
            dense[k] = q.float() * full
        else:
            stored[k] = dense[k] = v
    save_file({k: v.contiguous() for k, v in stored.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(raw))
    from eredu_b200.runtime.plan import inspect_artifact

    report = inspect_artifact(tmp_path)
    assert report.is_loadable, [(i.code, i.message) for i in report.issues]
    src = open_checkpoint(tmp_path)
    name = "layers.1.ffn.experts.2.w1.weight"
    assert src.mxfp4_scale_name(name) == "layers.1.ffn.experts.2.w1.scale" and torch.equal(src.get(name), dense[name])
    assert src.store.info(name)["dtype"] == "F4" and src.store.info(name.replace(".2.", ".3."))["dtype"] == "U8"
    assert torch.equal(src.get(name.replace(".2.", ".3.")), dense[name.replace(".2.", ".3.")])
    assert float((dense[name] - sd[name]).abs().max()) < 0.3 * float(sd[name].abs().max())      # a 4-bit rendering of the weights
    assert torch.equal(src.get("layers.0.attn.wq_b.weight"), dense["layers.0.attn.wq_b.weight"])
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    direct = DeepseekV4Model(cfg, dense.__getitem__, dense.__contains__)
    prompt = list(range(7, 25))
    assert torch.allclose(lm.prefill_logits(prompt), direct.forward(prompt, direct.new_cache()), atol=1e-5)
