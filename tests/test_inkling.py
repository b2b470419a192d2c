"""Inkling text decoder: relative-position attention without rotary embedding, short convolutions with state, dense and
routed feed-forward layers. No second implementation of the family is available here; the checks are the cache
invariants (cached = chunked = full pass) and direct restatements of the attention bias, the convolution and the router."""
import json

import pytest
import torch

from eredu_b200.models.inkling import InklingConfig, InklingModel, _ShortConv
from eredu_b200.ops import SamplingParams


def ink_cfg(**over):
    t = dict(hidden_size=40, num_hidden_layers=3, vocab_size=90, num_attention_heads=4, num_key_value_heads=2, head_dim=8,
             swa_num_attention_heads=2, swa_num_key_value_heads=1, swa_head_dim=8, sliding_window_size=5,
             layer_types=["sliding_attention", "full_attention", "sliding_attention"], dense_mlp_idx=1, sconv_kernel_size=3,
             use_sconv=True, rel_extent=7, d_rel=6, log_scaling_n_floor=4, log_scaling_alpha=0.3, rms_norm_eps=1e-6,
             use_embed_norm=True, unpadded_vocab_size=85, logits_mup_width_multiplier=2.0, intermediate_size=24,
             dense_intermediate_size=24, moe_intermediate_size=16, n_routed_experts=5, num_experts_per_tok=2, n_shared_experts=2,
             route_scale=1.2, shared_expert_sink=True, use_gate_bias=True, norm_after_topk=True, use_global_scale=True)
    t.update(over)
    return {"model_type": "inkling_mm_model", "text_config": t, "eos_token_id": 2}


def ink_state(cfg: InklingConfig, released=False, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, std=0.25: torch.randn(*s, generator=g) * std         # noqa: E731
    H = cfg.hidden_size
    sd = {"model.embed_tokens.weight": r(cfg.vocab_size, H, std=1.0), "model.embed_norm.weight": 1 + r(H, std=0.1),
          "model.norm.weight": 1 + r(H, std=0.1), "lm_head.weight": r(cfg.vocab_size, H)}
    for li in range(cfg.num_hidden_layers):
        p = f"model.layers.{li}."
        local = cfg.local_layers[li]
        hq, hkv, D = cfg.heads(local)
        ext = cfg.sliding_window_size if local else cfg.rel_extent
        sd[p + "input_layernorm.weight"], sd[p + "post_attention_layernorm.weight"] = 1 + r(H, std=0.1), 1 + r(H, std=0.1)
        a = p + "self_attn."
        sd[a + "q_proj.weight"], sd[a + "k_proj.weight"], sd[a + "v_proj.weight"] = r(hq * D, H), r(hkv * D, H), r(hkv * D, H)
        sd[a + "r_proj.weight"], sd[a + "o_proj.weight"] = r(hq * cfg.d_rel, H), r(H, hq * D)
        sd[a + "q_norm.weight"], sd[a + "k_norm.weight"] = 1 + r(D, std=0.1), 1 + r(D, std=0.1)
        sd[a + "rel_proj"] = r(cfg.d_rel, ext, std=0.8)
        sd[a + "k_sconv.weight"], sd[a + "v_sconv.weight"] = r(hkv * D, 1, 3, std=0.4), r(hkv * D, 1, 3, std=0.4)
        sd[p + "attn_sconv.weight"], sd[p + "mlp_sconv.weight"] = r(H, 1, 3, std=0.4), r(H, 1, 3, std=0.4)
        if cfg.dense_layers[li]:
            I = cfg.dense_intermediate_size
            sd[p + "dense.gate_proj.weight"], sd[p + "dense.up_proj.weight"], sd[p + "dense.down_proj.weight"] = r(I, H), r(I, H), r(H, I)
            sd[p + "dense_global_scale"] = torch.tensor([0.8])
        else:
            I, R, S = cfg.moe_intermediate_size, cfg.n_routed_experts, cfg.n_shared_experts
            m = p + "moe."
            sd[m + "router.weight"], sd[m + "router.bias"] = r(R + S, H, std=0.6), r(R, std=0.3)
            sd[m + "router.global_scale"] = torch.tensor([1.3])
            sd[m + "experts.gate_up_proj"], sd[m + "experts.down_proj"] = r(R, 2 * I, H), r(R, H, I)
            sd[m + "shared_experts.gate_up_proj"], sd[m + "shared_experts.down_proj"] = r(S, 2 * I, H), r(S, H, I)
    if not released:
        return sd
    ren = {"model.embed_tokens.weight": "model.llm.embed.weight", "model.embed_norm.weight": "model.llm.embed_norm.weight",
           "model.norm.weight": "model.llm.norm.weight", "lm_head.weight": "model.llm.unembed.weight"}
    sub = [("self_attn.q_proj", "attn.wq_du"), ("self_attn.k_proj", "attn.wk_dv"), ("self_attn.v_proj", "attn.wv_dv"),
           ("self_attn.r_proj", "attn.wr_du"), ("self_attn.o_proj", "attn.wo_ud"), ("self_attn.q_norm", "attn.q_norm"),
           ("self_attn.k_norm", "attn.k_norm"), ("self_attn.rel_proj", "attn.rel_logits_proj.proj"), ("self_attn.k_sconv", "attn.k_sconv"),
           ("self_attn.v_sconv", "attn.v_sconv"), ("input_layernorm", "attn_norm"), ("post_attention_layernorm", "mlp_norm"),
           ("dense.down_proj.weight", "mlp.w2_md.weight"), ("dense_global_scale", "mlp.global_scale"), ("moe.router.weight", "mlp.gate.weight"),
           ("moe.router.bias", "mlp.gate.bias"), ("moe.router.global_scale", "mlp.gate.global_scale"),
           ("moe.experts.gate_up_proj", "mlp.experts.w13_weight"), ("moe.experts.down_proj", "mlp.experts.w2_weight"),
           ("moe.shared_experts.gate_up_proj", "mlp.shared_experts.shared_w13_weight"),
           ("moe.shared_experts.down_proj", "mlp.shared_experts.shared_w2_weight")]
    out = {}
    for k, v in sd.items():
        if k in ren:
            out[ren[k]] = v
            continue
        if ".dense.gate_proj." in k:          # the released packing interleaves gate (even rows) and up (odd rows)
            li = k.split(".")[2]
            out[f"model.llm.layers.{li}.mlp.w13_dn.weight"] = torch.stack((v, sd[k.replace("gate_proj", "up_proj")]), 1).flatten(0, 1)
            continue
        if k.endswith("experts.gate_up_proj"):
            half = v.shape[1] // 2
            v = torch.stack((v[:, :half], v[:, half:]), 2).flatten(1, 2)
        if ".dense.up_proj." in k:
            continue
        n = k.replace("model.layers.", "model.llm.layers.")
        for a, b in sub:
            n = n.replace(a, b)
        out[n] = v
    return out


def build(**over):
    cfg = InklingConfig.from_dict(ink_cfg(**over))
    sd = ink_state(cfg)
    return InklingModel(cfg, sd.__getitem__, sd.__contains__), sd


def test_cached_chunked_and_full_passes_agree():
    model, _ = build()
    tokens = torch.randint(0, 85, (23,), generator=torch.Generator().manual_seed(1)).tolist()
    full = model.forward(tokens, model.new_cache(), all_rows=True)
    assert full.shape == (23, 85) and torch.isfinite(full).all()           # cut to the unpadded vocabulary
    cache = model.new_cache()
    rows = [model.forward(tokens[:4], cache)] + [model.forward([t], cache) for t in tokens[4:]]
    assert torch.allclose(rows[0], full[3], atol=2e-4)
    for i, row in enumerate(rows[1:]):
        assert torch.allclose(row, full[4 + i], atol=2e-4), i
    cache = model.new_cache()
    last = None
    for a, b in ((0, 1), (1, 9), (9, 10), (10, 23)):
        last = model.forward(tokens[a:b], cache)
    assert torch.allclose(last, full[-1], atol=2e-4)


def test_released_tensor_names_load_the_same_model():
    cfg = InklingConfig.from_dict(ink_cfg())
    a, b = ink_state(cfg), ink_state(cfg, released=True)
    assert not set(a) & set(b)
    ma, mb = InklingModel(cfg, a.__getitem__, a.__contains__), InklingModel(cfg, b.__getitem__, b.__contains__)
    tokens = list(range(3, 17))
    assert torch.equal(ma.forward(tokens, ma.new_cache()), mb.forward(tokens, mb.new_cache()))


def test_attention_restated_for_one_head():
    """One global layer, one query position: scores = q.k / D + tau * profile[distance], queries scaled by tau."""
    model, sd = build(num_hidden_layers=1, layer_types=["full_attention"], dense_mlp_idx=1)
    cfg = model.cfg
    w = model.layers[0]
    x = torch.randn(12, 40, generator=torch.Generator().manual_seed(2))
    got = model._attention(w, x, model.new_cache().layers[0], 0)
    hq, hkv, D = 4, 2, 8

    def conv(z, wt):                       # z [T, C]: causal depthwise convolution + skip
        pad = torch.cat((torch.zeros(2, z.shape[1]), z))
        return torch.stack([(pad[t:t + 3] * wt[:, 0, :].t()).sum(0) for t in range(z.shape[0])]) + z

    rms = lambda z, wt: z * torch.rsqrt(z.square().mean(-1, keepdim=True) + 1e-6) * wt       # noqa: E731
    p = "model.layers.0.self_attn."
    q = rms((x @ sd[p + "q_proj.weight"].t()).view(12, hq, D), sd[p + "q_norm.weight"])
    k = rms(conv(x @ sd[p + "k_proj.weight"].t(), sd[p + "k_sconv.weight"]).view(12, hkv, D), sd[p + "k_norm.weight"])
    v = conv(x @ sd[p + "v_proj.weight"].t(), sd[p + "v_sconv.weight"]).view(12, hkv, D)
    rel = (x @ sd[p + "r_proj.weight"].t()).view(12, hq, cfg.d_rel)
    t, h = 11, 3
    tau = 1.0 + 0.3 * torch.log(torch.tensor(12.0 / 4))
    prof = rel[t, h] @ sd[p + "rel_proj"]                                   # [extent 7]
    scores = torch.stack([(q[t, h] * tau) @ k[j, h // 2] / D + (tau * prof[t - j] if t - j < 7 else 0.0) for j in range(12)])
    ctx = torch.softmax(scores, 0) @ v[:, h // 2]
    out_all = got  # [T, H] after o_proj: compare through the projection of a one-hot head contribution
    o = sd[p + "o_proj.weight"]
    # rebuild the full attended row for position t from the model's own probabilities of the other heads
    rows = []
    for hh in range(hq):
        prof_h = rel[t, hh] @ sd[p + "rel_proj"]
        sc = torch.stack([(q[t, hh] * tau) @ k[j, hh // 2] / D + (tau * prof_h[t - j] if t - j < 7 else 0.0) for j in range(12)])
        rows.append(torch.softmax(sc, 0) @ v[:, hh // 2])
    assert torch.allclose(rows[h], ctx)
    assert torch.allclose(out_all[t], torch.cat(rows) @ o.t(), atol=1e-4)


def test_sliding_layers_forget_and_global_layers_do_not():
    local, _ = build(num_hidden_layers=1, layer_types=["sliding_attention"], dense_mlp_idx=1)
    a = torch.randint(0, 85, (16,), generator=torch.Generator().manual_seed(3)).tolist()
    b = list(a)
    b[2] = (b[2] + 1) % 85
    # position 15 sees keys 11..15; the convolutions reach two tokens further back: token 2 is out of reach
    assert torch.allclose(local.forward(a, local.new_cache()), local.forward(b, local.new_cache()), atol=1e-5)
    glob, _ = build(num_hidden_layers=1, layer_types=["full_attention"], dense_mlp_idx=1)
    assert not torch.allclose(glob.forward(a, glob.new_cache()), glob.forward(b, glob.new_cache()), atol=1e-5)


def test_short_convolution_state():
    w = torch.randn(6, 1, 3, generator=torch.Generator().manual_seed(4))
    conv = _ShortConv(w)
    x = torch.randn(9, 6, generator=torch.Generator().manual_seed(5))
    whole, _ = conv(x, None)
    y1, st = conv(x[:4], None)
    y2, st = conv(x[4:5], st)
    y3, st = conv(x[5:], st)
    assert torch.allclose(torch.cat((y1, y2, y3)), whole, atol=1e-6)
    assert torch.allclose(whole[5], x[5] + x[5] * w[:, 0, 2] + x[4] * w[:, 0, 1] + x[3] * w[:, 0, 0], atol=1e-6)
    assert torch.equal(st, x[7:])


def test_router_weights_come_from_one_softmax_over_chosen_and_shared_logits():
    model, sd = build()
    w = model.layers[1]                                                     # first routed layer
    x = torch.randn(3, 40, generator=torch.Generator().manual_seed(6))
    got = model._ffn(w, x)
    logits = x @ w["router"].t()
    want = torch.zeros(3, 40)

    def expert(z, gu, dn):
        h = z @ gu.t()
        return (torch.nn.functional.silu(h[:16]) * h[16:]) @ dn.t()

    for t in range(3):
        ids = torch.topk(torch.sigmoid(logits[t, :5]) + w["router_bias"], 2).indices
        both = torch.cat((logits[t, :5][ids], logits[t, 5:]))
        wt = torch.softmax(torch.nn.functional.logsigmoid(both), 0) * 1.2 * 1.3
        for j, e in enumerate(ids.tolist()):
            want[t] += expert(x[t], w["egu"][e], w["edn"][e]) * wt[j]
        for s in range(2):
            want[t] += expert(x[t], w["sgu"][s], w["sdn"][s]) * wt[2 + s]
    assert torch.allclose(got, want, atol=1e-4)


def test_loading_through_the_public_api(tmp_path):
    from safetensors.torch import save_file

    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.runtime.plan import inspect_artifact

    raw = ink_cfg()
    cfg = InklingConfig.from_dict(raw)
    sd = ink_state(cfg, released=True)
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(raw))
    report = inspect_artifact(tmp_path)
    assert report.is_loadable, [(i.code, i.message) for i in report.issues]
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    prompt = list(range(4, 20))
    direct = InklingModel(cfg, sd.__getitem__, sd.__contains__)
    want = direct.forward(prompt, direct.new_cache())
    assert torch.allclose(lm.prefill_logits(prompt), want, atol=1e-5)
    out = lm.generate([prompt], SamplingParams(temperature=0.0), 5)
    assert out[0][0] == int(want.argmax()) and len(out[0]) <= 5


def test_config_validation():
    with pytest.raises(ValueError, match="conflicts"):
        InklingConfig.from_dict(ink_cfg(local_layer_ids=[1]))
    with pytest.raises(ValueError, match="use_sconv"):
        InklingConfig.from_dict(ink_cfg(use_sconv=False))
    with pytest.raises(ValueError, match="unsupported"):
        InklingConfig.from_dict(ink_cfg(q_bias=True))
    cfg = InklingConfig.from_dict(ink_cfg(layer_types=None, local_layer_ids=[0, 2], dense_mlp_idx=None, mlp_layer_types=["dense", "moe", "moe"]))
    assert cfg.local_layers == [True, False, True] and cfg.dense_layers == [True, False, False]


def _tower_state(H=40, second=512, seed=7):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, std=0.05: torch.randn(*s, generator=g) * std         # noqa: E731
    specs = [(75, 128), (512, second), (second * 16, 4800), (9600, H)]
    sd = {}
    for i, (din, dout) in enumerate(specs):
        sd[f"model.visual.layers.linear_{i}.weight"] = r(dout, din)
        if i < 3:
            sd[f"model.visual.layers.norm_{i}.weight"] = 1 + r(dout, std=0.1)
    sd["model.visual.final_norm.weight"] = 1 + r(H, std=0.1)
    sd["audio.encoder.weight"] = r(4 * 9, H, std=1.0)
    sd["audio.final_norm.weight"] = 1 + r(H, std=0.1)
    return sd


def test_image_patches_follow_the_released_grid():
    from eredu_b200.models.inkling import IMAGE_MEAN, IMAGE_STD, image_patches

    img = torch.randint(0, 256, (50, 80, 3), generator=torch.Generator().manual_seed(1), dtype=torch.uint8)
    p = image_patches(img)
    assert p.shape == (2 * 3, 2, 40, 40, 3)                       # ceil(50 / 40) rows, 80 // 40 + 1 columns
    assert torch.equal(p[:, 0], p[:, 1])
    want = (float(img[45, 47, 1]) / 255 - IMAGE_MEAN[1]) / IMAGE_STD[1]
    assert abs(float(p[3 + 1, 0, 5, 7, 1]) - want) < 1e-6          # patch (row 1, col 1), pixel (5, 7)
    pad = (-1.0 / 255 - IMAGE_MEAN[0]) / IMAGE_STD[0]
    assert abs(float(p[2, 0, 0, 0, 0]) - pad) < 1e-6              # the extra column lies wholly outside the image


def test_hmlp_tower_against_a_restatement_and_the_splice():
    from eredu_b200.models.inkling import InklingAudio, InklingVision, image_patches, splice_media

    sd = _tower_state()
    vis = InklingVision({"text_hidden_size": 40, "patch_size": 40, "temporal_patch_size": 2, "num_channels": 3, "num_hidden_layers": 4},
                        sd.__getitem__, sd.__contains__)
    patches = image_patches(torch.randint(0, 256, (40, 39, 3), generator=torch.Generator().manual_seed(2), dtype=torch.uint8))
    out = vis(patches)
    assert out.shape == (1, 40)
    # restatement for the one patch: explicit neighbourhood gathers instead of reshapes
    rms = lambda z, w: z * torch.rsqrt(z.square().mean(-1, keepdim=True) + 1e-6) * w       # noqa: E731
    x = patches[0]                                                  # [2, 40, 40, 3]
    l0 = torch.zeros(2, 8, 8, 128)
    for t in range(2):
        for i in range(8):
            for j in range(8):
                l0[t, i, j] = sd["model.visual.layers.linear_0.weight"] @ x[t, 5 * i:5 * i + 5, 5 * j:5 * j + 5].reshape(-1)
    l0 = torch.nn.functional.gelu(rms(l0, sd["model.visual.layers.norm_0.weight"]))
    l1 = torch.zeros(2, 4, 4, 512)
    for t in range(2):
        for i in range(4):
            for j in range(4):
                l1[t, i, j] = sd["model.visual.layers.linear_1.weight"] @ l0[t, 2 * i:2 * i + 2, 2 * j:2 * j + 2].reshape(-1)
    l1 = torch.nn.functional.gelu(rms(l1, sd["model.visual.layers.norm_1.weight"]))
    l2 = torch.stack([sd["model.visual.layers.linear_2.weight"] @ l1[t].reshape(-1) for t in range(2)])
    l2 = torch.nn.functional.gelu(rms(l2, sd["model.visual.layers.norm_2.weight"]))
    l3 = sd["model.visual.layers.linear_3.weight"] @ l2.reshape(-1)
    want = rms(l3, sd["model.visual.final_norm.weight"])
    assert torch.allclose(out[0], want, atol=1e-4)
    # audio: the sum of one embedding per codebook, normalised
    aud = InklingAudio({"num_codebooks": 4, "codebook_size": 9}, sd.__getitem__, sd.__contains__)
    ids = torch.tensor([[0, 8, 3, 5], [2, 2, 2, 2], [1, 0, 7, 4]])
    a = aud(ids, valid_frames=2)
    e = sd["audio.encoder.weight"]
    assert a.shape == (2, 40) and torch.allclose(a[1], rms(e[2] + e[9 + 2] + e[18 + 2] + e[27 + 2], sd["audio.final_norm.weight"]), atol=1e-5)
    with pytest.raises(ValueError, match="codebook"):
        aud(torch.tensor([[0, 9, 0, 0]]))
    # soft tokens take the place of the placeholder rows, and only those
    model, _ = build()
    toks = [5, 6, 80, 7, 81, 81, 9]
    emb = splice_media(toks, 80, 81, [out], [a])
    assert emb[0].tolist() == [2, 4, 5]
    base = model.forward(toks, model.new_cache(), all_rows=True)
    with_media = model.forward(toks, model.new_cache(), all_rows=True, embeds=emb)
    assert torch.allclose(base[:2], with_media[:2]) and not torch.allclose(base[2:], with_media[2:])
    with pytest.raises(ValueError, match="placeholder"):
        splice_media(toks, 80, 81, [out, out], [a])


def test_media_parts_through_the_public_api(tmp_path):
    """An image, audio frames and ready embeddings between text parts: the API's typed parts give the same logits as the
    decoder fed with the spliced soft tokens, and a text-only checkpoint refuses media."""
    import numpy as np
    from safetensors.torch import save_file

    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.media import MultimodalPreparationError, RgbImage
    from eredu_b200.models.inkling import InklingAudio, InklingVision, image_patches, splice_media

    raw = ink_cfg(vocab_size=90)
    raw.update(image_token_id=80, audio_token_id=81,
               vision_config={"patch_size": 40, "temporal_patch_size": 2, "num_channels": 3, "num_hidden_layers": 4},
               audio_config={"num_codebooks": 4, "codebook_size": 9})
    cfg = InklingConfig.from_dict(raw)
    sd = {**ink_state(cfg), **_tower_state()}
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(raw))
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    assert lm.vision is not None and lm.audio is not None
    pixels = np.random.default_rng(3).integers(0, 256, (40, 39, 3), dtype=np.uint8)
    frames = torch.tensor([[0, 8, 3, 5], [2, 2, 2, 2], [1, 0, 7, 4]])
    ready = torch.randn(2, 40, generator=torch.Generator().manual_seed(5))
    segments = [[4, 5, 6], RgbImage(pixels), [7], {"audio_ids": frames, "valid_frames": 2}, {"image_embeds": ready}, [9, 10]]
    ids, (rows, values) = lm.multimodal_inputs(segments)
    assert ids == [4, 5, 6, 80, 7, 81, 81, 80, 80, 9, 10] and rows.tolist() == [3, 5, 6, 7, 8]
    # the same prompt by hand: towers, then the splice in order of appearance per modality
    vis = InklingVision({"text_hidden_size": 40, **raw["vision_config"]}, sd.__getitem__, sd.__contains__)
    aud = InklingAudio(raw["audio_config"], sd.__getitem__, sd.__contains__)
    img = vis(image_patches(torch.from_numpy(pixels)))
    emb = splice_media(ids, 80, 81, image_embeds=[img, ready], audio_embeds=[aud(frames, 2)])
    direct = InklingModel(cfg, sd.__getitem__, sd.__contains__)
    want = direct.forward(ids, direct.new_cache(), embeds=emb)
    seq = lm.engine.new_sequence(ids, SamplingParams(temperature=0.0), 4)
    got = lm.engine.feed_logits(seq, ids, (rows, values))
    assert torch.allclose(got, want, atol=1e-5)
    out = lm.generate_multimodal(segments, SamplingParams(temperature=0.0), max_new_tokens=3)
    assert out[0] == int(want.argmax()) or int(want.argmax()) == 2       # id 2 ends the sequence
    plain = direct.forward(ids, direct.new_cache())
    assert not torch.allclose(plain, want, atol=1e-3)                    # the soft tokens are what the decoder saw
    with pytest.raises(MultimodalPreparationError, match="media embeddings"):
        lm.multimodal_inputs([{"audio_embeds": torch.zeros(2, 8)}])
    # a checkpoint without towers
    text_dir = tmp_path / "text"
    text_dir.mkdir()
    raw_t = ink_cfg()
    save_file({k: v.contiguous() for k, v in ink_state(InklingConfig.from_dict(raw_t)).items()}, str(text_dir / "model.safetensors"))
    (text_dir / "config.json").write_text(json.dumps(raw_t))
    lm_t = LoadedModel.load(text_dir, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    with pytest.raises(MultimodalPreparationError, match="vision_config"):
        lm_t.multimodal_inputs([RgbImage(pixels)])
