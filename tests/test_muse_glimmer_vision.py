"""Muse-Glimmer vision tower and processor. No second implementation of the family is available here; the tower is
checked against a token-by-token restatement (explicit masks instead of chunked attention, explicit neighbour lookups
instead of reshapes), the processor against its definition, and the whole path through the public API."""
import json
import math

import numpy as np
import pytest
import torch

from eredu_b200.media import RgbImage
from eredu_b200.models.muse_glimmer_vision import (MuseGlimmerVision, MuseVisionConfig, MuseVisualProcessorConfig,
                                                  fold_neighbourhoods, image_to_patches, interpolation_plan, pack_patches,
                                                  rotary_tables, smart_resize, video_to_groups, window_order)

VISION = dict(model_type="muse_glimmer_vision", hidden_size=32, intermediate_size=48, num_attention_heads=2, num_hidden_layers=3,
              patch_size=4, patch_temporal=2, merge_size=2, pos_emb_height=3, pos_emb_width=3, max_position_embeddings=9,
              layer_norm_eps=1e-5, hidden_act="gelu", layer_types=["window_attention", "full_attention", "window_attention"],
              rope_parameters={"rope_type": "default", "rope_theta": 100.0})
LANG, PROJ = 64, 40


def tower_state(seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, std=0.2: torch.randn(*s, generator=g) * std          # noqa: E731
    H, I = 32, 48
    t = "model.vision_tower."
    sd = {t + "patch_embedder.patch_embedding.weight": r(H, 2 * 3 * 16), t + "patch_embedder.position_embedding_table.weight": r(9, H, std=0.5)}
    for n in ("ln_pre", "ln_post"):
        sd[t + n + ".weight"], sd[t + n + ".bias"] = 1 + r(H, std=0.1), r(H, std=0.1)
    for i in range(3):
        b = f"{t}layers.{i}."
        for n in ("norm1", "norm2"):
            sd[b + n + ".weight"], sd[b + n + ".bias"] = 1 + r(H, std=0.1), r(H, std=0.1)
        for n in ("q_proj", "k_proj", "v_proj", "proj"):
            sd[b + f"attn.{n}.weight"], sd[b + f"attn.{n}.bias"] = r(H, H), r(H, std=0.1)
        sd[b + "mlp.fc1.weight"], sd[b + "mlp.fc1.bias"] = r(I, H), r(I, std=0.1)
        sd[b + "mlp.fc2.weight"], sd[b + "mlp.fc2.bias"] = r(H, I), r(H, std=0.1)
    sd["model.vision_adapter.fc1.weight"], sd["model.vision_adapter.fc2.weight"] = r(PROJ, H * 4), r(PROJ, PROJ)
    sd["model.vision_projection.weight"] = r(LANG, PROJ)
    return sd


def restated_tower(sd, patches, grids):
    """Every patch keeps its raster position; attention uses a mask that says which patches share a window / a frame."""
    H, nh, D = 32, 2, 16
    t = "model.vision_tower."
    ln = lambda z, n: torch.nn.functional.layer_norm(z, (z.shape[-1],), sd[n + ".weight"], sd[n + ".bias"], 1e-5)    # noqa: E731
    coords = [(gi, f, y, x, h, w) for gi, (tt, h, w) in enumerate(grids) for f in range(tt) for y in range(h) for x in range(w)]
    N = len(coords)
    table = sd[t + "patch_embedder.position_embedding_table.weight"].view(3, 3, H)
    x = patches @ sd[t + "patch_embedder.patch_embedding.weight"].t()
    for n, (_, _, y, xx, h, w) in enumerate(coords):
        gy, gx = (y + 0.5) * 3 / h - 0.5, (xx + 0.5) * 3 / w - 0.5
        y0, x0 = math.floor(gy), math.floor(gx)
        for yy, wy in ((y0, 1 - (gy - y0)), (y0 + 1, gy - y0)):
            for xc, wx in ((x0, 1 - (gx - x0)), (x0 + 1, gx - x0)):
                if 0 <= yy < 3 and 0 <= xc < 3:
                    x[n] = x[n] + table[yy, xc] * (wy * wx)
    x = ln(x, t + "ln_pre")
    inv = [1.0 / 100.0 ** (i / 8) for i in range(0, 8, 2)]
    ang = torch.tensor([[(xx + 1) * v for v in inv] + [(y + 1) * v for v in inv] for (_, _, y, xx, _, _) in coords])
    ang = torch.cat((ang, ang), -1)
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    rot = lambda z: z * cos + torch.cat((-z[..., D // 2:], z[..., :D // 2]), -1) * sin                                  # noqa: E731
    same_frame = torch.tensor([[a[:2] == b[:2] for b in coords] for a in coords])
    same_window = torch.tensor([[a[:2] == b[:2] and a[2] // 3 == b[2] // 3 and a[3] // 3 == b[3] // 3 for b in coords] for a in coords])
    for i in range(3):
        b = f"{t}layers.{i}."
        lin = lambda z, n: z @ sd[b + n + ".weight"].t() + sd[b + n + ".bias"]                                            # noqa: E731
        y = ln(x, b + "norm1")
        q, k, v = (lin(y, f"attn.{n}").view(N, nh, D) for n in ("q_proj", "k_proj", "v_proj"))
        s = torch.einsum("qhd,khd->hqk", rot(q), rot(k)) / math.sqrt(D)
        mask = same_window if VISION["layer_types"][i] == "window_attention" else same_frame
        a = torch.einsum("hqk,khd->qhd", torch.softmax(s.masked_fill(~mask[None], float("-inf")), -1), v).reshape(N, H)
        x = x + lin(a, "attn.proj")
        x = x + lin(torch.nn.functional.gelu(lin(ln(x, b + "norm2"), "mlp.fc1")), "mlp.fc2")
    x = ln(x, t + "ln_post")
    where = {c[:4]: n for n, c in enumerate(coords)}
    rows = []
    for gi, (tt, h, w) in enumerate(grids):
        for f in range(tt):
            for oy in range(h // 2):
                for ox in range(w // 2):
                    cells = [x[where[(gi, f, 2 * oy + iy, 2 * ox + ix)]] for iy in range(2) for ix in range(2)]
                    rows.append(torch.stack(cells, 1).reshape(-1))            # channel-major: [C, 4]
    x = torch.stack(rows)
    x = torch.nn.functional.gelu(x @ sd["model.vision_adapter.fc1.weight"].t())
    x = torch.nn.functional.gelu(x @ sd["model.vision_adapter.fc2.weight"].t())
    x = x @ sd["model.vision_projection.weight"].t()
    return x * torch.rsqrt(x.square().mean(-1, keepdim=True) + 1e-5)


def test_tower_against_the_restatement():
    sd = tower_state()
    cfg = MuseVisionConfig.from_dict(VISION, LANG, PROJ)
    tower = MuseGlimmerVision(cfg, sd.__getitem__, sd.__contains__)
    grids = [(1, 4, 8), (2, 2, 4)]                       # windows of 3 x 3 patches: ragged windows at every edge
    patches = torch.randn(32 + 16, 96, generator=torch.Generator().manual_seed(4))
    got = tower(patches, grids)
    want = restated_tower(sd, patches, grids)
    assert got.shape == (8 + 4, LANG)
    assert float((got - want).abs().max()) < 2e-4
    with pytest.raises(ValueError, match="divisible"):
        tower(patches[:6], [(1, 2, 3)])
    with pytest.raises(ValueError, match="describes"):
        tower(patches[:7], [(1, 2, 4)])


def test_geometry_helpers():
    order, lengths = window_order([(1, 4, 5)], 3)
    # windows: rows 0-2 x cols 0-2, rows 0-2 x cols 3-4, row 3 x cols 0-2, row 3 x cols 3-4
    assert lengths == [9, 6, 3, 2] and sorted(order) == list(range(20))
    assert order[:9] == [0, 1, 2, 5, 6, 7, 10, 11, 12] and order[9:15] == [3, 4, 8, 9, 13, 14]
    idx, w = interpolation_plan([(1, 6, 3)], 3, 3)
    assert idx.shape == (18, 4) and torch.allclose(w[1::3].sum(1)[1:-1], torch.ones(4))           # interior rows sum to one
    assert float(w[0].sum()) < 1.0                       # the first of six rows reads above the table: that corner weighs nothing
    cos, sin = rotary_tables([(1, 2, 2)], 16, 100.0)
    assert cos.shape == (4, 16) and torch.allclose(cos[1, :4], cos[1, 8:12]) and torch.allclose(cos[1, 4:8], cos[0, 4:8])
    assert abs(float(sin[1, 0]) - math.sin(2.0)) < 1e-6                   # column 1 is coordinate 2 at frequency 1
    x = torch.arange(8 * 3, dtype=torch.float32).view(8, 3)
    f = fold_neighbourhoods(x, [(1, 2, 4)], 2)
    assert f.shape == (2, 12) and f[1].tolist()[:4] == [x[2, 0], x[3, 0], x[6, 0], x[7, 0]]


def test_processor_resize_rule_and_patch_layout():
    for h, w in ((1200, 800), (800, 1200), (28, 4096), (4096, 28)):
        th, tw = smart_resize(h, w, 28, 4096)
        assert th % 28 == 0 and tw % 28 == 0 and (th // 28) * (tw // 28) <= 4096
    assert smart_resize(100, 100, 28, 4096) == (84, 84)                   # 3.57 cells: floor wins the tie on aspect ratio
    assert smart_resize(10000, 10000, 28, 16) == (112, 112)
    cfg = MuseVisualProcessorConfig.from_dict({"patch_size": 4, "patch_temporal": 2, "merge_size": 2, "max_image_tokens": 6})
    assert cfg.temporal_patch_size == 2
    with pytest.raises(ValueError, match="Lanczos"):
        MuseVisualProcessorConfig.from_dict({"resample": 3})
    frames = [np.random.default_rng(i).standard_normal((3, 8, 12)).astype(np.float32) for i in range(2)]
    p, grid = pack_patches(frames, cfg, False)
    assert grid == (1, 2, 3) and p.shape == (6, 2 * 3 * 16)
    # patch (row 1, column 2), temporal slice 1, channel 2, pixel (3, 1)
    assert float(p[1 * 3 + 2, 1 * 48 + 2 * 16 + 3 * 4 + 1]) == float(frames[1][2, 4 + 3, 8 + 1])
    still, _ = pack_patches(frames[:1], cfg, True)
    assert torch.equal(still[:, :48], still[:, 48:])
    image = RgbImage(np.random.default_rng(3).integers(0, 256, (30, 60, 3), dtype=np.uint8))
    p, grid = image_to_patches(image, cfg)
    assert grid[1] % 2 == 0 and grid[2] % 2 == 0 and (grid[1] // 2) * (grid[2] // 2) <= 6 and grid[2] > grid[1]
    assert float(p.abs().max()) <= 1.0 + 1e-6                              # mean 0.5, std 0.5


def test_video_groups():
    from eredu_b200.media.request import Video

    rng = np.random.default_rng(0)
    video = Video([RgbImage(rng.integers(0, 256, (16, 16, 3), dtype=np.uint8)) for _ in range(10)], fps=4.0)
    cfg = MuseVisualProcessorConfig.from_dict({"patch_size": 4, "patch_temporal": 2, "merge_size": 2, "max_video_frame_tokens": 4, "fps": 2.0})
    groups = video_to_groups(video, cfg)
    assert len(groups) == 2                              # 10 frames at 4 fps sampled at 2 fps -> 5 -> 4 frames -> 2 groups
    assert [g[2] for g in groups] == [(1, 4, 4)] * 2 and groups[0][0] == 0.0 and groups[1][0] == 6 / 4.0
    assert len(video_to_groups(video, cfg, frame_count=1)) == 1            # at least one whole group


def test_images_through_the_public_api(tmp_path):
    from safetensors.torch import save_file

    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.ops import SamplingParams
    from test_muse_glimmer import TEXT, dense_reference, state

    sd = {**state(), **tower_state()}
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({
        "model_type": "muse_glimmer", "architectures": ["MuseGlimmerForConditionalGeneration"], "text_config": TEXT, "eos_token_id": 3,
        "vision_config": VISION, "image_token_id": 190, "video_token_id": 191, "out_hidden_size": 32, "projector_hidden_size": PROJ}))
    (tmp_path / "processor_config.json").write_text(json.dumps({
        "image_processor": {"patch_size": 4, "patch_temporal": 2, "merge_size": 2, "max_image_tokens": 6},
        "video_processor": {"patch_size": 4, "patch_temporal": 2, "merge_size": 2, "max_video_frame_tokens": 4}}))
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    assert lm.vision is not None, lm.vision_error
    image = RgbImage(np.random.default_rng(5).integers(0, 256, (24, 40, 3), dtype=np.uint8))
    segments = [[5, 6, 7], image, [8, 9]]
    ids, mm = lm.multimodal_inputs(segments, wrap=False)
    n = len(ids) - 5
    assert 1 <= n <= 6 and ids[3:3 + n] == [190] * n and mm["rows"].tolist() == list(range(3, 3 + n))
    rms = mm["values"].float().square().mean(-1)
    assert torch.allclose(rms, torch.ones_like(rms), atol=1e-3)          # the rows arrive normalised
    # the decoder sees the tower rows in place of the normalised placeholder embeddings: restate with a patched table
    seq = lm.engine.new_sequence(ids, SamplingParams(temperature=0.0), 4)
    got = lm.engine.feed_logits(seq, ids, mm)
    lm.engine.release(seq)
    sd2 = dict(sd)
    table = sd["model.language_model.embed_tokens.weight"].clone()
    fresh = list(range(192, 192 + n))                    # unused ids stand in for the soft tokens
    table[fresh] = mm["values"].float()                  # already unit RMS: the reference's embedding norm leaves them as they are
    sd2["model.language_model.embed_tokens.weight"] = table
    want = dense_reference(sd2, ids[:3] + fresh + ids[3 + n:])
    assert float((got.float() - want[-1]).abs().max()) < 5e-4
    out = lm.generate_multimodal(segments, SamplingParams(temperature=0.0), max_new_tokens=3, wrap=False)
    assert out[0] == int(want[-1].argmax()) or int(want[-1].argmax()) == 3
