"""Gemma 4 vision tower, multimodal embedder and image prompts against Hugging Face Transformers."""
import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

from eredu_b200.models.gemma4_vision import Gemma4VisionConfig, Gemma4VisionTower, image_to_patches, target_size

TEXT = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
            head_dim=16, global_head_dim=32, sliding_window=8, max_position_embeddings=128,
            layer_types=["sliding_attention", "sliding_attention", "full_attention"], pad_token_id=0, num_kv_shared_layers=0,
            hidden_size_per_layer_input=8, vocab_size_per_layer_input=320, use_bidirectional_attention="vision")
VISION = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=2, head_dim=16,
              patch_size=4, pooling_kernel_size=2, position_embedding_size=16)


def hf_g4(**vision_kw):
    cfg = transformers.Gemma4Config(text_config=TEXT, vision_config=dict(VISION, **vision_kw), audio_config=None, image_token_id=300,
                                    video_token_id=301, audio_token_id=302, boi_token_id=303, eoi_token_id=304)
    torch.manual_seed(0)
    m = transformers.Gemma4ForConditionalGeneration(cfg).eval().float()
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for name, p in m.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn(p.shape, generator=g) * 0.1)
            if "position_embedding_table" in name:
                p.copy_(torch.randn(p.shape, generator=g) * 0.2)
        for name, b in m.named_buffers():
            if name.endswith("layer_scalar"):
                b.fill_(0.9)
            if name.endswith(("input_min", "output_min")):
                b.fill_(-0.8)
            if name.endswith(("input_max", "output_max")):
                b.fill_(0.9)
            if name.endswith("std_bias"):
                b.copy_(torch.randn(b.shape, generator=g) * 0.1)
            if name.endswith("std_scale"):
                b.copy_(torch.rand(b.shape, generator=g) + 0.5)
    return m


@pytest.mark.parametrize("vision_kw", [{}, {"use_clipped_linears": True, "standardize": True}])
def test_tower_and_embedder_match_transformers(vision_kw):
    m = hf_g4(**vision_kw)
    sd = m.state_dict()
    cfg = Gemma4VisionConfig.from_dict(dict(VISION, rope_parameters={"rope_theta": 100.0}, **vision_kw))
    tower = Gemma4VisionTower(cfg, sd.__getitem__, sd.__contains__)
    gh, gw = 4, 6
    g = torch.Generator().manual_seed(2)
    patches = torch.rand(gh * gw, 48, generator=g)
    ys, xs = np.divmod(np.arange(gh * gw), gw)
    pos = torch.from_numpy(np.stack((xs, ys), -1))
    with torch.no_grad():
        ref = m.model.get_image_features(patches[None], pos[None], return_dict=True)
    pooled = tower.encode(patches, pos)
    assert pooled.shape == (6, 32) and torch.allclose(pooled, ref.last_hidden_state, atol=2e-4), \
        float((pooled - ref.last_hidden_state).abs().max())
    soft = tower.embed(pooled)
    assert soft.shape == (6, 64) and torch.allclose(soft, ref.pooler_output, atol=2e-4)
    with pytest.raises(ValueError):
        tower.encode(patches[:-1], pos[:-1])                       # not a whole grid


def test_resize_rule_and_patch_layout():
    from eredu_b200.media import RgbImage

    # 280 soft tokens x 3 x 3 pooling = 2520 patches of 16 px: sides are multiples of 48
    assert target_size(1000, 1000, 16, 2520, 3) == (768, 768)
    assert target_size(480, 1920, 16, 2520, 3) == (384, 1584)
    assert target_size(10, 4000, 16, 2520, 3) == (48, 13440)       # a side that rounds to zero becomes one pooled row
    cfg = Gemma4VisionConfig.from_dict(VISION)
    rng = np.random.default_rng(0)
    img = RgbImage(rng.integers(0, 255, (16, 24, 3), dtype=np.uint8))
    patches, pos, soft = image_to_patches(img, cfg, max_soft_tokens=6)     # budget 24 patches of 4 px: the image as it is
    assert patches.shape == (24, 48) and soft == 6 and pos[:7].tolist() == [[0, 0], [1, 0], [2, 0], [3, 0], [4, 0], [5, 0], [0, 1]]
    # patch 7 = row 1, column 1; inside a patch pixels run row-major with the channels last
    want = np.asarray(img.pixels, dtype=np.float32)[4:8, 4:8].reshape(-1) / 255.0
    assert np.allclose(patches[7].numpy(), want)


@pytest.mark.parametrize("bidirectional", [True, False])
def test_image_prompt_logits_match_transformers(tmp_path, bidirectional):
    """Soft tokens replace the padding embedding of their rows (the per-layer inputs see the padding token); with
    ``use_bidirectional_attention = "vision"`` the soft tokens of one image attend to each other in both directions, in the
    sliding layers too."""
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.media import RgbImage

    global TEXT
    saved = TEXT
    TEXT = dict(TEXT, use_bidirectional_attention="vision" if bidirectional else None)
    try:
        m = hf_g4()
    finally:
        TEXT = saved
    m.save_pretrained(tmp_path, safe_serialization=True)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=128))
    assert lm.vision is not None and lm.vision_tokens["image_token_id"] == 300 and lm.vision_tokens["boi_token_id"] == 303
    rng = np.random.default_rng(0)
    img_a = RgbImage(rng.integers(0, 255, (16, 24, 3), dtype=np.uint8))      # 4 x 6 patches -> 6 soft tokens
    img_b = RgbImage(rng.integers(0, 255, (8, 8, 3), dtype=np.uint8))        # upscaled to the budget: 4 x 4 patches -> 4 soft tokens
    segments = [[5, 6, 7], img_a, [8, 9], img_b, [10, 11, 12, 13]]
    ids, mm = lm.multimodal_inputs(segments, image_limits=dict(max_soft_tokens=6))
    assert len(mm["rows"]) == 10 and ids[3] == 303 and ids[10] == 304 and all(ids[r] == 0 for r in mm["rows"])
    assert (mm["bidir_groups"] is not None) == bidirectional
    # Transformers gets the same patches (padded to one length per batch entry, padding marked by position -1)
    from eredu_b200.models.gemma4_vision import image_to_patches as g4_patches

    pa, xa, _ = g4_patches(img_a, lm.vision.cfg, 6)
    pb, xb, _ = g4_patches(img_b, lm.vision.cfg, 6)
    pv = torch.zeros(2, 24, 48)
    pp = torch.full((2, 24, 2), -1, dtype=torch.long)
    pv[0], pp[0] = pa, xa
    pv[1, :16], pp[1, :16] = pb, xb
    hf_ids = list(ids)
    for r in mm["rows"]:
        hf_ids[r] = 300
    types = torch.tensor([[1 if t == 300 else 0 for t in hf_ids]])
    with torch.no_grad():
        out = m(input_ids=torch.tensor([hf_ids]), pixel_values=pv, image_position_ids=pp, mm_token_type_ids=types)
    ref = out.logits[0, -1]
    seq = lm.engine.new_sequence(ids, max_new_tokens=4)
    got = lm.engine.feed_logits(seq, ids, mm).float().cpu()
    assert torch.allclose(got, ref, atol=2e-3), float((got - ref).abs().max())
    # decode continues causally after the prompt
    nxt = int(ref.argmax())
    with torch.no_grad():
        ref2 = m(input_ids=torch.tensor([hf_ids + [nxt]]), pixel_values=pv, image_position_ids=pp,
                 mm_token_type_ids=torch.tensor([types[0].tolist() + [0]])).logits[0, -1]
    got2 = lm.engine.step_logits(seq, nxt).float().cpu()
    lm.engine.release(seq)
    assert torch.allclose(got2, ref2, atol=2e-3), float((got2 - ref2).abs().max())
