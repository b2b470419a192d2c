"""Qwen3-VL vision tower and processor against Hugging Face Transformers."""
import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

from eredu_b200.models.qwen_vl import VisionConfig, VisionTower, image_to_patches, mrope_positions, smart_resize

VISION = dict(depth=3, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4, spatial_merge_size=2,
              temporal_patch_size=2, out_hidden_size=64, num_position_embeddings=36, deepstack_visual_indexes=[0, 2])
TEXT = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
            num_key_value_heads=2, head_dim=32, max_position_embeddings=256,
            rope_scaling={"rope_type": "default", "mrope_section": [8, 4, 4], "mrope_interleaved": True})


def hf_vl():
    cfg = transformers.Qwen3VLConfig(text_config=TEXT, vision_config=VISION, tie_word_embeddings=False, image_token_id=300,
                                     video_token_id=301, vision_start_token_id=302, vision_end_token_id=303)
    torch.manual_seed(0)
    m = transformers.Qwen3VLForConditionalGeneration(cfg).eval().float()
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for _, p in m.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn(p.shape, generator=g) * 0.1)
    return m


def test_vision_tower_matches_transformers():
    m = hf_vl()
    sd = m.state_dict()
    tower = VisionTower(VisionConfig.from_dict(VISION), lambda n: sd[n])
    grids = [(1, 4, 6), (1, 8, 4)]
    n = sum(t * h * w for t, h, w in grids)
    patches = torch.randn(n, 3 * 2 * 4 * 4, generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        ref = m.model.visual(patches, grid_thw=torch.tensor(grids))
    feats, deep = tower.forward(patches, grids)
    assert feats.shape == (n // 4, 64) and len(deep) == 2
    assert torch.allclose(feats, ref.pooler_output, atol=2e-4), float((feats - ref.pooler_output).abs().max())
    for a, b in zip(deep, ref.deepstack_features):
        assert torch.allclose(a, b, atol=2e-4)


def test_processor_patch_layout_and_resize():
    from eredu_b200.media import RgbImage

    assert smart_resize(100, 70, 8, 64, 10**6) == (96, 72)                  # 12.5 rounds half to even, like the published processor
    assert smart_resize(1000, 1000, 8, 64, 40000)[0] * smart_resize(1000, 1000, 8, 64, 40000)[1] <= 40000
    assert smart_resize(4, 4, 8, 256, 10**6) == (16, 16)
    cfg = VisionConfig.from_dict(VISION)
    rng = np.random.default_rng(0)
    img = RgbImage(rng.integers(0, 255, (16, 24, 3), dtype=np.uint8))       # already a multiple of patch * merge = 8
    patches, grid = image_to_patches(img, cfg, min_pixels=64, max_pixels=10**6)
    assert grid == (1, 4, 6) and patches.shape == (24, 3 * 2 * 4 * 4)
    norm = img.pixels.astype(np.float32) / 255.0 * 2 - 1
    # patch 0 is the top-left patch, patch 1 its right neighbour, patch 2 the one BELOW patch 0 (merge-block order)
    first = patches[0].view(3, 2, 4, 4)
    assert torch.allclose(first[:, 0], torch.from_numpy(norm[:4, :4].transpose(2, 0, 1)), atol=1e-6)
    assert torch.equal(first[:, 0], first[:, 1])                             # the still frame is repeated in time
    assert torch.allclose(patches[1].view(3, 2, 4, 4)[:, 0], torch.from_numpy(norm[:4, 4:8].transpose(2, 0, 1)), atol=1e-6)
    assert torch.allclose(patches[2].view(3, 2, 4, 4)[:, 0], torch.from_numpy(norm[4:8, :4].transpose(2, 0, 1)), atol=1e-6)
    assert torch.allclose(patches[4].view(3, 2, 4, 4)[:, 0], torch.from_numpy(norm[:4, 8:12].transpose(2, 0, 1)), atol=1e-6)


def test_mrope_positions_match_transformers():
    m = hf_vl()
    IMG = 300
    grids = [(1, 4, 6)]
    ids = [5, 6, 302] + [IMG] * 6 + [303, 7, 8, 9]
    pos, delta = mrope_positions(ids, IMG, grids, 2)
    ref, ref_delta = m.model.get_rope_index(torch.tensor([ids]), image_grid_thw=torch.tensor(grids),
                                            mm_token_type_ids=torch.tensor([[1 if t == IMG else 0 for t in ids]]))
    assert torch.equal(pos, ref[:, 0]) and delta == int(ref_delta)
    with pytest.raises(ValueError):
        mrope_positions([IMG] * 5, IMG, grids, 2)
