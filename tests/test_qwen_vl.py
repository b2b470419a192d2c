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


def test_image_prompt_logits_and_decode_match_transformers(tmp_path):
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.media import MultimodalPreparationError, RgbImage

    m = hf_vl()
    m.save_pretrained(tmp_path, safe_serialization=True)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=128))
    assert lm.vision is not None and lm.vision_tokens["image_token_id"] == 300
    rng = np.random.default_rng(0)
    img_a = RgbImage(rng.integers(0, 255, (16, 24, 3), dtype=np.uint8))
    img_b = RgbImage(rng.integers(0, 255, (8, 8, 3), dtype=np.uint8))
    segments = [[5, 6, 7], img_a, [8, 9], img_b, [10, 11, 12]]
    ids, mm = lm.multimodal_inputs(segments, min_pixels=64, max_pixels=10**6)
    assert ids.count(300) == 6 + 1 and ids[3] == 302 and mm["values"].shape == (7, 64) and len(mm["deepstack"]) == 2
    # the same pixels through Transformers: patches in its layout are exactly what our processor produced
    from eredu_b200.models.qwen_vl import image_to_patches

    pa, ga = image_to_patches(img_a, lm.vision.cfg, 64, 10**6)
    pb, gb = image_to_patches(img_b, lm.vision.cfg, 64, 10**6)
    with torch.no_grad():
        out = m(input_ids=torch.tensor([ids]), pixel_values=torch.cat((pa, pb)), image_grid_thw=torch.tensor([ga, gb]),
                mm_token_type_ids=torch.tensor([[1 if t == 300 else 0 for t in ids]]))
    ref = out.logits[0, -1]
    seq = lm.engine.new_sequence(ids, max_new_tokens=8)
    got = lm.engine.feed_logits(seq, ids, mm)
    assert torch.allclose(got.float().cpu(), ref, atol=2e-3), float((got.float().cpu() - ref).abs().max())
    # decode after the images: positions continue at index + delta, as in Transformers' generation
    with torch.no_grad():
        gen = m.generate(input_ids=torch.tensor([ids]), pixel_values=torch.cat((pa, pb)), image_grid_thw=torch.tensor([ga, gb]),
                         mm_token_type_ids=torch.tensor([[1 if t == 300 else 0 for t in ids]]),
                         max_new_tokens=6, do_sample=False)[0, len(ids):].tolist()
    lm.engine.release(seq)
    ours = lm.generate_multimodal(segments, max_new_tokens=6, min_pixels=64, max_pixels=10**6)
    assert ours == gen[:len(ours)] and len(ours) >= 1
    # a text-only checkpoint refuses image parts
    lm.vision = None
    with pytest.raises(MultimodalPreparationError):
        lm.multimodal_inputs(segments)


def test_chat_segments_cut_the_prompt_at_image_placeholders(tmp_path):
    from eredu_b200.api import LoadedModel
    from eredu_b200.media import RgbImage, load_image

    class FakeLM(LoadedModel):
        def __init__(self):
            pass

        def prepare_chat(self, messages, **kw):
            from types import SimpleNamespace

            text = "".join("<|vision_start|><|image_pad|><|vision_end|>" if c["type"] == "image" else c["text"]
                           for m in messages for c in m["content"])
            return SimpleNamespace(prompt="<|im_start|>user\n" + text + "<|im_end|>")

    a, b = RgbImage(np.zeros((2, 2, 3), np.uint8)), RgbImage(np.ones((2, 2, 3), np.uint8))
    msgs = [{"role": "user", "content": [{"type": "image"}, {"type": "text", "text": "compare"}, {"type": "image"}]}]
    segs = FakeLM().chat_segments(msgs, [a, b])
    assert segs == ["<|im_start|>user\n<|vision_start|>", a, "<|vision_end|>compare<|vision_start|>", b, "<|vision_end|><|im_end|>"]
    with pytest.raises(ValueError):
        FakeLM().chat_segments(msgs, [a])
    Image = pytest.importorskip("PIL.Image")
    Image.fromarray(np.full((3, 5, 3), 200, np.uint8)).save(tmp_path / "x.png")
    im = load_image(tmp_path / "x.png")
    assert (im.height, im.width) == (3, 5) and int(im.pixels[0, 0, 0]) == 200


def test_video_prompt_matches_transformers(tmp_path):
    """A video is sampled, padded to whole temporal patches and enters the decoder as one framed placeholder run per
    temporal group; tower features, three-axis positions and logits agree with Transformers on the same frames."""
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.media.request import Video
    from eredu_b200.media import RgbImage
    from eredu_b200.models.qwen_vl import video_to_patches

    m = hf_vl()
    m.save_pretrained(tmp_path, safe_serialization=True)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=256))
    assert lm.vision_tokens["video_token_id"] == 301
    rng = np.random.default_rng(1)
    video = Video([RgbImage(rng.integers(0, 255, (16, 16, 3), dtype=np.uint8)) for _ in range(10)], fps=4.0)
    limits = dict(target_fps=2.0, min_frames=2, max_frames=8, min_pixels=64, max_pixels=10**6)
    patches, grid, stamps = video_to_patches(video, lm.vision.cfg, **limits)
    # 10 frames at 4 fps for 2 fps -> 5 sampled (0, 2, 4, 7, 9 by round-half-even), padded to 6 -> 3 temporal groups
    assert grid == (3, 4, 4) and patches.shape == (48, 3 * 2 * 4 * 4) and len(stamps) == 3
    assert stamps == pytest.approx([(0 + 2) / 8, (4 + 7) / 8, (9 + 9) / 8])
    img = RgbImage(rng.integers(0, 255, (8, 8, 3), dtype=np.uint8))
    segments = [[5, 6], video, [7], img, [8, 9]]
    ids, mm = lm.multimodal_inputs(segments, min_pixels=64, max_pixels=10**6, video_limits=limits)
    assert ids.count(301) == 3 * 4 and ids.count(300) == 1 and ids.count(302) == 4 and mm["values"].shape == (13, 64)
    pi, gi = image_to_patches(img, lm.vision.cfg, 64, 10**6)
    types = torch.tensor([[1 if t == 300 else 2 if t == 301 else 0 for t in ids]])
    with torch.no_grad():
        out = m(input_ids=torch.tensor([ids]), pixel_values=pi, image_grid_thw=torch.tensor([gi]), pixel_values_videos=patches,
                video_grid_thw=torch.tensor([grid]), mm_token_type_ids=types)
        ref_pos, ref_delta = m.model.get_rope_index(torch.tensor([ids]), image_grid_thw=torch.tensor([gi]),
                                                    video_grid_thw=torch.tensor([grid]), mm_token_type_ids=types)
    assert torch.equal(mm["rope_positions"], ref_pos[:, 0]) and mm["rope_delta"] == int(ref_delta)
    seq = lm.engine.new_sequence(ids, max_new_tokens=4)
    got = lm.engine.feed_logits(seq, ids, mm)
    lm.engine.release(seq)
    assert torch.allclose(got.float().cpu(), out.logits[0, -1], atol=2e-3), float((got.float().cpu() - out.logits[0, -1]).abs().max())
    assert len(lm.generate_multimodal(segments, max_new_tokens=3, min_pixels=64, max_pixels=10**6, video_limits=limits)) >= 1


def test_qwen3_5_hybrid_decoder_with_its_vision_tower_matches_transformers(tmp_path):
    """Qwen3.5 vision-language checkpoints: the gated-delta / attention hybrid decoder under ``model.language_model``, a
    tower without DeepStack taps under ``model.visual``, three-axis rotary positions on a quarter of the head."""
    import os

    from safetensors.torch import save_file

    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.media import RgbImage

    vision = {k: v for k, v in VISION.items() if k != "deepstack_visual_indexes"}
    text = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                num_key_value_heads=2, head_dim=32, max_position_embeddings=256, linear_num_value_heads=4, linear_num_key_heads=2,
                linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4, full_attention_interval=4,
                rope_parameters={"rope_type": "default", "mrope_section": [2, 1, 1], "mrope_interleaved": True,
                                 "rope_theta": 10000.0, "partial_rotary_factor": 0.25})
    cfg = transformers.Qwen3_5Config(text_config=text, vision_config=vision, tie_word_embeddings=False, image_token_id=300,
                                     video_token_id=301, vision_start_token_id=302, vision_end_token_id=303)
    torch.manual_seed(0)
    m = transformers.Qwen3_5ForConditionalGeneration(cfg).eval().float()
    # written by hand under the published tensor names (model.language_model.*, model.visual.*, lm_head.weight)
    save_file({k: v.contiguous() for k, v in m.state_dict().items()}, os.path.join(tmp_path, "model.safetensors"))
    cfg.save_pretrained(tmp_path)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=128))
    assert lm.vision is not None and lm.vision.cfg.deepstack_visual_indexes == () and lm.config.model_type == "qwen3_5_text"
    rng = np.random.default_rng(0)
    img_a = RgbImage(rng.integers(0, 255, (16, 24, 3), dtype=np.uint8))
    img_b = RgbImage(rng.integers(0, 255, (8, 8, 3), dtype=np.uint8))
    segments = [[5, 6, 7], img_a, [8, 9], img_b, [10, 11, 12]]
    ids, mm = lm.multimodal_inputs(segments, min_pixels=64, max_pixels=10**6)
    pa, ga = image_to_patches(img_a, lm.vision.cfg, 64, 10**6)
    pb, gb = image_to_patches(img_b, lm.vision.cfg, 64, 10**6)
    kw = dict(pixel_values=torch.cat((pa, pb)), image_grid_thw=torch.tensor([ga, gb]),
              mm_token_type_ids=torch.tensor([[1 if t == 300 else 0 for t in ids]]))
    with torch.no_grad():
        ref = m(input_ids=torch.tensor([ids]), **kw).logits[0, -1]
    seq = lm.engine.new_sequence(ids, max_new_tokens=8)
    got = lm.engine.feed_logits(seq, ids, mm)
    assert torch.allclose(got.float().cpu(), ref, atol=2e-3), float((got.float().cpu() - ref).abs().max())
    lm.engine.release(seq)
    with torch.no_grad():
        gen = m.generate(input_ids=torch.tensor([ids]), max_new_tokens=5, do_sample=False, **kw)[0, len(ids):].tolist()
    ours = lm.generate_multimodal(segments, max_new_tokens=5, min_pixels=64, max_pixels=10**6)
    assert ours == gen[:len(ours)] and len(ours) >= 1
