"""Gemma 4 audio tower, embedder and audio prompts against Hugging Face Transformers."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from eredu_b200.models.gemma4_audio import Gemma4AudioConfig, Gemma4AudioTower

TEXT = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
            head_dim=16, global_head_dim=32, sliding_window=8, max_position_embeddings=128,
            layer_types=["sliding_attention", "sliding_attention", "full_attention"], pad_token_id=0, num_kv_shared_layers=0,
            hidden_size_per_layer_input=8, vocab_size_per_layer_input=320)
AUDIO = dict(hidden_size=64, num_attention_heads=4, num_hidden_layers=2, output_proj_dims=48, subsampling_conv_channels=[16, 8],
             conv_kernel_size=5)
MEL = 16        # (channels[0] / 4) frequency bins survive the two stride-2 convolutions


def shake(m):
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for _, p in m.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn(p.shape, generator=g) * 0.2)
        for n, b in m.named_buffers():
            if n.endswith(("input_min", "output_min")):
                b.fill_(-2.5)
            if n.endswith(("input_max", "output_max")):
                b.fill_(2.5)
            if n.endswith("layer_scalar"):
                b.fill_(0.9)
    return g


@pytest.mark.parametrize("frames", [53, 12, 97])
def test_tower_matches_transformers(frames):
    cfg = transformers.Gemma4AudioConfig(**AUDIO)
    torch.manual_seed(0)
    m = transformers.Gemma4AudioModel(cfg).eval().float()
    g = shake(m)
    sd = {"model.audio_tower." + k: v for k, v in m.state_dict().items()}
    feats = torch.randn(frames, MEL, generator=g)
    with torch.no_grad():
        ref = m(feats[None], torch.ones(1, frames, dtype=torch.bool)).last_hidden_state[0]
    tower = Gemma4AudioTower(Gemma4AudioConfig.from_dict(cfg.to_dict()), sd.__getitem__, sd.__contains__)
    got = tower.encode(feats)
    assert got.shape == ref.shape == (tower.soft_token_count(frames), 48)
    assert torch.allclose(got, ref, atol=2e-5), float((got - ref).abs().max())
    with pytest.raises(RuntimeError, match="embedder"):
        tower.embed(got)


def test_audio_prompt_logits_match_transformers(tmp_path):
    """An audio clip enters the decoder as <boa> <audio> x n <eoa>: the placeholder rows are embedded as the padding token
    (also for the per-layer inputs) and take the embedded soft tokens; they attend causally."""
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.media import MultimodalPreparationError

    cfg = transformers.Gemma4Config(text_config=TEXT, vision_config=None, audio_config=AUDIO, image_token_id=300, video_token_id=301,
                                    audio_token_id=302, boi_token_id=303, eoi_token_id=304, boa_token_id=305, eoa_token_index=306)
    torch.manual_seed(0)
    m = transformers.Gemma4ForConditionalGeneration(cfg).eval().float()
    g = shake(m)
    m.save_pretrained(tmp_path, safe_serialization=True)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=128))
    assert lm.audio is not None and lm.vision is None and lm.audio_tokens == {"audio_token_id": 302, "boa_token_id": 305, "eoa_token_id": 306}
    clip_a, clip_b = torch.randn(37, MEL, generator=g), torch.randn(18, MEL, generator=g)
    segments = [[5, 6, 7], clip_a, [8, 9], clip_b, [10, 11, 12, 13]]
    ids, mm = lm.multimodal_inputs(segments)
    na, nb = lm.audio.soft_token_count(37), lm.audio.soft_token_count(18)
    assert len(mm["rows"]) == na + nb and ids[3] == 305 and ids[4 + na] == 306 and mm["bidir_groups"] is None
    hf_ids = list(ids)
    for r in mm["rows"]:
        hf_ids[r] = 302
    feats = torch.zeros(2, 37, MEL)
    mask = torch.zeros(2, 37, dtype=torch.bool)
    feats[0], mask[0] = clip_a, True
    feats[1, :18], mask[1, :18] = clip_b, True
    with torch.no_grad():
        ref = m(input_ids=torch.tensor([hf_ids]), input_features=feats, input_features_mask=mask).logits[0, -1]
    seq = lm.engine.new_sequence(ids, max_new_tokens=4)
    got = lm.engine.feed_logits(seq, ids, mm).float().cpu()
    assert torch.allclose(got, ref, atol=2e-3), float((got - ref).abs().max())
    nxt = int(ref.argmax())
    with torch.no_grad():
        ref2 = m(input_ids=torch.tensor([hf_ids + [nxt]]), input_features=feats, input_features_mask=mask).logits[0, -1]
    got2 = lm.engine.step_logits(seq, nxt).float().cpu()
    lm.engine.release(seq)
    assert torch.allclose(got2, ref2, atol=2e-3), float((got2 - ref2).abs().max())
    # an image part has no tower to go to
    import numpy as np

    from eredu_b200.media import RgbImage

    with pytest.raises(MultimodalPreparationError, match="vision"):
        lm.multimodal_inputs([[1, 2], RgbImage(np.zeros((8, 8, 3), np.uint8))])
