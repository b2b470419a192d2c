"""Mimi codec against Transformers' MimiModel on the same (tiny, random) weights: codes, reconstruction, streaming."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from eredu_b200.codec import Mimi, MimiConfig


def tiny(tmp_path, **kw):
    d = dict(hidden_size=32, num_filters=8, num_residual_layers=1, upsampling_ratios=[4, 2], codebook_size=16, codebook_dim=8,
             num_quantizers=4, num_semantic_quantizers=1, vector_quantization_hidden_dimension=8, num_hidden_layers=2,
             num_attention_heads=4, num_key_value_heads=4, head_dim=8, intermediate_size=64, sliding_window=16, frame_rate=150.0,
             upsample_groups=32, sampling_rate=2400, max_position_embeddings=256)
    d.update(kw)
    torch.manual_seed(0)
    m = transformers.MimiModel(transformers.MimiConfig(**d)).eval()
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for name, p in m.named_parameters():
            if "layer_scale" in name:
                p.copy_(torch.rand(p.shape, generator=g) * 0.5 + 0.25)      # the published 0.01 would hide the transformer
            elif p.dim() == 1:
                p.add_(torch.randn(p.shape, generator=g) * 0.1)
        for name, b in m.named_buffers():
            if name.endswith("embed_sum"):
                b.copy_(torch.randn(b.shape, generator=g))
            elif name.endswith("cluster_usage"):
                b.copy_(torch.rand(b.shape, generator=g) + 0.5)
    for mod in m.modules():
        if hasattr(mod, "_embed"):
            mod._embed = None
    m.save_pretrained(tmp_path, safe_serialization=True)
    return m


@pytest.mark.parametrize("residual_layers,length", [(1, 640), (2, 1000)])
def test_codes_and_reconstruction_match_transformers(tmp_path, residual_layers, length):
    hf = tiny(tmp_path, num_residual_layers=residual_layers)
    codec = Mimi.load(tmp_path)
    cfg = codec.cfg
    assert cfg.frame_size == 16 and cfg.downsample_stride == 2 and cfg.encoder_hop == 8
    pcm = torch.randn(2, 1, length, generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        want_codes = hf.encode(pcm).audio_codes
        want_pcm = hf.decode(want_codes).audio_values
    codes = codec.encode(pcm)
    assert codes.shape == want_codes.shape and torch.equal(codes, want_codes)
    got = codec.decode(codes)
    assert got.shape == want_pcm.shape and torch.allclose(got, want_pcm, atol=2e-5)
    # a leading subset of the codebooks decodes too (Moshi reads 8 of 32)
    with torch.no_grad():
        want2 = hf.decode(want_codes[:, :2]).audio_values
    assert torch.allclose(codec.decode(codes[:, :2]), want2, atol=2e-5)
    assert torch.equal(codec.encode(pcm, num_codebooks=2), want_codes[:, :2])
    with pytest.raises(ValueError):
        codec.decode(torch.zeros(1, 5, 3, dtype=torch.long))


def test_streaming_equals_one_shot(tmp_path):
    tiny(tmp_path)
    codec = Mimi.load(tmp_path)
    F_ = codec.cfg.frame_size
    pcm = torch.randn(1, 1, 40 * F_, generator=torch.Generator().manual_seed(5))         # 40 frames: beyond the window of 16
    codes = codec.encode(pcm)
    audio = codec.decode(codes)
    # encoder: ragged chunks; frames come out as they complete
    codec.reset_encode_state()
    got, at = [], 0
    for n in (5, F_ * 3 + 7, 1, F_ * 10, F_ * 30):
        out = codec.encode_step(pcm[..., at:at + n])
        at += n
        if out is not None:
            got.append(out)
    assert at >= pcm.shape[-1] and torch.equal(torch.cat(got, -1), codes)
    # decoder: one frame, then several at a time
    codec.reset_decode_state()
    parts, at = [], 0
    for n in (1, 1, 5, 13, 20):
        parts.append(codec.decode_step(codes[..., at:at + n]))
        at += n
    assert torch.allclose(torch.cat(parts, -1), audio, atol=2e-5)
    # a new stream starts clean
    codec.reset_decode_state()
    assert torch.allclose(codec.decode_step(codes[..., :4]), audio[..., :4 * F_], atol=2e-5)


def test_configuration():
    cfg = MimiConfig.v0_1(8)
    assert cfg.frame_size == 1920 and cfg.encoder_hop == 960 and cfg.downsample_stride == 2 and cfg.num_quantizers == 8
    assert cfg.attn_head_dim == 64
    with pytest.raises(ValueError):
        MimiConfig.from_dict({"num_quantizers": 1, "num_semantic_quantizers": 1})
    with pytest.raises(ValueError):
        MimiConfig.from_dict({"frame_rate": 7.0})
