"""Media preprocessing: image views / resampling / normalisation, log-mel features, video frame sampling."""
import numpy as np
import pytest

from eredu_b200 import media as M
from eredu_b200.media.image import MediaError


def test_image_view_and_normalisation():
    # two 1-pixel rows six bytes apart: the padding between them is dropped
    view = M.RgbImage.with_row_stride(bytes([255, 0, 0, 9, 9, 9, 0, 255, 0]), 1, 2, 6)
    norm = M.rescale_and_normalize_rgb8(view, 1.0 / 255.0, [0.5] * 3, [0.5] * 3)
    assert norm.data.reshape(-1).tolist() == [1.0, -1.0, -1.0, 1.0, -1.0, -1.0] and norm.get(1, 1, 0) == 1.0
    assert (norm.channels, norm.height, norm.width) == (3, 2, 1)
    same = M.resize_rgb8_bicubic(M.RgbImage.with_row_stride(bytes([1, 2, 3, 0, 4, 5, 6]), 1, 2, 4), 1, 2)
    assert same.pixels.reshape(-1).tolist() == [1, 2, 3, 4, 5, 6]
    with pytest.raises(MediaError):
        M.RgbImage.with_row_stride(bytes(5), 1, 2, 3)
    with pytest.raises(MediaError):
        M.rescale_and_normalize_rgb8(view, 1.0, [0] * 3, [1, 0, 1])
    with pytest.raises(MediaError):
        M.resize_rgb8_lanczos3(view, 0, 4)


@pytest.mark.parametrize("fn,pil", [(M.resize_rgb8_bicubic, "BICUBIC"), (M.resize_rgb8_lanczos3, "LANCZOS")])
@pytest.mark.parametrize("size", [(48, 32), (200, 150), (64, 200)])
def test_resampling_agrees_with_an_independent_implementation(fn, pil, size):
    Image = pytest.importorskip("PIL.Image")
    rng = np.random.default_rng(0)
    # smooth content plus an edge: resampling filters differ most on noise, which no preprocessing pipeline feeds them
    yy, xx = np.mgrid[0:96, 0:128]
    img = np.stack([127 + 100 * np.sin(xx / 9.0), 127 + 100 * np.cos(yy / 7.0), (xx > 64) * 200.0], -1)
    img = np.clip(img + rng.normal(0, 2, img.shape), 0, 255).astype(np.uint8)
    out = fn(M.RgbImage(img), size[0], size[1]).pixels
    ref = np.asarray(Image.fromarray(img).resize(size, getattr(Image.Resampling, pil)))
    assert out.shape == ref.shape == (size[1], size[0], 3)
    diff = np.abs(out.astype(int) - ref.astype(int))
    assert diff.max() <= 3 and diff.mean() < 0.5
    flat = np.full((10, 14, 3), 77, dtype=np.uint8)
    assert np.all(fn(M.RgbImage(flat), 33, 5).pixels == 77)          # the weights of every output sample sum to one


def test_log_mel_features():
    cfg = M.LogMelConfig()
    feats = M.extract_log_mel(M.AudioWaveform(np.zeros(16000, dtype=np.float32), 16000), cfg)
    assert feats.frames == 99 and feats.mel_bins == 128 and feats.mask.all() and np.isfinite(feats.values).all()
    assert np.allclose(feats.values, np.log(1e-3), atol=1e-6)
    # a pure tone lights up the filter around its frequency
    t = np.arange(16000) / 16000.0
    tone = M.extract_log_mel(M.AudioWaveform(np.sin(2 * np.pi * 1000.0 * t).astype(np.float32), 16000), cfg)
    mel_of = lambda f: 2595.0 * np.log10(1.0 + f / 700.0)                          # noqa: E731
    expect = int(round(mel_of(1000.0) / mel_of(8000.0) * 129)) - 1
    assert abs(int(tone.values[50].argmax()) - expect) <= 1
    # direct evaluation of one frame: windowed DFT magnitude through the triangular filters
    from eredu_b200.media.audio import htk_mel_filters

    x = np.random.default_rng(1).normal(size=4000).astype(np.float32)
    got = M.extract_log_mel(M.AudioWaveform(x, 16000), cfg)
    padded = np.concatenate([np.zeros(160, np.float32), x, np.zeros(200, np.float32)])
    f = 7
    frame = padded[f * 160:f * 160 + 320] * (0.5 - 0.5 * np.cos(2 * np.pi * np.arange(320) / 320))
    k = np.arange(257)[:, None] * np.arange(320)[None, :]
    mag = np.abs((frame[None, :] * np.exp(-2j * np.pi * k / 512)).sum(1))
    assert np.allclose(got.values[f], np.log(mag @ htk_mel_filters(cfg) + 1e-3), atol=2e-3)
    # frames whose end point lies in the padding are masked and zeroed; truncation applies before padding
    assert got.frames == (160 + 4096 - 321) // 160 + 1 and not got.mask[-1] and np.all(got.values[-1] == 0)
    short = M.extract_log_mel(M.AudioWaveform(x, 16000), M.LogMelConfig(max_samples=1000))
    assert short.frames == (160 + 1024 - 321) // 160 + 1
    with pytest.raises(MediaError):
        M.extract_log_mel(M.AudioWaveform(x, 8000), cfg)
    with pytest.raises(MediaError):
        M.AudioWaveform(np.array([np.nan], dtype=np.float32), 16000)


def test_video_sampling():
    assert M.uniform_sample_indices(10, 4) == [0, 3, 6, 9]
    assert M.uniform_sample_indices(3, 8) == [0, 1, 2] and M.uniform_sample_indices(5, 1) == [0]
    assert M.uniform_sample_indices(6, 3) == [0, 2, 5]                 # 2.5 rounds to the even neighbour
    assert M.sampled_frame_count(300, 30.0, 2.0, 4, 16) == 16 and M.sampled_frame_count(60, 30.0, 2.0, 4, 16) == 4
    assert M.sampled_frame_count(3, 30.0, 2.0, 4, 16) == 3
    idx = M.pad_frame_indices([0, 2, 4], 2)
    assert idx == [0, 2, 4, 4]
    assert M.temporal_group_timestamps(idx, 2.0, 2) == [0.5, 2.0]
    assert M.frame_timestamps([0, 15, 30], 30.0) == [0.0, 0.5, 1.0]
    assert M.format_mm_ss(125.9) == "02:05"
    frames = [M.RgbImage(np.zeros((4, 6, 3), np.uint8)), M.RgbImage(np.zeros((4, 6, 3), np.uint8))]
    assert M.validate_rgb_frames(frames) == (6, 4)
    with pytest.raises(MediaError):
        M.validate_rgb_frames(frames + [M.RgbImage(np.zeros((5, 6, 3), np.uint8))])
    for bad in (lambda: M.uniform_sample_indices(0, 1), lambda: M.sampled_frame_count(10, 0.0, 1.0, 1, 2),
                lambda: M.format_mm_ss(-1.0), lambda: M.temporal_group_timestamps([0, 1, 2], 1.0, 2)):
        with pytest.raises(MediaError):
            bad()


def test_multimodal_request_values():
    im = M.RgbImage(np.zeros((2, 2, 3), np.uint8))
    req = M.MultimodalRequest().text("describe").image(im).text("briefly")
    assert req.modalities() == {"text", "image"} and len(req.parts) == 3
    with pytest.raises(M.MultimodalPreparationError, match="image"):
        M.prepare_for_text_model(req, lambda s: [1])
    segs = M.prepare_for_text_model(M.MultimodalRequest().text("ab").text("c"), lambda s: [ord(c) for c in s])
    assert [s.token_ids for s in segs] == [[97, 98], [99]] and all(s.kind == "text" for s in segs)
    with pytest.raises(MediaError):
        M.Video([im, M.RgbImage(np.zeros((3, 2, 3), np.uint8))], 24.0)
