"""Mono PCM validation and semicausal periodic-Hann HTK log-mel features
(eredu/src/backend/mlx/runtime/media/audio.rs:9-200): the waveform is truncated to ``max_samples``, zero-padded on the
right to a multiple of ``pad_to_multiple`` and on the left by half a frame; frame f covers samples
[f * hop, f * hop + frame_length) and is valid when its end point (one past the frame) falls on real audio; the value is
``ln(sum_k |FFT|_k * mel[k, m] + mel_floor)``; invalid frames are zeroed."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .image import MediaError


@dataclass
class AudioWaveform:
    samples: np.ndarray
    sample_rate: int

    def __post_init__(self):
        self.samples = np.asarray(self.samples, dtype=np.float32).reshape(-1)
        if self.samples.size == 0:
            raise MediaError("audio waveform must not be empty")
        if self.sample_rate <= 0:
            raise MediaError("audio sample rate must be positive")
        if not np.all(np.isfinite(self.samples)):
            raise MediaError("audio waveform samples must all be finite")


@dataclass
class LogMelConfig:
    sample_rate: int = 16000
    frame_length: int = 320
    hop_length: int = 160
    fft_length: int = 512
    mel_bins: int = 128
    min_frequency: float = 0.0
    max_frequency: float = 8000.0
    mel_floor: float = 1e-3
    max_samples: int = 480000
    pad_to_multiple: int = 128


@dataclass
class LogMelFeatures:
    values: np.ndarray   # float32 [frames, mel_bins]
    mask: np.ndarray     # bool [frames]

    @property
    def frames(self) -> int:
        return int(self.values.shape[0])

    @property
    def mel_bins(self) -> int:
        return int(self.values.shape[1])


def htk_mel_filters(cfg: LogMelConfig) -> np.ndarray:
    """Triangular filters [fft_length / 2 + 1, mel_bins] with HTK mel spacing (no area normalisation)."""
    bins = cfg.fft_length // 2 + 1
    to_mel = lambda f: 2595.0 * np.log10(1.0 + f / 700.0)          # noqa: E731
    to_hz = lambda m: 700.0 * (10.0 ** (m / 2595.0) - 1.0)         # noqa: E731
    lo, hi = to_mel(cfg.min_frequency), to_mel(cfg.max_frequency)
    centres = to_hz(lo + (hi - lo) * np.arange(cfg.mel_bins + 2) / (cfg.mel_bins + 1))
    hz = cfg.sample_rate * 0.5 * np.arange(bins) / (bins - 1)
    down = (hz[:, None] - centres[None, :-2]) / (centres[None, 1:-1] - centres[None, :-2])
    up = (centres[None, 2:] - hz[:, None]) / (centres[None, 2:] - centres[None, 1:-1])
    return np.maximum(np.minimum(down, up), 0.0).astype(np.float32)


def extract_log_mel(waveform: AudioWaveform, cfg: LogMelConfig) -> LogMelFeatures:
    if waveform.sample_rate != cfg.sample_rate:
        raise MediaError(f"audio processor requires {cfg.sample_rate} Hz PCM, got {waveform.sample_rate} Hz")
    if (cfg.frame_length <= 0 or cfg.hop_length <= 0 or cfg.fft_length < cfg.frame_length or cfg.mel_bins <= 0
            or cfg.pad_to_multiple <= 0):
        raise MediaError("invalid log-mel processor configuration")
    real = min(waveform.samples.size, cfg.max_samples)
    padded_n = -(-real // cfg.pad_to_multiple) * cfg.pad_to_multiple
    left = cfg.frame_length // 2
    span = cfg.frame_length + 1
    total = left + padded_n
    frames = max(total - span, 0) // cfg.hop_length + 1
    padded = np.zeros(max(total, (frames - 1) * cfg.hop_length + cfg.frame_length), dtype=np.float32)
    padded[left:left + real] = waveform.samples[:real]
    window = (0.5 - 0.5 * np.cos(2.0 * np.pi * np.arange(cfg.frame_length) / cfg.frame_length)).astype(np.float32)
    idx = np.arange(frames)[:, None] * cfg.hop_length + np.arange(cfg.frame_length)[None, :]
    spec = np.abs(np.fft.rfft(padded[idx] * window[None, :], n=cfg.fft_length, axis=1)).astype(np.float32)
    values = np.log(spec @ htk_mel_filters(cfg) + np.float32(cfg.mel_floor)).astype(np.float32)
    end = np.arange(frames) * cfg.hop_length + span - 1
    mask = (end >= left) & (end < left + real)
    values[~mask] = 0.0
    return LogMelFeatures(values, mask)
