"""RoPE frequency tables: default, linear, Llama-3, YaRN, proportional (partial rotary).

Formulas follow eredu/src/backend/mlx/nn/rope.rs:111-226 (Llama-3 wavelength banding :111-194).
The kernels take ``inv_freq`` ([rotary_dim/2] fp32) and an attention factor that scales cos/sin.
"""
from __future__ import annotations

import math

import torch

from .config import ModelConfig


def base_inv_freq(theta: float, rot: int) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float64) / rot))


def llama3_inv_freq(inv_freq: torch.Tensor, factor: float, low_freq_factor: float, high_freq_factor: float,
                    original_max: int) -> torch.Tensor:
    low_wavelen = original_max / low_freq_factor
    high_wavelen = original_max / high_freq_factor
    wavelen = 2 * math.pi / inv_freq
    scaled = inv_freq / factor
    smooth = (original_max / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
    mid = (1 - smooth) * scaled + smooth * inv_freq
    out = torch.where(wavelen > low_wavelen, scaled, inv_freq)
    is_mid = (wavelen <= low_wavelen) & (wavelen >= high_wavelen)
    return torch.where(is_mid, mid, out)


def yarn_inv_freq(theta: float, rot: int, factor: float, original_max: int, beta_fast: float = 32.0,
                  beta_slow: float = 1.0, mscale: float = 1.0, mscale_all_dim: float = 0.0):
    def correction_dim(num_rot):
        return (rot * math.log(original_max / (num_rot * 2 * math.pi))) / (2 * math.log(theta))

    low = max(math.floor(correction_dim(beta_fast)), 0)
    high = min(math.ceil(correction_dim(beta_slow)), rot - 1)
    if low == high:
        high += 0.001
    pos_freqs = theta ** (torch.arange(0, rot, 2, dtype=torch.float64) / rot)
    extrapolation = 1.0 / pos_freqs
    interpolation = 1.0 / (factor * pos_freqs)
    ramp = ((torch.arange(rot // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
    mask = 1 - ramp
    inv_freq = interpolation * (1 - mask) + extrapolation * mask

    def get_mscale(scale, m):
        return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

    if mscale_all_dim:
        attn_factor = get_mscale(factor, mscale) / get_mscale(factor, mscale_all_dim)
    else:
        attn_factor = get_mscale(factor, 1.0)
    return inv_freq, attn_factor


def rope_tables(cfg: ModelConfig) -> tuple[torch.Tensor, float]:
    """(inv_freq fp32 [rot/2], attention factor)."""
    rot = cfg.rotary_dim
    inv = base_inv_freq(cfg.rope_theta, rot)
    factor_out = 1.0
    sc = cfg.rope_scaling
    if sc:
        kind = sc.get("rope_type", sc.get("type", "default"))
        factor = float(sc.get("factor", 1.0))
        if kind == "linear":
            inv = inv / factor
        elif kind == "llama3":
            inv = llama3_inv_freq(inv, factor, float(sc.get("low_freq_factor", 1.0)),
                                  float(sc.get("high_freq_factor", 4.0)),
                                  int(sc.get("original_max_position_embeddings", 8192)))
        elif kind == "yarn":
            inv, factor_out = yarn_inv_freq(cfg.rope_theta, rot, factor,
                                            int(sc.get("original_max_position_embeddings") or cfg.max_position_embeddings),
                                            float(sc.get("beta_fast", 32.0)), float(sc.get("beta_slow", 1.0)),
                                            float(sc.get("mscale", 1.0)), float(sc.get("mscale_all_dim", 0.0)))
            if "attention_factor" in sc and sc["attention_factor"] is not None:
                factor_out = float(sc["attention_factor"])
        elif kind in ("default", "none", "mrope", "dynamic"):
            pass
        else:
            raise ValueError(f"unsupported rope scaling type {kind!r}")
    return inv.to(torch.float32), float(factor_out)
