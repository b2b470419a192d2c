"""Gemma 4 vision tower: image patches -> soft tokens in the decoder's embedding space.

Counterpart of the reference's Gemma 4 vision path (eredu/src/backend/mlx/architectures/gemma4/, vision tower and
multimodal embedder). Structure:

* patches ``[N, 3 P^2]`` with pixel values in [0, 1] are mapped to [-1, 1], projected, and get the sum of two learned
  position embeddings (one table per axis, indexed by the patch's x and y);
* encoder blocks with sandwich RMSNorms, q / k RMSNorm (learned scale) and a scale-free v RMSNorm, a two-axis rotary embedding
  (the head dimension is split in halves for x and y, each rotated on its own), full bidirectional attention with scale 1,
  gated GELU feed-forward; linears may clamp their inputs and outputs to ranges stored with the weights;
* k x k average pooling over the patch grid, multiplication by sqrt(hidden), optional standardisation;
* the multimodal embedder: scale-free RMSNorm, then a projection to the decoder width.

Inside the decoder the soft tokens of one image attend to each other in both directions (``bidirectional groups`` of
``ops.attention_ref``). ``tests/test_gemma4_vision.py`` checks tower, embedder and image-prompt logits against Transformers.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch
import torch.nn.functional as F


@dataclass
class Gemma4VisionConfig:
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 16
    num_attention_heads: int = 12
    num_key_value_heads: int = 12
    head_dim: int = 64
    patch_size: int = 16
    pooling_kernel_size: int = 3
    position_embedding_size: int = 10240
    rms_norm_eps: float = 1e-6
    rope_theta: float = 100.0
    hidden_activation: str = "gelu_pytorch_tanh"
    use_clipped_linears: bool = False
    standardize: bool = False

    @classmethod
    def from_dict(cls, d: dict) -> "Gemma4VisionConfig":
        kw = {k: d[k] for k in cls.__dataclass_fields__ if k in d and d[k] is not None}
        rp = d.get("rope_parameters") or {}
        if "rope_theta" in rp:
            kw["rope_theta"] = float(rp["rope_theta"])
        return cls(**kw)


def _rms(x, w, eps):
    xf = x.float()
    y = xf * torch.pow(xf.pow(2).mean(-1, keepdim=True) + eps, -0.5)
    return (y * w.float() if w is not None else y).to(x.dtype)


class _Linear:
    """Weight plus the optional clamp ranges of a clippable linear."""

    def __init__(self, get, has, name: str, device, dtype, clipped: bool):
        self.w = get(name + ".linear.weight").to(device=device, dtype=dtype).contiguous()
        self.lim = None
        if clipped and has(name + ".input_min"):
            self.lim = tuple(float(get(f"{name}.{k}")) for k in ("input_min", "input_max", "output_min", "output_max"))

    def __call__(self, x):
        if self.lim is None:
            return F.linear(x, self.w)
        return F.linear(x.clamp(self.lim[0], self.lim[1]), self.w).clamp(self.lim[2], self.lim[3])


class Gemma4VisionTower:
    def __init__(self, cfg: Gemma4VisionConfig, get, has, device="cpu", dtype=torch.float32, prefix="model.vision_tower.",
                 embed_prefix="model.embed_vision."):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        up = lambda n, dt=None: get(n).to(device=self.device, dtype=dt or dtype).contiguous()       # noqa: E731
        self.input_proj = up(prefix + "patch_embedder.input_proj.weight")
        self.pos_table = up(prefix + "patch_embedder.position_embedding_table")                     # [2, size, hidden]
        self.layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"{prefix}encoder.layers.{i}."
            lw = {n: _Linear(get, has, p + path, self.device, dtype, cfg.use_clipped_linears)
                  for n, path in (("q", "self_attn.q_proj"), ("k", "self_attn.k_proj"), ("v", "self_attn.v_proj"),
                                  ("o", "self_attn.o_proj"), ("gate", "mlp.gate_proj"), ("up", "mlp.up_proj"),
                                  ("down", "mlp.down_proj"))}
            for n in ("self_attn.q_norm", "self_attn.k_norm", "input_layernorm", "post_attention_layernorm",
                      "pre_feedforward_layernorm", "post_feedforward_layernorm"):
                lw[n] = up(p + n + ".weight", torch.float32)
            self.layers.append(lw)
        self.std = (up(prefix + "std_bias", torch.float32), up(prefix + "std_scale", torch.float32)) if cfg.standardize else None
        self.embed_proj = up(embed_prefix + "embedding_projection.weight")
        if cfg.hidden_activation not in ("gelu_pytorch_tanh", "gelu", "silu"):
            raise ValueError(f"unsupported vision activation {cfg.hidden_activation!r}")

    def _act(self, x):
        name = self.cfg.hidden_activation
        return F.gelu(x, approximate="tanh") if name == "gelu_pytorch_tanh" else F.gelu(x) if name == "gelu" else F.silu(x)

    def _rotary(self, positions):
        """cos / sin [N, D]: the first half of the head dimension turns with x, the second with y."""
        D = self.cfg.head_dim
        half = D // 2
        inv = 1.0 / (self.cfg.rope_theta ** (torch.arange(0, half, 2, dtype=torch.float32, device=self.device) / half))
        parts = []
        for axis in range(2):
            f = positions[:, axis].float()[:, None] * inv[None, :]
            parts.append(torch.cat((f, f), -1))
        ang = torch.cat(parts, -1)
        return ang.cos(), ang.sin()

    @staticmethod
    def _rotate(x, cos, sin):
        """x [N, H, D]; each half of D is a rotary embedding of its own (split-half inside the half)."""
        D = x.shape[-1]
        out = []
        for lo in (0, D // 2):
            part, c, s = x[..., lo:lo + D // 2], cos[:, None, lo:lo + D // 2], sin[:, None, lo:lo + D // 2]
            q = part.shape[-1] // 2
            rot = torch.cat((-part[..., q:], part[..., :q]), -1)
            out.append(part * c + rot * s)
        return torch.cat(out, -1)

    @torch.no_grad()
    def encode(self, patches: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """One image: patches [N, 3 P^2] in [0, 1] (row-major over the patch grid), positions [N, 2] as (x, y).
        Returns the pooled encoder output [N / k^2, hidden] (before the multimodal embedder)."""
        cfg = self.cfg
        positions = positions.to(self.device)
        x = F.linear((2.0 * (patches.to(self.device, torch.float32) - 0.5)).to(self.dtype), self.input_proj)
        x = x + self.pos_table[0][positions[:, 0]] + self.pos_table[1][positions[:, 1]]
        cos, sin = self._rotary(positions)
        cos, sin = cos.to(self.dtype), sin.to(self.dtype)
        N, Hq, Hkv, D, eps = x.shape[0], cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps
        for lw in self.layers:
            h = _rms(x, lw["input_layernorm"], eps)
            q = self._rotate(_rms(lw["q"](h).view(N, Hq, D), lw["self_attn.q_norm"], eps), cos, sin)
            k = self._rotate(_rms(lw["k"](h).view(N, Hkv, D), lw["self_attn.k_norm"], eps), cos, sin)
            v = _rms(lw["v"](h).view(N, Hkv, D), None, eps)
            if Hkv != Hq:
                k, v = k.repeat_interleave(Hq // Hkv, 1), v.repeat_interleave(Hq // Hkv, 1)
            a = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None], scale=1.0)[0]
            x = x + _rms(lw["o"](a.transpose(0, 1).reshape(N, Hq * D)), lw["post_attention_layernorm"], eps)
            h = _rms(x, lw["pre_feedforward_layernorm"], eps)
            x = x + _rms(lw["down"](self._act(lw["gate"](h)) * lw["up"](h)), lw["post_feedforward_layernorm"], eps)
        kk = cfg.pooling_kernel_size
        gw, gh = int(positions[:, 0].max()) + 1, int(positions[:, 1].max()) + 1
        if gw * gh != N or gw % kk or gh % kk:
            raise ValueError(f"a {gw} x {gh} patch grid cannot be pooled {kk} x {kk}")
        grid = torch.zeros((gh, gw, x.shape[1]), dtype=torch.float32, device=self.device)
        grid[positions[:, 1], positions[:, 0]] = x.float()
        pooled = grid.view(gh // kk, kk, gw // kk, kk, -1).mean((1, 3)).reshape(-1, x.shape[1]) * math.sqrt(cfg.hidden_size)
        if self.std is not None:
            pooled = (pooled - self.std[0]) * self.std[1]
        return pooled.to(self.dtype)

    @torch.no_grad()
    def embed(self, pooled: torch.Tensor) -> torch.Tensor:
        """Soft tokens in the decoder's embedding space."""
        return F.linear(_rms(pooled, None, self.cfg.rms_norm_eps), self.embed_proj)

    def forward(self, patches, positions) -> torch.Tensor:
        return self.embed(self.encode(patches, positions))


def target_size(height: int, width: int, patch_size: int, max_patches: int, pooling: int) -> tuple[int, int]:
    """Largest size with the image's aspect ratio that gives at most ``max_patches`` patches and whose sides are multiples
    of ``pooling * patch_size``; a side that would round to zero becomes one such multiple."""
    side = pooling * patch_size
    factor = math.sqrt(max_patches * patch_size ** 2 / (height * width))
    th, tw = int(math.floor(factor * height / side)) * side, int(math.floor(factor * width / side)) * side
    if th == 0 and tw == 0:
        raise ValueError("the image would be resized to 0 x 0")
    longest = (max_patches // pooling ** 2) * side
    if th == 0:
        th, tw = side, min(int(math.floor(width / height)) * side, longest)
    elif tw == 0:
        tw, th = side, min(int(math.floor(height / width)) * side, longest)
    if th * tw > max_patches * patch_size ** 2:
        raise ValueError("resized image exceeds the patch budget")
    return th, tw


def image_to_patches(image, cfg: Gemma4VisionConfig, max_soft_tokens: int = 280):
    """``media.RgbImage`` -> (patches float32 [N, 3 P^2] in [0, 1], channel-last inside a patch, row-major over the grid;
    positions int64 [N, 2] as (x, y); soft-token count)."""
    from ..media import resize_rgb8_bicubic

    P, kk = cfg.patch_size, cfg.pooling_kernel_size
    H, W = target_size(image.height, image.width, P, max_soft_tokens * kk * kk, kk)
    img = image if (H, W) == (image.height, image.width) else resize_rgb8_bicubic(image, W, H)
    arr = np.asarray(img.pixels, dtype=np.float32) / 255.0                                   # [H, W, 3]
    gh, gw = H // P, W // P
    patches = arr.reshape(gh, P, gw, P, 3).transpose(0, 2, 1, 3, 4).reshape(gh * gw, P * P * 3)
    ys, xs = np.divmod(np.arange(gh * gw), gw)
    return torch.from_numpy(np.ascontiguousarray(patches)), torch.from_numpy(np.stack((xs, ys), -1)), gh * gw // (kk * kk)
