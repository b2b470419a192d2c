"""Muse-Glimmer vision tower, adapter and language projection, with the family's image / video processor.

Behavioural counterpart of eredu/src/backend/mlx/architectures/muse_glimmer/vision.rs and processor.rs:

* processor (processor.rs:334-500): the image is resized (Lanczos-3) to a grid of ``patch_size * merge_size`` cells chosen
  from the floor / ceil candidates of the ideal grid under the token budget, closest to the source aspect ratio; rescaled,
  normalised; patches are emitted in raster order, each ``[temporal, channel, y, x]`` with a still image repeated over the
  temporal extent. A video is sampled, padded to whole temporal groups, and every group becomes a part of its own.
* tower (vision.rs:377-647): linear patch embedding plus a learned position table read by bilinear interpolation
  (half-pixel centres, out-of-table corners weigh nothing); LayerNorm before and after the blocks; blocks are pre-norm
  attention (biased q / k / v / output projections, two-axis rotary embedding with 1-based coordinates laid out
  ``[w, h, w, h]`` over the head) and a GELU feed-forward. ``layer_types`` says which blocks attend inside square windows
  of ``pos_emb_height`` patches and which over the whole frame; tokens are kept in window order between the first and the
  last block so that every window is one contiguous run.
* head (vision.rs:625-647): ``merge_size x merge_size`` neighbourhoods are folded channel-major into one row, two GELU
  layers (the adapter), a projection to the decoder's width and a weight-free RMSNorm (eps 1e-5): the rows replace the
  normalised embeddings of the image placeholder tokens.

The GEMMs are this repository's (``ops.linear``); attention runs per window / frame through the fused SDPA of the tensor
library on bf16 and through plain fp32 matmuls on CPU. Not built: tensor parallelism of the tower, the collapsed-temporal
projector of the GGUF release.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

from .. import ops
from ..media import RgbImage, rescale_and_normalize_rgb8, resize_rgb8_lanczos3
from ..media.image import MediaError
from ..media.video import pad_frame_indices, uniform_sample_indices, validate_rgb_frames


# ------------------------------------------------------------------------------------------------- processor
@dataclass
class MuseVisualProcessorConfig:
    do_resize: bool = True
    do_rescale: bool = True
    rescale_factor: float = 1.0 / 255.0
    do_normalize: bool = True
    image_mean: tuple = (0.5, 0.5, 0.5)
    image_std: tuple = (0.5, 0.5, 0.5)
    patch_size: int = 14
    temporal_patch_size: int = 2
    merge_size: int = 2
    max_image_tokens: int = 4096
    max_video_frame_tokens: int = 144
    num_frames: int = 96
    fps: float = 2.0
    do_sample_frames: bool = True
    resample: int = 1

    @classmethod
    def from_dict(cls, d: dict, kind: str = "image") -> "MuseVisualProcessorConfig":
        d = dict(d or {})
        if "patch_temporal" in d and "temporal_patch_size" not in d:
            d["temporal_patch_size"] = d["patch_temporal"]
        known = {k: d[k] for k in cls.__dataclass_fields__ if k in d}
        c = cls(**known)
        if min(c.patch_size, c.temporal_patch_size, c.merge_size, c.max_image_tokens, c.max_video_frame_tokens) <= 0:
            raise ValueError(f"Muse-Glimmer {kind} processor dimensions and token limits must be positive")
        if int(c.resample) != 1:
            raise ValueError(f"Muse-Glimmer {kind} processor requires Lanczos resample mode 1, got {c.resample}")
        return c


def load_processor(model_dir) -> tuple:
    """(image config, video config) from ``processor_config.json``; defaults when the file is absent."""
    p = Path(model_dir) / "processor_config.json"
    if not p.exists():
        return MuseVisualProcessorConfig(), MuseVisualProcessorConfig()
    raw = json.loads(p.read_text())
    return (MuseVisualProcessorConfig.from_dict(raw.get("image_processor"), "image"),
            MuseVisualProcessorConfig.from_dict(raw.get("video_processor"), "video"))


def smart_resize(height: int, width: int, cell: int, max_tokens: int) -> tuple:
    """Target (height, width): whole cells, at most ``max_tokens`` of them, aspect ratio as close to the source as the
    floor / ceil candidates allow (first candidate wins ties: rows floor-first, then columns floor-first)."""
    if min(height, width, cell, max_tokens) <= 0:
        raise MediaError("Muse-Glimmer smart resize requires positive dimensions")
    ih, iw = height / cell, width / cell
    ratio = iw / ih
    if ih * iw > max_tokens:
        ih = math.sqrt(max_tokens / ratio)
        iw = ih * ratio
    cands = []
    for h in (math.floor(ih), math.ceil(ih)):
        for w in (math.floor(iw), math.ceil(iw)):
            if h > 0 and w > 0 and h * w <= max_tokens and (h, w) not in cands:
                cands.append((h, w))
    if not cands:
        cands.append((max(int(round(ih)), 1), max(int(round(iw)), 1)))
    src = height / width
    best = min(cands, key=lambda c: abs(c[0] / c[1] - src))      # min() keeps the first of equal keys
    return best[0] * cell, best[1] * cell


def _normalised(image: RgbImage, target: tuple, cfg: MuseVisualProcessorConfig) -> np.ndarray:
    h, w = target if cfg.do_resize else (image.height, image.width)
    resized = resize_rgb8_lanczos3(image, w, h)
    mean, std = (cfg.image_mean, cfg.image_std) if cfg.do_normalize else ((0.0,) * 3, (1.0,) * 3)
    return rescale_and_normalize_rgb8(resized, cfg.rescale_factor if cfg.do_rescale else 1.0, mean, std).data   # [3, H, W]


def pack_patches(frames: list, cfg: MuseVisualProcessorConfig, duplicate_image: bool) -> tuple:
    """Normalised frames ``[3, H, W]`` -> (patches fp32 [gh * gw, T * 3 * P * P], grid (1, gh, gw)); a still image
    (``duplicate_image``) fills every temporal slice."""
    if not frames:
        raise MediaError("Muse-Glimmer patch input is empty")
    P, T = cfg.patch_size, cfg.temporal_patch_size
    C, H, W = frames[0].shape
    if H % P or W % P:
        raise MediaError(f"Muse-Glimmer processed media {W}x{H} is not divisible by patch size {P}")
    if any(f.shape != frames[0].shape for f in frames):
        raise MediaError("Muse-Glimmer video frames must have identical dimensions")
    if not duplicate_image and len(frames) != T:
        raise MediaError(f"Muse-Glimmer video group has {len(frames)} frames, expected {T}")
    stack = np.stack([frames[0]] * T if duplicate_image else frames)                      # [T, C, H, W]
    gh, gw = H // P, W // P
    x = stack.reshape(T, C, gh, P, gw, P).transpose(2, 4, 0, 1, 3, 5).reshape(gh * gw, T * C * P * P)
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)), (1, gh, gw)


def image_to_patches(image: RgbImage, cfg: MuseVisualProcessorConfig) -> tuple:
    target = smart_resize(image.height, image.width, cfg.patch_size * cfg.merge_size, cfg.max_image_tokens)
    return pack_patches([_normalised(image, target, cfg)], cfg, True)


def video_to_groups(video, cfg: MuseVisualProcessorConfig, frame_count=None) -> list:
    """One (seconds, patches, grid) per temporal group of a ``media.request.Video`` (processor.rs:236-310): frames are
    sampled at the processor's rate (or ``frame_count`` of them), the count is rounded down to whole groups (at least
    one), the last frame repeats to fill the final group; a group's time is its first sampled frame's."""
    validate_rgb_frames(video.frames)
    total, T = len(video.frames), cfg.temporal_patch_size
    if frame_count is not None:
        want = min(int(frame_count), total)
    elif cfg.do_sample_frames:
        want = min(int(total * cfg.fps / video.fps), cfg.num_frames, total)
    else:
        want = total
    want = max(want, T) // T * T
    idx = uniform_sample_indices(total, max(min(want, total), 1))
    padded = pad_frame_indices(idx, T)
    first = video.frames[0]
    target = smart_resize(first.height, first.width, cfg.patch_size * cfg.merge_size, cfg.max_video_frame_tokens)
    frames = [_normalised(video.frames[i], target, cfg) for i in padded]
    out = []
    for g in range(len(frames) // T):
        src = idx[g * T] if g * T < len(idx) else idx[-1]
        patches, grid = pack_patches(frames[g * T:(g + 1) * T], cfg, False)
        out.append((src / video.fps, patches, grid))
    return out


# ------------------------------------------------------------------------------------------------- geometry
def window_order(grids: list, window: int) -> tuple:
    """Permutation that lists the patches window by window (square windows of ``window`` patches, raster order of
    windows inside a frame and of patches inside a window) and the length of every non-empty window."""
    if window <= 0:
        raise ValueError("the attention window must hold at least one patch")
    index, lengths, base = [], [], 0
    for t, h, w in grids:
        for f in range(t):
            for wy in range(0, h, window):
                for wx in range(0, w, window):
                    ys, xs = range(wy, min(wy + window, h)), range(wx, min(wx + window, w))
                    index.extend(base + f * h * w + y * w + x for y in ys for x in xs)
                    lengths.append(len(ys) * len(xs))
        base += t * h * w
    return index, lengths


def interpolation_plan(grids: list, side_h: int, side_w: int) -> tuple:
    """Four table rows and weights per patch: bilinear read of the ``side_h x side_w`` position table at the patch's
    centre in table coordinates; corners outside the table keep a clamped index and weight 0."""
    idx, wts = [], []
    for t, h, w in grids:
        gy = (np.arange(h, dtype=np.float32) + np.float32(0.5)) * np.float32(side_h) / np.float32(h) - np.float32(0.5)
        gx = (np.arange(w, dtype=np.float32) + np.float32(0.5)) * np.float32(side_w) / np.float32(w) - np.float32(0.5)
        y0, x0 = np.floor(gy).astype(np.int64), np.floor(gx).astype(np.int64)
        yf, xf = (gy - y0).astype(np.float32), (gx - x0).astype(np.float32)
        fi, fw = [], []
        for dy, dx in ((0, 0), (0, 1), (1, 0), (1, 1)):
            yy, xx = (y0 + dy)[:, None], (x0 + dx)[None, :]
            wy, wx = (yf if dy else 1 - yf)[:, None], (xf if dx else 1 - xf)[None, :]
            ok = (yy >= 0) & (yy < side_h) & (xx >= 0) & (xx < side_w)
            fi.append((np.clip(yy, 0, side_h - 1) * side_w + np.clip(xx, 0, side_w - 1)).reshape(-1))
            fw.append(np.where(ok, wy * wx, 0.0).astype(np.float32).reshape(-1))
        fi, fw = np.stack(fi, 1), np.stack(fw, 1)                                           # [h * w, 4]
        idx.extend([fi] * t)
        wts.extend([fw] * t)
    return torch.from_numpy(np.concatenate(idx)), torch.from_numpy(np.concatenate(wts))


def rotary_tables(grids: list, head_dim: int, theta: float) -> tuple:
    """cos / sin [patches, head_dim]: angles of the 1-based column then row coordinate over ``head_dim / 4`` frequencies
    each, the pair repeated to fill the head (``[w, h, w, h]``)."""
    spatial = head_dim // 2
    if spatial % 2:
        raise ValueError("Muse-Glimmer vision RoPE spatial dimension must be even")
    inv = 1.0 / (theta ** (torch.arange(0, spatial, 2, dtype=torch.float32) / spatial))
    rows = []
    for t, h, w in grids:
        fw = (torch.arange(1, w + 1, dtype=torch.float32)[:, None] * inv)[None, :, :].expand(h, w, -1)
        fh = (torch.arange(1, h + 1, dtype=torch.float32)[:, None] * inv)[:, None, :].expand(h, w, -1)
        ang = torch.cat((fw, fh, fw, fh), -1).reshape(h * w, head_dim)
        rows.extend([ang] * t)
    ang = torch.cat(rows)
    return ang.cos(), ang.sin()


def fold_neighbourhoods(x: torch.Tensor, grids: list, m: int) -> torch.Tensor:
    """[patches, C] -> [patches / m^2, C * m^2]: every ``m x m`` neighbourhood becomes one row, channel-major (channel c
    of the neighbourhood's cells sits at columns ``c * m^2 ...``)."""
    out, off = [], 0
    for t, h, w in grids:
        n = t * h * w
        c = x[off:off + n].view(t, h // m, m, w // m, m, -1)                     # t, oy, iy, ox, ix, C
        out.append(c.permute(0, 1, 3, 5, 2, 4).reshape(t * (h // m) * (w // m), -1))
        off += n
    return torch.cat(out)


# ------------------------------------------------------------------------------------------------- tower
@dataclass
class MuseVisionConfig:
    hidden_size: int
    intermediate_size: int
    num_heads: int
    patch_size: int
    temporal_patch_size: int
    merge_size: int
    pos_height: int
    pos_width: int
    layer_norm_eps: float
    rope_theta: float
    windowed: list = field(default_factory=list)        # per block: True = window attention
    language_hidden_size: int = 0
    projector_hidden_size: int = 4096

    @classmethod
    def from_dict(cls, d: dict, language_hidden_size: int, projector_hidden_size: int = 4096) -> "MuseVisionConfig":
        if d.get("model_type") != "muse_glimmer_vision":
            raise ValueError(f"Muse-Glimmer vision model_type must be muse_glimmer_vision, got {d.get('model_type')!r}")
        H, I, nh = int(d["hidden_size"]), int(d["intermediate_size"]), int(d["num_attention_heads"])
        P, T, m = int(d["patch_size"]), int(d["patch_temporal"]), int(d["merge_size"])
        ph, pw = int(d["pos_emb_height"]), int(d["pos_emb_width"])
        eps = float(d["layer_norm_eps"])
        if (d.get("hidden_act") != "gelu" or min(H, I, nh, P, T, m, ph, pw) <= 0 or H % nh or eps <= 0
                or ph * pw != int(d["max_position_embeddings"])):
            raise ValueError("Muse-Glimmer vision geometry or activation is invalid")
        kinds = list(d["layer_types"])
        if int(d["num_hidden_layers"]) <= 0 or len(kinds) != int(d["num_hidden_layers"]):
            raise ValueError(f"Muse-Glimmer vision layer_types has {len(kinds)} entries, expected {d['num_hidden_layers']}")
        bad = [k for k in kinds if k not in ("window_attention", "full_attention")]
        if bad:
            raise ValueError(f"Muse-Glimmer vision has unsupported layer type {bad[0]!r}")
        rp = d.get("rope_parameters") or {}
        theta = float(rp.get("rope_theta") or 0.0)
        if not (math.isfinite(theta) and theta > 0):
            raise ValueError("Muse-Glimmer vision rope_parameters.rope_theta must be positive")
        if rp.get("rope_type") != "default":
            raise ValueError("Muse-Glimmer vision supports only default 2-D RoPE")
        return cls(H, I, nh, P, T, m, ph, pw, eps, theta, [k == "window_attention" for k in kinds],
                   int(language_hidden_size), int(projector_hidden_size))


class MuseGlimmerVision:
    """``(patches [N, T * 3 * P * P], grids [(t, h, w), ...]) -> [sum t * h/m * w/m, language_hidden]``."""

    def __init__(self, cfg: MuseVisionConfig, get, has, device="cpu", dtype=torch.float32, prefix: str = "model."):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        up = lambda n, dt=None: get(prefix + n).to(device=self.device, dtype=dt or dtype).contiguous()     # noqa: E731
        opt = lambda n: up(n) if has(prefix + n) else None                                                  # noqa: E731
        H, m = cfg.hidden_size, cfg.merge_size
        self.patch_w = up("vision_tower.patch_embedder.patch_embedding.weight")
        if tuple(self.patch_w.shape) != (H, cfg.temporal_patch_size * 3 * cfg.patch_size ** 2):
            raise ValueError(f"patch embedding has shape {tuple(self.patch_w.shape)}")
        self.pos_table = up("vision_tower.patch_embedder.position_embedding_table.weight", torch.float32)
        if self.pos_table.shape[0] != cfg.pos_height * cfg.pos_width:
            raise ValueError("the position table does not match pos_emb_height x pos_emb_width")
        ln = lambda n: (up(n + ".weight", torch.float32), up(n + ".bias", torch.float32))                   # noqa: E731
        self.ln_pre, self.ln_post = ln("vision_tower.ln_pre"), ln("vision_tower.ln_post")
        self.blocks = []
        for i in range(len(cfg.windowed)):
            b = f"vision_tower.layers.{i}."
            w = {"norm1": ln(b + "norm1"), "norm2": ln(b + "norm2")}
            # one GEMM for q, k and v
            w["qkv"] = torch.cat([up(b + f"attn.{n}.weight") for n in ("q_proj", "k_proj", "v_proj")], 0).contiguous()
            biases = [opt(b + f"attn.{n}.bias") for n in ("q_proj", "k_proj", "v_proj")]
            w["qkv_b"] = torch.cat([x if x is not None else torch.zeros(H, device=self.device, dtype=dtype) for x in biases]) \
                if any(x is not None for x in biases) else None
            for n, key in (("attn.proj", "proj"), ("mlp.fc1", "fc1"), ("mlp.fc2", "fc2")):
                w[key], w[key + "_b"] = up(b + n + ".weight"), opt(b + n + ".bias")
            self.blocks.append(w)
        self.fc1, self.fc2 = up("vision_adapter.fc1.weight"), up("vision_adapter.fc2.weight")
        self.proj = up("vision_projection.weight")
        if self.fc1.shape[1] != H * m * m or self.proj.shape[0] != cfg.language_hidden_size:
            raise ValueError("the vision adapter does not match the tower / decoder widths")

    def _ln(self, x, wb):
        return F.layer_norm(x.float(), (x.shape[-1],), wb[0], wb[1], self.cfg.layer_norm_eps).to(self.dtype)

    def _attention(self, w, x, lengths, cos, sin):
        cfg = self.cfg
        N, nh = x.shape[0], cfg.num_heads
        D = cfg.hidden_size // nh
        qkv = ops.linear(x, w["qkv"], bias=w["qkv_b"]).view(N, 3, nh, D)
        half = D // 2

        def rot(t):
            t = t.float()
            return (t * cos[:, None, :] + torch.cat((-t[..., half:], t[..., :half]), -1) * sin[:, None, :]).to(self.dtype)

        q, k, v = rot(qkv[:, 0]), rot(qkv[:, 1]), qkv[:, 2]
        out = torch.empty((N, nh, D), dtype=self.dtype, device=x.device)
        # runs of equal length attend as one batch
        start, runs = 0, {}
        for n in lengths:
            runs.setdefault(n, []).append(start)
            start += n
        if start != N:
            raise ValueError(f"Muse-Glimmer vision chunks cover {start} tokens, expected {N}")
        for n, starts in runs.items():
            rows = (torch.tensor(starts, device=x.device)[:, None] + torch.arange(n, device=x.device)[None, :]).reshape(-1)
            take = lambda t: t[rows].view(len(starts), n, nh, D).transpose(1, 2)             # noqa: E731
            o = F.scaled_dot_product_attention(take(q), take(k), take(v), scale=D ** -0.5)
            out[rows] = o.transpose(1, 2).reshape(-1, nh, D)
        return ops.linear(out.view(N, nh * D), w["proj"], bias=w["proj_b"])

    @torch.no_grad()
    def __call__(self, patches: torch.Tensor, grids: list) -> torch.Tensor:
        cfg = self.cfg
        grids = [tuple(int(v) for v in g) for g in grids]
        if not grids or any(min(g) <= 0 or g[1] % cfg.merge_size or g[2] % cfg.merge_size for g in grids):
            raise ValueError("Muse-Glimmer vision grid must be positive and spatially divisible by merge_size")
        if patches.dim() != 2 or patches.shape[1] != self.patch_w.shape[1]:
            raise ValueError(f"Muse-Glimmer vision pixels must be shaped [patches, {self.patch_w.shape[1]}], got {tuple(patches.shape)}")
        if sum(t * h * w for t, h, w in grids) != patches.shape[0]:
            raise ValueError(f"Muse-Glimmer vision grid describes {sum(t * h * w for t, h, w in grids)} patches, tensor has {patches.shape[0]}")
        dev = self.device
        x = ops.linear(patches.to(dev, self.dtype).contiguous(), self.patch_w)
        pi, pw = interpolation_plan(grids, cfg.pos_height, cfg.pos_width)
        pos = (self.pos_table[pi.to(dev)] * pw.to(dev)[..., None]).sum(1)
        x = self._ln(x.float() + pos, self.ln_pre)
        order, win_lengths = window_order(grids, cfg.pos_height)
        full_lengths = [h * w for t, h, w in grids for _ in range(t)]
        order_t = torch.tensor(order, device=dev)
        cos, sin = rotary_tables(grids, cfg.hidden_size // cfg.num_heads, cfg.rope_theta)
        cos, sin = cos.to(dev)[order_t], sin.to(dev)[order_t]
        x = x[order_t]
        # in window order a frame is still one contiguous run (its windows follow each other), so both kinds of block use
        # the same token order
        for w, windowed in zip(self.blocks, cfg.windowed):
            x = x + self._attention(w, self._ln(x, w["norm1"]), win_lengths if windowed else full_lengths, cos, sin)
            y = F.gelu(ops.linear(self._ln(x, w["norm2"]), w["fc1"], bias=w["fc1_b"]).float()).to(self.dtype)
            x = x + ops.linear(y, w["fc2"], bias=w["fc2_b"])
        back = torch.empty_like(order_t)
        back[order_t] = torch.arange(order_t.numel(), device=dev)
        x = self._ln(x[back], self.ln_post)
        x = fold_neighbourhoods(x, grids, cfg.merge_size).contiguous()
        x = F.gelu(ops.linear(x, self.fc1).float()).to(self.dtype)
        x = F.gelu(ops.linear(x, self.fc2).float()).to(self.dtype)
        x = ops.linear(x, self.proj).float()
        return (x * torch.rsqrt(x.square().mean(-1, keepdim=True) + 1e-5)).to(self.dtype)


def load_muse_glimmer_vision(raw_config: dict, language_hidden_size: int, get, has, device, dtype, prefix: str = "model."):
    """The tower of a checkpoint whose top-level configuration carries ``vision_config`` (and ``projector_hidden_size``)."""
    cfg = MuseVisionConfig.from_dict(raw_config["vision_config"], language_hidden_size,
                                     int(raw_config.get("projector_hidden_size") or 4096))
    out = raw_config.get("out_hidden_size")
    if out is not None and int(out) != cfg.hidden_size:
        raise ValueError("Muse-Glimmer out_hidden_size must equal the vision hidden size")
    return MuseGlimmerVision(cfg, get, has, device, dtype, prefix)
