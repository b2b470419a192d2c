"""Qwen3-VL vision side: the image tower, the patch processor and the positions / feature injection of the decoder.

Behavioural counterpart of eredu/src/backend/mlx/architectures/qwen/vl/ (vision tower, MRoPE, DeepStack; the reference
follows the published Qwen3-VL model). Tower: patches ``[C, 2, P, P]`` -> linear patch embedding + bilinearly interpolated
learned position grid -> pre-LayerNorm blocks with 2-D rotary attention inside each image and a GELU MLP -> a merger
that folds each ``merge x merge`` block of patches into one decoder-width vector; selected blocks also feed DeepStack
mergers whose outputs are added to the hidden states of the first decoder layers at the image positions.

The tower is tensor operations on the model's device (its GEMMs are small and run once per image); the decoder part
reuses the Qwen3 / Qwen3-MoE path with three-axis rotary positions for prompts that contain images.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn.functional as F


@dataclass
class VisionConfig:
    depth: int = 27
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 3584
    num_position_embeddings: int = 2304
    deepstack_visual_indexes: tuple = (8, 16, 24)
    hidden_act: str = "gelu_pytorch_tanh"

    @classmethod
    def from_dict(cls, d: dict) -> "VisionConfig":
        known = {k: d[k] for k in cls.__dataclass_fields__ if k in d}
        # a configuration that does not name DeepStack taps has none (the Qwen3.5 tower: patch embedding, blocks, one
        # merger); Qwen3-VL configurations always carry the list
        known["deepstack_visual_indexes"] = tuple(known.get("deepstack_visual_indexes") or ())
        return cls(**known)


def _act(name: str):
    if name in ("gelu_pytorch_tanh", "gelu_tanh"):
        return lambda t: F.gelu(t, approximate="tanh")
    if name == "gelu":
        return F.gelu
    if name in ("silu", "swish"):
        return F.silu
    raise ValueError(f"unsupported vision activation {name!r}")


class VisionTower:
    """Weights + forward of the image tower (inference only, explicit tensors)."""

    def __init__(self, cfg: VisionConfig, get, device="cpu", dtype=torch.float32, prefix="model.visual."):
        self.cfg = cfg
        self.device, self.dtype = torch.device(device), dtype
        up = lambda n: get(prefix + n).to(device=self.device, dtype=dtype).contiguous()      # noqa: E731
        self.patch_w = up("patch_embed.proj.weight").reshape(cfg.hidden_size, -1)
        self.patch_b = up("patch_embed.proj.bias")
        self.pos_embed = up("pos_embed.weight")
        self.blocks = []
        for i in range(cfg.depth):
            b = f"blocks.{i}."
            self.blocks.append({k: up(b + k) for k in (
                "norm1.weight", "norm1.bias", "norm2.weight", "norm2.bias", "attn.qkv.weight", "attn.qkv.bias", "attn.proj.weight",
                "attn.proj.bias", "mlp.linear_fc1.weight", "mlp.linear_fc1.bias", "mlp.linear_fc2.weight", "mlp.linear_fc2.bias")})
        merger = lambda p: {k: up(p + k) for k in ("norm.weight", "norm.bias", "linear_fc1.weight", "linear_fc1.bias",   # noqa: E731
                                                    "linear_fc2.weight", "linear_fc2.bias")}
        self.merger = merger("merger.")
        self.deepstack = [merger(f"deepstack_merger_list.{i}.") for i in range(len(cfg.deepstack_visual_indexes))]
        self.act = _act(cfg.hidden_act)

    # ---- positions
    def _block_order_coords(self, h: int, w: int):
        """(row, col) of every patch of an h x w grid in merge-block order: blocks row-major, patches inside a block
        row-major."""
        m = self.cfg.spatial_merge_size
        rows = torch.arange(h, device=self.device).view(h // m, m, 1, 1).expand(h // m, m, w // m, m)
        cols = torch.arange(w, device=self.device).view(1, 1, w // m, m).expand(h // m, m, w // m, m)
        order = (0, 2, 1, 3)
        return rows.permute(order).reshape(-1), cols.permute(order).reshape(-1)

    def _pos_embed(self, grids) -> torch.Tensor:
        side = int(self.cfg.num_position_embeddings ** 0.5)
        table = self.pos_embed.view(side, side, -1)
        out = []
        for t, h, w in grids:
            ys = torch.linspace(0, side - 1, h, device=self.device)
            xs = torch.linspace(0, side - 1, w, device=self.device)
            y0, x0 = ys.floor().long(), xs.floor().long()
            y1, x1 = (y0 + 1).clamp(max=side - 1), (x0 + 1).clamp(max=side - 1)
            dy, dx = (ys - y0).to(self.dtype)[:, None, None], (xs - x0).to(self.dtype)[None, :, None]
            grid = (table[y0][:, x0] * (1 - dy) * (1 - dx) + table[y0][:, x1] * (1 - dy) * dx
                    + table[y1][:, x0] * dy * (1 - dx) + table[y1][:, x1] * dy * dx)             # [h, w, hidden]
            r, c = self._block_order_coords(h, w)
            out.append(grid[r, c].repeat(t, 1))
        return torch.cat(out, 0)

    def _rotary(self, grids):
        hd = self.cfg.hidden_size // self.cfg.num_heads
        inv = 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, dtype=torch.float32, device=self.device) / (hd // 2)))
        parts = []
        for t, h, w in grids:
            r, c = self._block_order_coords(h, w)
            f = torch.cat((r.float()[:, None] * inv[None, :], c.float()[:, None] * inv[None, :]), -1)   # [h*w, hd/2]
            parts.append(f.repeat(t, 1))
        f = torch.cat(parts, 0)
        emb = torch.cat((f, f), -1)
        return emb.cos(), emb.sin()

    # ---- forward
    @torch.no_grad()
    def forward(self, patches: torch.Tensor, grids):
        """patches [N, C * Tp * P * P] in merge-block order; grids: list of (t, h, w) patch counts per image.
        Returns (features [N / merge^2, out_hidden], DeepStack features list of the same shape)."""
        cfg = self.cfg
        x = F.linear(patches.to(self.device, self.dtype), self.patch_w, self.patch_b) + self._pos_embed(grids)
        cos, sin = self._rotary(grids)
        cos, sin = cos[:, None, :].to(self.dtype), sin[:, None, :].to(self.dtype)
        H, hd = cfg.num_heads, cfg.hidden_size // cfg.num_heads
        lengths = [h * w for t, h, w in grids for _ in range(t)]
        deep = []
        for i, b in enumerate(self.blocks):
            y = F.layer_norm(x, (cfg.hidden_size,), b["norm1.weight"], b["norm1.bias"], 1e-6)
            qkv = F.linear(y, b["attn.qkv.weight"], b["attn.qkv.bias"]).view(-1, 3, H, hd)
            q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]

            def rot(t):
                half = hd // 2
                return t * cos + torch.cat((-t[..., half:], t[..., :half]), -1) * sin

            q, k = rot(q), rot(k)
            outs, s0 = [], 0
            for n in lengths:      # attention never crosses an image (or a frame)
                a = F.scaled_dot_product_attention(q[s0:s0 + n].transpose(0, 1)[None], k[s0:s0 + n].transpose(0, 1)[None],
                                                   v[s0:s0 + n].transpose(0, 1)[None])[0]
                outs.append(a.transpose(0, 1).reshape(n, H * hd))
                s0 += n
            x = x + F.linear(torch.cat(outs, 0), b["attn.proj.weight"], b["attn.proj.bias"])
            y = F.layer_norm(x, (cfg.hidden_size,), b["norm2.weight"], b["norm2.bias"], 1e-6)
            x = x + F.linear(self.act(F.linear(y, b["mlp.linear_fc1.weight"], b["mlp.linear_fc1.bias"])),
                             b["mlp.linear_fc2.weight"], b["mlp.linear_fc2.bias"])
            if i in cfg.deepstack_visual_indexes:
                deep.append(self._merge(self.deepstack[cfg.deepstack_visual_indexes.index(i)], x, post_shuffle=True))
        return self._merge(self.merger, x, post_shuffle=False), deep

    def _merge(self, w, x, post_shuffle: bool):
        cfg = self.cfg
        wide = cfg.hidden_size * cfg.spatial_merge_size ** 2
        if post_shuffle:
            y = F.layer_norm(x.reshape(-1, wide), (wide,), w["norm.weight"], w["norm.bias"], 1e-6)
        else:
            y = F.layer_norm(x, (cfg.hidden_size,), w["norm.weight"], w["norm.bias"], 1e-6).reshape(-1, wide)
        return F.linear(F.gelu(F.linear(y, w["linear_fc1.weight"], w["linear_fc1.bias"])), w["linear_fc2.weight"],
                        w["linear_fc2.bias"])


# ---------------------------------------------------------------------------------------------- processor
def smart_resize(height: int, width: int, factor: int, min_pixels: int, max_pixels: int) -> tuple[int, int]:
    """Target size: both sides multiples of ``factor``, area within [min_pixels, max_pixels], aspect kept as far as the
    rounding allows."""
    if max(height, width) / min(height, width) > 200:
        raise ValueError("aspect ratio must be below 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def image_to_patches(image, cfg: VisionConfig, min_pixels: int = 64 * 32 * 32, max_pixels: int = 16384 * 32 * 32,
                     mean=(0.5, 0.5, 0.5), std=(0.5, 0.5, 0.5)):
    """RgbImage -> (patches float32 [N, C * Tp * P * P] in merge-block order, (1, h_patches, w_patches))."""
    from ..media import rescale_and_normalize_rgb8, resize_rgb8_bicubic

    P, m, Tp = cfg.patch_size, cfg.spatial_merge_size, cfg.temporal_patch_size
    H, W = smart_resize(image.height, image.width, P * m, min_pixels, max_pixels)
    norm = rescale_and_normalize_rgb8(resize_rgb8_bicubic(image, W, H), 1.0 / 255.0, mean, std).data     # [C, H, W]
    frames = np.repeat(norm[None], Tp, axis=0)                                                            # a still image fills the temporal patch
    gh, gw = H // P, W // P
    C = norm.shape[0]
    x = frames.reshape(1, Tp, C, gh // m, m, P, gw // m, m, P)
    x = x.transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)              # (t, block row, block col, in-block row, in-block col, C, Tp, P, P)
    return torch.from_numpy(np.ascontiguousarray(x).reshape(gh * gw, C * Tp * P * P)), (1, gh, gw)


def video_to_patches(video, cfg: VisionConfig, target_fps: float = 2.0, min_frames: int = 4, max_frames: int = 768,
                     min_pixels: int = 128 * 32 * 32, max_pixels: int = 768 * 32 * 32, mean=(0.5, 0.5, 0.5), std=(0.5, 0.5, 0.5)):
    """``media.Video`` -> (patches [t * gh * gw, C * Tp * P * P] in merge-block order per temporal group, (t, gh, gw),
    timestamps): frames are sampled uniformly at ``target_fps`` (between ``min_frames`` and ``max_frames``), padded by
    repeating the last one to whole temporal patches, resized together (the pixel budget is per frame) and grouped
    ``temporal_patch_size`` at a time; every group gets the mean time of its first and last frame
    (eredu/src/backend/mlx/architectures/qwen/vl/ video preparation; runtime/media/video.rs for the sampling rules)."""
    from ..media import rescale_and_normalize_rgb8, resize_rgb8_bicubic
    from ..media.video import pad_frame_indices, sampled_frame_count, temporal_group_timestamps, uniform_sample_indices

    P, m, Tp = cfg.patch_size, cfg.spatial_merge_size, cfg.temporal_patch_size
    total = len(video.frames)
    count = sampled_frame_count(total, video.fps, target_fps, min(min_frames, total), max_frames)
    indices = pad_frame_indices(uniform_sample_indices(total, count), Tp)
    stamps = temporal_group_timestamps(indices, video.fps, Tp)
    first = video.frames[0]
    H, W = smart_resize(first.height, first.width, P * m, min_pixels, max_pixels)
    frames = np.stack([rescale_and_normalize_rgb8(resize_rgb8_bicubic(video.frames[i], W, H), 1.0 / 255.0, mean, std).data
                       for i in indices])                                                     # [T, C, H, W]
    t, gh, gw = len(indices) // Tp, H // P, W // P
    C = frames.shape[1]
    x = frames.reshape(t, Tp, C, gh // m, m, P, gw // m, m, P)
    x = x.transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)
    return torch.from_numpy(np.ascontiguousarray(x).reshape(t * gh * gw, C * Tp * P * P)), (t, gh, gw), stamps


# ---------------------------------------------------------------------------------------------- decoder positions
def mrope_positions(token_ids, image_token_id, grids, merge: int):
    """Three-axis (t, h, w) rotary positions of a prompt whose image placeholders are runs of ``image_token_id`` (an id,
    or several: a video contributes one (1, h, w) grid per temporal group, each a run of the video placeholder):
    text tokens advance all three axes together; an image of t x (h/merge) x (w/merge) merged tokens keeps t at the
    run's start and spreads h and w over its grid; the next text token continues after the largest position used.
    Returns (positions int64 [3, T], delta) where a later decode token at index i has position i + delta on all axes."""
    pos = torch.zeros((3, len(token_ids)), dtype=torch.int64)
    i, nxt, g = 0, 0, 0
    T = len(token_ids)
    marks = {int(image_token_id)} if isinstance(image_token_id, int) else {int(x) for x in image_token_id}
    while i < T:
        if token_ids[i] in marks:
            t, h, w = grids[g]
            g += 1
            hh, ww = h // merge, w // merge
            n = t * hh * ww
            if token_ids[i:i + n] != [token_ids[i]] * n:
                raise ValueError("image placeholder run does not match the image grid")
            tt = torch.arange(t).view(t, 1, 1).expand(t, hh, ww).reshape(-1)
            ys = torch.arange(hh).view(1, hh, 1).expand(t, hh, ww).reshape(-1)
            xs = torch.arange(ww).view(1, 1, ww).expand(t, hh, ww).reshape(-1)
            pos[:, i:i + n] = torch.stack((tt, ys, xs)) + nxt
            nxt = int(pos[:, i:i + n].max()) + 1
            i += n
        else:
            pos[:, i] = nxt
            nxt += 1
            i += 1
    return pos, nxt - T
