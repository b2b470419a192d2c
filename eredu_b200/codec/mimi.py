"""Mimi: the streaming neural audio codec of Moshi / PersonaPlex (24 kHz PCM <-> 12.5 Hz frames of residual codebook indices).

Counterpart of the reference's codec crate (eredu-codec/src/mimi.rs:39-105 configuration, :203-266 ``encode`` / ``decode`` /
``encode_step`` / ``decode_step`` / latent entry points, :1392-1640 split residual vector quantiser). Structure::

    pcm -> SEANet encoder (causal convolutions, strides 4-5-6-8) -> transformer (RoPE, sliding window, layer scale)
        -> stride-2 downsampling -> split residual VQ (1 semantic + n acoustic codebooks) -> codes [B, n_q, frames]
    codes -> codebook sums -> depthwise x2 upsampling -> transformer -> SEANet decoder (transposed convolutions) -> pcm

Every operator is causal, so the streaming entry points (``encode_step`` / ``decode_step``: whole frames at a time, state kept
between calls) produce exactly what the one-shot calls produce; ``tests/test_mimi.py`` checks both against Transformers'
``MimiModel`` on the same weights. Tensor names are those of the Hugging Face checkpoint (``kyutai/mimi``).
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

import torch
import torch.nn.functional as F


@dataclass
class MimiConfig:
    sampling_rate: int = 24000
    frame_rate: float = 12.5
    audio_channels: int = 1
    hidden_size: int = 512
    num_filters: int = 64
    num_residual_layers: int = 1
    upsampling_ratios: list = field(default_factory=lambda: [8, 6, 5, 4])
    kernel_size: int = 7
    last_kernel_size: int = 3
    residual_kernel_size: int = 3
    dilation_growth_rate: int = 2
    compress: int = 2
    pad_mode: str = "constant"
    codebook_size: int = 2048
    codebook_dim: int = 256
    num_quantizers: int = 32
    num_semantic_quantizers: int = 1
    vector_quantization_hidden_dimension: int = 256
    upsample_groups: int = 512
    num_hidden_layers: int = 8
    num_attention_heads: int = 8
    num_key_value_heads: int = 8
    head_dim: Optional[int] = None
    intermediate_size: int = 2048
    sliding_window: int = 250
    rope_theta: float = 10000.0
    norm_eps: float = 1e-5
    layer_scale_initial_scale: float = 0.01

    @classmethod
    def v0_1(cls, num_codebooks: Optional[int] = None) -> "MimiConfig":
        """The published 24 kHz / 12.5 Hz model; Moshi uses the first 8 of its 32 codebooks."""
        return cls(num_quantizers=int(num_codebooks or 32))

    @classmethod
    def from_dict(cls, d: dict) -> "MimiConfig":
        known = {f for f in cls.__dataclass_fields__}
        kw = {k: v for k, v in d.items() if k in known and v is not None}
        if "frame_rate" not in kw and d.get("_frame_rate") is not None:
            kw["frame_rate"] = float(d["_frame_rate"])
        rp = d.get("rope_parameters") or {}
        if "rope_theta" in rp:
            kw["rope_theta"] = float(rp["rope_theta"])
        cfg = cls(**kw)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.num_semantic_quantizers >= self.num_quantizers:
            raise ValueError("the semantic codebooks must leave at least one acoustic codebook")
        if self.hidden_size % self.num_attention_heads:
            raise ValueError("hidden_size must be divisible by the number of attention heads")
        hop = self.encoder_hop
        if abs(self.sampling_rate / hop / self.frame_rate - round(self.sampling_rate / hop / self.frame_rate)) > 1e-6:
            raise ValueError("the frame rate must divide the encoder's output rate")

    @property
    def encoder_hop(self) -> int:
        return int(math.prod(self.upsampling_ratios))

    @property
    def downsample_stride(self) -> int:
        return int(round(self.sampling_rate / self.encoder_hop / self.frame_rate))

    @property
    def frame_size(self) -> int:
        """PCM samples per codec frame."""
        return self.encoder_hop * self.downsample_stride

    @property
    def attn_head_dim(self) -> int:
        return self.head_dim or self.hidden_size // self.num_attention_heads


# ---------------------------------------------------------------------------------------------------------------
# Causal convolutions. One-shot calls pad on the left by (effective kernel - stride) and, when the length is not a
# whole number of strides, on the right up to the next one. Streaming calls take whole strides at a time and carry the
# left context (convolution) or the overlapping tail (transposed convolution) between calls.

class _Conv:
    def __init__(self, w, b, stride=1, dilation=1, groups=1, pad_mode="constant"):
        self.w, self.b = w, b
        self.stride, self.dilation, self.groups, self.pad_mode = stride, dilation, groups, pad_mode
        self.k_eff = (w.shape[-1] - 1) * dilation + 1
        self.pad = self.k_eff - stride

    def _left(self, x, n, first):
        if n == 0:
            return x[..., :0]
        if self.pad_mode == "replicate" and first:
            return x[..., :1].expand(*x.shape[:-1], n)
        return x.new_zeros(*x.shape[:-1], n)

    def __call__(self, x, state: Optional[dict] = None, key=None):
        if state is None:
            T = x.shape[-1]
            frames = math.ceil((T - self.k_eff + self.pad) / self.stride + 1) - 1
            extra = max(0, frames * self.stride + self.k_eff - self.pad - T)
            if self.pad_mode == "replicate":
                x = F.pad(x, (self.pad, extra), mode="replicate") if x.shape[-1] > 0 else x
            else:
                x = F.pad(x, (self.pad, extra))
            return F.conv1d(x, self.w, self.b, self.stride, 0, self.dilation, self.groups)
        if x.shape[-1] % self.stride:
            raise ValueError("streaming convolutions take whole strides")
        ctx = state.get(key)
        if ctx is None:
            ctx = self._left(x, self.pad, first=True)
        buf = torch.cat((ctx, x), dim=-1)
        state[key] = buf[..., buf.shape[-1] - self.pad:] if self.pad else buf[..., :0]
        return F.conv1d(buf, self.w, self.b, self.stride, 0, self.dilation, self.groups)


class _ConvTranspose:
    def __init__(self, w, b, stride, groups=1):
        self.w, self.b, self.stride, self.groups = w, b, stride, groups
        self.tail = w.shape[-1] - stride                        # samples of every call that overlap the next one

    def __call__(self, x, state: Optional[dict] = None, key=None):
        y = F.conv_transpose1d(x, self.w, None, self.stride, groups=self.groups)
        n = x.shape[-1] * self.stride
        if state is not None:
            carry = state.get(key)
            if carry is not None and self.tail:
                y = torch.cat((y[..., :self.tail] + carry, y[..., self.tail:]), dim=-1)
            state[key] = y[..., n:]
        y = y[..., :n]                                           # causal: everything that overhangs is trimmed on the right
        return y if self.b is None else y + self.b.view(1, -1, 1)


class _ResBlock:
    """ELU -> dilated convolution to hidden / compress -> ELU -> 1x1 convolution back, plus the identity."""

    def __init__(self, convs):
        self.convs = convs

    def __call__(self, x, state, key):
        h = x
        for j, c in enumerate(self.convs):
            h = c(F.elu(h), state, (key, j))
        return x + h


class _SeaNet:
    """Sequence of convolutions / residual blocks / transposed convolutions with ELU before every strided or final one."""

    def __init__(self, steps):
        self.steps = steps               # list of (kind, module): "conv" | "elu_conv" | "res" | "elu_convtr"

    def __call__(self, x, state: Optional[dict] = None, name=""):
        for i, (kind, mod) in enumerate(self.steps):
            key = (name, i)
            if kind == "res":
                x = mod(x, state, key)
            else:
                x = mod(F.elu(x) if kind.startswith("elu_") else x, state, key)
        return x


def _build_encoder(cfg: MimiConfig, get) -> _SeaNet:
    conv = lambda p, **kw: _Conv(get(p + ".conv.weight"), get(p + ".conv.bias"), pad_mode=cfg.pad_mode, **kw)   # noqa: E731
    steps = [("conv", conv("encoder.layers.0"))]
    idx = 1
    for ratio in reversed(cfg.upsampling_ratios):
        for j in range(cfg.num_residual_layers):
            p = f"encoder.layers.{idx}.block."
            steps.append(("res", _ResBlock([conv(p + "1", dilation=cfg.dilation_growth_rate ** j), conv(p + "3")])))
            idx += 1
        idx += 1                                                  # the ELU occupies an index of its own
        steps.append(("elu_conv", conv(f"encoder.layers.{idx}", stride=ratio)))
        idx += 1
    idx += 1
    steps.append(("elu_conv", conv(f"encoder.layers.{idx}")))
    return _SeaNet(steps)


def _build_decoder(cfg: MimiConfig, get) -> _SeaNet:
    conv = lambda p, **kw: _Conv(get(p + ".conv.weight"), get(p + ".conv.bias"), pad_mode=cfg.pad_mode, **kw)   # noqa: E731
    steps = [("conv", conv("decoder.layers.0"))]
    idx = 1
    for ratio in cfg.upsampling_ratios:
        idx += 1                                                  # ELU
        p = f"decoder.layers.{idx}"
        steps.append(("elu_convtr", _ConvTranspose(get(p + ".conv.weight"), get(p + ".conv.bias"), ratio)))
        idx += 1
        for j in range(cfg.num_residual_layers):
            p = f"decoder.layers.{idx}.block."
            steps.append(("res", _ResBlock([conv(p + "1", dilation=cfg.dilation_growth_rate ** j), conv(p + "3")])))
            idx += 1
    idx += 1
    steps.append(("elu_conv", conv(f"decoder.layers.{idx}")))
    return _SeaNet(steps)


# ---------------------------------------------------------------------------------------------------------------
class _Transformer:
    """Pre-norm transformer over frames [B, T, C]: LayerNorm, rotary causal attention inside a sliding window, GELU
    feed-forward, a learned per-channel scale on both branches. ``state`` holds the keys / values of the window."""

    def __init__(self, cfg: MimiConfig, get, prefix: str):
        self.cfg = cfg
        self.layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"{prefix}.layers.{i}."
            self.layers.append({k: get(p + n) for k, n in (
                ("q", "self_attn.q_proj.weight"), ("k", "self_attn.k_proj.weight"), ("v", "self_attn.v_proj.weight"),
                ("o", "self_attn.o_proj.weight"), ("fc1", "mlp.fc1.weight"), ("fc2", "mlp.fc2.weight"),
                ("ln1_w", "input_layernorm.weight"), ("ln1_b", "input_layernorm.bias"),
                ("ln2_w", "post_attention_layernorm.weight"), ("ln2_b", "post_attention_layernorm.bias"),
                ("s1", "self_attn_layer_scale.scale"), ("s2", "mlp_layer_scale.scale"))})
        D = cfg.attn_head_dim
        self.inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))

    def _rope(self, x, pos):
        ang = pos.to(torch.float32)[:, None] * self.inv_freq.to(x.device)[None, :]          # [T, D/2]
        cos, sin = torch.cat((ang.cos(), ang.cos()), -1), torch.cat((ang.sin(), ang.sin()), -1)
        half = x.shape[-1] // 2
        rot = torch.cat((-x[..., half:], x[..., :half]), -1)
        return (x.float() * cos + rot.float() * sin).to(x.dtype)

    def __call__(self, x, state: Optional[dict] = None, name=""):
        cfg = self.cfg
        B, T, C = x.shape
        Hq, Hkv, D, W = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.attn_head_dim, cfg.sliding_window
        start = 0 if state is None else state.get((name, "pos"), 0)
        pos = torch.arange(start, start + T, device=x.device)
        for li, lw in enumerate(self.layers):
            h = F.layer_norm(x, (C,), lw["ln1_w"], lw["ln1_b"], cfg.norm_eps)
            q = self._rope(F.linear(h, lw["q"]).view(B, T, Hq, D).transpose(1, 2), pos)
            k = self._rope(F.linear(h, lw["k"]).view(B, T, Hkv, D).transpose(1, 2), pos)
            v = F.linear(h, lw["v"]).view(B, T, Hkv, D).transpose(1, 2)
            kpos = pos
            if state is not None:
                old = state.get((name, li))
                if old is not None:
                    k, v, kpos = torch.cat((old[0], k), 2), torch.cat((old[1], v), 2), torch.cat((old[2], pos))
                keep = max(0, k.shape[2] - (W - 1))               # the next query sees at most W - 1 earlier frames
                state[(name, li)] = (k[:, :, keep:], v[:, :, keep:], kpos[keep:])
            if Hkv != Hq:
                k, v = k.repeat_interleave(Hq // Hkv, 1), v.repeat_interleave(Hq // Hkv, 1)
            rel = pos[:, None] - kpos[None, :]
            mask = (rel >= 0) & (rel < W)
            a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
            x = x + lw["s1"] * F.linear(a.transpose(1, 2).reshape(B, T, Hq * D), lw["o"])
            h = F.layer_norm(x, (C,), lw["ln2_w"], lw["ln2_b"], cfg.norm_eps)
            x = x + lw["s2"] * F.linear(F.gelu(F.linear(h, lw["fc1"])), lw["fc2"])
        if state is not None:
            state[(name, "pos")] = start + T
        return x


class _ResidualVQ:
    """``input_proj`` (1x1) -> residual nearest-centroid search over the layers' codebooks; decoding sums the chosen
    centroids and applies ``output_proj``. Centroids are the running sums divided by the running usage counts."""

    def __init__(self, get, prefix: str, n_layers: int, eps: float = 1e-5):
        self.w_in, self.w_out = get(prefix + ".input_proj.weight"), get(prefix + ".output_proj.weight")
        self.books = []
        for i in range(n_layers):
            p = f"{prefix}.layers.{i}.codebook."
            self.books.append(get(p + "embed_sum") / get(p + "cluster_usage").clamp(min=eps)[:, None])

    def encode(self, x, n: Optional[int] = None):
        r = F.conv1d(x, self.w_in).transpose(1, 2)                                    # [B, T, d]
        out = []
        for book in self.books[:n]:
            idx = torch.cdist(r.float(), book.float()[None]).argmin(-1)
            r = r - book[idx]
            out.append(idx)
        return torch.stack(out, 1)                                                    # [B, n, T]

    def decode(self, codes):
        q = sum(self.books[i][codes[:, i]] for i in range(codes.shape[1]))           # [B, T, d]
        return F.conv1d(q.transpose(1, 2), self.w_out)


# ---------------------------------------------------------------------------------------------------------------
class Mimi:
    """The codec. ``encode`` / ``decode`` work on whole clips; ``encode_step`` / ``decode_step`` on whole frames with
    state carried between calls (``reset_encode_state`` / ``reset_decode_state`` start a new stream)."""

    def __init__(self, cfg: MimiConfig, get, device="cpu", dtype=torch.float32):
        cfg.validate()
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        cache: dict = {}

        def fetch(name):
            if name not in cache:
                cache[name] = get(name).to(device=self.device, dtype=dtype).contiguous()
            return cache[name]

        self.encoder = _build_encoder(cfg, fetch)
        self.decoder = _build_decoder(cfg, fetch)
        self.encoder_transformer = _Transformer(cfg, fetch, "encoder_transformer")
        self.decoder_transformer = _Transformer(cfg, fetch, "decoder_transformer")
        s = cfg.downsample_stride
        self.downsample = self.upsample = None
        if s > 1:
            self.downsample = _Conv(fetch("downsample.conv.weight"), None, stride=s, pad_mode="replicate")
            up = fetch("upsample.conv.weight")
            self.upsample = _ConvTranspose(up, None, s, groups=up.shape[0] // max(1, up.shape[1]) if up.shape[1] == 1 else 1)
        n_sem = cfg.num_semantic_quantizers
        self.semantic = _ResidualVQ(fetch, "quantizer.semantic_residual_vector_quantizer", n_sem)
        self.acoustic = _ResidualVQ(fetch, "quantizer.acoustic_residual_vector_quantizer", cfg.num_quantizers - n_sem)
        self._enc_state: dict = {}
        self._dec_state: dict = {}
        self._pcm_tail = None

    @classmethod
    def load(cls, path, device="cpu", dtype=torch.float32, num_codebooks: Optional[int] = None) -> "Mimi":
        """A Hugging Face Mimi directory (``config.json`` + SafeTensors). ``num_codebooks`` keeps only the first codebooks
        (Moshi reads 8 of the published 32)."""
        import numpy as np

        from ..formats.checkpoint import _ST_TO_TORCH
        from ..lib import _eredu_host as H

        path = Path(path)
        cfg = MimiConfig.from_dict(json.loads((path / "config.json").read_text()))
        if num_codebooks is not None:
            if not cfg.num_semantic_quantizers < num_codebooks <= cfg.num_quantizers:
                raise ValueError(f"num_codebooks must be in ({cfg.num_semantic_quantizers}, {cfg.num_quantizers}]")
            cfg.num_quantizers = int(num_codebooks)
        store = H.SafetensorsStore(str(path), 4)

        def get(name):
            t = torch.from_numpy(np.array(store.tensor(name)))          # a private copy: the mapping can go away
            want = _ST_TO_TORCH[store.info(name)["dtype"]]
            return t if t.dtype == want else t.view(want)

        return cls(cfg, get, device, dtype)

    # ---- one-shot
    @torch.no_grad()
    def encode_latent(self, pcm: torch.Tensor, state: Optional[dict] = None) -> torch.Tensor:
        """PCM [B, channels, samples] -> latent frames [B, hidden, frames] (what the quantiser sees)."""
        x = self.encoder(pcm.to(self.device, self.dtype), state, "enc")
        x = self.encoder_transformer(x.transpose(1, 2), state, "enc_tr").transpose(1, 2)
        return self.downsample(x, state, "down") if self.downsample is not None else x

    @torch.no_grad()
    def quantize(self, latent: torch.Tensor, num_codebooks: Optional[int] = None) -> torch.Tensor:
        n = num_codebooks or self.cfg.num_quantizers
        n_sem = self.cfg.num_semantic_quantizers
        codes = self.semantic.encode(latent, min(n, n_sem))
        if n > n_sem:
            codes = torch.cat((codes, self.acoustic.encode(latent, n - n_sem)), 1)   # both start from the same latent
        return codes

    def encode(self, pcm: torch.Tensor, num_codebooks: Optional[int] = None) -> torch.Tensor:
        """PCM [B, channels, samples] -> codes [B, n_q, frames] (int64)."""
        return self.quantize(self.encode_latent(pcm), num_codebooks)

    @torch.no_grad()
    def dequantize(self, codes: torch.Tensor) -> torch.Tensor:
        n_sem = self.cfg.num_semantic_quantizers
        if codes.shape[1] > self.cfg.num_quantizers:
            raise ValueError(f"{codes.shape[1]} codebooks given, the codec has {self.cfg.num_quantizers}")
        codes = codes.to(self.device)
        x = self.semantic.decode(codes[:, :n_sem])
        if codes.shape[1] > n_sem:
            x = x + self.acoustic.decode(codes[:, n_sem:])
        return x

    @torch.no_grad()
    def decode_latent(self, latent: torch.Tensor, state: Optional[dict] = None) -> torch.Tensor:
        x = self.upsample(latent, state, "up") if self.upsample is not None else latent
        x = self.decoder_transformer(x.transpose(1, 2), state, "dec_tr").transpose(1, 2)
        return self.decoder(x, state, "dec")

    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        """codes [B, n_q', frames] (any leading subset of the codebooks) -> PCM [B, channels, frames * frame_size]."""
        return self.decode_latent(self.dequantize(codes))

    # ---- streaming
    def reset_encode_state(self) -> None:
        self._enc_state, self._pcm_tail = {}, None

    def reset_decode_state(self) -> None:
        self._dec_state = {}

    def encode_step(self, pcm: torch.Tensor, num_codebooks: Optional[int] = None) -> Optional[torch.Tensor]:
        """Feed any amount of PCM; returns the codes of the frames completed so far (None while less than one frame is
        buffered). Samples beyond the last whole frame wait for the next call."""
        pcm = pcm.to(self.device, self.dtype)
        if self._pcm_tail is not None:
            pcm = torch.cat((self._pcm_tail, pcm), -1)
        whole = pcm.shape[-1] // self.cfg.frame_size * self.cfg.frame_size
        self._pcm_tail = pcm[..., whole:]
        if whole == 0:
            return None
        return self.quantize(self.encode_latent(pcm[..., :whole], self._enc_state), num_codebooks)

    def decode_step(self, codes: torch.Tensor) -> torch.Tensor:
        """Codes of one or more new frames [B, n_q', frames] -> their PCM."""
        return self.decode_latent(self.dequantize(codes), self._dec_state)
