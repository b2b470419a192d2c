"""Gemma 4 audio tower and its embedder.

Architecture (eredu/src/backend/mlx/architectures/gemma4/audio.rs; the same network as Transformers'
``Gemma4AudioModel``, which the tests use as the oracle): log-mel frames ``[T, F]`` are sub-sampled four times in time
and frequency by two strided 3x3 convolutions (each followed by a bias-free LayerNorm over channels and ReLU) and
projected to the tower width; a stack of conformer blocks follows - half-step feed-forward, local self-attention with a
relative-position term, a gated depthwise ("light") convolution, another half-step feed-forward, an output norm - and a
biased projection to the soft-token width. ``embed`` is the multimodal embedder: a weight-free RMSNorm and a projection
into the decoder's hidden size.

The attention is local: frame i sees the ``context_left - 1`` frames ending at i and the ``context_right - 1`` after it. The reference
implementations block the sequence and unfold context windows; here one clip is attended densely under the same band
mask, with the relative term ``q_i · W_rel · sinusoid(i - j)`` added for the distances the table covers
(0 .. context_left - 1), soft-capped with tanh, which gives the same numbers without the blocking machinery. Clips are
encoded one at a time (no padding, no padding mask). Tensor operations only.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .gemma4_vision import _Linear, _rms


@dataclass
class Gemma4AudioConfig:
    hidden_size: int = 1024
    num_attention_heads: int = 8
    num_hidden_layers: int = 12
    attention_chunk_size: int = 12
    attention_context_left: int = 13
    attention_context_right: int = 0
    attention_logit_cap: float = 50.0
    attention_invalid_logits_value: float = -1e9
    conv_kernel_size: int = 5
    gradient_clipping: float = 1e10
    hidden_act: str = "silu"
    output_proj_dims: int = 1536
    residual_weight: float = 0.5
    rms_norm_eps: float = 1e-6
    subsampling_conv_channels: tuple = (128, 32)
    use_clipped_linears: bool = True

    @classmethod
    def from_dict(cls, d: dict) -> "Gemma4AudioConfig":
        known = {k: d[k] for k in cls.__dataclass_fields__ if k in d}
        if "subsampling_conv_channels" in known:
            known["subsampling_conv_channels"] = tuple(known["subsampling_conv_channels"])
        return cls(**known)


class Gemma4AudioTower:
    def __init__(self, cfg: Gemma4AudioConfig, get, has, device="cpu", dtype=torch.float32, prefix="model.audio_tower.",
                 embed_prefix="model.embed_audio."):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        if cfg.hidden_act not in ("silu", "swish"):
            raise ValueError(f"unsupported audio activation {cfg.hidden_act!r}")
        up = lambda n, dt=None: get(n).to(device=self.device, dtype=dt or dtype).contiguous()       # noqa: E731
        lin = lambda n: _Linear(get, has, n, self.device, dtype, cfg.use_clipped_linears)          # noqa: E731
        sp = prefix + "subsample_conv_projection."
        self.convs = [(up(sp + f"layer{i}.conv.weight"), up(sp + f"layer{i}.norm.weight", torch.float32)) for i in range(2)]
        self.input_proj = up(sp + "input_proj_linear.weight")
        self.layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"{prefix}layers.{i}."
            lw = {}
            for ff in ("feed_forward1", "feed_forward2"):
                lw[ff] = (up(p + ff + ".pre_layer_norm.weight", torch.float32), lin(p + ff + ".ffw_layer_1"),
                          lin(p + ff + ".ffw_layer_2"), up(p + ff + ".post_layer_norm.weight", torch.float32))
            for n in ("q_proj", "k_proj", "v_proj", "post"):
                lw[n] = lin(p + "self_attn." + n)
            lw["rel_k"] = up(p + "self_attn.relative_k_proj.weight")
            lw["per_dim_scale"] = up(p + "self_attn.per_dim_scale", torch.float32)
            lw["lconv"] = (up(p + "lconv1d.pre_layer_norm.weight", torch.float32), lin(p + "lconv1d.linear_start"),
                           up(p + "lconv1d.depthwise_conv1d.weight"), up(p + "lconv1d.conv_norm.weight", torch.float32),
                           lin(p + "lconv1d.linear_end"))
            for n in ("norm_pre_attn", "norm_post_attn", "norm_out"):
                lw[n] = up(p + n + ".weight", torch.float32)
            self.layers.append(lw)
        self.out_w, self.out_b = up(prefix + "output_proj.weight"), up(prefix + "output_proj.bias")
        self.embed_proj = up(embed_prefix + "embedding_projection.weight") if has(embed_prefix + "embedding_projection.weight") else None
        H = cfg.hidden_size
        n_scales = H // 2
        inc = math.log(10000.0) / max(n_scales - 1, 1)
        inv = torch.exp(torch.arange(n_scales, dtype=torch.float32) * -inc)
        dist = torch.arange(cfg.attention_context_left, dtype=torch.float32)[:, None]      # distances 0 .. context_left - 1
        self.rel_table = torch.cat((torch.sin(dist * inv), torch.cos(dist * inv)), -1).to(device=self.device, dtype=dtype)

    # ------------------------------------------------------------------ pieces
    def soft_token_count(self, frames: int) -> int:
        """Soft tokens a clip of ``frames`` log-mel frames becomes: two stride-2 convolutions with padding 1."""
        t = (frames + 1) // 2
        return (t + 1) // 2

    def _subsample(self, feats: torch.Tensor) -> torch.Tensor:
        x = feats.to(self.dtype)[None, None]                               # [1, 1, T, F]
        for w, nw in self.convs:
            x = F.conv2d(x, w, stride=2, padding=1)
            x = F.relu(F.layer_norm(x.permute(0, 2, 3, 1), (x.shape[1],), nw.to(x.dtype), None, self.cfg.rms_norm_eps))
            x = x.permute(0, 3, 1, 2)
        T = x.shape[2]
        x = x.permute(0, 2, 3, 1).reshape(T, -1)                           # [T', F' * C]
        return F.linear(x, self.input_proj)

    def _ffn(self, x, w):
        pre, l1, l2, post = w
        gc = min(self.cfg.gradient_clipping, torch.finfo(self.dtype).max)
        h = _rms(x.clamp(-gc, gc), pre, 1e-6)
        h = l2(F.silu(l1(h)))
        return _rms(h.clamp(-gc, gc), post, 1e-6) * self.cfg.residual_weight + x

    def _attention(self, x, lw):
        cfg = self.cfg
        T, H = x.shape
        nh = cfg.num_attention_heads
        D = H // nh
        q = lw["q_proj"](x).float().view(T, nh, D)
        k = lw["k_proj"](x).float().view(T, nh, D)
        v = lw["v_proj"](x).float().view(T, nh, D)
        q = q * ((D ** -0.5) / math.log(2)) * F.softplus(lw["per_dim_scale"])
        k = k * (math.log(1 + math.e) / math.log(2))
        logits = torch.einsum("ihd,jhd->hij", q, k)                         # content term
        rel = F.linear(self.rel_table, lw["rel_k"]).float().view(-1, nh, D)  # [distances, heads, D]
        qr = torch.einsum("ihd,phd->hip", q, rel)                           # [heads, T, distances]
        left, right = cfg.attention_context_left - 1, cfg.attention_context_right
        i = torch.arange(T, device=x.device)
        dist = i[:, None] - i[None, :]                                       # i - j
        band = ((dist >= 0) & (dist < left)) | ((dist < 0) & (-dist < right))    # windows are exclusive of their far edge
        has_rel = (dist >= 0) & (dist < rel.shape[0])
        logits = logits + torch.where(has_rel, qr.gather(2, dist.clamp(0, rel.shape[0] - 1)[None].expand(nh, -1, -1)),
                                      torch.zeros((), device=x.device))
        cap = cfg.attention_logit_cap
        logits = torch.tanh(logits / cap) * cap
        logits = logits.masked_fill(~band[None], cfg.attention_invalid_logits_value)
        probs = torch.softmax(logits, dim=-1, dtype=torch.float32)
        out = torch.einsum("hij,jhd->ihd", probs, v).reshape(T, H)
        return lw["post"](out.to(self.dtype))

    def _light_conv(self, x, w):
        pre, start, dw, cnorm, end = w
        cfg = self.cfg
        h = F.glu(start(_rms(x, pre, cfg.rms_norm_eps)), dim=-1)            # [T, H]
        h = F.conv1d(F.pad(h.t()[None], (cfg.conv_kernel_size - 1, 0)), dw, groups=h.shape[1])[0].t()
        gc = min(cfg.gradient_clipping, torch.finfo(self.dtype).max)
        h = F.silu(_rms(h.clamp(-gc, gc), cnorm, cfg.rms_norm_eps))
        return end(h) + x

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def encode(self, features: torch.Tensor) -> torch.Tensor:
        """Log-mel frames [T, F] -> soft tokens [ceil(ceil(T/2)/2), output_proj_dims]."""
        gc = min(self.cfg.gradient_clipping, torch.finfo(self.dtype).max)
        x = self._subsample(features.to(self.device))
        for lw in self.layers:
            x = self._ffn(x, lw["feed_forward1"])
            res = x
            h = _rms(x.clamp(-gc, gc), lw["norm_pre_attn"], 1e-6)
            h = self._attention(h, lw)
            x = _rms(h.clamp(-gc, gc), lw["norm_post_attn"], 1e-6) + res
            x = self._light_conv(x, lw["lconv"])
            x = self._ffn(x, lw["feed_forward2"])
            x = _rms(x.clamp(-gc, gc), lw["norm_out"], 1e-6)
        return F.linear(x, self.out_w, self.out_b)

    def embed(self, soft: torch.Tensor) -> torch.Tensor:
        if self.embed_proj is None:
            raise RuntimeError("this checkpoint carries an audio tower without its embedder")
        return F.linear(_rms(soft, None, self.cfg.rms_norm_eps), self.embed_proj)

    def forward(self, features: torch.Tensor) -> torch.Tensor:
        return self.embed(self.encode(features))
