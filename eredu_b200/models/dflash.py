"""DFlash: the block drafter released with Muse-Glimmer (``model_type: muse_glimmer_assistant``).

Architecture (eredu/src/backend/mlx/architectures/muse_glimmer/assistant.rs, driven by mtp.rs): the drafter proposes a
whole block in ONE pass. Its input block is the target's embedding of ``[newest token, mask, mask, ...]``; its context
is the target's own activity - the outputs of a few target layers (``target_layer_ids``) for every committed token,
concatenated, projected by ``encoder.fc`` and RMS-normalised. Every drafter layer keeps keys and values of that encoded
context (its own ``k_proj`` / ``v_proj``, per-head RMSNorm on the keys, rotary embedding at the tokens' absolute
positions; at most ``sliding_window`` tokens are retained) and attends from the block to ``[context | block]``: context
keys causally and inside the window, block keys in both directions (assistant.rs:398-478). Pre-norm blocks with SwiGLU;
the final norm's rows 1 .. give the proposal states, which go through the TARGET's output head and logit scaling.

The block's width is what the request asks for (one anchor plus k masks, up to ``block_size``): attention inside the
block is bidirectional, so padding to the trained width would change the distributions (mtp.rs:228-237).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from .. import ops


@dataclass
class DFlashConfig:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    block_size: int
    mask_token_id: int
    target_layer_ids: list = field(default_factory=list)
    rms_norm_eps: float = 1e-6
    rope_theta: float = 500000.0
    sliding_window: int = 2048

    @classmethod
    def from_dict(cls, d: dict) -> "DFlashConfig":
        import dataclasses

        if str(d.get("model_type", "muse_glimmer_assistant")) != "muse_glimmer_assistant":
            raise ValueError(f"not a DFlash assistant config: {d.get('model_type')!r}")
        if d.get("hidden_act", "silu") != "silu" or any(t != "sliding_attention" for t in d.get("layer_types", [])):
            raise ValueError("DFlash assistants use SiLU and sliding attention on every layer")
        known = {f.name: d[f.name] for f in dataclasses.fields(cls) if f.name in d and d[f.name] is not None}
        rp = d.get("rope_parameters") or {}
        if "rope_theta" in rp:
            known["rope_theta"] = float(rp["rope_theta"])
        missing = [f.name for f in dataclasses.fields(cls)
                   if f.name not in known and f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING]
        if missing:
            raise ValueError(f"DFlash config lacks {missing}")
        cfg = cls(**known)
        cfg.target_layer_ids = [int(i) for i in cfg.target_layer_ids]
        if not cfg.target_layer_ids or cfg.block_size < 2 or cfg.num_attention_heads % cfg.num_key_value_heads:
            raise ValueError("DFlash config needs target layers, a block of at least two tokens and grouped heads")
        return cfg


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def _rope(x, positions, inv_freq):
    ang = positions.float()[:, None] * inv_freq[None, :]
    cos, sin = torch.cat((ang.cos(), ang.cos()), -1)[:, None, :], torch.cat((ang.sin(), ang.sin()), -1)[:, None, :]
    half = x.shape[-1] // 2
    return x * cos + torch.cat((-x[..., half:], x[..., :half]), -1) * sin


class DFlashContext:
    """Per request: the encoded context's keys / values of every drafter layer for positions ``[start, end)``."""

    def __init__(self):
        self.keys, self.values = None, None          # lists over layers of [n, Hkv, D]
        self.start = self.end = 0

    def clone(self):
        c = DFlashContext()
        c.keys = None if self.keys is None else [k.clone() for k in self.keys]
        c.values = None if self.values is None else [v.clone() for v in self.values]
        c.start, c.end = self.start, self.end
        return c


class DFlash:
    def __init__(self, cfg: DFlashConfig, get, has, device="cpu", dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        up = lambda t, dt=None: t.to(device=self.device, dtype=dt or dtype).contiguous()          # noqa: E731
        f32 = lambda n: up(get(n), torch.float32)                                                  # noqa: E731
        H, D = cfg.hidden_size, cfg.head_dim
        self.fc = up(get("encoder.fc.weight"))
        if tuple(self.fc.shape) != (H, H * len(cfg.target_layer_ids)):
            raise ValueError(f"encoder.fc.weight has shape {tuple(self.fc.shape)}, expected {(H, H * len(cfg.target_layer_ids))}")
        self.enc_norm = f32("encoder.output_norm_enc.weight")
        self.norm = f32("norm.weight")
        self.inv_freq = (1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))).to(self.device)
        self.layers = []
        for li in range(cfg.num_hidden_layers):
            p = f"layers.{li}."
            w = {n: up(get(p + f"self_attn.{n}.weight")) for n in ("q_proj", "k_proj", "v_proj", "o_proj")}
            w["q_norm"], w["k_norm"] = f32(p + "self_attn.q_norm.weight"), f32(p + "self_attn.k_norm.weight")
            w["in_norm"], w["post_norm"] = f32(p + "input_layernorm.weight"), f32(p + "post_attention_layernorm.weight")
            w["gate_up"] = up(torch.cat((get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")), 0))
            w["down"] = up(get(p + "mlp.down_proj.weight"))
            self.layers.append(w)

    @property
    def max_proposals(self) -> int:
        return self.cfg.block_size - 1

    # ------------------------------------------------------------------ context
    @torch.no_grad()
    def extend_context(self, ctx: DFlashContext, target_states: torch.Tensor, end: int) -> DFlashContext:
        """``target_states`` [n, H * layers]: the concatenated target-layer outputs of the n newest committed tokens, which
        end at absolute position ``end``. Keeps the last ``sliding_window`` positions."""
        cfg = self.cfg
        n = target_states.shape[0]
        if n == 0:
            return ctx
        if ctx.keys is not None and ctx.end != end - n:
            raise ValueError(f"context ends at {ctx.end}, the new states start at {end - n}")
        enc = _rms(ops.linear(target_states.to(self.device, self.dtype).contiguous(), self.fc), self.enc_norm, cfg.rms_norm_eps)
        pos = torch.arange(end - n, end, device=self.device)
        keys, values = [], []
        for li, w in enumerate(self.layers):
            k = _rms(ops.linear(enc, w["k_proj"]).view(n, cfg.num_key_value_heads, cfg.head_dim), w["k_norm"], cfg.rms_norm_eps)
            k = _rope(k.float(), pos, self.inv_freq)
            v = ops.linear(enc, w["v_proj"]).view(n, cfg.num_key_value_heads, cfg.head_dim).float()
            if ctx.keys is not None:
                k, v = torch.cat((ctx.keys[li], k)), torch.cat((ctx.values[li], v))
            keys.append(k[-cfg.sliding_window:])
            values.append(v[-cfg.sliding_window:])
        out = DFlashContext()
        out.keys, out.values = keys, values
        out.end = end
        out.start = end - keys[0].shape[0]
        return out

    # ------------------------------------------------------------------ one block
    @torch.no_grad()
    def propose(self, block_embeds: torch.Tensor, ctx: DFlashContext) -> torch.Tensor:
        """``block_embeds`` [1 + k, H]: the target's embeddings of the anchor and k mask tokens; the block sits at absolute
        positions ``ctx.end ..``. Returns the k proposal states [k, H] (to be projected by the target's head)."""
        cfg = self.cfg
        T = block_embeds.shape[0]
        if T < 2 or T > cfg.block_size or ctx.keys is None:
            raise ValueError("a DFlash block holds an anchor and 1 .. block_size - 1 masks, behind a non-empty context")
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        n = ctx.end - ctx.start
        pos = torch.arange(ctx.end, ctx.end + T, device=self.device)
        kpos = torch.arange(ctx.start, ctx.end, device=self.device)
        dist = pos[:, None] - kpos[None, :]
        allowed = torch.cat(((dist >= 0) & (dist < cfg.sliding_window), torch.ones((T, T), dtype=torch.bool, device=self.device)), 1)
        h = block_embeds.to(self.device, self.dtype)
        g = Hq // Hkv
        for w, ck, cv in zip(self.layers, ctx.keys, ctx.values):
            x = _rms(h, w["in_norm"], cfg.rms_norm_eps)
            q = _rope(_rms(ops.linear(x, w["q_proj"]).view(T, Hq, D), w["q_norm"], cfg.rms_norm_eps).float(), pos, self.inv_freq)
            k = _rope(_rms(ops.linear(x, w["k_proj"]).view(T, Hkv, D), w["k_norm"], cfg.rms_norm_eps).float(), pos, self.inv_freq)
            v = ops.linear(x, w["v_proj"]).view(T, Hkv, D).float()
            keys, values = torch.cat((ck, k)), torch.cat((cv, v))                             # [n + T, Hkv, D]
            s = torch.einsum("tkgd,nkd->tkgn", q.view(T, Hkv, g, D), keys) * (D ** -0.5)
            s = s.masked_fill(~allowed[:, None, None, :], float("-inf"))
            a = torch.einsum("tkgn,nkd->tkgd", torch.softmax(s, -1), values).reshape(T, Hq * D)
            h = h + ops.linear(a.to(self.dtype), w["o_proj"])
            y = _rms(h, w["post_norm"], cfg.rms_norm_eps)
            gu = ops.linear(y, w["gate_up"]).float()
            inter = gu.shape[1] // 2
            h = h + ops.linear((F.silu(gu[:, :inter]) * gu[:, inter:]).to(self.dtype), w["down"])
        assert n == ctx.keys[0].shape[0]
        return _rms(h, self.norm, cfg.rms_norm_eps)[1:]


def load_dflash(path, device="cpu", dtype=torch.float32) -> DFlash:
    """A DFlash directory: ``config.json`` + safetensors with the module-tree names (``encoder.fc.weight``,
    ``layers.N.self_attn.q_proj.weight``, ``norm.weight`` ...)."""
    import json
    from pathlib import Path

    from safetensors import safe_open

    path = Path(path)
    with open(path / "config.json") as f:
        cfg = DFlashConfig.from_dict(json.load(f))
    where = {}
    for shard in sorted(path.glob("*.safetensors")):
        h = safe_open(str(shard), framework="pt", device="cpu")
        for name in h.keys():
            where[name] = h
    if not where:
        raise FileNotFoundError(f"{path}: no safetensors shards")
    return DFlash(cfg, lambda n: where[n].get_tensor(n), where.__contains__, device, dtype)
