"""Moshi / PersonaPlex: a temporal transformer over frames and a depth transformer over the codebooks of one frame.

Counterpart of the reference's realtime speech family (eredu/src/backend/mlx/architectures/moshi/, 6.0k lines: temporal +
depth transformers, tensor parallel only; the codec is ``eredu_b200.codec.Mimi``). Per frame t:

* the temporal transformer reads the SUM of the text-token embedding and the embeddings of the 2 K audio tokens of the
  frame (K codebooks the model spoke, K it heard) and gives text logits and the normalised hidden state ``h_t``;
* the depth transformer runs over K positions: position k reads ``input_projection_k(h_t)`` plus the embedding of the token
  chosen just before (the text token at k = 0, codebook k-1 afterwards) and gives the logits of codebook k. Its linear maps
  have one weight per position; it uses no rotary embedding.

Tensor names are those of the Hugging Face checkpoint (``kyutai/moshiko-pytorch-bf16`` converted); ``tests/test_moshi.py``
checks both transformers against Transformers' ``MoshiForConditionalGeneration`` on the same weights.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from .. import ops


@dataclass
class MoshiConfig:
    vocab_size: int = 32000
    audio_vocab_size: int = 2048
    hidden_size: int = 4096
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    head_dim: Optional[int] = None
    ffn_dim: int = 22528
    num_codebooks: int = 8
    sliding_window: int = 3000
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-8
    depth: dict = field(default_factory=dict)        # the same keys for the depth transformer
    audio_encoder: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: dict) -> "MoshiConfig":
        def pick(src):
            out = {k: src[k] for k in ("vocab_size", "audio_vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                                       "num_key_value_heads", "head_dim", "ffn_dim", "num_codebooks", "sliding_window",
                                       "rms_norm_eps") if src.get(k) is not None}
            rp = src.get("rope_parameters") or {}
            theta = rp.get("rope_theta", src.get("rope_theta"))
            if theta is not None:
                out["rope_theta"] = float(theta)
            return out

        depth = pick(d.get("depth_decoder_config") or {})
        depth["input_size"] = (d.get("depth_decoder_config") or {}).get("input_size", d.get("hidden_size"))
        cfg = cls(depth=depth, audio_encoder=dict(d.get("audio_encoder_config") or {}), **pick(d))
        if cfg.hidden_size % cfg.num_attention_heads or cfg.ffn_dim % 2:
            raise ValueError("invalid Moshi geometry")
        if int(depth.get("num_codebooks", cfg.num_codebooks)) != cfg.num_codebooks:
            raise ValueError("the depth transformer must cover the model's codebooks")
        return cfg


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def _rope(x, pos, theta):
    """Split-half rotary embedding; x [B, H, T, D], pos [T]."""
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32, device=x.device) / D))
    ang = pos.to(torch.float32)[:, None] * inv[None, :]
    cos, sin = torch.cat((ang.cos(), ang.cos()), -1), torch.cat((ang.sin(), ang.sin()), -1)
    rot = torch.cat((-x[..., D // 2:], x[..., :D // 2]), -1)
    return (x.float() * cos + rot.float() * sin).to(x.dtype)


def _linear(x, w):
    """[.., K] x [N, K]^T through the GEMM kernel on CUDA (2-D view), plain matmul elsewhere."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        return ops.linear(x.reshape(-1, x.shape[-1]).contiguous(), w).view(*x.shape[:-1], w.shape[0])
    return F.linear(x, w)


class MoshiLm:
    """Both transformers of one checkpoint. ``TemporalState`` carries the temporal transformer's keys / values of the
    window; the depth transformer starts from an empty cache at every frame."""

    def __init__(self, cfg: MoshiConfig, get: Callable[[str], torch.Tensor], device="cpu", dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        up = lambda n, dt=None: get(n).to(device=self.device, dtype=dt or dtype).contiguous()      # noqa: E731
        K = cfg.num_codebooks
        self.text_embed = up("decoder.model.embed_tokens.weight")
        self.audio_embed = [up(f"embed_tokens.{i}.weight") for i in range(2 * K)]      # K spoken, then K heard
        self.layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"decoder.model.layers.{i}."
            self.layers.append(dict(
                qkv=torch.cat([up(p + f"self_attn.{n}_proj.linear.weight") for n in "qkv"], 0), o=up(p + "self_attn.o_proj.linear.weight"),
                fc1=up(p + "mlp.fc1.weight"), fc2=up(p + "mlp.fc2.weight"),
                n1=up(p + "input_layernorm.weight", torch.float32), n2=up(p + "post_attention_layernorm.weight", torch.float32)))
        self.norm = up("decoder.model.norm.weight", torch.float32)
        self.text_head = up("decoder.lm_head.weight")
        d = cfg.depth
        self.d_hidden, self.d_heads = int(d["hidden_size"]), int(d["num_attention_heads"])
        self.d_kv = int(d.get("num_key_value_heads", self.d_heads))
        self.d_eps = float(d.get("rms_norm_eps", cfg.rms_norm_eps))
        self.d_text_embed = up("depth_decoder.text_embed_tokens.weight")
        self.d_audio_embed = [up(f"depth_decoder.embed_tokens.{i}.weight") for i in range(K - 1)]
        self.d_in = up("depth_decoder.input_projections.weight")                          # [K, d_hidden, hidden]
        self.d_layers = []
        for i in range(int(d["num_hidden_layers"])):
            p = f"depth_decoder.layers.{i}."
            self.d_layers.append(dict(
                q=up(p + "self_attn.q_proj.linear.weight"), k=up(p + "self_attn.k_proj.linear.weight"),
                v=up(p + "self_attn.v_proj.linear.weight"), o=up(p + "self_attn.o_proj.linear.weight"),
                fc1=up(p + "mlp.fc1.weight"), fc2=up(p + "mlp.fc2.weight"),
                n1=up(p + "input_layernorm.weight", torch.float32), n2=up(p + "post_attention_layernorm.weight", torch.float32)))
        self.d_heads_w = up("depth_decoder.lm_heads.weight")                              # [K, audio_vocab, d_hidden]

    @classmethod
    def load(cls, path, device="cpu", dtype=None) -> "MoshiLm":
        import numpy as np

        from ..formats.checkpoint import _ST_TO_TORCH
        from ..lib import _eredu_host as H

        path = Path(path)
        cfg = MoshiConfig.from_dict(json.loads((path / "config.json").read_text()))
        store = H.SafetensorsStore(str(path), 4)

        def get(name):
            t = torch.from_numpy(np.array(store.tensor(name)))
            want = _ST_TO_TORCH[store.info(name)["dtype"]]
            return t if t.dtype == want else t.view(want)

        dev = torch.device(device)
        return cls(cfg, get, dev, dtype or (torch.bfloat16 if dev.type == "cuda" else torch.float32))

    # ---- temporal transformer
    def embed_frame(self, text_ids, spoken_codes=None, heard_codes=None):
        """text_ids [B, T]; spoken / heard codes [B, K, T] (None or negative entries contribute nothing)."""
        x = F.embedding(text_ids.to(self.device), self.text_embed)
        K = self.cfg.num_codebooks
        for base, codes in ((0, spoken_codes), (K, heard_codes)):
            if codes is None:
                continue
            codes = codes.to(self.device)
            for k in range(codes.shape[1]):
                c = codes[:, k]
                e = F.embedding(c.clamp_min(0), self.audio_embed[base + k])
                x = x + torch.where((c >= 0)[..., None], e, torch.zeros_like(e))
        return x

    @torch.no_grad()
    def temporal(self, x, state: Optional[dict] = None):
        """Frame embeddings [B, T, H] -> (text logits [B, T, V] fp32, normalised hidden [B, T, H]). ``state`` (a dict that
        starts empty) makes the call incremental."""
        cfg = self.cfg
        B, T, H = x.shape
        Hq, Hkv = cfg.num_attention_heads, cfg.num_key_value_heads
        D = cfg.head_dim or H // Hq
        W = cfg.sliding_window
        start = 0 if state is None else state.get("pos", 0)
        pos = torch.arange(start, start + T, device=x.device)
        for li, lw in enumerate(self.layers):
            h = _rms(x, lw["n1"], cfg.rms_norm_eps)
            qkv = _linear(h, lw["qkv"])
            q, k, v = qkv.split((Hq * D, Hkv * D, Hkv * D), -1)
            q = _rope(q.view(B, T, Hq, D).transpose(1, 2), pos, cfg.rope_theta)
            k = _rope(k.view(B, T, Hkv, D).transpose(1, 2), pos, cfg.rope_theta)
            v = v.view(B, T, Hkv, D).transpose(1, 2)
            kpos = pos
            if state is not None:
                old = state.get(li)
                if old is not None:
                    k, v, kpos = torch.cat((old[0], k), 2), torch.cat((old[1], v), 2), torch.cat((old[2], pos))
                keep = max(0, k.shape[2] - (W - 1)) if W else 0
                state[li] = (k[:, :, keep:], v[:, :, keep:], kpos[keep:])
            if Hkv != Hq:
                k, v = k.repeat_interleave(Hq // Hkv, 1), v.repeat_interleave(Hq // Hkv, 1)
            rel = pos[:, None] - kpos[None, :]
            mask = (rel >= 0) & ((rel < W) if W else True)
            a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
            x = x + _linear(a.transpose(1, 2).reshape(B, T, Hq * D), lw["o"])
            h = _linear(_rms(x, lw["n2"], cfg.rms_norm_eps), lw["fc1"])
            gate, upv = h.split(h.shape[-1] // 2, -1)
            x = x + _linear(F.silu(gate) * upv, lw["fc2"])
        if state is not None:
            state["pos"] = start + T
        hidden = _rms(x, self.norm, cfg.rms_norm_eps)
        return _linear(hidden, self.text_head).float(), hidden

    # ---- depth transformer
    def _depth_position(self, k: int, x, cache: list):
        """One codebook position: x [B, d_hidden] (already input_projection_k(h) + previous token's embedding) -> hidden."""
        B = x.shape[0]
        Hq, Hkv = self.d_heads, self.d_kv
        D = self.d_hidden // Hq
        for li, lw in enumerate(self.d_layers):
            h = _rms(x, lw["n1"], self.d_eps)
            q = F.linear(h, lw["q"][k]).view(B, Hq, 1, D)
            kk = F.linear(h, lw["k"][k]).view(B, Hkv, 1, D)
            vv = F.linear(h, lw["v"][k]).view(B, Hkv, 1, D)
            if cache[li] is not None:
                kk, vv = torch.cat((cache[li][0], kk), 2), torch.cat((cache[li][1], vv), 2)
            cache[li] = (kk, vv)
            if Hkv != Hq:
                kk, vv = kk.repeat_interleave(Hq // Hkv, 1), vv.repeat_interleave(Hq // Hkv, 1)
            a = F.scaled_dot_product_attention(q, kk, vv)                          # one query over positions 0..k
            x = x + F.linear(a.reshape(B, Hq * D), lw["o"][k])
            h = F.linear(_rms(x, lw["n2"], self.d_eps), lw["fc1"][k])
            gate, upv = h.split(h.shape[-1] // 2, -1)
            x = x + F.linear(F.silu(gate) * upv, lw["fc2"][k])
        return x

    @torch.no_grad()
    def depth_logits(self, hidden, text_token, audio_tokens):
        """Teacher-forced pass: hidden [B, H] of one frame, its text token [B] and its K codebook tokens [B, K] (the last one
        is not read) -> logits [B, K, audio_vocab] fp32."""
        K = self.cfg.num_codebooks
        cache = [None] * len(self.d_layers)
        out = []
        for k in range(K):
            prev = F.embedding(text_token, self.d_text_embed) if k == 0 else F.embedding(audio_tokens[:, k - 1], self.d_audio_embed[k - 1])
            x = prev + F.linear(hidden, self.d_in[k])
            g = self._depth_position(k, x, cache)
            out.append(F.linear(g, self.d_heads_w[k]).float())
        return torch.stack(out, 1)

    @torch.no_grad()
    def depth_generate(self, hidden, text_token, choose: Optional[Callable] = None):
        """The K codebook tokens of one frame, one after the other. ``choose(k, logits [B, V]) -> [B]`` picks a token
        (default: argmax)."""
        K = self.cfg.num_codebooks
        cache = [None] * len(self.d_layers)
        prev = F.embedding(text_token, self.d_text_embed)
        tokens = []
        for k in range(K):
            g = self._depth_position(k, prev + F.linear(hidden, self.d_in[k]), cache)
            logits = F.linear(g, self.d_heads_w[k]).float()
            tok = logits.argmax(-1) if choose is None else choose(k, logits)
            tokens.append(tok)
            if k + 1 < K:
                prev = F.embedding(tok, self.d_audio_embed[k])
        return torch.stack(tokens, 1)
