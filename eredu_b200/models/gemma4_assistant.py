"""Gemma 4 assistant drafter: the external multi-token-prediction model that ships next to a Gemma 4 checkpoint.

Architecture (eredu/src/backend/mlx/architectures/gemma4/assistant.rs): a short stack of Gemma 4 blocks whose attention
layers own no keys or values - every layer reads the K / V that the TARGET wrote for the last layer of the same attention
kind (sliding or global). A draft step takes the target-embedded last token (scaled by sqrt(backbone width)) concatenated
with a hidden state of the backbone's width (the target's pre-norm hidden state of the last cached token on the first
step, the drafter's own ``post_projection`` output afterwards), projects the pair down (``pre_projection``), runs the
blocks at position ``cache_len - 1 + step`` over the target's committed cache (nothing is appended: all steps of a
round see the same keys), normalises, and produces logits through one of three heads: tied embeddings, an untied
``lm_head``, or the ordered masked embedder (score ``num_centroids`` centroids, keep the best ``top_k`` groups, evaluate
only the tokens ``token_ordering`` lists for those groups and leave every other logit one below the smallest evaluated
one - assistant.rs:186-273).

The blocks are Gemma 4's: sandwich norms, per-head q RMSNorm, score scale 1, GeGLU, learned layer scalar; no per-layer
inputs and no sparse block. Tensor operations around this repository's GEMMs, like the Gemma 4 decoder itself.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from .. import ops
from .gemma4 import _rms, _rope, rope_tables


@dataclass
class Gemma4AssistantConfig:
    backbone_hidden_size: int
    text: object                               # ModelConfig of the assistant body
    use_ordered_embeddings: bool = False
    num_centroids: int = 2048
    centroid_intermediate_top_k: int = 32
    tie_word_embeddings: bool = True
    block_size: int = 4
    extra: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: dict) -> "Gemma4AssistantConfig":
        from .config import ModelConfig

        if "text_config" not in d or "backbone_hidden_size" not in d:
            raise ValueError("a Gemma 4 assistant config needs text_config and backbone_hidden_size")
        text = dict(d["text_config"])
        text.setdefault("model_type", "gemma4_text")
        text.setdefault("architectures", ["Gemma4ForCausalLM"])
        return cls(backbone_hidden_size=int(d["backbone_hidden_size"]), text=ModelConfig.from_hf_dict(text),
                   use_ordered_embeddings=bool(d.get("use_ordered_embeddings", False)),
                   num_centroids=int(d.get("num_centroids", 2048)),
                   centroid_intermediate_top_k=int(d.get("centroid_intermediate_top_k", 32)),
                   tie_word_embeddings=bool(d.get("tie_word_embeddings", True)), block_size=int(d.get("block_size", 4)))


def donor_layers(target_cfg) -> dict:
    """Attention kind -> the target layer whose K / V the assistant reads: the last layer of that kind that owns its cache."""
    from .gemma4 import geometry

    out = {}
    for li, (sliding, _, _, _, donor) in enumerate(geometry(target_cfg)):
        if donor is None:
            out["sliding_attention" if sliding else "full_attention"] = li
    return out


class Gemma4Assistant:
    def __init__(self, cfg: Gemma4AssistantConfig, get, has, target_model, device=None, dtype=None):
        self.cfg = cfg
        tc = cfg.text
        self.target = target_model
        self.device = torch.device(device) if device is not None else target_model.device
        self.dtype = dtype or target_model.dtype
        tcfg = target_model.cfg
        if tcfg.hidden_size != cfg.backbone_hidden_size:
            raise ValueError(f"assistant was trained for backbone width {cfg.backbone_hidden_size}, target has {tcfg.hidden_size}")
        if tc.vocab_size != tcfg.vocab_size:
            raise ValueError("assistant and target must share the vocabulary")
        if tc.extra["gemma4"].get("enable_moe_block"):
            raise NotImplementedError("assistant bodies with a sparse block are not supported")
        if target_model.par.tp_size > 1:
            raise NotImplementedError("the assistant drafter runs next to an unsharded target")
        up = lambda t, dt=None: t.to(device=self.device, dtype=dt or self.dtype).contiguous()       # noqa: E731
        f32 = lambda n: up(get(n), torch.float32)                                                   # noqa: E731
        g = tc.extra["gemma4"]
        self.eps = tc.rms_norm_eps
        self.inv_freq = {k: v.to(self.device) for k, v in rope_tables(tc).items()}
        self.donors = donor_layers(tcfg)
        tg = tcfg.extra["gemma4"]
        self.layers = []
        for li in range(tc.num_hidden_layers):
            kind = tc.layer_types[li]
            if kind not in self.donors:
                raise ValueError(f"assistant layer {li} is {kind} but the target owns no cache of that kind")
            sliding = kind == "sliding_attention"
            D = tc.head_dim if sliding or not g.get("global_head_dim") else int(g["global_head_dim"])
            tD = tcfg.head_dim if sliding or not tg.get("global_head_dim") else int(tg["global_head_dim"])
            if D != tD:
                raise ValueError(f"assistant layer {li} has head size {D}, the target's {kind} cache has {tD}")
            p = f"model.layers.{li}."
            w = {n: f32(p + n + ".weight") for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm",
                                                     "post_feedforward_layernorm")}
            w["scalar"] = f32(p + "layer_scalar") if has(p + "layer_scalar") else None
            w["q"], w["o"] = up(get(p + "self_attn.q_proj.weight")), up(get(p + "self_attn.o_proj.weight"))
            w["q_norm"] = f32(p + "self_attn.q_norm.weight")
            w["gate_up"] = up(torch.cat((get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")), 0))
            w["down"] = up(get(p + "mlp.down_proj.weight"))
            w["kind"], w["sliding"], w["D"] = kind, sliding, D
            self.layers.append(w)
        self.norm = f32("model.norm.weight")
        self.embed = up(get("model.embed_tokens.weight"))
        self.pre = up(get("pre_projection.weight"))
        self.post = up(get("post_projection.weight"))
        self.lm_head = None if cfg.tie_word_embeddings else up(get("lm_head.weight"))
        self.centroids = self.ordering = None
        if cfg.use_ordered_embeddings:
            if tc.vocab_size % cfg.num_centroids:
                raise ValueError("the vocabulary does not divide into the configured number of centroid groups")
            self.centroids = up(get("masked_embedding.centroids.weight"))
            self.ordering = get("masked_embedding.token_ordering").to(device=self.device, dtype=torch.int64).view(
                cfg.num_centroids, tc.vocab_size // cfg.num_centroids)
        self.softcap = float(g.get("final_logit_softcapping") or 0.0)

    @property
    def max_proposals(self) -> int:
        return max(1, self.cfg.block_size - 1)

    # ------------------------------------------------------------------ pieces
    def _attend(self, q, w, kv, block_table, cache_lens, q_pos):
        """q [B, Hq, D] over the target's cache of this layer's kind: keys 0 .. cache_len - 1, and on sliding layers only
        those less than a window behind the query position."""
        tcfg = self.target.cfg
        src = self.donors[w["kind"]]
        k_pool, v_pool = kv.layer(src)
        nkv = self.target.g4["geometry"][src][2]
        D = w["D"]
        B, Hq, _ = q.shape
        out = torch.empty_like(q, dtype=torch.float32)
        window = int(tcfg.sliding_window or 0) if w["sliding"] else 0
        for b in range(B):
            n = int(cache_lens[b])
            k = ops.core._gather_kv(k_pool[:, :nkv, :, :D], block_table[b], n).float()       # [nkv, n, D]
            v = ops.core._gather_kv(v_pool[:, :nkv, :, :D], block_table[b], n).float()
            qb = q[b].float().view(nkv, Hq // nkv, D)
            s = torch.einsum("ngd,nkd->ngk", qb, k)
            if window > 0:
                far = torch.arange(n, device=q.device) <= int(q_pos[b]) - window
                s = s.masked_fill(far[None, None, :], float("-inf"))
            out[b] = torch.einsum("ngk,nkd->ngd", torch.softmax(s, -1), v).reshape(Hq, D)
        return out

    def _logits(self, h):
        tc = self.cfg.text
        if self.centroids is not None:
            B = h.shape[0]
            scores = F.linear(h.float(), self.centroids.float())
            top = torch.topk(scores, self.cfg.centroid_intermediate_top_k, dim=-1).indices          # [B, k]
            ids = self.ordering[top].reshape(B, -1)                                                  # [B, k * per]
            rows = self.embed[ids].float()                                                           # [B, n, H]
            sel = torch.einsum("bh,bnh->bn", h.float(), rows)
            out = torch.full((B, tc.vocab_size), float(sel.min()) - 1.0, dtype=torch.float32, device=h.device)
            out.scatter_(1, ids, sel)
            return out
        logits = ops.linear(h, self.lm_head if self.lm_head is not None else self.embed, out_dtype=torch.float32)
        if self.softcap > 0:
            logits = torch.tanh(logits / self.softcap) * self.softcap
        return logits

    # ------------------------------------------------------------------ one draft step
    @torch.no_grad()
    def draft_step(self, token_ids, hidden, kv, block_table, cache_lens, step: int):
        """token_ids [B]: the newest token of every sequence; hidden [B, backbone]: what pairs with it; the target's cache
        holds ``cache_lens[b]`` tokens of sequence b. Returns (logits [B, V] fp32, the hidden rows for the next step)."""
        dt = self.dtype
        tc = self.cfg.text
        emb = self.target.embed[token_ids.long()].float() * (self.cfg.backbone_hidden_size ** 0.5)
        h = ops.linear(torch.cat((emb, hidden.float()), -1).to(dt), self.pre)
        B = h.shape[0]
        q_pos = (cache_lens.to(torch.int64) - 1 + step).clamp_min(0)
        for w in self.layers:
            D = w["D"]
            Hq = w["q"].shape[0] // D
            x = _rms(h, w["input_layernorm"], self.eps).to(dt)
            q = _rope(_rms(ops.linear(x, w["q"]).view(B, Hq, D), w["q_norm"], self.eps), q_pos, self.inv_freq[w["kind"]])
            a = self._attend(q, w, kv, block_table, cache_lens, q_pos)
            a = ops.linear(a.reshape(B, Hq * D).to(dt), w["o"])
            h = h + _rms(a, w["post_attention_layernorm"], self.eps).to(dt)
            y = _rms(h, w["pre_feedforward_layernorm"], self.eps).to(dt)
            gu = ops.linear(y, w["gate_up"]).float()
            inter = gu.shape[1] // 2
            y = ops.linear((F.gelu(gu[:, :inter], approximate="tanh") * gu[:, inter:]).to(dt), w["down"])
            h = h + _rms(y, w["post_feedforward_layernorm"], self.eps).to(dt)
            if w["scalar"] is not None:
                h = (h.float() * w["scalar"]).to(dt)
        h = _rms(h, self.norm, self.eps).to(dt)
        return self._logits(h), ops.linear(h, self.post)


def load_gemma4_assistant(path, target_model, device=None, dtype=None) -> Gemma4Assistant:
    """An assistant directory (``config.json`` + safetensors shards, tensor names as the module tree: ``model.*``,
    ``pre_projection``, ``post_projection``, ``lm_head``, ``masked_embedding.*``) next to a loaded Gemma 4 target.
    Reference: load_gemma4_assistant_model_with_options, eredu/src/backend/mlx/architectures/gemma4/assistant.rs:499-588."""
    import json
    from pathlib import Path

    from safetensors import safe_open

    path = Path(path)
    with open(path / "config.json") as f:
        raw = json.load(f)
    if raw.get("quantization") and raw.get("use_ordered_embeddings"):
        raise ValueError("an affine-quantised assistant cannot use ordered masked embeddings: that head indexes dense embedding rows")
    cfg = Gemma4AssistantConfig.from_dict(raw)
    handles, where = [], {}
    for shard in sorted(path.glob("*.safetensors")):
        h = safe_open(str(shard), framework="pt", device="cpu")
        handles.append(h)
        for name in h.keys():
            where[name] = h
    if not where:
        raise FileNotFoundError(f"{path}: no safetensors shards")
    return Gemma4Assistant(cfg, lambda n: where[n].get_tensor(n), where.__contains__, target_model, device, dtype)
