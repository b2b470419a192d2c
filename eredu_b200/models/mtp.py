"""Checkpoint-embedded next-token prediction layers used as the drafter of speculative decoding.

Two checkpoint layouts carry such a layer:

* Qwen3-Next / Qwen3.5 (``mtp_num_hidden_layers``): ``mtp.pre_fc_norm_embedding``, ``mtp.pre_fc_norm_hidden``, ``mtp.fc``
  ``[H, 2H]``, one full-attention decoder block ``mtp.layers.0.*``, ``mtp.norm``; the vocabulary head is the model's own
  (eredu/src/backend/mlx/architectures/qwen/hybrid/qwen3_5.rs:4533-4640).
* DeepSeek-V3 (``num_nextn_predict_layers``): decoder layer ``L = num_hidden_layers`` with ``enorm``, ``hnorm``, ``eh_proj``
  ``[H, 2H]``, the block itself, ``shared_head.norm`` and ``shared_head.head`` (and a copy of the embedding)
  (eredu/src/backend/mlx/architectures/deepseek_v3/layerwise.rs:82-262).

* Nemotron-H (``num_nextn_predict_layers`` + ``mtp_hybrid_override_pattern`` of ``*`` / ``E`` markers): ``mtp.layers.j`` for
  the ``P`` blocks of a prediction step (same tensor names as a backbone block), ``enorm`` / ``hnorm`` / ``eh_proj`` on the
  step's first block, ``final_layernorm`` on its last; embedding and head are the model's own
  (eredu/src/backend/mlx/architectures/nemotron_h/layerwise.rs:88-330, checkpoint.rs:114-178). The first step's blocks
  draft at every depth.

All compute, for the hidden state ``h_i`` that enters the target's final norm at position i and the token ``t_{i+1}``::

    x = proj(concat(norm_e(embed(t_{i+1})), norm_h(h_i)));  g = block(x) at position i;  logits(t_{i+2}) = head(norm(g))

and ``g`` stands in for the target's hidden state when more than one token is drafted.

The block runs as a one-layer model of the same family (its own paged KV pool of one layer) that receives ``x`` through the
activation input pipeline stages use, so every attention form the family has (latent attention, gated attention, sparse
feed-forward) is the family's own code.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Optional

import torch

from .. import ops


def _layout(cfg, has) -> Optional[dict]:
    """Tensor-name mapping of the one-layer head model, or None when the checkpoint has no usable prediction layer."""
    if cfg.mtp_layers <= 0:
        return None
    L = cfg.num_hidden_layers
    if has("mtp.fc.weight"):
        return {"layer": "mtp.layers.0.", "norm": "mtp.norm.weight", "head": None, "embed": None, "proj": "mtp.fc.weight",
                "norm_e": "mtp.pre_fc_norm_embedding.weight", "norm_h": "mtp.pre_fc_norm_hidden.weight"}
    for root in ("mtp.layers.", "model.mtp.layers."):
        if cfg.model_type == "nemotron_h" and has(root + "0.eh_proj.weight"):
            pattern = str(cfg.extra.get("mtp_hybrid_override_pattern", ""))
            if not pattern or any(ch not in "*E" for ch in pattern):
                raise ValueError("Nemotron-H prediction layers need an mtp_hybrid_override_pattern made of '*' and 'E'")
            P = len(pattern)
            return {"layers": root, "pattern": pattern, "norm": f"{root}{P - 1}.final_layernorm.weight", "head": None, "embed": None,
                    "proj": root + "0.eh_proj.weight", "norm_e": root + "0.enorm.weight", "norm_h": root + "0.hnorm.weight"}
    p = f"model.layers.{L}."
    if has(p + "eh_proj.weight"):
        return {"layer": p, "norm": p + "shared_head.norm.weight",
                "head": p + "shared_head.head.weight" if has(p + "shared_head.head.weight") else None,
                "embed": p + "embed_tokens.weight" if has(p + "embed_tokens.weight") else None,
                "proj": p + "eh_proj.weight", "norm_e": p + "enorm.weight", "norm_h": p + "hnorm.weight"}
    return None


class EmbeddedMtp:
    """The prediction layer of a checkpoint: ``fuse`` makes the block input, ``model`` is the one-layer head model."""

    def __init__(self, model, proj, norm_e, norm_h, embed):
        self.model = model
        self.proj, self.norm_e, self.norm_h, self.embed = proj, norm_e, norm_h, embed
        self.cfg = model.cfg

    def fuse(self, token_ids: torch.Tensor, hidden: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        e = ops.embedding(token_ids, self.embed, 0, cfg.embedding_scale)
        e, _ = ops.rmsnorm(e.contiguous(), self.norm_e, cfg.rms_norm_eps, weight_offset=cfg.norm_weight_offset)
        h, _ = ops.rmsnorm(hidden.to(e.dtype).contiguous(), self.norm_h, cfg.rms_norm_eps, weight_offset=cfg.norm_weight_offset)
        return ops.linear(torch.cat((e, h), dim=-1).contiguous(), self.proj)

    def weight_bytes(self) -> int:
        own = sum(t.numel() * t.element_size() for t in (self.proj, self.norm_e, self.norm_h))
        return own + self.model.weight_bytes()


def head_config(cfg, pattern=None):
    """Configuration of the head model: one full-attention (or latent-attention) block, sparse where the family's later
    layers are; for Nemotron-H the blocks its pattern names ('*' attention, 'E' sparse feed-forward)."""
    extra = {k: v for k, v in cfg.extra.items() if k not in ("mtp_num_hidden_layers", "num_nextn_predict_layers",
                                                             "mtp_hybrid_override_pattern")}
    if pattern:
        marks = {"*": "attention_only", "E": "moe_only"}
        return dataclasses.replace(cfg, num_hidden_layers=len(pattern), layer_types=[marks[ch] for ch in pattern], extra=extra)
    kw = dict(num_hidden_layers=1, extra=extra)
    if cfg.layer_types:
        kw["layer_types"] = ["full_attention"]
    if cfg.is_moe:
        kw["mlp_only_layers"] = []
        kw["decoder_sparse_step"] = 1
    return dataclasses.replace(cfg, **kw)


def build_embedded_mtp(cfg, get: Callable, has: Callable, target, device, dtype, moe_factory=None,
                       quantizer=None) -> Optional[EmbeddedMtp]:
    """Reads the prediction layer next to an already built ``target`` model (single rank). Embedding and vocabulary head
    are the target's own tensors unless the checkpoint stores separate ones for the layer."""
    names = _layout(cfg, has)
    if names is None:
        return None
    from .llama import build_from_tensors

    def remap(name: str) -> str:
        if "layers" in names:                       # several blocks per step: model.layers.j.* -> <root>j.*
            if name.startswith("model.layers."):
                return names["layers"] + name[len("model.layers."):]
        elif name.startswith("model.layers.0."):
            return names["layer"] + name[len("model.layers.0."):]
        if name == "model.norm.weight":
            return names["norm"]
        if name == "lm_head.weight" and names["head"]:
            return names["head"]
        if name == "model.embed_tokens.weight" and names["embed"]:
            return names["embed"]
        return name

    hcfg = head_config(cfg, names.get("pattern"))
    model = build_from_tensors(hcfg, lambda n: get(remap(n)), lambda n: has(remap(n)), device, dtype, None, moe_factory,
                               quantizer)
    # share what the checkpoint shares: no second copy of the vocabulary matrices on the device
    folded = getattr(model, "head_folded", False) or getattr(target, "head_folded", False)
    if names["embed"] is None and target.embed is not None:
        if model.lm_head is model.embed and not folded:
            model.lm_head = target.embed
        model.embed = target.embed
    if names["head"] is None and target.lm_head is not None and not folded:
        # a head with its final norm folded in is specific to that norm: the two models then keep their own copies
        model.lm_head = target.lm_head
    up = lambda n, dt: get(n).to(device=model.device, dtype=dt).contiguous()      # noqa: E731
    return EmbeddedMtp(model, up(names["proj"], dtype), up(names["norm_e"], torch.float32), up(names["norm_h"], torch.float32),
                       model.embed)
