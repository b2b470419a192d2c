"""Inkling text decoder (``model_type: inkling_mm_model``).

Behavioural counterpart of eredu/src/backend/mlx/architectures/inkling/model.rs (text side):

* no rotary embedding: position enters through a learned relative term. ``r_proj`` gives every query head a ``d_rel``-wide
  code; ``rel_proj [d_rel, extent]`` turns it into one bias per distance 0 .. extent - 1 (extent = the window on sliding
  layers, ``rel_extent`` on global ones), added to the scores; beyond the extent the bias is zero (model.rs:1377-1425);
* scores are ``q . k / head_dim`` (not its square root) with per-head RMSNorm on q and k; global layers multiply the query
  and the bias by ``1 + alpha * log(max((position + 1) / n_floor, 1))`` (model.rs:1351-1374);
* sliding layers have their own head counts (``swa_*``) and an exact window ``0 <= p - k < window``;
* four depthwise causal convolutions with a skip per layer - on the projected keys, on the projected values, on the
  attention output and on the feed-forward output - each with a ``kernel - 1`` token state (model.rs:1467-1478,
  2165-2204; nn/convolution.rs:87-111);
* feed-forward: dense SwiGLU (times a learned global scale) on the first ``dense_mlp_idx`` layers, otherwise routed
  experts chosen by ``sigmoid(logit) + bias``; the weights of the chosen experts AND of the shared experts come from one
  softmax over the log-sigmoids of their logits, times ``route_scale`` and a learned global scale (model.rs:1514-1531);
* the embedding is RMS-normalised; logits are taken from ``hidden / logits_mup_width_multiplier`` and cut to the unpadded
  vocabulary (model.rs:2769-2806).

Tensor names: the canonical ``model.layers.N.self_attn.*`` spelling or the released ``model.llm.layers.N.attn.*`` one
(architectures/inkling/checkpoint.rs:35-330). Canonical fused ``gate_up`` banks hold the gate rows first; the released
``w13`` tensors interleave gate and up rows and are de-interleaved at load.

The per-layer state (keys, values and four convolution tails) is kept per sequence; the family runs on
``runtime.unpaged.UnpagedEngine``.

Media ingress (model.rs:2808-3243, processor.rs:237-284): images are cut into 40 x 40 patches (row-major, one extra column,
missing pixels at raw value -1, CLIP normalisation, each patch doubled in time) and every patch becomes ONE soft token
through the hMLP tower - four linear layers that fold 5 x 5, 2 x 2, 4 x 4 pixel neighbourhoods and finally the two time
steps into the channel dimension, RMSNorm + GELU between them, an RMSNorm at the end; audio arrives as frames of
``num_codebooks`` discrete ids, a frame's soft token is the RMSNorm of the sum of its codebook embeddings. Soft tokens
replace the (normalised) embeddings at the image / audio placeholder ids.

Not built: the dMel audio front end (waveform to codebook ids), the prediction layers, tensor / expert parallelism, GGUF
checkpoints of this family.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn.functional as F

from .. import ops


@dataclass
class InklingConfig:
    hidden_size: int
    num_hidden_layers: int
    vocab_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    sliding_window_size: int
    sconv_kernel_size: int
    rel_extent: int
    d_rel: int
    intermediate_size: int
    n_routed_experts: int
    num_experts_per_tok: int
    n_shared_experts: int
    swa_num_attention_heads: Optional[int] = None
    swa_num_key_value_heads: Optional[int] = None
    swa_head_dim: Optional[int] = None
    local_layers: list = field(default_factory=list)        # per layer: sliding?
    dense_layers: list = field(default_factory=list)        # per layer: dense feed-forward?
    log_scaling_n_floor: Optional[int] = None
    log_scaling_alpha: float = 0.0
    rms_norm_eps: float = 1e-6
    unpadded_vocab_size: Optional[int] = None
    logits_mup_width_multiplier: float = 1.0
    dense_intermediate_size: Optional[int] = None
    moe_intermediate_size: Optional[int] = None
    route_scale: float = 1.0

    @classmethod
    def from_dict(cls, d: dict) -> "InklingConfig":
        import dataclasses

        t = dict(d.get("text_config") or d)
        for flag in ("use_sconv", "use_embed_norm", "shared_expert_sink", "use_gate_bias", "norm_after_topk", "use_global_scale"):
            if not t.get(flag, True):
                raise ValueError(f"Inkling config turns off {flag}: only the released variant is supported")
        if t.get("gate_activation", "sigmoid") != "sigmoid" or t.get("hidden_act", "silu") != "silu" or t.get("q_bias") or t.get("o_bias") \
                or (t.get("final_logit_softcapping") or 0.0) != 0.0:
            raise ValueError("Inkling config uses an unsupported attention, routing or logit variant")
        L = int(t["num_hidden_layers"])
        local = None
        if t.get("local_layer_ids") is not None:
            ids = [int(i) for i in t["local_layer_ids"]]
            if any(i < 0 or i >= L for i in ids) or len(set(ids)) != len(ids):
                raise ValueError("Inkling local_layer_ids must be distinct layers of the model")
            local = [i in ids for i in range(L)]
        if t.get("layer_types") is not None:
            kinds = list(t["layer_types"])
            if len(kinds) != L or any(k not in ("sliding_attention", "full_attention") for k in kinds):
                raise ValueError("Inkling layer_types must name sliding_attention or full_attention for every layer")
            by_type = [k == "sliding_attention" for k in kinds]
            if local is not None and local != by_type:
                raise ValueError("Inkling local_layer_ids conflicts with layer_types")
            local = by_type
        dense = None
        if t.get("mlp_layer_types") is not None:
            kinds = list(t["mlp_layer_types"])
            if len(kinds) != L or any(k not in ("dense", "moe") for k in kinds):
                raise ValueError("Inkling mlp_layer_types must name dense or moe for every layer")
            dense = [k == "dense" for k in kinds]
        if t.get("dense_mlp_idx") is not None:
            th = int(t["dense_mlp_idx"])
            if th < 0 or th > L:
                raise ValueError("Inkling dense_mlp_idx is outside the model")
            by_th = [i < th for i in range(L)]
            if dense is not None and dense != by_th:
                raise ValueError("Inkling dense_mlp_idx conflicts with mlp_layer_types")
            dense = by_th
        known = {f.name: t[f.name] for f in dataclasses.fields(cls) if f.name in t and t[f.name] is not None}
        missing = [f.name for f in dataclasses.fields(cls)
                   if f.name not in known and f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING]
        if missing:
            raise ValueError(f"Inkling config lacks {missing}")
        cfg = cls(**known)
        cfg.local_layers = local if local is not None else [False] * L
        cfg.dense_layers = dense if dense is not None else [False] * L
        for loc in (False, True):
            hq, hkv, D = cfg.heads(loc)
            if hq <= 0 or hkv <= 0 or hq % hkv or (loc and D != cfg.head_dim):
                raise ValueError("Inkling attention head geometry is inconsistent")
        return cfg

    def heads(self, local: bool):
        if local:
            return (self.swa_num_attention_heads or self.num_attention_heads,
                    self.swa_num_key_value_heads or self.num_key_value_heads, self.swa_head_dim or self.head_dim)
        return self.num_attention_heads, self.num_key_value_heads, self.head_dim


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


class _ShortConv:
    """Depthwise causal convolution plus the input itself, in fp32; ``state`` holds the last ``kernel - 1`` inputs."""

    def __init__(self, weight):
        self.weight = weight.float()                         # [C, 1, K]
        self.k = weight.shape[-1]

    def __call__(self, x, state):
        xf = x.float()
        C = xf.shape[1]
        tail = state if state is not None else xf.new_zeros((self.k - 1, C))
        padded = torch.cat((tail, xf))
        y = F.conv1d(padded.t()[None], self.weight, groups=C)[0].t()
        return (y + xf).to(x.dtype), padded[padded.shape[0] - (self.k - 1):].clone()


class InklingLayerCache:
    def __init__(self):
        self.k = self.v = None                               # [n, Hkv, D]
        self.conv = [None, None, None, None]                 # keys, values, attention output, feed-forward output

    def clone(self):
        c = InklingLayerCache()
        c.k = None if self.k is None else self.k.clone()
        c.v = None if self.v is None else self.v.clone()
        c.conv = [None if s is None else s.clone() for s in self.conv]
        return c


class InklingCache:
    def __init__(self, layers: int):
        self.layers = [InklingLayerCache() for _ in range(layers)]
        self.length = 0

    def clone(self):
        c = InklingCache(0)
        c.layers, c.length = [l.clone() for l in self.layers], self.length
        return c


class InklingModel:
    def __init__(self, cfg: InklingConfig, get, has, device="cpu", dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        up = lambda t, dt=None: t.to(device=self.device, dtype=dt or dtype).contiguous()          # noqa: E731

        def fetch(canonical, released):
            return get(canonical) if has(canonical) else get(released)

        def present(canonical, released):
            return has(canonical) or has(released)

        def fused(canonical, released, axis):
            """A gate / up bank as [gate rows; up rows]: the canonical tensors hold that, the released ``w13`` tensors
            interleave them row by row - gate on the even rows, up on the odd ones (layerwise.rs:2312-2337, 3987-4003)."""
            if has(canonical):
                return get(canonical)
            t = get(released)
            if t.shape[axis] % 2:
                raise ValueError(f"{released} has an odd interleaved width")
            idx = torch.cat((torch.arange(0, t.shape[axis], 2), torch.arange(1, t.shape[axis], 2)))
            return t.index_select(axis, idx)

        f32 = lambda c, r: up(fetch(c, r), torch.float32)                                           # noqa: E731
        self.embed = up(fetch("model.embed_tokens.weight", "model.llm.embed.weight"))
        self.embed_norm = f32("model.embed_norm.weight", "model.llm.embed_norm.weight")
        self.norm = f32("model.norm.weight", "model.llm.norm.weight")
        self.lm_head = up(fetch("lm_head.weight", "model.llm.unembed.weight"))
        self.layers = []
        for li in range(cfg.num_hidden_layers):
            c, r = f"model.layers.{li}.", f"model.llm.layers.{li}."
            local = cfg.local_layers[li]
            hq, hkv, D = cfg.heads(local)
            w = {"local": local, "hq": hq, "hkv": hkv, "D": D,
                 "extent": cfg.sliding_window_size if local else cfg.rel_extent}
            w["in_norm"] = f32(c + "input_layernorm.weight", r + "attn_norm.weight")
            w["post_norm"] = f32(c + "post_attention_layernorm.weight", r + "mlp_norm.weight")
            for name, rel in (("q_proj", "wq_du"), ("k_proj", "wk_dv"), ("v_proj", "wv_dv"), ("r_proj", "wr_du"), ("o_proj", "wo_ud")):
                w[name] = up(fetch(c + f"self_attn.{name}.weight", r + f"attn.{rel}.weight"))
            w["q_norm"] = f32(c + "self_attn.q_norm.weight", r + "attn.q_norm.weight")
            w["k_norm"] = f32(c + "self_attn.k_norm.weight", r + "attn.k_norm.weight")
            w["rel_proj"] = f32(c + "self_attn.rel_proj", r + "attn.rel_logits_proj.proj")
            if tuple(w["rel_proj"].shape) != (cfg.d_rel, w["extent"]):
                raise ValueError(f"layer {li}: rel_proj has shape {tuple(w['rel_proj'].shape)}, expected {(cfg.d_rel, w['extent'])}")
            w["k_sconv"] = _ShortConv(up(fetch(c + "self_attn.k_sconv.weight", r + "attn.k_sconv.weight"), torch.float32))
            w["v_sconv"] = _ShortConv(up(fetch(c + "self_attn.v_sconv.weight", r + "attn.v_sconv.weight"), torch.float32))
            w["attn_sconv"] = _ShortConv(f32(c + "attn_sconv.weight", r + "attn_sconv.weight"))
            w["mlp_sconv"] = _ShortConv(f32(c + "mlp_sconv.weight", r + "mlp_sconv.weight"))
            if cfg.dense_layers[li]:
                if has(c + "dense.gate_proj.weight"):
                    gu = torch.cat((get(c + "dense.gate_proj.weight"), get(c + "dense.up_proj.weight")), 0)
                else:
                    gu = fused(c + "dense.gate_up_proj.weight", r + "mlp.w13_dn.weight", 0)
                w["dense_gu"] = up(gu)
                w["dense_dn"] = up(fetch(c + "dense.down_proj.weight", r + "mlp.w2_md.weight"))
                w["dense_scale"] = f32(c + "dense_global_scale", r + "mlp.global_scale") \
                    if present(c + "dense_global_scale", r + "mlp.global_scale") else None
            else:
                w["router"] = f32(c + "moe.router.weight", r + "mlp.gate.weight")
                w["router_bias"] = f32(c + "moe.router.bias", r + "mlp.gate.bias")
                w["router_scale"] = f32(c + "moe.router.global_scale", r + "mlp.gate.global_scale")
                w["egu"] = up(fused(c + "moe.experts.gate_up_proj", r + "mlp.experts.w13_weight", 1))
                w["edn"] = up(fetch(c + "moe.experts.down_proj", r + "mlp.experts.w2_weight"))
                w["sgu"] = up(fused(c + "moe.shared_experts.gate_up_proj", r + "mlp.shared_experts.shared_w13_weight", 1))
                w["sdn"] = up(fetch(c + "moe.shared_experts.down_proj", r + "mlp.shared_experts.shared_w2_weight"))
            self.layers.append(w)

    def new_cache(self) -> InklingCache:
        return InklingCache(self.cfg.num_hidden_layers)

    # ------------------------------------------------------------------ attention
    def _attention(self, w, x, lc: InklingLayerCache, offset: int):
        cfg = self.cfg
        T = x.shape[0]
        hq, hkv, D = w["hq"], w["hkv"], w["D"]
        q = ops.linear(x, w["q_proj"])
        k, lc.conv[0] = w["k_sconv"](ops.linear(x, w["k_proj"]), lc.conv[0])
        v, lc.conv[1] = w["v_sconv"](ops.linear(x, w["v_proj"]), lc.conv[1])
        rel = ops.linear(x, w["r_proj"]).float().view(T, hq, cfg.d_rel)
        q = _rms(q.view(T, hq, D), w["q_norm"], cfg.rms_norm_eps).float()
        k = _rms(k.view(T, hkv, D), w["k_norm"], cfg.rms_norm_eps)
        v = v.view(T, hkv, D)
        lc.k = k if lc.k is None else torch.cat((lc.k, k))
        lc.v = v if lc.v is None else torch.cat((lc.v, v))
        keys, values = lc.k.float(), lc.v.float()
        n = keys.shape[0]
        pos = torch.arange(offset, offset + T, device=x.device)
        dist = pos[:, None] - torch.arange(n, device=x.device)[None, :]                    # [T, n]
        valid = dist >= 0
        if w["local"]:
            valid = valid & (dist < cfg.sliding_window_size)
        profiles = torch.einsum("thr,re->the", rel, w["rel_proj"])                         # [T, hq, extent]
        bias = torch.gather(profiles, 2, dist.clamp(0, w["extent"] - 1)[:, None, :].expand(T, hq, n))
        bias = torch.where(((dist >= 0) & (dist < w["extent"]))[:, None, :], bias, torch.zeros((), device=x.device))
        if not w["local"] and cfg.log_scaling_n_floor:
            tau = 1.0 + cfg.log_scaling_alpha * torch.log(((pos + 1).float() / cfg.log_scaling_n_floor).clamp_min(1.0))
            q = q * tau[:, None, None]
            bias = bias * tau[:, None, None]
        g = hq // hkv
        scores = torch.einsum("tkgd,nkd->tkgn", q.view(T, hkv, g, D) / D, keys).reshape(T, hq, n) + bias
        scores = scores.masked_fill(~valid[:, None, :], float("-inf"))
        probs = torch.softmax(scores, -1)
        out = torch.einsum("tkgn,nkd->tkgd", probs.view(T, hkv, g, n), values).reshape(T, hq * D)
        return ops.linear(out.to(self.dtype), w["o_proj"])

    # ------------------------------------------------------------------ feed-forward
    def _swiglu(self, x, gu, dn):
        h = ops.linear(x, gu).float()
        i = h.shape[1] // 2
        return ops.linear((F.silu(h[:, :i]) * h[:, i:]).to(self.dtype), dn).float()

    def _ffn(self, w, x):
        cfg = self.cfg
        if "dense_gu" in w:
            y = self._swiglu(x, w["dense_gu"], w["dense_dn"])
            return (y * w["dense_scale"] if w["dense_scale"] is not None else y).to(self.dtype)
        T = x.shape[0]
        R, S, k = cfg.n_routed_experts, cfg.n_shared_experts, cfg.num_experts_per_tok
        logits = x.float() @ w["router"].t()
        routed, shared = logits[:, :R], logits[:, R:]
        ids = torch.topk(torch.sigmoid(routed) + w["router_bias"], k, dim=-1).indices
        both = torch.cat((torch.gather(routed, 1, ids), shared), -1)
        wt = torch.softmax(F.logsigmoid(both), -1) * cfg.route_scale * w["router_scale"]
        y = torch.zeros((T, cfg.hidden_size), dtype=torch.float32, device=x.device)
        for e in ids.unique().tolist():
            rows, slot = (ids == e).nonzero(as_tuple=True)
            y.index_add_(0, rows, self._swiglu(x[rows], w["egu"][e], w["edn"][e]) * wt[rows, slot, None])
        for s in range(S):
            y += self._swiglu(x, w["sgu"][s], w["sdn"][s]) * wt[:, k + s, None]
        return y.to(self.dtype)

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, token_ids, cache: InklingCache, all_rows: bool = False, embeds=None):
        """``embeds``: (rows, values) from :func:`splice_media` - soft tokens that take the place of the normalised
        embeddings at those rows of this call."""
        cfg = self.cfg
        token_ids = torch.as_tensor(token_ids, device=self.device)
        offset = cache.length
        h = _rms(self.embed[token_ids.long()].to(self.dtype), self.embed_norm, cfg.rms_norm_eps)
        if embeds is not None:
            rows, values = embeds
            h = h.index_copy(0, rows.to(self.device), values.to(device=self.device, dtype=self.dtype))
        for w, lc in zip(self.layers, cache.layers):
            a = self._attention(w, _rms(h, w["in_norm"], cfg.rms_norm_eps), lc, offset)
            a, lc.conv[2] = w["attn_sconv"](a, lc.conv[2])
            h = h + a
            f = self._ffn(w, _rms(h, w["post_norm"], cfg.rms_norm_eps))
            f, lc.conv[3] = w["mlp_sconv"](f, lc.conv[3])
            h = h + f
        cache.length = offset + token_ids.shape[0]
        h = _rms(h, self.norm, cfg.rms_norm_eps)
        if not all_rows:
            h = h[-1:]
        logits = ops.linear((h.float() / cfg.logits_mup_width_multiplier).to(self.dtype), self.lm_head, out_dtype=torch.float32)
        if cfg.unpadded_vocab_size and cfg.unpadded_vocab_size < logits.shape[-1]:
            logits = logits[:, :cfg.unpadded_vocab_size]
        return logits if all_rows else logits[0]


# ---------------------------------------------------------------------------------------------- media ingress
IMAGE_MEAN = (0.48145466, 0.4578275, 0.40821073)
IMAGE_STD = (0.26862954, 0.2613026, 0.2757771)


def image_patches(image: torch.Tensor) -> torch.Tensor:
    """``image`` uint8 / float [H, W, 3] with raw 0..255 values -> [rows * cols, 2, 40, 40, 3]: ``ceil(H / 40)`` rows and
    ``W // 40 + 1`` columns of patches (the released processor keeps a final partial or empty column), pixels beyond the
    image at raw value -1, normalised, both time steps equal."""
    H, W, C = image.shape
    if C != 3:
        raise ValueError("Inkling images are RGB")
    rows, cols = (H + 39) // 40, W // 40 + 1
    canvas = torch.full((rows * 40, cols * 40, 3), -1.0, dtype=torch.float32)
    canvas[:H, :W] = image.float()
    canvas = (canvas / 255.0 - torch.tensor(IMAGE_MEAN)) / torch.tensor(IMAGE_STD)
    p = canvas.view(rows, 40, cols, 40, 3).permute(0, 2, 1, 3, 4).reshape(rows * cols, 1, 40, 40, 3)
    return p.expand(-1, 2, -1, -1, -1).contiguous()


class InklingVision:
    """The hMLP tower: ``[P, 2, 40, 40, 3]`` patches -> ``[P, hidden]`` soft tokens."""

    def __init__(self, vcfg: dict, get, has, device="cpu", dtype=torch.float32):
        H = int(vcfg.get("text_hidden_size", vcfg.get("decoder_dmodel")))
        geometry = (int(vcfg.get("temporal_patch_size", 2)), int(vcfg.get("patch_size", 40)),
                    int(vcfg.get("num_hidden_layers", vcfg.get("n_layers", 4))), int(vcfg.get("num_channels", vcfg.get("n_channels", 3))))
        if geometry != (2, 40, 4, 3) or vcfg.get("vision_encoder_type", "hmlp") != "hmlp":
            raise ValueError(f"the hMLP tower supports (temporal 2, patch 40, 4 layers, 3 channels), got {geometry}")
        second = 320 if H == 4096 else 512
        self.specs = [(75, 128, 1, 5), (512, second, 1, 2), (second * 16, 4800, 1, 4), (9600, H, 2, 1)]
        self.eps = float(vcfg.get("rms_norm_eps", 1e-6))
        self.device, self.dtype = torch.device(device), dtype
        up = lambda t, dt=None: t.to(device=self.device, dtype=dt or dtype).contiguous()          # noqa: E731
        pick = lambda a, b: get(a) if has(a) else get(b)                                            # noqa: E731
        self.layers = []
        for i, (din, dout, _, _) in enumerate(self.specs):
            w = up(pick(f"visual.layers.{i}.projection.weight", f"model.visual.layers.linear_{i}.weight"))
            if tuple(w.shape) != (dout, din):
                raise ValueError(f"hMLP layer {i} has shape {tuple(w.shape)}, expected {(dout, din)}")
            norm = up(pick(f"visual.layers.{i}.layer_norm.weight", f"model.visual.layers.norm_{i}.weight"), torch.float32) \
                if i + 1 < len(self.specs) else None
            self.layers.append((w, norm))
        self.final_norm = up(pick("visual.final_norm.weight", "model.visual.final_norm.weight"), torch.float32)

    @staticmethod
    def _fold(x, t_fold, hw_fold):
        P, T, Hh, Ww, C = x.shape
        if T % t_fold or Hh % hw_fold or Ww % hw_fold:
            raise ValueError(f"fold ({t_fold}, {hw_fold}) does not divide {tuple(x.shape)}")
        x = x.reshape(P, T // t_fold, t_fold, Hh // hw_fold, hw_fold, Ww // hw_fold, hw_fold, C)
        return x.permute(0, 1, 3, 5, 2, 4, 6, 7).reshape(P, T // t_fold, Hh // hw_fold, Ww // hw_fold, t_fold * hw_fold * hw_fold * C)

    @torch.no_grad()
    def __call__(self, patches: torch.Tensor) -> torch.Tensor:
        if patches.dim() != 5 or tuple(patches.shape[1:]) != (2, 40, 40, 3):
            raise ValueError(f"image patches must be [patches, 2, 40, 40, 3], got {tuple(patches.shape)}")
        x = patches.to(self.device, self.dtype)
        for (w, norm), (_, _, tf, hf) in zip(self.layers, self.specs):
            x = self._fold(x, tf, hf)
            lead = x.shape[:-1]
            x = ops.linear(x.reshape(-1, x.shape[-1]).contiguous(), w).view(*lead, w.shape[0])
            if norm is not None:
                x = F.gelu(_rms(x, norm, self.eps).float()).to(self.dtype)
        return _rms(x, self.final_norm, self.eps).reshape(-1, x.shape[-1])


class InklingAudio:
    """Frames of codebook ids ``[frames, codebooks]`` -> ``[frames, hidden]``: summed codebook embeddings, RMS-normalised."""

    def __init__(self, acfg: dict, get, has, device="cpu", dtype=torch.float32):
        self.codebooks = int(acfg.get("num_codebooks", acfg.get("n_mel_bins")))
        self.size = int(acfg.get("codebook_size", acfg.get("mel_vocab_size")))
        self.eps = float(acfg.get("rms_norm_eps", 1e-6))
        self.device, self.dtype = torch.device(device), dtype
        pick = lambda a, b: get(a) if has(a) else get(b)                                            # noqa: E731
        self.table = pick("audio.encoder.weight", "model.audio.encoder.weight").to(device=self.device, dtype=dtype)
        if self.table.shape[0] != self.codebooks * self.size:
            raise ValueError("the audio embedding table does not match the codebook geometry")
        self.final_norm = pick("audio.final_norm.weight", "model.audio.final_norm.weight").to(device=self.device, dtype=torch.float32)

    @torch.no_grad()
    def __call__(self, ids: torch.Tensor, valid_frames=None) -> torch.Tensor:
        if ids.dim() != 2 or ids.shape[1] != self.codebooks:
            raise ValueError(f"audio ids must be [frames, {self.codebooks}], got {tuple(ids.shape)}")
        ids = ids.to(self.device).long()
        if int(ids.min()) < 0 or int(ids.max()) >= self.size:
            raise ValueError("audio id outside its codebook")
        offs = torch.arange(self.codebooks, device=self.device) * self.size
        x = self.table[ids + offs[None, :]].float().sum(1)
        x = _rms(x.to(self.dtype), self.final_norm, self.eps)
        return x if valid_frames is None else x[:int(valid_frames)]


def splice_media(token_ids, image_token_id: int, audio_token_id: int, image_embeds=(), audio_embeds=()):
    """Rows of ``token_ids`` that hold placeholder ids and the soft tokens that replace them, in order of appearance.
    Returns (rows int64 [n], values [n, hidden]) for ``InklingModel.forward(..., embeds=)``."""
    ids = torch.as_tensor(token_ids)
    rows, vals = [], []
    for tid, parts, name in ((image_token_id, image_embeds, "image"), (audio_token_id, audio_embeds, "audio")):
        where = (ids == tid).nonzero(as_tuple=True)[0]
        have = sum(int(p.shape[0]) for p in parts)
        if where.numel() != have:
            raise ValueError(f"{where.numel()} {name} placeholder tokens for {have} {name} soft tokens")
        if have:
            rows.append(where)
            vals.append(torch.cat([p for p in parts]))
    if not rows:
        return None
    return torch.cat(rows), torch.cat(vals)
