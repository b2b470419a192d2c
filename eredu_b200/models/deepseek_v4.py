"""DeepSeek-V4 text decoder.

Behavioural counterpart of eredu/src/backend/mlx/architectures/deepseek_v4/{attention,layers,model}.rs:

* residual scheme: ``hc_mult`` residual streams per token mixed by hyper-connections (``ops.hyper_connections``); every
  sub-layer reads a learned collapse of the streams and writes back through ``expand``; a hyper-head collapses them
  before the final norm (model.rs:760-782, 916-971);
* attention (attention.rs:878-1078): low-rank query (``wq_a`` -> RMSNorm -> ``wq_b``, a weight-free RMSNorm per head),
  ONE shared key / value head (``wkv`` -> RMSNorm; keys are the values), interleaved RoPE on the trailing
  ``qk_rope_head_dim`` channels of queries and keys and the INVERSE rotation on the attention output, a learned sink
  logit per head, a grouped low-rank output projection (``wo_a`` per group of heads, then ``wo_b``). Three layer kinds by
  ``compress_ratios[layer]``:
    - 0: local - a sliding window over the token keys;
    - r (not 0, not 4): compressed - the window plus every pooled token, where a pooled token is a gated softmax pooling
      of ``r`` consecutive source tokens (``Compressor``: ``wkv`` / ``wgate`` + a learned position term, RMSNorm, RoPE at the
      window's first position with frequencies scaled by r); pooled token i is visible from position p when its window
      is complete, ``i < (p + 1) // r`` (runtime/cache/kv.rs: PoolingCache::make_mask);
    - 4: sparse - overlapping pooling (each pooled token also sees the previous window through a second half of the
      projections) and an indexer (own compressor, ``index_n_heads`` ReLU-scored heads weighted by ``weights_proj``) that
      keeps the ``index_topk`` best pooled tokens per query; with no more pooled tokens than that, all are attended;
* feed-forward (layers.rs): routed SwiGLU experts (clamped: gate <= limit, |up| <= limit) plus an unclamped shared
  expert; router scores ``sqrt(softplus(logits))``, selection by score + correction bias, weights normalised and scaled;
  the first ``num_hash_layers`` layers route by token id through ``tid2eid`` instead of by score.

The local window is applied by position, ``0 <= p - k < sliding_window``, for every call shape (the reference's resident
cache lets a multi-token prefill see its whole call; one-token decode steps are identical), so cached, chunked and
full passes agree exactly here.

The cache of this family is not a paged K / V pool: per layer a token-key tensor, one or two pooled streams and their
open windows. The model therefore runs on ``runtime.unpaged.UnpagedEngine`` (one sequence at a time, tensor operations
around this repository's GEMMs). Not built: the prediction (MTP) layers and the DSpark drafter, tensor / expert
parallelism for this family, FP4 expert banks.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn.functional as F

from .. import ops
from ..ops.hyper_connections import HyperConnection, HyperHead, expand, weightless_rms_norm


@dataclass
class DeepseekV4Config:
    hidden_size: int
    moe_intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    head_dim: int
    qk_rope_head_dim: int
    q_lora_rank: int
    o_lora_rank: int
    o_groups: int
    vocab_size: int
    index_n_heads: int
    index_head_dim: int
    index_topk: int
    n_routed_experts: int
    num_experts_per_tok: int
    max_position_embeddings: int = 65536
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    compress_rope_theta: float = 160000.0
    rope_scaling: Optional[dict] = None
    sliding_window: int = 128
    compress_ratios: list = field(default_factory=list)
    hc_mult: int = 4
    hc_sinkhorn_iters: int = 20
    hc_eps: float = 1e-6
    n_shared_experts: int = 1
    num_hash_layers: int = 0
    norm_topk_prob: bool = True
    routed_scaling_factor: float = 1.0
    swiglu_limit: float = 0.0
    tie_word_embeddings: bool = False

    @classmethod
    def from_dict(cls, d: dict) -> "DeepseekV4Config":
        import dataclasses

        known = {k: d[k] for k in cls.__dataclass_fields__ if k in d and d[k] is not None}
        missing = [f.name for f in dataclasses.fields(cls)
                   if f.name not in known and f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING]
        if missing:
            raise ValueError(f"DeepSeek-V4 config lacks {missing}")
        cfg = cls(**known)
        cfg.compress_ratios = [int(r) for r in (cfg.compress_ratios or [0] * cfg.num_hidden_layers)]
        if len(cfg.compress_ratios) < cfg.num_hidden_layers:
            raise ValueError("compress_ratios must name every layer")
        if cfg.num_attention_heads % cfg.o_groups:
            raise ValueError("attention heads must divide into the output groups")
        if str(d.get("scoring_func", "sqrtsoftplus")).lower() not in ("sqrtsoftplus", "sqrt_softplus"):
            raise ValueError(f"unsupported DeepSeek-V4 router scoring {d.get('scoring_func')!r}")
        return cfg


def _rms(x, w, eps):
    return (weightless_rms_norm(x.float(), eps) * w.float()).to(x.dtype)


class _Rope:
    """Interleaved rotation of the trailing ``dims`` channels; YaRN blends the frequencies of compressed layers
    (attention.rs:41-121). ``scale``: positions advance by ``scale`` source tokens per index (pooled streams)."""

    def __init__(self, cfg: DeepseekV4Config, base: float, yarn: bool, device):
        dims = cfg.qk_rope_head_dim
        inv = [1.0 / base ** (i / dims) for i in range(0, dims, 2)]
        rs = cfg.rope_scaling
        if yarn and rs:
            factor = float(rs["factor"])
            orig = float(rs["original_max_position_embeddings"])

            def correction(rot):
                return dims * math.log(orig / (rot * 2 * math.pi)) / (2 * math.log(base))

            low = max(math.floor(correction(float(rs.get("beta_fast", 32)))), 0.0)
            high = min(math.ceil(correction(float(rs.get("beta_slow", 1)))), dims - 1.0)
            if low == high:
                high += 0.001
            for i in range(len(inv)):
                ramp = min(max((i - low) / (high - low), 0.0), 1.0)
                smooth = 1.0 - ramp
                inv[i] = inv[i] / factor * (1.0 - smooth) + inv[i] * smooth
        self.inv = torch.tensor(inv, dtype=torch.float32, device=device)
        self.dims = dims

    def __call__(self, x, positions, inverse=False):
        """x [T, ..., D]; positions [T] (source-token positions)."""
        ang = positions.float()[:, None] * self.inv[None, :]
        if inverse:
            ang = -ang
        shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (self.dims // 2,)
        cos, sin = ang.cos().view(shape), ang.sin().view(shape)
        xf = x.float()
        head, tail = xf[..., :x.shape[-1] - self.dims], xf[..., x.shape[-1] - self.dims:]
        a, b = tail[..., 0::2], tail[..., 1::2]
        rot = torch.stack((a * cos - b * sin, a * sin + b * cos), -1).flatten(-2)
        return torch.cat((head, rot), -1).to(x.dtype)


class PoolingState:
    """An append-only pooled stream with its open window (runtime/cache/kv.rs: PoolingCache)."""

    def __init__(self):
        self.pending_values = self.pending_gates = None      # [< ratio, width]
        self.overlap_values = self.overlap_gates = None      # [ratio, head_dim]: first half of the last complete window
        self.pooled = None                                   # [P, head_dim]
        self.processed = 0

    def clone(self):
        c = PoolingState()
        for k, v in vars(self).items():
            setattr(c, k, v.clone() if torch.is_tensor(v) else v)
        return c


class _Compressor:
    def __init__(self, cfg, ratio, head_dim, get, prefix, up, device):
        self.ratio, self.head_dim, self.overlap = ratio, head_dim, ratio == 4
        self.wkv, self.wgate = up(get(prefix + "wkv.weight")), up(get(prefix + "wgate.weight"))
        self.ape = get(prefix + "ape").to(device=device, dtype=torch.float32)
        self.norm = get(prefix + "norm.weight").to(device=device, dtype=torch.float32)
        self.rope = _Rope(cfg, cfg.compress_rope_theta, True, device)
        self.eps = cfg.rms_norm_eps
        width = head_dim * (2 if self.overlap else 1)
        if tuple(self.wkv.shape) != (width, cfg.hidden_size) or tuple(self.ape.shape) != (ratio, width):
            raise ValueError(f"{prefix}: compressor tensors do not match ratio {ratio} and head size {head_dim}")

    def __call__(self, x, state: PoolingState, offset: int):
        """x [T, H] at source positions offset ..; appends the newly completed pooled tokens and returns all of them."""
        if offset != state.processed:
            raise ValueError(f"pooling stream expected source offset {state.processed}, got {offset}")
        r, D = self.ratio, self.head_dim
        values, gates = ops.linear(x, self.wkv).float(), ops.linear(x, self.wgate).float()
        pend = 0 if state.pending_values is None else state.pending_values.shape[0]
        if pend:
            values, gates = torch.cat((state.pending_values, values)), torch.cat((state.pending_gates, gates))
        total = values.shape[0]
        usable = total // r * r
        state.processed += total - pend
        state.pending_values = values[usable:] if usable < total else None
        state.pending_gates = gates[usable:] if usable < total else None
        base = offset - pend
        if usable:
            n = usable // r
            v = values[:usable].view(n, r, -1)
            g = gates[:usable].view(n, r, -1) + self.ape
            if self.overlap:
                first_v = state.overlap_values[None] if state.overlap_values is not None else v.new_zeros(1, r, D)
                first_g = state.overlap_gates[None] if state.overlap_gates is not None else g.new_full((1, r, D), float("-inf"))
                prev_v, prev_g = torch.cat((first_v, v[:-1, :, :D])), torch.cat((first_g, g[:-1, :, :D]))
                state.overlap_values, state.overlap_gates = v[-1, :, :D].clone(), g[-1, :, :D].clone()
                v, g = torch.cat((prev_v, v[:, :, D:]), 1), torch.cat((prev_g, g[:, :, D:]), 1)
            pooled = (v * torch.softmax(g, dim=1)).sum(1)                                   # [n, D]
            pooled = weightless_rms_norm(pooled, self.eps) * self.norm
            # pooled token i stands at source position base + i * r (frequencies scaled by r over index base / r + i)
            pos = torch.arange(n, device=x.device) * r + (base // r) * r
            pooled = self.rope(pooled[:, None, :], pos)[:, 0].to(x.dtype)
            state.pooled = pooled if state.pooled is None else torch.cat((state.pooled, pooled))
        if state.pooled is None:
            return x.new_zeros((0, D))
        return state.pooled


class LayerCache:
    def __init__(self, ratio):
        self.keys = None                                     # [n, D] token keys (= values) of every position so far
        self.pool = PoolingState() if ratio else None
        self.index_pool = PoolingState() if ratio == 4 else None

    def clone(self):
        c = LayerCache(0)
        c.keys = None if self.keys is None else self.keys.clone()
        c.pool = None if self.pool is None else self.pool.clone()
        c.index_pool = None if self.index_pool is None else self.index_pool.clone()
        return c


class SequenceCache:
    def __init__(self, ratios):
        self.layers = [LayerCache(r) for r in ratios]
        self.length = 0

    def clone(self):
        c = SequenceCache([])
        c.layers, c.length = [l.clone() for l in self.layers], self.length
        return c


class DeepseekV4Model:
    def __init__(self, cfg: DeepseekV4Config, get, has, device="cpu", dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        up = lambda t, dt=None: t.to(device=self.device, dtype=dt or dtype).contiguous()          # noqa: E731
        f32 = lambda n: up(get(n), torch.float32)                                                  # noqa: E731
        H, n = cfg.hidden_size, cfg.hc_mult
        self.embed = up(get("embed.weight"))
        self.norm = f32("norm.weight")
        self.head = self.embed if cfg.tie_word_embeddings and not has("head.weight") else up(get("head.weight"))
        self.hc_head = HyperHead(f32("hc_head_fn"), f32("hc_head_base"), f32("hc_head_scale"), n, H, cfg.rms_norm_eps, cfg.hc_eps)
        self.layers = []
        for li in range(cfg.num_hidden_layers):
            p = f"layers.{li}."
            ratio = cfg.compress_ratios[li]
            w = {"ratio": ratio}
            for kind in ("attn", "ffn"):
                w[kind + "_hc"] = HyperConnection(f32(p + f"hc_{kind}_fn"), f32(p + f"hc_{kind}_base"), f32(p + f"hc_{kind}_scale"),
                                                  n, H, cfg.hc_sinkhorn_iters, cfg.hc_eps)
                w[kind + "_norm"] = f32(p + kind + "_norm.weight")
            a = p + "attn."
            for name in ("wq_a", "wq_b", "wkv", "wo_b"):
                w[name] = up(get(a + name + ".weight"))
            wo_a = get(a + "wo_a.weight")
            if tuple(wo_a.shape) != (cfg.o_groups * cfg.o_lora_rank, cfg.num_attention_heads * cfg.head_dim // cfg.o_groups):
                raise ValueError(f"{a}wo_a.weight has shape {tuple(wo_a.shape)}")
            w["wo_a"] = up(wo_a).view(cfg.o_groups, cfg.o_lora_rank, -1)
            w["q_norm"], w["kv_norm"] = f32(a + "q_norm.weight"), f32(a + "kv_norm.weight")
            w["sink"] = f32(a + "attn_sink")
            w["rope"] = _Rope(cfg, cfg.compress_rope_theta if ratio else cfg.rope_theta, ratio != 0, self.device)
            if ratio:
                w["compressor"] = _Compressor(cfg, ratio, cfg.head_dim, get, a + "compressor.", up, self.device)
            if ratio == 4:
                w["idx_wq_b"] = up(get(a + "indexer.wq_b.weight"))
                w["idx_weights"] = up(get(a + "indexer.weights_proj.weight"))
                w["idx_compressor"] = _Compressor(cfg, ratio, cfg.index_head_dim, get, a + "indexer.compressor.", up, self.device)
            f = p + "ffn."
            w["gate"] = f32(f + "gate.weight")
            w["tid2eid"] = get(f + "gate.tid2eid").to(device=self.device, dtype=torch.int64) if li < cfg.num_hash_layers else None
            w["gate_bias"] = f32(f + "gate.bias") if li >= cfg.num_hash_layers and has(f + "gate.bias") else None
            w["shared_gu"] = up(torch.cat((get(f + "shared_experts.w1.weight"), get(f + "shared_experts.w3.weight")), 0))
            w["shared_dn"] = up(get(f + "shared_experts.w2.weight"))
            if has(f + "experts.gate_up_proj"):              # stacked banks [E, 2 I, H] / [E, H, I]
                w["egu"], w["edn"] = up(get(f + "experts.gate_up_proj")), up(get(f + "experts.down_proj"))
            else:
                w["egu"] = up(torch.stack([torch.cat((get(f + f"experts.{e}.w1.weight"), get(f + f"experts.{e}.w3.weight")), 0)
                                           for e in range(cfg.n_routed_experts)]))
                w["edn"] = up(torch.stack([get(f + f"experts.{e}.w2.weight") for e in range(cfg.n_routed_experts)]))
            self.layers.append(w)

    # ------------------------------------------------------------------ cache
    def new_cache(self) -> SequenceCache:
        return SequenceCache(self.cfg.compress_ratios[:self.cfg.num_hidden_layers])

    # ------------------------------------------------------------------ attention
    def _attention(self, w, x, cache: LayerCache, offset: int):
        cfg = self.cfg
        T = x.shape[0]
        Hq, D = cfg.num_attention_heads, cfg.head_dim
        pos = torch.arange(offset, offset + T, device=x.device)
        qr = _rms(ops.linear(x, w["wq_a"]), w["q_norm"], cfg.rms_norm_eps)
        q = weightless_rms_norm(ops.linear(qr, w["wq_b"]).float().view(T, Hq, D), cfg.rms_norm_eps)
        q = w["rope"](q, pos)                                                              # fp32 [T, Hq, D]
        kv = w["rope"](_rms(ops.linear(x, w["wkv"]), w["kv_norm"], cfg.rms_norm_eps)[:, None, :], pos)[:, 0]
        cache.keys = kv if cache.keys is None else torch.cat((cache.keys, kv))
        keys = cache.keys.float()                                                          # [n, D]
        kpos = torch.arange(keys.shape[0], device=x.device)
        dist = pos[:, None] - kpos[None, :]
        local_ok = (dist >= 0) & (dist < cfg.sliding_window)                               # [T, n]
        scale = D ** -0.5
        local_scores = torch.einsum("thd,kd->htk", q, keys) * scale
        local_scores = local_scores.masked_fill(~local_ok[None], float("-inf"))
        sink = w["sink"][:, None, None].expand(Hq, T, 1)
        ratio = w["ratio"]
        if ratio == 0:
            probs = torch.softmax(torch.cat((local_scores, sink), -1), -1)
            out = torch.einsum("htk,kd->thd", probs[..., :-1], keys)
        else:
            pooled = w["compressor"](x, cache.pool, offset).float()                        # [P, D]
            P = pooled.shape[0]
            visible = torch.arange(P, device=x.device)[None, :] < ((pos + 1) // ratio)[:, None]      # [T, P]
            selected = None
            if ratio == 4:
                idx_pooled = w["idx_compressor"](x, cache.index_pool, offset).float()      # [P, Di]
                if P > cfg.index_topk:
                    Hi, Di = cfg.index_n_heads, cfg.index_head_dim
                    qi = w["rope"](ops.linear(qr, w["idx_wq_b"]).float().view(T, Hi, Di), pos)
                    s = torch.relu(torch.einsum("thd,pd->thp", qi, idx_pooled)) * (Di ** -0.5)
                    hw = ops.linear(x, w["idx_weights"]).float() * (Hi ** -0.5)            # [T, Hi]
                    s = (s * hw[:, :, None]).sum(1).masked_fill(~visible, float("-inf"))   # [T, P]
                    selected = torch.topk(s, cfg.index_topk, dim=-1).indices               # [T, k]
            if selected is None:
                pooled_scores = torch.einsum("thd,pd->htp", q, pooled) * scale
                pooled_scores = pooled_scores.masked_fill(~visible[None], float("-inf"))
                probs = torch.softmax(torch.cat((local_scores, pooled_scores, sink), -1), -1)
                n = keys.shape[0]
                out = torch.einsum("htk,kd->thd", probs[..., :n], keys) + torch.einsum("htp,pd->thd", probs[..., n:n + P], pooled)
            else:
                sel = pooled[selected]                                                     # [T, k, D]
                sel_ok = torch.gather(visible, 1, selected)                                # [T, k]
                pooled_scores = torch.einsum("thd,tkd->htk", q, sel) * scale
                pooled_scores = pooled_scores.masked_fill(~sel_ok[None], float("-inf"))
                probs = torch.softmax(torch.cat((local_scores, pooled_scores, sink), -1), -1)
                n, k = keys.shape[0], selected.shape[1]
                out = torch.einsum("htk,kd->thd", probs[..., :n], keys) + torch.einsum("htk,tkd->thd", probs[..., n:n + k], sel)
        out = w["rope"](out, pos, inverse=True)                                            # the values carried the key rotation
        G = cfg.o_groups
        grouped = out.reshape(T, G, (Hq // G) * D).to(self.dtype)
        low = torch.einsum("tgi,gri->tgr", grouped.float(), w["wo_a"].float()).reshape(T, G * cfg.o_lora_rank).to(self.dtype)
        return ops.linear(low, w["wo_b"])

    # ------------------------------------------------------------------ feed-forward
    def _ffn(self, w, x, token_ids):
        cfg = self.cfg
        T = x.shape[0]
        scores = torch.sqrt(F.softplus(x.float() @ w["gate"].t()))
        if w["tid2eid"] is not None:
            ids = w["tid2eid"][token_ids.long()]                                           # [T, k]
        else:
            choose = scores if w["gate_bias"] is None else scores + w["gate_bias"]
            ids = torch.topk(choose, cfg.num_experts_per_tok, dim=-1).indices
        wt = torch.gather(scores, 1, ids)
        if cfg.norm_topk_prob:
            wt = wt / (wt.sum(-1, keepdim=True) + 1e-20)
        wt = wt * cfg.routed_scaling_factor
        y = torch.zeros((T, cfg.hidden_size), dtype=torch.float32, device=x.device)
        lim = cfg.swiglu_limit
        for e in ids.unique().tolist():
            rows, slot = (ids == e).nonzero(as_tuple=True)
            gu = ops.linear(x[rows], w["egu"][e]).float()
            inter = gu.shape[1] // 2
            g, u = gu[:, :inter], gu[:, inter:]
            if lim > 0:
                g, u = g.clamp(max=lim), u.clamp(-lim, lim)
            out = ops.linear((F.silu(g) * u).to(self.dtype), w["edn"][e]).float()
            y.index_add_(0, rows, out * wt[rows, slot, None])
        sgu = ops.linear(x, w["shared_gu"]).float()
        si = sgu.shape[1] // 2
        shared = ops.linear((F.silu(sgu[:, :si]) * sgu[:, si:]).to(self.dtype), w["shared_dn"]).float()
        return (y + shared).to(self.dtype)

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, token_ids, cache: SequenceCache, all_rows: bool = False):
        """Feeds ``token_ids`` [T] behind the cached prefix. Returns fp32 logits of the last row ([V]) or of all rows."""
        cfg = self.cfg
        token_ids = torch.as_tensor(token_ids, device=self.device)
        offset = cache.length
        h = self.embed[token_ids.long()].to(self.dtype)
        streams = h[:, None, :].expand(-1, cfg.hc_mult, -1).contiguous()
        for w, lc in zip(self.layers, cache.layers):
            x, post, comb = w["attn_hc"].collapse(streams, cfg.rms_norm_eps)
            a = self._attention(w, _rms(x, w["attn_norm"], cfg.rms_norm_eps), lc, offset)
            streams = expand(a, streams, post, comb)
            x, post, comb = w["ffn_hc"].collapse(streams, cfg.rms_norm_eps)
            f = self._ffn(w, _rms(x, w["ffn_norm"], cfg.rms_norm_eps), token_ids)
            streams = expand(f, streams, post, comb)
        cache.length = offset + token_ids.shape[0]
        hidden = _rms(self.hc_head(streams), self.norm, cfg.rms_norm_eps)
        if not all_rows:
            hidden = hidden[-1:]
        logits = ops.linear(hidden, self.head, out_dtype=torch.float32)
        return logits if all_rows else logits[0]
