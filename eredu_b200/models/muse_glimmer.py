"""Muse-Glimmer text decoder (``model_type: muse_glimmer``; the decoder sits under ``model.language_model.*``).

Behavioural counterpart of eredu/src/backend/mlx/architectures/muse_glimmer/mod.rs (dense text side):

* the token embedding goes through a weight-free RMSNorm (mod.rs:1700-1702);
* sandwich-normalised blocks: norms before AND after attention and feed-forward, the two "post" norms with their own
  epsilon; the released checkpoints store ``scale - 1`` in the four block norms ("centered" weights, mod.rs:530-549), the
  final norm stores its scale as is;
* attention (mod.rs:864-905, 727-757): weight-free RMSNorm per head on queries and keys, queries times
  ``qk_scale_factor``, scores times ``1 / sqrt(head_dim)``; rotary embedding only on the layers whose entry in
  ``layer_rope_theta`` is non-zero; sliding-window layers by ``layer_types``; the attended values are multiplied by
  ``sigmoid(gate_proj(x))`` before the output projection;
* SwiGLU feed-forward; logits are ``softcap * tanh(logits * output_multiplier / softcap)`` (mod.rs:551-559).

The key / value cache is an ordinary grouped-query cache, so the family runs on the paged engine (batching, prefix reuse,
sampling kernels); the block is tensor operations around this repository's GEMMs over the paged pool, with the attention
kernels (tcgen05 prefill, split-KV decode) for head sizes 64 and 128; the dense variant's decode step is captured in a
CUDA graph. The routed-expert variant of the feed-forward (softmax top-k over fused expert banks) runs as a loop over
the chosen experts and decodes eagerly. The vision tower lives in ``muse_glimmer_vision.py``, the DFlash block
drafter in ``dflash.py``. Under tensor parallelism heads, the output gate and the feed-forward rows are split and every
row-parallel sum is taken before its norm.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import ops


def _wrms(x, eps):
    xf = x.float()
    return xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)


def _rope(x, positions, inv_freq):
    ang = positions.float()[:, None] * inv_freq[None, :]
    cos, sin = torch.cat((ang.cos(), ang.cos()), -1)[:, None, :], torch.cat((ang.sin(), ang.sin()), -1)[:, None, :]
    half = x.shape[-1] // 2
    return x * cos + torch.cat((-x[..., half:], x[..., :half]), -1) * sin


def build(model, cfg, get, has, up):
    from .llama import LayerWeights
    from .rope import rope_tables

    g = cfg.extra["muse_glimmer"]
    # Tensor parallelism: query heads (and the output gate, which has one column per query channel) are split evenly, key /
    # value heads are split or, when there are fewer than ranks, the one head a rank's queries read is kept; feed-forward
    # and expert intermediates are split by rows / columns. The sandwich norms act on complete sums, so every
    # row-parallel projection is reduced before its norm; its bias is added once, after the sum.
    tp, r = model.par.tp_size, model.par.tp_rank
    D = cfg.head_dim
    q0, qn = r * model.n_q_local * D, model.n_q_local * D
    kv0 = (r * model.n_kv_local if model.kv_rep == 1 else r // model.kv_rep) * D
    kvn = model.n_kv_local * D
    rows = {"q_proj": (q0, qn), "gate_proj": (q0, qn), "k_proj": (kv0, kvn), "v_proj": (kv0, kvn)}
    sparse = int(g.get("num_experts") or 0) > 0
    L = cfg.num_hidden_layers
    thetas = list(g.get("layer_rope_theta") or [cfg.rope_theta] * L)
    kinds = list(g.get("layer_types") or ["full_attention"] * L)
    if len(thetas) != L or len(kinds) != L:
        raise ValueError("Muse-Glimmer layer_rope_theta and layer_types must name every layer")
    inv, _ = rope_tables(cfg)
    model.mg = {"inv_freq": inv.to(model.device), "uses_rope": [float(t) != 0.0 for t in thetas],
                "sliding": [k == "sliding_attention" for k in kinds], "post_eps": float(g.get("post_norm_eps") or cfg.rms_norm_eps),
                "qk_scale": float(g.get("qk_scale_factor") or 1.0)}

    def split(n_total):
        if n_total % tp:
            raise NotImplementedError(f"an intermediate size of {n_total} does not divide over {tp} tensor ranks")
        return r * (n_total // tp), n_total // tp

    for li in range(model.first_layer, model.last_layer):
        p = f"model.layers.{li}."
        f32 = lambda n: up(get(p + n), torch.float32)                                  # noqa: E731
        w = {n: 1.0 + f32(n + ".weight") for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm",
                                                   "post_feedforward_layernorm")}       # stored centered: scale - 1
        a = "self_attn."
        for n, (lo, cnt) in rows.items():
            w[n] = up(get(p + a + n + ".weight")[lo:lo + cnt])
            w[n + "_b"] = up(get(p + a + n + ".bias")[lo:lo + cnt]) if has(p + a + n + ".bias") else None
        w["o_proj"] = up(get(p + a + "o_proj.weight")[:, q0:q0 + qn])
        w["o_proj_b"] = up(get(p + a + "o_proj.bias")) if has(p + a + "o_proj.bias") else None
        if sparse:
            # Qwen3-style routed experts (mod.rs:932-1040): softmax over all experts, top-k, optional renormalisation;
            # fused banks [E, 2 I, H] hold the gate rows first
            w["router"] = f32("mlp.gate.weight")
            egu, edn = get(p + "mlp.experts.gate_up_proj"), get(p + "mlp.experts.down_proj")
            inter = egu.shape[1] // 2
            lo, cnt = split(inter)
            w["egu"] = up(torch.cat((egu[:, lo:lo + cnt], egu[:, inter + lo:inter + lo + cnt]), 1))
            w["edn"] = up(edn[:, :, lo:lo + cnt])
        else:
            wg, wu, wd = get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight"), get(p + "mlp.down_proj.weight")
            lo, cnt = split(wg.shape[0])
            w["gate_up"] = up(torch.cat((wg[lo:lo + cnt], wu[lo:lo + cnt]), 0))
            w["down"] = up(wd[:, lo:lo + cnt])
        lw = LayerWeights(attn_norm=w["input_layernorm"], wqkv=None, wo=None, ffn_norm=None)
        lw.block_kind = "muse_glimmer"
        lw.extra = w
        model.layers.append(lw)


def block_forward(model, li, lw, h, batch, kv):
    cfg, w, mg = model.cfg, lw.extra, model.mg
    eps, dt = cfg.rms_norm_eps, h.dtype
    M = h.shape[0]
    Hq, Hkv, D = model.n_q_local, model.n_kv_local, cfg.head_dim
    tp = model.par.tp_size

    def reduced(partial, bias=None):
        """A row-parallel projection: summed over the tensor ranks, its bias added once."""
        if tp > 1:
            partial = model.tp_ops.all_reduce(partial.to(dt).contiguous())
        return partial if bias is None else partial + bias

    x = (_wrms(h, eps) * w["input_layernorm"]).to(dt)
    q = _wrms(ops.linear(x, w["q_proj"], bias=w["q_proj_b"]).view(M, Hq, D), eps) * mg["qk_scale"]
    k = _wrms(ops.linear(x, w["k_proj"], bias=w["k_proj_b"]).view(M, Hkv, D), eps)
    v = ops.linear(x, w["v_proj"], bias=w["v_proj_b"]).view(M, Hkv, D)
    if mg["uses_rope"][li]:
        q, k = _rope(q, batch.positions, mg["inv_freq"]), _rope(k, batch.positions, mg["inv_freq"])
    k_cache, v_cache = kv.layer(li)
    # rows without a slot (padding of a captured decode batch) land in page 0, which no sequence owns: the scatter
    # keeps a fixed shape, so the step can be captured in a CUDA graph
    slot = batch.slots.clamp_min(0)
    page, off = slot // ops.PAGE, slot % ops.PAGE
    k_cache[page, :, off] = k.to(k_cache.dtype)
    v_cache[page, :, off] = v.to(v_cache.dtype)
    window = int(cfg.sliding_window or 0) if mg["sliding"][li] else 0
    if h.is_cuda and D in ops.KERNEL_HEAD_DIMS and dt == torch.bfloat16:
        # head sizes with attention kernels: tcgen05 prefill, split-KV decode (the cache rows were written above)
        qc = q.to(dt).contiguous()
        if batch.is_prefill:
            attn = ops.attention_prefill(qc, k_cache, v_cache, batch.block_table, batch.seq_lens, batch.cu_q, batch.max_q_len,
                                         D ** -0.5, window=window)
        else:
            attn = ops.attention_decode(qc, k_cache, v_cache, batch.block_table, batch.seq_lens, batch.q_per_seq, D ** -0.5,
                                        splits=batch.splits, window=window, scratch=batch.scratch)
    else:
        q_lens = (batch.cu_q[1:] - batch.cu_q[:-1]).tolist() if batch.is_prefill else [batch.q_per_seq] * batch.seq_lens.shape[0]
        attn = ops.attention_ref(q.to(dt), k_cache, v_cache, batch.block_table, batch.seq_lens, q_lens, D ** -0.5, window=window)
    gate = torch.sigmoid(ops.linear(x, w["gate_proj"], bias=w["gate_proj_b"]).float())
    a = reduced(ops.linear((attn.reshape(M, Hq * D).float() * gate).to(dt), w["o_proj"]), w["o_proj_b"])
    h = h + (_wrms(a, mg["post_eps"]) * w["post_attention_layernorm"]).to(dt)
    y = (_wrms(h, eps) * w["pre_feedforward_layernorm"]).to(dt)
    if "router" in w:
        g = cfg.extra["muse_glimmer"]
        probs = torch.softmax(y.float() @ w["router"].t(), -1)
        top_w, top_i = torch.topk(probs, int(g["num_experts_per_tok"]), dim=-1)
        if g.get("norm_topk_prob"):
            top_w = top_w / top_w.sum(-1, keepdim=True)
        out = torch.zeros((M, cfg.hidden_size), dtype=torch.float32, device=h.device)
        for e in top_i.unique().tolist():
            rows, slot = (top_i == e).nonzero(as_tuple=True)
            eu = ops.linear(y[rows], w["egu"][e]).float()
            ie = eu.shape[1] // 2
            out.index_add_(0, rows, ops.linear((F.silu(eu[:, :ie]) * eu[:, ie:]).to(dt), w["edn"][e]).float() * top_w[rows, slot, None])
        y = reduced(out)
    else:
        gu = ops.linear(y, w["gate_up"]).float()
        inter = gu.shape[1] // 2
        y = reduced(ops.linear((F.silu(gu[:, :inter]) * gu[:, inter:]).to(dt), w["down"]))
    return h + (_wrms(y, mg["post_eps"]) * w["post_feedforward_layernorm"]).to(dt)
