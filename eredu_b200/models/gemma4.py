"""Gemma 4 text decoder.

Behavioural counterpart of eredu/src/backend/mlx/architectures/gemma4/model.rs (text side): sandwich-normalised blocks
(norm before AND after attention and FFN), GeGLU FFN (double width on KV-sharing layers when configured), an optional
sparse block that runs NEXT TO the dense FFN, per-layer input embeddings gated into every block, a learned scalar per
layer, soft-capped logits; attention with per-head q / k RMSNorm, an unscaled value norm, score scale 1, sliding and
global layers with their OWN head size, KV head count and RoPE (global: "proportional" - only a leading share of the
frequency pairs rotates), optional keys-as-values on global layers, and a tail of layers that reuse the K/V of the last
earlier layer of their type instead of computing their own.

Head sizes here (256 / 512) have no attention kernel, and the cache geometry differs per layer type: the block is
tensor operations around this repository's GEMMs over sliced views of one paged pool, and the model decodes eagerly.
Tensor parallelism, the vision / audio towers and the external MTP assistant are not built.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import ops


def _rms(x, w, eps):
    xf = x.float()
    y = xf * torch.pow(xf.pow(2).mean(-1, keepdim=True) + eps, -0.5)
    return y if w is None else y * w.float()


def geometry(cfg):
    """Per layer: (is_sliding, head_dim, kv_heads, keys_are_values, donor layer or None)."""
    g = cfg.extra["gemma4"]
    L = cfg.num_hidden_layers
    types = cfg.layer_types
    first_shared = L - int(g.get("num_kv_shared_layers", 0) or 0)
    out = []
    for li in range(L):
        sliding = types[li] == "sliding_attention"
        D = cfg.head_dim if sliding or not g.get("global_head_dim") else int(g["global_head_dim"])
        k_eq_v = bool(g.get("attention_k_eq_v", False)) and not sliding
        nkv = int(g["num_global_key_value_heads"]) if k_eq_v else cfg.num_key_value_heads
        donor = None
        if 0 < first_shared <= li:
            prev = types[:first_shared]
            donor = len(prev) - 1 - prev[::-1].index(types[li])
        out.append((sliding, D, nkv, k_eq_v, donor))
    return out


def rope_tables(cfg):
    """inv_freq [D/2] per layer type; 'proportional' rotates only the first share of the frequency pairs."""
    g = cfg.extra["gemma4"]
    rp = g.get("rope_parameters") or {}
    out = {}
    for kind in set(cfg.layer_types):
        p = rp.get(kind) or {"rope_type": "default", "rope_theta": 10000.0}
        base = float(p.get("rope_theta", 10000.0))
        if p.get("rope_type", "default") == "proportional":
            D = int(g.get("global_head_dim") or cfg.head_dim) if kind == "full_attention" else cfg.head_dim
            n_rot = int(float(p.get("partial_rotary_factor", 1.0)) * D // 2)
            inv = 1.0 / (base ** (torch.arange(0, 2 * n_rot, 2, dtype=torch.float32) / D))
            inv = torch.cat((inv, torch.zeros(D // 2 - n_rot))) / float(p.get("factor", 1.0))
        elif p.get("rope_type", "default") == "default":
            D = cfg.head_dim
            inv = 1.0 / (base ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
        else:
            raise ValueError(f"unsupported Gemma 4 rope type {p.get('rope_type')!r}")
        out[kind] = inv
    return out


def build(model, cfg, get, has, up):
    """Populate ``model.layers`` (one dict of tensors per layer in ``LayerWeights.extra``) and the per-layer-input tables."""
    from .llama import LayerWeights

    g = cfg.extra["gemma4"]
    tp, r = model.par.tp_size, model.par.tp_rank
    geo = geometry(cfg)
    Hq = cfg.num_attention_heads
    if tp > 1:
        # Tensor parallelism: query heads are split evenly; a layer type's key / value heads are split when there are at
        # least as many as ranks and otherwise the one head a rank's queries read is kept (replication); feed-forward
        # and expert intermediates are split by rows / columns. Per-layer-input tables and norms are replicated. The
        # sandwich norms act on complete sums, so every row-parallel projection is reduced before its norm.
        if Hq % tp:
            raise NotImplementedError(f"{Hq} attention heads do not divide over {tp} tensor ranks")
        local = []
        for sliding, D, nkv, k_eq_v, donor in geo:
            if nkv % tp == 0:
                kv0, kvn = r * (nkv // tp), nkv // tp
            elif tp % nkv == 0:
                kv0, kvn = r // (tp // nkv), 1
            else:
                raise NotImplementedError(f"{nkv} key / value heads cannot be laid out over {tp} tensor ranks")
            local.append((sliding, D, kvn, k_eq_v, donor, kv0))
    else:
        local = [t + (0,) for t in geo]
    model.g4_heads = Hq // tp
    model.g4 = {"geometry": [t[:5] for t in local], "inv_freq": {k: v.to(model.device) for k, v in rope_tables(cfg).items()}}
    P = int(g.get("hidden_size_per_layer_input") or 0)
    if P:
        model.g4["embed_per_layer"] = up(get("model.embed_tokens_per_layer.weight"))
        model.g4["ple_proj"] = up(get("model.per_layer_model_projection.weight"))
        model.g4["ple_norm"] = up(get("model.per_layer_projection_norm.weight"), torch.float32)
    for li in range(model.first_layer, model.last_layer):
        p = f"model.layers.{li}."
        f32 = lambda n: up(get(p + n), torch.float32)                                  # noqa: E731
        w = {n: f32(n + ".weight") for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm",
                                             "post_feedforward_layernorm")}
        w["scalar"] = f32("layer_scalar") if has(p + "layer_scalar") else None
        a = "self_attn."
        _, D, kvn, _, _, kv0 = local[li]
        Hl = Hq // tp
        wq, wo = get(p + a + "q_proj.weight"), get(p + a + "o_proj.weight")
        if tp > 1:
            wq, wo = wq[r * Hl * D:(r + 1) * Hl * D], wo[:, r * Hl * D:(r + 1) * Hl * D]
        w["q"], w["o"] = up(wq), up(wo)
        w["q_norm"], w["k_norm"] = f32(a + "q_norm.weight"), f32(a + "k_norm.weight")
        if geo[li][4] is None or has(p + a + "k_proj.weight"):
            kv_rows = (lambda t: t[kv0 * D:(kv0 + kvn) * D]) if tp > 1 else (lambda t: t)
            w["k"] = up(kv_rows(get(p + a + "k_proj.weight")))
            w["v"] = up(kv_rows(get(p + a + "v_proj.weight"))) if has(p + a + "v_proj.weight") else None
        wg, wu, wd = get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight"), get(p + "mlp.down_proj.weight")
        if tp > 1:
            n = wg.shape[0] // tp
            wg, wu, wd = wg[r * n:(r + 1) * n], wu[r * n:(r + 1) * n], wd[:, r * n:(r + 1) * n]
        w["gate_up"] = up(torch.cat((wg, wu), 0))
        w["down"] = up(wd)
        if P:
            w["ple_gate"], w["ple_out"] = up(get(p + "per_layer_input_gate.weight")), up(get(p + "per_layer_projection.weight"))
            w["ple_post"] = f32("post_per_layer_input_norm.weight")
        if g.get("enable_moe_block"):
            w["router_proj"] = up(get(p + "router.proj.weight"))
            w["router_scale"], w["expert_scale"] = f32("router.scale"), f32("router.per_expert_scale")
            egu, edn = get(p + "experts.gate_up_proj"), get(p + "experts.down_proj")          # [E, 2 I, H], [E, H, I]
            if tp > 1:
                ie = egu.shape[1] // 2
                n = ie // tp
                egu = torch.cat((egu[:, r * n:(r + 1) * n], egu[:, ie + r * n:ie + (r + 1) * n]), 1)
                edn = edn[:, :, r * n:(r + 1) * n]
            w["experts_gu"], w["experts_dn"] = up(egu), up(edn)
            for n in ("post_feedforward_layernorm_1", "post_feedforward_layernorm_2", "pre_feedforward_layernorm_2"):
                w[n] = f32(n + ".weight")
        lw = LayerWeights(attn_norm=w["input_layernorm"], wqkv=None, wo=None, ffn_norm=None)
        lw.block_kind = "gemma4"
        lw.extra = w
        model.layers.append(lw)


def per_layer_inputs(model, token_ids, h):
    """[M, L, P]: the token's per-layer embedding plus a projection of its main embedding, normalised and averaged."""
    cfg, g4 = model.cfg, model.g4
    if "embed_per_layer" not in g4:
        return None
    g = cfg.extra["gemma4"]
    P, L = int(g["hidden_size_per_layer_input"]), cfg.num_hidden_layers
    M = token_ids.shape[0]
    emb = g4["embed_per_layer"][token_ids.long()].float().view(M, L, P) * (P ** 0.5)
    proj = (ops.linear(h, g4["ple_proj"]).float() * (cfg.hidden_size ** -0.5)).view(M, L, P)
    proj = _rms(proj, g4["ple_norm"], cfg.rms_norm_eps)
    return (proj + emb) * (2.0 ** -0.5)


def _rope(x, positions, inv_freq):
    ang = positions.float()[:, None] * inv_freq[None, :]
    cos, sin = torch.cat((ang.cos(), ang.cos()), -1)[:, None, :], torch.cat((ang.sin(), ang.sin()), -1)[:, None, :]
    half = x.shape[-1] // 2
    return x * cos + torch.cat((-x[..., half:], x[..., :half]), -1) * sin


def block_forward(model, li, lw, h, batch, kv):
    cfg, w = model.cfg, lw.extra
    g = cfg.extra["gemma4"]
    eps = cfg.rms_norm_eps
    sliding, D, nkv, k_eq_v, donor = model.g4["geometry"][li]
    M = h.shape[0]
    Hq = model.g4_heads
    dt = h.dtype
    tp = model.par.tp_size

    def reduced(partial):
        """Sum of a row-parallel projection over the tensor ranks (the norms that follow need the complete value)."""
        return model.tp_ops.all_reduce(partial.contiguous()) if tp > 1 else partial

    inv = model.g4["inv_freq"][cfg.layer_types[li]]
    x = _rms(h, w["input_layernorm"], eps).to(dt)
    q = _rope(_rms(ops.linear(x, w["q"]).view(M, Hq, D), w["q_norm"], eps), batch.positions, inv)
    src = li if donor is None else donor
    k_pool, v_pool = kv.layer(src)
    k_cache, v_cache = k_pool[:, :nkv, :, :D], v_pool[:, :nkv, :, :D]           # this layer type's slice of the shared pool
    if donor is None:
        k_raw = ops.linear(x, w["k"]).view(M, nkv, D)
        v_raw = k_raw if w.get("v") is None else ops.linear(x, w["v"]).view(M, nkv, D)
        k = _rope(_rms(k_raw, w["k_norm"], eps), batch.positions, inv)
        v = _rms(v_raw, None, eps)
        ok = batch.slots >= 0
        page, off = batch.slots[ok] // ops.PAGE, batch.slots[ok] % ops.PAGE
        k_cache[page, :, off] = k[ok].to(k_cache.dtype)
        v_cache[page, :, off] = v[ok].to(v_cache.dtype)
    q_lens = (batch.cu_q[1:] - batch.cu_q[:-1]).tolist() if batch.is_prefill else [batch.q_per_seq] * batch.seq_lens.shape[0]
    attn = ops.attention_ref(q.to(dt), k_cache, v_cache, batch.block_table, batch.seq_lens, q_lens, 1.0,
                             window=int(cfg.sliding_window or 0) if sliding else 0, bidir=batch.bidir_groups)
    a = reduced(ops.linear(attn.reshape(M, Hq * D).to(dt), w["o"]))
    h = h + _rms(a, w["post_attention_layernorm"], eps).to(dt)

    res = h
    y = _rms(h, w["pre_feedforward_layernorm"], eps).to(dt)
    gu = ops.linear(y, w["gate_up"]).float()
    inter = gu.shape[1] // 2
    y = reduced(ops.linear((F.gelu(gu[:, :inter], approximate="tanh") * gu[:, inter:]).to(dt), w["down"]))
    if "router_proj" in w:
        y1 = _rms(y, w["post_feedforward_layernorm_1"], eps)
        r = _rms(res, None, eps) * w["router_scale"] * (cfg.hidden_size ** -0.5)
        probs = torch.softmax(ops.linear(r.to(dt), w["router_proj"]).float(), -1)
        top_w, top_i = torch.topk(probs, int(g["top_k_experts"]), dim=-1)
        top_w = top_w / top_w.sum(-1, keepdim=True) * w["expert_scale"][top_i]
        z = _rms(res, w["pre_feedforward_layernorm_2"], eps).to(dt)
        y2 = torch.zeros((M, cfg.hidden_size), dtype=torch.float32, device=h.device)
        for e in top_i.unique().tolist():
            rows, slot = (top_i == e).nonzero(as_tuple=True)
            eu = ops.linear(z[rows], w["experts_gu"][e]).float()
            ie = eu.shape[1] // 2
            out = ops.linear((F.gelu(eu[:, :ie], approximate="tanh") * eu[:, ie:]).to(dt), w["experts_dn"][e]).float()
            y2.index_add_(0, rows, out * top_w[rows, slot, None])
        y2 = reduced(y2.to(dt)).float() if tp > 1 else y2
        y = (y1 + _rms(y2, w["post_feedforward_layernorm_2"], eps)).to(dt)
    h = res + _rms(y, w["post_feedforward_layernorm"], eps).to(dt)

    if "ple_gate" in w:
        gate = F.gelu(ops.linear(h, w["ple_gate"]).float(), approximate="tanh") * batch.per_layer_inputs[:, li]
        h = h + _rms(ops.linear(gate.to(dt), w["ple_out"]), w["ple_post"], eps).to(dt)
    if w["scalar"] is not None:
        h = (h.float() * w["scalar"]).to(dt)
    return h
