"""Qwen3-Next / Qwen3.5 hybrid decoders: gated delta networks ("linear_attention" layers) between gated softmax
attention layers, zero-centred RMSNorm weights, a sparse FFN with a sigmoid-gated shared expert.

Architecture: eredu/src/backend/mlx/architectures/qwen/hybrid/qwen3_5.rs (norms :1391-1457, gated full attention
:1581-1652, linear attention :2015-2084 with its causal convolution :1914-1956 and l2-normalised, 1/sqrt(dk)-scaled
queries :1958-1981, sparse block with shared-expert gate :2927-3275); checkpoint layouts (fused ``in_proj_qkvz`` /
``in_proj_ba`` grouped by key head, or split ``in_proj_qkv`` / ``_z`` / ``_b`` / ``_a``): hybrid/checkpoint.rs:360-440.

Per gated-delta layer and token:  [qkv | z | b | a] = in_proj(norm(x));  qkv <- silu(causal_conv(qkv));
q, k <- l2norm;  q <- q / sqrt(dk);  beta = sigmoid(b);  g = -exp(A_log) * softplus(a + dt_bias);
o = gated_delta_scan(q, k, v, g, beta);  y = out_proj(rmsnorm(o) * w * silu(z)).
The convolution tail and the recurrent matrix of every sequence live in state slots of the KV cache object.
Under tensor parallelism a key head with its value heads is the unit of sharding; the output projection is
row-parallel.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import ops


def split_fused_projections(cfg, qkvz: torch.Tensor, ba: torch.Tensor):
    """De-interleave the fused checkpoint layout: rows are grouped by key head as
    [q (dk) | k (dk) | v (r * dv) | z (r * dv)] and [b (r) | a (r)] with r = value heads per key head."""
    Hk, Hv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    r = Hv // Hk
    H = qkvz.shape[1]
    g = qkvz.view(Hk, 2 * dk + 2 * r * dv, H)
    q, k, v, z = g[:, :dk], g[:, dk:2 * dk], g[:, 2 * dk:2 * dk + r * dv], g[:, 2 * dk + r * dv:]
    qkv = torch.cat((q.reshape(Hk * dk, H), k.reshape(Hk * dk, H), v.reshape(Hv * dv, H)), 0)
    gb = ba.view(Hk, 2 * r, H)
    return qkv, z.reshape(Hv * dv, H), gb[:, :r].reshape(Hv, H), gb[:, r:].reshape(Hv, H)


def build_linear_attention_layer(model, cfg, p, get, has, up):
    from .llama import LayerWeights

    la = p + "linear_attn."
    if has(la + "in_proj_qkvz.weight"):
        qkv, z, b, a = split_fused_projections(cfg, get(la + "in_proj_qkvz.weight"), get(la + "in_proj_ba.weight"))
    else:
        qkv, z, b, a = (get(la + f"in_proj_{n}.weight") for n in ("qkv", "z", "b", "a"))
    conv = get(la + "conv1d.weight")
    conv = conv.reshape(conv.shape[0], -1)
    dt_bias, a_log, w_out = get(la + "dt_bias"), get(la + "A_log"), get(la + "out_proj.weight")
    tp, r = model.par.tp_size, model.par.tp_rank
    if tp > 1:
        # a key head with the value heads that share it is the unit: rank r owns key heads [r Hk/tp, (r+1) Hk/tp),
        # their value heads, the matching convolution channels and decay parameters, and the columns of out_proj
        Hk, Hv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
        if Hk % tp != 0:
            raise ValueError(f"{Hk} linear-attention key heads cannot be split over {tp} tensor ranks")
        rep = Hv // Hk
        k0, k1 = r * (Hk // tp), (r + 1) * (Hk // tp)
        v0, v1 = k0 * rep, k1 * rep
        key_dim = Hk * dk
        rows = torch.cat((torch.arange(k0 * dk, k1 * dk), key_dim + torch.arange(k0 * dk, k1 * dk),
                          2 * key_dim + torch.arange(v0 * dv, v1 * dv)))
        qkv, conv = qkv[rows], conv[rows]
        z, b, a = z[v0 * dv:v1 * dv], b[v0:v1], a[v0:v1]
        dt_bias, a_log, w_out = dt_bias[v0:v1], a_log[v0:v1], w_out[:, v0 * dv:v1 * dv]
    lw = LayerWeights(attn_norm=up(get(p + "input_layernorm.weight"), torch.float32), wqkv=None, wo=None,
                      ffn_norm=up(get(p + "post_attention_layernorm.weight"), torch.float32))
    lw.la_in = up(torch.cat((qkv, z, b, a), 0))
    lw.la_conv_w = up(conv, torch.float32)
    lw.la_dt_bias = up(dt_bias, torch.float32)
    lw.la_A_log = up(a_log, torch.float32)
    lw.la_norm_w = up(get(la + "norm.weight"), torch.float32)
    lw.la_out = up(w_out)
    return lw


def linear_attention_forward(model, li, lw, h, ssq, batch, kv):
    """The gated-delta operator of one layer; returns (h + out_proj(...), ssq')."""
    cfg = model.cfg
    tp = model.par.tp_size
    Hk, Hv = cfg.linear_num_key_heads // tp, cfg.linear_num_value_heads // tp       # this rank's heads
    dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
    key_dim, value_dim = Hk * dk, Hv * dv
    conv_dim = 2 * key_dim + value_dim
    proj = model._normed_linear(h, ssq, lw.fold_attn, lw.attn_norm, lw.la_in, lw, "la_in")
    M = proj.shape[0]
    conv_state, rec_state = kv.linear_attention_state(li)
    state_idx = kv.page_to_slot[batch.block_table[:, 0].long()].to(torch.int32).view(-1, 1).contiguous()
    mixed = ops.short_conv(proj, lw.la_conv_w, None, conv_state, state_idx, batch.cu_q if batch.is_prefill else None,
                           batch.q_per_seq, batch.positions, batch.slots, batch.max_q_len, mode=1, x_off=0)
    z = proj[:, conv_dim:conv_dim + value_dim].float().view(M, Hv, dv)
    b = proj[:, conv_dim + value_dim:conv_dim + value_dim + Hv].float()
    a = proj[:, conv_dim + value_dim + Hv:conv_dim + value_dim + 2 * Hv].float()
    q = mixed[:, :key_dim].float().view(M, Hk, dk)
    k = mixed[:, key_dim:2 * key_dim].float().view(M, Hk, dk)
    v = mixed[:, 2 * key_dim:].view(M, Hv, dv)
    q = q * torch.rsqrt(q.square().sum(-1, keepdim=True) + 1e-6) * (dk ** -0.5)
    k = k * torch.rsqrt(k.square().sum(-1, keepdim=True) + 1e-6)
    rep = Hv // Hk
    if rep > 1:
        q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    q, k = q.to(v.dtype), k.to(v.dtype)
    beta = torch.sigmoid(b)
    g = -torch.exp(lw.la_A_log)[None, :] * F.softplus(a + lw.la_dt_bias[None, :])
    slots = state_idx.view(-1).long()
    if batch.is_prefill:
        bounds = batch.cu_q.tolist()
        outs = []
        for i in range(len(bounds) - 1):
            r0, r1 = bounds[i], bounds[i + 1]
            if r1 <= r0:
                continue
            s = int(slots[i])
            S, o = ops.gated_delta_scan(q[None, r0:r1], k[None, r0:r1], v[None, r0:r1], g[None, r0:r1], beta[None, r0:r1],
                                        rec_state[s:s + 1])
            rec_state[s] = S[0]
            outs.append(o[0])
        core = torch.cat(outs, 0)
    else:
        B, T = slots.shape[0], batch.q_per_seq
        old = rec_state.index_select(0, slots)
        S, o = ops.gated_delta_scan(q.view(B, T, Hv, dk), k.view(B, T, Hv, dk), v.view(B, T, Hv, dv), g.view(B, T, Hv),
                                    beta.view(B, T, Hv), old)
        active = (batch.slots.view(B, T)[:, 0] >= 0).view(B, 1, 1, 1)
        rec_state.index_copy_(0, slots, torch.where(active, S, old))   # idle rows of the decode batch keep their state
        core = o.reshape(M, Hv, dv)
    cf = core.float()
    normed = cf * torch.rsqrt(cf.square().mean(-1, keepdim=True) + cfg.rms_norm_eps) * lw.la_norm_w[None, None, :]
    y = (normed * F.silu(z)).reshape(M, value_dim).to(h.dtype)
    return model._row_linear_ssq(lw, "la_out", y, lw.la_out, h, None, lw.fold_ffn)


def random_linear_attention_state(cfg, p, mat, out, std):
    """Random tensors of one gated-delta layer in the split checkpoint layout (tests, benchmarks)."""
    H = cfg.hidden_size
    Hk, Hv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    la = p + "linear_attn."
    mat(la + "in_proj_qkv.weight", 2 * Hk * dk + Hv * dv, H)
    mat(la + "in_proj_z.weight", Hv * dv, H)
    mat(la + "in_proj_b.weight", Hv, H)
    mat(la + "in_proj_a.weight", Hv, H)
    mat(la + "conv1d.weight", 2 * Hk * dk + Hv * dv, 1, cfg.linear_conv_kernel_dim)
    out[la + "conv1d.weight"] = out[la + "conv1d.weight"] * (0.5 / std)
    mat(la + "dt_bias", Hv)
    mat(la + "A_log", Hv)
    out[la + "norm.weight"] = torch.ones(dv, dtype=out[la + "dt_bias"].dtype, device=out[la + "dt_bias"].device)
    mat(la + "out_proj.weight", H, Hv * dv)
