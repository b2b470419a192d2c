"""Kimi Linear: Kimi Delta Attention (KDA) layers - a gated delta rule with one decay per key CHANNEL - between
latent-attention (MLA, no positional rotation) layers, over a DeepSeek-style sparse FFN.

Architecture: eredu/src/backend/mlx/architectures/kimi_linear/model.rs (KDA module :996-1110, forward :1113-1226:
q / k / v projections each through a causal depthwise convolution + SiLU, RMS-normalised q (scale 1/D) and k (scale
1/sqrt(D)), ``log_decay = -exp(A_log) * softplus(f_b(f_a(x)) + dt_bias)`` per channel, ``beta = sigmoid(b(x))``, the gated
delta scan, ``o_norm(core) * sigmoid(g_b(g_a(x)))``, ``o_proj``; layer schedule from 1-based ``kda_layers`` /
``full_attn_layers`` :71-90; sparse layers: index >= first_k_dense_replace and index % moe_layer_freq == 0).
Checkpoints spell the sparse block ``block_sparse_moe`` with experts ``w1 / w3 / w2``.
"""
from __future__ import annotations

import re

import torch
import torch.nn.functional as F

from .. import ops

_LAYER = re.compile(r"^model\.layers\.(\d+)\.mlp\.(.+)$")
_EXPERT = re.compile(r"^experts\.(\d+)\.(gate|up|down)_proj\.weight$")
_W = {"gate": "w1", "up": "w3", "down": "w2"}


def checkpoint_name(canonical: str) -> str:
    m = _LAYER.match(canonical)
    if not m:
        return canonical
    rest = m.group(2)
    e = _EXPERT.match(rest)
    if e:
        rest = f"experts.{e.group(1)}.{_W[e.group(2)]}.weight"
    return f"model.layers.{m.group(1)}.block_sparse_moe.{rest}"


def canonical_access(get, has):
    def g(name):
        alt = checkpoint_name(name)
        return get(alt) if alt != name and has(alt) else get(name)

    def h(name):
        alt = checkpoint_name(name)
        return (alt != name and has(alt)) or has(name)

    return g, h


def build_kda_layer(model, cfg, p, get, has, up):
    from .llama import LayerWeights

    # Tensor parallelism splits the layer by heads: q / k / v / beta rows, the convolution channels, the expanded decay
    # and gate projections, the per-head rates and the output projection's inputs; the two low-rank bottlenecks (f_a,
    # g_a) and the output norm are replicated, the output projection is summed over the ranks.
    tp, r = model.par.tp_size, model.par.tp_rank
    H, D = cfg.linear_num_value_heads, cfg.linear_value_head_dim
    if H % tp:
        raise NotImplementedError(f"{H} KDA heads do not divide over {tp} tensor ranks")
    Hl = H // tp
    rows = (lambda t, per: t[r * Hl * per:(r + 1) * Hl * per]) if tp > 1 else (lambda t, per: t)
    a = p + "self_attn."
    lw = LayerWeights(attn_norm=up(get(p + "input_layernorm.weight"), torch.float32), wqkv=None, wo=None,
                      ffn_norm=up(get(p + "post_attention_layernorm.weight"), torch.float32))
    # one input GEMM: [q | k | v | f_a | b | g_a]
    lw.kda_in = up(torch.cat([rows(get(a + "q_proj.weight"), D), rows(get(a + "k_proj.weight"), D), rows(get(a + "v_proj.weight"), D),
                              get(a + "f_a_proj.weight"), rows(get(a + "b_proj.weight"), 1), get(a + "g_a_proj.weight")], 0))
    conv = torch.cat([rows(get(a + f"{n}_conv1d.weight"), D) for n in "qkv"], 0)
    lw.kda_conv_w = up(conv.reshape(conv.shape[0], -1), torch.float32)
    lw.kda_f_b = up(rows(get(a + "f_b_proj.weight"), D))
    lw.kda_g_b = up(rows(get(a + "g_b_proj.weight"), D))
    lw.kda_A_log = up(rows(get(a + "A_log").reshape(-1), 1), torch.float32)          # one rate per head
    lw.kda_dt_bias = up(rows(get(a + "dt_bias").reshape(-1), D), torch.float32)      # one bias per channel
    lw.kda_o_norm = up(get(a + "o_norm.weight"), torch.float32)
    wo = get(a + "o_proj.weight")
    lw.wo = up(wo[:, r * Hl * D:(r + 1) * Hl * D] if tp > 1 else wo)
    return lw


def kda_forward(model, li, lw, h, ssq, batch, kv):
    cfg = model.cfg
    H, D = cfg.linear_num_value_heads // model.par.tp_size, cfg.linear_value_head_dim
    P = H * D
    proj = model._normed_linear(h, ssq, lw.fold_attn, lw.attn_norm, lw.kda_in, lw, "kda_in")
    M = proj.shape[0]
    conv_state, rec_state = kv.linear_attention_state(li)
    state_idx = kv.page_to_slot[batch.block_table[:, 0].long()].to(torch.int32).view(-1, 1).contiguous()
    qkv = ops.short_conv(proj, lw.kda_conv_w, None, conv_state, state_idx, batch.cu_q if batch.is_prefill else None,
                         batch.q_per_seq, batch.positions, batch.slots, batch.max_q_len, mode=1, x_off=0)
    f_a = proj[:, 3 * P:3 * P + D].contiguous()
    b = proj[:, 3 * P + D:3 * P + D + H].float()
    g_a = proj[:, 3 * P + D + H:3 * P + 2 * D + H].contiguous()

    def rms_scaled(t, scale):
        tf = t.float().view(M, H, D)
        return tf * torch.rsqrt(tf.square().mean(-1, keepdim=True) + 1e-6) * scale

    q = rms_scaled(qkv[:, :P], 1.0 / D).to(h.dtype)
    k = rms_scaled(qkv[:, P:2 * P], D ** -0.5).to(h.dtype)
    v = qkv[:, 2 * P:].view(M, H, D)
    decay_logits = ops.linear(f_a, lw.kda_f_b).float().view(M, H, D)
    log_decay = -torch.exp(lw.kda_A_log)[None, :, None] * F.softplus(decay_logits + lw.kda_dt_bias.view(1, H, D))
    beta = torch.sigmoid(b)
    slots = state_idx.view(-1).long()
    if batch.is_prefill:
        bounds = batch.cu_q.tolist()
        outs = []
        for i in range(len(bounds) - 1):
            r0, r1 = bounds[i], bounds[i + 1]
            if r1 <= r0:
                continue
            s = int(slots[i])
            S, o = ops.gated_delta_scan(q[None, r0:r1], k[None, r0:r1], v[None, r0:r1], log_decay[None, r0:r1].contiguous(),
                                        beta[None, r0:r1], rec_state[s:s + 1])
            rec_state[s] = S[0]
            outs.append(o[0])
        core = torch.cat(outs, 0)
    else:
        B, T = slots.shape[0], batch.q_per_seq
        old = rec_state.index_select(0, slots)
        S, o = ops.gated_delta_scan(q.view(B, T, H, D), k.view(B, T, H, D), v.view(B, T, H, D), log_decay.view(B, T, H, D),
                                    beta.view(B, T, H), old)
        active = (batch.slots.view(B, T)[:, 0] >= 0).view(B, 1, 1, 1)
        rec_state.index_copy_(0, slots, torch.where(active, S, old))
        core = o.reshape(M, H, D)
    gate = torch.sigmoid(ops.linear(g_a, lw.kda_g_b).float().view(M, H, D))
    cf = core.float()
    normed = cf * torch.rsqrt(cf.square().mean(-1, keepdim=True) + cfg.rms_norm_eps) * lw.kda_o_norm[None, None, :]
    y = (normed * gate).reshape(M, P).to(h.dtype)
    return model._row_linear_ssq(lw, "o", y, lw.wo, h, None, lw.fold_ffn)


def random_kda_state(cfg, p, mat, ones, out, std):
    Hd, H, D = cfg.hidden_size, cfg.linear_num_value_heads, cfg.linear_value_head_dim
    P = H * D
    a = p + "self_attn."
    for n in ("q_proj", "k_proj", "v_proj"):
        mat(a + f"{n}.weight", P, Hd)
    for n in "qkv":
        mat(a + f"{n}_conv1d.weight", P, 1, cfg.linear_conv_kernel_dim)
        out[a + f"{n}_conv1d.weight"] = out[a + f"{n}_conv1d.weight"] * (0.5 / std)
    mat(a + "f_a_proj.weight", D, Hd)
    mat(a + "f_b_proj.weight", P, D)
    mat(a + "b_proj.weight", H, Hd)
    mat(a + "g_a_proj.weight", D, Hd)
    mat(a + "g_b_proj.weight", P, D)
    mat(a + "A_log", 1, 1, H, 1)
    mat(a + "dt_bias", P)
    ones(a + "o_norm.weight", D)
    mat(a + "o_proj.weight", Hd, P)
