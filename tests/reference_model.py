"""Independent dense (non-paged, no cache) PyTorch implementation of the Llama-family forward used as the
oracle for the engine: full recompute of the whole sequence at every step."""
import math

import torch
import torch.nn.functional as F

from eredu_b200.models.rope import rope_tables


def rms(x, w, eps, off=0.0):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (w + off)


def rope(x, pos, inv_freq, factor, interleaved, rot):
    # x: [T, heads, D]
    ang = pos.float()[:, None] * inv_freq[None, :]
    cos, sin = (ang.cos() * factor)[:, None, :], (ang.sin() * factor)[:, None, :]
    xr, xp = x[..., :rot], x[..., rot:]
    if interleaved:
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack((a * cos - b * sin, b * cos + a * sin), -1).flatten(-2)
    else:
        a, b = xr[..., : rot // 2], xr[..., rot // 2:]
        out = torch.cat((a * cos - b * sin, b * cos + a * sin), -1)
    return torch.cat((out, xp), -1)


def forward_logits(cfg, sd, tokens, moe_fn=None):
    """sd: HF-named fp32 state dict; tokens: list[int]. Returns logits [T, V] (fp32)."""
    sd = {k: v.float() for k, v in sd.items()}
    T = len(tokens)
    D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    inv, factor = rope_tables(cfg)
    if not cfg.use_rope:
        inv = torch.zeros_like(inv)
    pos = torch.arange(T)
    h = sd["model.embed_tokens.weight"][torch.tensor(tokens)] * cfg.embedding_scale
    for li in range(cfg.num_hidden_layers):
        p = f"model.layers.{li}."
        if cfg.model_type == "nemotron_h":
            h = h + _nemotron_mixer(cfg, sd, li, p, rms(h, sd[p + "norm.weight"], cfg.rms_norm_eps), moe_fn)
            continue
        x = rms(h, sd[p + "input_layernorm.weight"], cfg.rms_norm_eps, cfg.norm_weight_offset)
        if cfg.layer_is_linear_attention(li):
            h = h + _gated_delta_layer(cfg, sd, p + "linear_attn.", x)
            h = _ffn(cfg, sd, li, p, h, moe_fn)
            continue
        if cfg.layer_is_conv(li):
            # LFM2 gated short convolution: causal depthwise conv1d over B * X, gated by C
            Cc = cfg.hidden_size
            pj = F.linear(x, sd[p + "conv.in_proj.weight"], sd.get(p + "conv.in_proj.bias"))
            bx = (pj[:, :Cc] * pj[:, 2 * Cc:]).t()[None]
            L = cfg.conv_l_cache
            y = F.conv1d(F.pad(bx, (L - 1, 0)), sd[p + "conv.conv.weight"].view(Cc, 1, L), sd.get(p + "conv.conv.bias"),
                         groups=Cc)[0].t()
            h = h + F.linear(pj[:, Cc:2 * Cc] * y, sd[p + "conv.out_proj.weight"], sd.get(p + "conv.out_proj.bias"))
            h = _ffn(cfg, sd, li, p, h, moe_fn)
            continue
        if cfg.layer_is_kda(li):
            h = h + _kda_layer(cfg, sd, p + "self_attn.", x)
            h = _ffn(cfg, sd, li, p, h, moe_fn)
            continue
        if cfg.is_mla:
            h = h + _mla_attention(cfg, sd, p + "self_attn.", x, pos, inv, factor)
            h = _ffn(cfg, sd, li, p, h, moe_fn)
            continue
        gate = None
        if cfg.attn_output_gate:
            qg = F.linear(x, sd[p + "self_attn.q_proj.weight"]).view(T, Hq, 2 * D)
            q, gate = qg[..., :D], qg[..., D:].reshape(T, Hq * D)
        else:
            q = F.linear(x, sd[p + "self_attn.q_proj.weight"], sd.get(p + "self_attn.q_proj.bias")).view(T, Hq, D)
        k = F.linear(x, sd[p + "self_attn.k_proj.weight"], sd.get(p + "self_attn.k_proj.bias")).view(T, Hkv, D)
        v = F.linear(x, sd[p + "self_attn.v_proj.weight"], sd.get(p + "self_attn.v_proj.bias")).view(T, Hkv, D)
        if p + "self_attn.q_norm.weight" in sd:
            q = rms(q, sd[p + "self_attn.q_norm.weight"], cfg.rms_norm_eps, cfg.norm_weight_offset)
            k = rms(k, sd[p + "self_attn.k_norm.weight"], cfg.rms_norm_eps, cfg.norm_weight_offset)
        q = rope(q, pos, inv, factor, cfg.rope_traditional, cfg.rotary_dim)
        k = rope(k, pos, inv, factor, cfg.rope_traditional, cfg.rotary_dim)
        g = Hq // Hkv
        k, v = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(D)
        mask = pos[None, :] <= pos[:, None]
        w = cfg.layer_window(li)
        if w > 0:
            mask = mask & (pos[None, :] > pos[:, None] - w)
        s = s.masked_fill(~mask[None], float("-inf"))
        if p + "self_attn.sinks" in sd:   # a learned per-head logit that only takes probability mass
            sink = sd[p + "self_attn.sinks"].view(Hq, 1, 1).expand(Hq, T, 1)
            probs = torch.softmax(torch.cat((s, sink), -1), -1)[..., :-1]
        else:
            probs = torch.softmax(s, -1)
        a = torch.einsum("hqk,khd->qhd", probs, v).reshape(T, Hq * D)
        if gate is not None:
            a = a * torch.sigmoid(gate)
        h = h + F.linear(a, sd[p + "self_attn.o_proj.weight"], sd.get(p + "self_attn.o_proj.bias"))
        h = _ffn(cfg, sd, li, p, h, moe_fn)
    x = rms(h, sd["model.norm.weight"], cfg.rms_norm_eps, cfg.norm_weight_offset)
    head = sd.get("lm_head.weight", sd["model.embed_tokens.weight"])
    return F.linear(x, head)


def _kda_layer(cfg, sd, a, x):
    """Kimi Delta Attention over a whole sequence: per-channel decay, token by token."""
    T = x.shape[0]
    H, D, K = cfg.linear_num_value_heads, cfg.linear_value_head_dim, cfg.linear_conv_kernel_dim
    P = H * D

    def conv_silu(name):
        y = F.linear(x, sd[a + f"{name}_proj.weight"])
        return F.silu(F.conv1d(F.pad(y.t()[None], (K - 1, 0)), sd[a + f"{name}_conv1d.weight"].view(P, 1, K), groups=P)[0].t())

    def rms_scaled(t, scale):
        t = t.view(T, H, D)
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6) * scale

    q, k, v = rms_scaled(conv_silu("q"), 1.0 / D), rms_scaled(conv_silu("k"), D ** -0.5), conv_silu("v").view(T, H, D)
    logits = F.linear(F.linear(x, sd[a + "f_a_proj.weight"]), sd[a + "f_b_proj.weight"]).view(T, H, D)
    g = -torch.exp(sd[a + "A_log"].view(1, H, 1)) * F.softplus(logits + sd[a + "dt_bias"].view(1, H, D))
    beta = torch.sigmoid(F.linear(x, sd[a + "b_proj.weight"]))
    S = torch.zeros(H, D, D)
    outs = []
    for t in range(T):
        S = S * torch.exp(g[t])[:, :, None]
        mem = torch.einsum("hkv,hk->hv", S, k[t])
        S = S + torch.einsum("hk,hv->hkv", k[t], (v[t] - mem) * beta[t][:, None])
        outs.append(torch.einsum("hkv,hk->hv", S, q[t]))
    o = torch.stack(outs)
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * sd[a + "o_norm.weight"]
    gate = torch.sigmoid(F.linear(F.linear(x, sd[a + "g_a_proj.weight"]), sd[a + "g_b_proj.weight"])).view(T, H, D)
    return F.linear((o * gate).reshape(T, P), sd[a + "o_proj.weight"])


def _mla_attention(cfg, sd, a, x, pos, inv, factor):
    """DeepSeek latent attention in the plain (decompressed) form: per-head keys and values are materialised."""
    T = x.shape[0]
    Hq, nope, rp, vd = cfg.num_attention_heads, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
    if cfg.q_lora_rank:
        q = F.linear(rms(F.linear(x, sd[a + "q_a_proj.weight"]), sd[a + "q_a_layernorm.weight"], cfg.rms_norm_eps),
                     sd[a + "q_b_proj.weight"])
    else:
        q = F.linear(x, sd[a + "q_proj.weight"])
    q = q.view(T, Hq, nope + rp)
    ckv = F.linear(x, sd[a + "kv_a_proj_with_mqa.weight"])
    c, k_pe = ckv[:, :cfg.kv_lora_rank], ckv[:, cfg.kv_lora_rank:].view(T, 1, rp)
    kv = F.linear(rms(c, sd[a + "kv_a_layernorm.weight"], cfg.rms_norm_eps), sd[a + "kv_b_proj.weight"]).view(T, Hq, nope + vd)
    k_nope, v = kv[..., :nope], kv[..., nope:]
    q_pe = rope(q[..., nope:], pos, inv, factor, cfg.rope_traditional, rp)
    k_pe = rope(k_pe, pos, inv, factor, cfg.rope_traditional, rp)
    qf = torch.cat((q[..., :nope], q_pe), -1)
    kf = torch.cat((k_nope, k_pe.expand(T, Hq, rp)), -1)
    sc = cfg.rope_scaling or {}
    mult = 1.0
    if sc.get("mscale_all_dim") and float(sc.get("factor", 1.0)) > 1.0:
        mult = (0.1 * float(sc["mscale_all_dim"]) * math.log(float(sc["factor"])) + 1.0) ** 2
    s_ = torch.einsum("qhd,khd->hqk", qf, kf) * ((nope + rp) ** -0.5 * mult)
    s_ = s_.masked_fill(~(pos[None, :] <= pos[:, None])[None], float("-inf"))
    o = torch.einsum("hqk,khd->qhd", torch.softmax(s_, -1), v).reshape(T, Hq * vd)
    return F.linear(o, sd[a + "o_proj.weight"])


def _nemotron_mixer(cfg, sd, li, p, x, moe_fn):
    """One Nemotron-H mixer over a whole sequence (no cache): Mamba-2, attention without rotation, relu^2 MLP or experts."""
    T = x.shape[0]
    kind = cfg.layer_types[li]
    mx = p + "mixer."
    if kind == "mlp_only":
        return F.linear(torch.relu(F.linear(x, sd[mx + "up_proj.weight"])) ** 2, sd[mx + "down_proj.weight"])
    if kind == "moe_only":
        return moe_fn(cfg, sd, li, x)
    if kind == "attention_only":
        D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
        q = F.linear(x, sd[mx + "q_proj.weight"]).view(T, Hq, D)
        k = F.linear(x, sd[mx + "k_proj.weight"]).view(T, Hkv, D).repeat_interleave(Hq // Hkv, 1)
        v = F.linear(x, sd[mx + "v_proj.weight"]).view(T, Hkv, D).repeat_interleave(Hq // Hkv, 1)
        s_ = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(D)
        s_ = s_.masked_fill(~(torch.arange(T)[None, :] <= torch.arange(T)[:, None])[None], float("-inf"))
        a = torch.einsum("hqk,khd->qhd", torch.softmax(s_, -1), v).reshape(T, Hq * D)
        return F.linear(a, sd[mx + "o_proj.weight"])
    Hm, P, N, G, K = cfg.mamba_num_heads, cfg.mamba_head_dim, cfg.ssm_state_size, cfg.mamba_n_groups, cfg.mamba_conv_kernel
    inter = Hm * P
    conv_dim = inter + 2 * G * N
    proj = F.linear(x, sd[mx + "in_proj.weight"])
    gate, xbc, dt = proj[:, :inter], proj[:, inter:inter + conv_dim], proj[:, inter + conv_dim:]
    xbc = F.silu(F.conv1d(F.pad(xbc.t()[None], (K - 1, 0)), sd[mx + "conv1d.weight"].view(conv_dim, 1, K),
                          sd.get(mx + "conv1d.bias"), groups=conv_dim)[0].t())
    xs = xbc[:, :inter].view(T, Hm, P)
    Bm = xbc[:, inter:inter + G * N].view(T, G, N).repeat_interleave(Hm // G, 1)
    Cm = xbc[:, inter + G * N:].view(T, G, N).repeat_interleave(Hm // G, 1)
    dt = torch.clamp_min(F.softplus(dt + sd[mx + "dt_bias"]), cfg.time_step_min)
    A = -torch.exp(sd[mx + "A_log"])
    S = torch.zeros(Hm, P, N)
    ys = []
    for t in range(T):
        S = S * torch.exp(dt[t] * A)[:, None, None] + torch.einsum("hp,hn->hpn", xs[t], dt[t][:, None] * Bm[t])
        ys.append(torch.einsum("hpn,hn->hp", S, Cm[t]) + sd[mx + "D"][:, None] * xs[t])
    y = torch.stack(ys).reshape(T, inter) * F.silu(gate)
    y = y.view(T, G, inter // G)
    y = (y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps)).reshape(T, inter) * sd[mx + "norm.weight"]
    return F.linear(y, sd[mx + "out_proj.weight"])


def _gated_delta_layer(cfg, sd, la, x):
    """Qwen3-Next gated delta network over a whole sequence, written token by token."""
    T = x.shape[0]
    Hk, Hv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    K = cfg.linear_conv_kernel_dim
    qkv = F.linear(x, sd[la + "in_proj_qkv.weight"])
    z = F.linear(x, sd[la + "in_proj_z.weight"]).view(T, Hv, dv)
    beta = torch.sigmoid(F.linear(x, sd[la + "in_proj_b.weight"]))
    a = F.linear(x, sd[la + "in_proj_a.weight"])
    C = qkv.shape[1]
    conv = F.conv1d(F.pad(qkv.t()[None], (K - 1, 0)), sd[la + "conv1d.weight"].view(C, 1, K), groups=C)[0].t()
    qkv = F.silu(conv)
    q, k, v = qkv[:, :Hk * dk].view(T, Hk, dk), qkv[:, Hk * dk:2 * Hk * dk].view(T, Hk, dk), qkv[:, 2 * Hk * dk:].view(T, Hv, dv)
    l2 = lambda t: t / torch.sqrt(t.pow(2).sum(-1, keepdim=True) + 1e-6)       # noqa: E731
    q, k = l2(q) / math.sqrt(dk), l2(k)
    r = Hv // Hk
    q, k = q.repeat_interleave(r, 1), k.repeat_interleave(r, 1)
    g = -torch.exp(sd[la + "A_log"]) * F.softplus(a + sd[la + "dt_bias"])
    S = torch.zeros(Hv, dk, dv)
    outs = []
    for t in range(T):
        S = S * torch.exp(g[t])[:, None, None]
        mem = torch.einsum("hkv,hk->hv", S, k[t])
        S = S + torch.einsum("hk,hv->hkv", k[t], (v[t] - mem) * beta[t][:, None])
        outs.append(torch.einsum("hkv,hk->hv", S, q[t]))
    o = torch.stack(outs)                                                     # [T, Hv, dv]
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * sd[la + "norm.weight"]
    return F.linear((o * F.silu(z)).reshape(T, Hv * dv), sd[la + "out_proj.weight"])


def _ffn(cfg, sd, li, p, h, moe_fn):
    x = rms(h, sd[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps, cfg.norm_weight_offset)
    if cfg.layer_is_moe(li):
        return h + moe_fn(cfg, sd, li, x)
    gate = F.linear(x, sd[p + "mlp.gate_proj.weight"])
    up = F.linear(x, sd[p + "mlp.up_proj.weight"])
    return h + F.linear(F.silu(gate) * up, sd[p + "mlp.down_proj.weight"])


def greedy(cfg, sd, prompt, n, moe_fn=None):
    toks = list(prompt)
    out = []
    for _ in range(n):
        t = int(torch.argmax(forward_logits(cfg, sd, toks, moe_fn)[-1]))
        out.append(t)
        toks.append(t)
    return out
