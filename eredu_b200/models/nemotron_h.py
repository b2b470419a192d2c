"""Nemotron-H: a stack of single-mixer blocks - Mamba-2, attention (no positional rotation), relu^2 MLP or sparse
relu^2 experts - each ``h + mixer(norm(h))``.

Architecture: eredu/src/backend/mlx/architectures/nemotron_h/model.rs (pattern markers :74-90, Mamba-2 mixer
:2117-2170 with its causal convolution + SiLU :1850-1883, token update :1929-1962, time-step floor :2090-2096 and grouped
gated RMSNorm :870-932; relu^2 MLP :998-1001; sigmoid router with correction bias and group-limited top-k); tensor
names: ``backbone.embeddings``, ``backbone.layers.N.norm``, ``backbone.layers.N.mixer.*``, ``backbone.norm_f``.

The Mamba-2 input projection is laid out as [z (gate) | x B C | dt]; x B C pass through the depthwise causal
convolution (state slots in the cache object, like the gated-delta layers), B and C are shared by the heads of a group.
"""
from __future__ import annotations

import re

import torch
import torch.nn.functional as F

from .. import ops

_LAYER = re.compile(r"^model\.layers\.(\d+)\.(.+)$")


def checkpoint_names(canonical: str) -> list[str]:
    """Spellings of a canonical tensor name in Nemotron-H checkpoints: the original ``backbone.*`` tree and the
    ``model.*`` tree of newer exports (``embeddings`` / ``norm_f`` instead of ``embed_tokens`` / ``norm``)."""
    if canonical == "model.embed_tokens.weight":
        return ["backbone.embeddings.weight", "backbone.embedding.weight", "model.embeddings.weight"]
    if canonical == "model.norm.weight":
        return ["backbone.norm_f.weight", "model.norm_f.weight"]
    m = _LAYER.match(canonical)
    if not m:
        return []
    return [f"backbone.layers.{m.group(1)}.{m.group(2)}"]


def checkpoint_name(canonical: str) -> str:
    alts = checkpoint_names(canonical)
    return alts[0] if alts else canonical


def canonical_access(get, has):
    def resolve(name):
        for alt in checkpoint_names(name):
            if has(alt):
                return alt
        return name

    return (lambda name: get(resolve(name))), (lambda name: has(resolve(name)))


def to_checkpoint_names(state: dict) -> dict:
    return {checkpoint_name(k): v for k, v in state.items()}


def mamba_dims(cfg, tp: int = 1):
    heads = cfg.mamba_num_heads // tp
    groups = max(1, cfg.mamba_n_groups // tp)
    inter = heads * cfg.mamba_head_dim
    conv_dim = inter + 2 * groups * cfg.ssm_state_size
    return heads, groups, inter, conv_dim


def build_block(model, cfg, li, p, get, has, up, moe_factory):
    """One Nemotron-H block as LayerWeights (``block_kind`` names the mixer)."""
    from .llama import LayerWeights, shard_attention

    tp, r = model.par.tp_size, model.par.tp_rank
    kind = cfg.layer_types[li]
    lw = LayerWeights(attn_norm=up(get(p + "norm.weight"), torch.float32), wqkv=None, wo=None, ffn_norm=None)
    lw.block_kind = kind
    mx = p + "mixer."
    bias = lambda n: up(get(n)) if has(n) else None                                   # noqa: E731
    if kind == "mamba":
        # Tensor parallelism splits the mixer by heads: a rank keeps H / tp heads with their gate and value channels,
        # G / tp groups of B / C, its slice of the convolution, of the grouped norm and of the output projection's inputs
        # (whole groups per rank, so the grouped RMSNorm stays local); the output projection is summed over the ranks.
        H_all, G_all, N, P = cfg.mamba_num_heads, cfg.mamba_n_groups, cfg.ssm_state_size, cfg.mamba_head_dim
        if tp > 1 and (H_all % tp or G_all % tp):
            raise NotImplementedError(f"Mamba heads ({H_all}) and groups ({G_all}) must divide over {tp} tensor ranks")
        inter_all = H_all * P
        w_in = get(mx + "in_proj.weight")
        if tp > 1 and w_in.shape[0] != 2 * inter_all + 2 * G_all * N + H_all:
            raise NotImplementedError("tensor parallelism needs the plain [gate | x | B | C | dt] input projection")
        hs, gs = H_all // tp, G_all // tp

        def parts(t, lead: int):
            """Rows of this rank from a tensor laid out as [lead blocks of `inter` | B | C | (dt)]."""
            if tp == 1:
                return t
            out, off = [], 0
            for _ in range(lead):
                out.append(t[off + r * hs * P:off + (r + 1) * hs * P])
                off += inter_all
            for _ in range(2):
                out.append(t[off + r * gs * N:off + (r + 1) * gs * N])
                off += G_all * N
            if t.shape[0] > off:
                out.append(t[off + r * hs:off + (r + 1) * hs])
            return torch.cat(out, 0)

        head = (lambda t: t[r * hs:(r + 1) * hs]) if tp > 1 else (lambda t: t)
        lw.m_in = up(parts(w_in, 2))
        lw.m_in_b = up(parts(get(mx + "in_proj.bias"), 2)) if has(mx + "in_proj.bias") else None
        conv = get(mx + "conv1d.weight")
        lw.m_conv_w = up(parts(conv.reshape(conv.shape[0], -1), 1), torch.float32)
        lw.m_conv_b = up(parts(get(mx + "conv1d.bias"), 1), torch.float32) if has(mx + "conv1d.bias") else None
        lw.m_A_log = up(head(get(mx + "A_log")), torch.float32)
        lw.m_D = up(head(get(mx + "D")), torch.float32)
        lw.m_dt_bias = up(head(get(mx + "dt_bias")), torch.float32)
        nw, ow = get(mx + "norm.weight"), get(mx + "out_proj.weight")
        lw.m_norm_w = up(nw[r * hs * P:(r + 1) * hs * P] if tp > 1 else nw, torch.float32)
        lw.m_out = up(ow[:, r * hs * P:(r + 1) * hs * P] if tp > 1 else ow)
        lw.m_out_b = bias(mx + "out_proj.bias")
    elif kind == "attention_only":
        wq, wk, wv, wo = (get(mx + f"{n}_proj.weight") for n in "qkvo")
        wqkv, wo_l, _ = shard_attention(cfg, model.par, wq, wk, wv, wo)
        lw.wqkv, lw.wo = up(wqkv), up(wo_l)
    elif kind == "mlp_only":
        w_up, w_dn = get(mx + "up_proj.weight"), get(mx + "down_proj.weight")   # a single up projection: relu^2, no gate
        if tp > 1:
            n = w_up.shape[0] // tp
            w_up, w_dn = w_up[r * n:(r + 1) * n], w_dn[:, r * n:(r + 1) * n]
        lw.w_gate_up, lw.w_down = up(w_up), up(w_dn)
    else:
        lw.moe = moe_factory(model, li, get, has)
    return lw


def block_forward(model, li, lw, h, batch, kv):
    cfg = model.cfg
    x, _ = ops.rmsnorm(h, lw.attn_norm, cfg.rms_norm_eps)
    kind = lw.block_kind
    if kind == "mlp_only":
        a = ops.linear(x, lw.w_gate_up)
        a = torch.relu(a).square_()
        return model._row_linear(lw, "down", a, lw.w_down, h)
    if kind == "moe_only":
        return lw.moe(x, residual=h)
    if kind == "attention_only":
        qkv = ops.linear(x, lw.wqkv)
        k_cache, v_cache = kv.layer(li)
        q = ops.rope_kv(qkv, batch.positions, batch.slots, model.inv_freq, k_cache, v_cache, model.n_q_local, model.n_kv_local,
                        cfg.head_dim, rot=cfg.head_dim)         # inv_freq is zero for this family: rotation is the identity
        if batch.is_prefill:
            attn = ops.attention_prefill(q, k_cache, v_cache, batch.block_table, batch.seq_lens, batch.cu_q, batch.max_q_len,
                                         model.scale)
        else:
            attn = ops.attention_decode(q, k_cache, v_cache, batch.block_table, batch.seq_lens, batch.q_per_seq, model.scale,
                                        splits=batch.splits, scratch=batch.scratch)
        return model._row_linear(lw, "o", attn.view(attn.shape[0], -1), lw.wo, h)
    return mamba_forward(model, li, lw, x, batch, kv, h)


def mamba_forward(model, li, lw, x, batch, kv, residual):
    cfg = model.cfg
    heads, groups, inter, conv_dim = mamba_dims(cfg, model.par.tp_size)
    P, N = cfg.mamba_head_dim, cfg.ssm_state_size
    proj = ops.linear(x, lw.m_in, bias=lw.m_in_b)
    M = proj.shape[0]
    d_mlp2 = proj.shape[1] - (inter + conv_dim + heads)         # leading [2 d_mlp] block of older checkpoints (usually 0)
    gate = proj[:, d_mlp2:d_mlp2 + inter].float()
    dt_raw = proj[:, d_mlp2 + inter + conv_dim:].float()
    conv_state, ssm_state = kv.linear_attention_state(li)
    state_idx = kv.page_to_slot[batch.block_table[:, 0].long()].to(torch.int32).view(-1, 1).contiguous()
    xbc = ops.short_conv(proj, lw.m_conv_w, lw.m_conv_b, conv_state, state_idx, batch.cu_q if batch.is_prefill else None,
                         batch.q_per_seq, batch.positions, batch.slots, batch.max_q_len, mode=1, x_off=d_mlp2 + inter)
    xs = xbc[:, :inter].view(M, heads, P)
    Bs = xbc[:, inter:inter + groups * N].reshape(M, groups, N)        # one B / C per group: the scan maps heads to groups
    Cs = xbc[:, inter + groups * N:].reshape(M, groups, N)
    dt = torch.clamp_min(F.softplus(dt_raw + lw.m_dt_bias[None, :]), cfg.time_step_min)
    A = -torch.exp(lw.m_A_log)
    slots = state_idx.view(-1).long()
    if batch.is_prefill:
        bounds = batch.cu_q.tolist()
        outs = []
        for i in range(len(bounds) - 1):
            r0, r1 = bounds[i], bounds[i + 1]
            if r1 <= r0:
                continue
            s = int(slots[i])
            S, y = ops.mamba2_scan(xs[None, r0:r1], Bs[None, r0:r1], Cs[None, r0:r1], dt[None, r0:r1], A, lw.m_D,
                                   ssm_state[s:s + 1])
            ssm_state[s] = S[0]
            outs.append(y[0])
        y = torch.cat(outs, 0)
    else:
        Bn, T = slots.shape[0], batch.q_per_seq
        old = ssm_state.index_select(0, slots)
        S, y = ops.mamba2_scan(xs.reshape(Bn, T, heads, P), Bs.view(Bn, T, groups, N), Cs.view(Bn, T, groups, N),
                               dt.view(Bn, T, heads), A, lw.m_D, old)
        active = (batch.slots.view(Bn, T)[:, 0] >= 0).view(Bn, 1, 1, 1)
        ssm_state.index_copy_(0, slots, torch.where(active, S, old))
        y = y.reshape(M, heads, P)
    # grouped gated RMSNorm: (y * silu(gate)) normalised within each group of inter / groups channels
    gated = y.reshape(M, inter).float() * F.silu(gate)
    grouped = gated.view(M, groups, inter // groups)
    normed = (grouped * torch.rsqrt(grouped.square().mean(-1, keepdim=True) + cfg.rms_norm_eps)).view(M, inter)
    out = (normed.to(x.dtype) * lw.m_norm_w.to(x.dtype)[None, :])
    return model._row_linear(lw, "m_out", out, lw.m_out, residual, bias=lw.m_out_b)


def random_block_state(cfg, li, p, mat, out, std):
    H = cfg.hidden_size
    kind = cfg.layer_types[li]
    mx = p + "mixer."
    out[p + "norm.weight"] = torch.ones(H)
    if kind == "mamba":
        heads, groups, inter, conv_dim = mamba_dims(cfg)
        mat(mx + "in_proj.weight", inter + conv_dim + heads, H)
        mat(mx + "conv1d.weight", conv_dim, 1, cfg.mamba_conv_kernel)
        out[mx + "conv1d.weight"] = out[mx + "conv1d.weight"] * (0.5 / std)
        if cfg.mamba_conv_bias:
            mat(mx + "conv1d.bias", conv_dim)
        mat(mx + "A_log", heads)
        mat(mx + "D", heads)
        mat(mx + "dt_bias", heads)
        out[mx + "norm.weight"] = torch.ones(inter)
        mat(mx + "out_proj.weight", H, inter)
    elif kind == "attention_only":
        D = cfg.head_dim
        mat(mx + "q_proj.weight", cfg.num_attention_heads * D, H)
        mat(mx + "k_proj.weight", cfg.num_key_value_heads * D, H)
        mat(mx + "v_proj.weight", cfg.num_key_value_heads * D, H)
        mat(mx + "o_proj.weight", H, cfg.num_attention_heads * D)
    elif kind == "mlp_only":
        mat(mx + "up_proj.weight", cfg.intermediate_size, H)
        mat(mx + "down_proj.weight", H, cfg.intermediate_size)
    else:
        mat(mx + "gate.weight", cfg.num_experts, H)
        mat(mx + "gate.e_score_correction_bias", cfg.num_experts)
        for e in range(cfg.num_experts):
            mat(mx + f"experts.{e}.up_proj.weight", cfg.moe_intermediate_size, H)
            mat(mx + f"experts.{e}.down_proj.weight", H, cfg.moe_intermediate_size)
        if cfg.shared_expert_intermediate_size:
            mat(mx + "shared_experts.up_proj.weight", cfg.shared_expert_intermediate_size, H)
            mat(mx + "shared_experts.down_proj.weight", H, cfg.shared_expert_intermediate_size)
