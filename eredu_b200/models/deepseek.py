"""DeepSeek-V3 / R1 multi-head latent attention (MLA).

Architecture: eredu/src/backend/mlx/architectures/deepseek_v3/model.rs (projections :1120-1240, softmax scale
``1/sqrt(qk_head_dim) * yarn multiplier`` :1164-1170, RoPE on the ``qk_rope_head_dim`` slice only :1231-1238; cache of the
compressed latent: ``CompressedLatentCache`` in runtime/cache/kv.rs). Per token the cache holds ONE row shared by all
heads: the normalised latent ``c`` (``kv_lora_rank``) followed by the rotated positional key (``qk_rope_head_dim``).

Attention runs in the absorbed form, so the per-head keys and values are never materialised:
``score = (q_nope W_uk) . c + q_pe . k_pe``,  ``out = (softmax(score) . c) W_uv^T``  with W_uk / W_uv the two halves of
``kv_b_proj``. The key width (576 for the published models) has no attention kernel: the layer is tensor operations
around this repository's GEMMs, and such models decode eagerly. Tensor parallelism shards the heads (q_b / kv_b rows,
o_proj columns); the latent projection and its cache are replicated.
"""
from __future__ import annotations

import torch

from .. import ops


def build_mla_layer(model, cfg, p, get, has, up):
    from .llama import LayerWeights

    tp, r = model.par.tp_size, model.par.tp_rank
    heads = cfg.num_attention_heads
    if heads % tp != 0:
        raise ValueError(f"{heads} attention heads cannot be split over {tp} tensor ranks")
    hl = heads // tp
    qd, vd, nope = cfg.qk_nope_head_dim + cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.qk_nope_head_dim
    a = p + "self_attn."
    lw = LayerWeights(attn_norm=up(get(p + "input_layernorm.weight"), torch.float32), wqkv=None, wo=None,
                      ffn_norm=up(get(p + "post_attention_layernorm.weight"), torch.float32))
    kv_a = get(a + "kv_a_proj_with_mqa.weight")
    if cfg.q_lora_rank:
        lw.mla_in = up(torch.cat((get(a + "q_a_proj.weight"), kv_a), 0))          # [q_lora + kv_lora + rope, H]
        lw.mla_q_norm = up(get(a + "q_a_layernorm.weight"), torch.float32)
        lw.mla_q_b = up(get(a + "q_b_proj.weight")[r * hl * qd:(r + 1) * hl * qd])
    else:
        lw.mla_in = up(torch.cat((get(a + "q_proj.weight")[r * hl * qd:(r + 1) * hl * qd], kv_a), 0))
    lw.mla_kv_norm = up(get(a + "kv_a_layernorm.weight"), torch.float32)
    kv_b = get(a + "kv_b_proj.weight").view(heads, nope + vd, cfg.kv_lora_rank)[r * hl:(r + 1) * hl]
    lw.mla_w_uk = up(kv_b[:, :nope])                                                # [heads_local, nope, kv_lora]
    lw.mla_w_uv = up(kv_b[:, nope:])                                                # [heads_local, v, kv_lora]
    lw.wo = up(get(a + "o_proj.weight")[:, r * hl * vd:(r + 1) * hl * vd])
    return lw


def _rope(x, positions, inv_freq, factor, interleaved):
    """x [M, heads, rot] -> rotated, fp32."""
    ang = positions.float()[:, None] * inv_freq[None, :]
    cos, sin = (ang.cos() * factor)[:, None, :], (ang.sin() * factor)[:, None, :]
    xf = x.float()
    if interleaved:
        a, b = xf[..., 0::2], xf[..., 1::2]
        return torch.stack((a * cos - b * sin, b * cos + a * sin), -1).flatten(-2)
    half = xf.shape[-1] // 2
    a, b = xf[..., :half], xf[..., half:]
    return torch.cat((a * cos - b * sin, b * cos + a * sin), -1)


def _rms(x, w, eps):
    xf = x.float()
    return xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps) * w


def mla_forward(model, li, lw, h, ssq, batch, kv):
    cfg = model.cfg
    hl = lw.mla_w_uk.shape[0]
    nope, rope, vd, lora = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
    proj = model._normed_linear(h, ssq, lw.fold_attn, lw.attn_norm, lw.mla_in, lw, "mla_in")
    M = proj.shape[0]
    if lw.mla_q_b is not None:
        qa = _rms(proj[:, :cfg.q_lora_rank], lw.mla_q_norm, cfg.rms_norm_eps).to(h.dtype)
        q = ops.linear(qa, lw.mla_q_b)
        rest = proj[:, cfg.q_lora_rank:]
    else:
        q = proj[:, :hl * (nope + rope)]
        rest = proj[:, hl * (nope + rope):]
    q = q.reshape(M, hl, nope + rope)
    latent = _rms(rest[:, :lora], lw.mla_kv_norm, cfg.rms_norm_eps)
    k_pe = _rope(rest[:, lora:lora + rope].reshape(M, 1, rope), batch.positions, model.inv_freq, model.attn_factor,
                 cfg.rope_traditional)[:, 0]
    q_pe = _rope(q[..., nope:], batch.positions, model.inv_freq, model.attn_factor, cfg.rope_traditional)
    q_abs = torch.einsum("mhn,hnc->mhc", q[..., :nope].float(), lw.mla_w_uk.float())      # queries in latent space
    # append this step's rows: one [latent | rotated key] row per token, shared by every head
    k_cache, _ = kv.layer(li)
    flat = k_cache.view(-1, k_cache.shape[-1])                       # one KV head: row index = page * 16 + offset = slot
    rows = torch.cat((latent, k_pe), -1).to(flat.dtype)
    keep = batch.slots >= 0                                          # idle rows of a decode batch carry slot -1
    flat[batch.slots[keep]] = rows[keep]
    scale = (nope + rope) ** -0.5 * _yarn_multiplier(cfg)
    out = torch.zeros((M, hl, vd), dtype=torch.float32, device=h.device)
    seq_lens = batch.seq_lens.tolist()
    bounds = batch.cu_q.tolist() if batch.is_prefill else [i * batch.q_per_seq for i in range(len(seq_lens) + 1)]
    for b, kv_len in enumerate(seq_lens):
        r0, r1 = bounds[b], bounds[b + 1]
        if r1 <= r0 or kv_len <= 0:
            continue
        n_pages = (kv_len + ops.PAGE - 1) // ops.PAGE
        ctx = k_cache[batch.block_table[b, :n_pages].long(), 0].reshape(-1, lora + rope)[:kv_len].float()   # [T, lora + rope]
        c, kp = ctx[:, :lora], ctx[:, lora:]
        s = (torch.einsum("qhc,tc->hqt", q_abs[r0:r1], c) + torch.einsum("qhr,tr->hqt", q_pe[r0:r1], kp)) * scale
        ql = r1 - r0
        qpos = torch.arange(kv_len - ql, kv_len, device=h.device)[:, None]
        s = s.masked_fill(torch.arange(kv_len, device=h.device)[None, :] > qpos, float("-inf"))
        o_lat = torch.einsum("hqt,tc->qhc", torch.softmax(s, -1), c)
        out[r0:r1] = torch.einsum("qhc,hvc->qhv", o_lat, lw.mla_w_uv.float())
    attn = out.reshape(M, hl * vd).to(h.dtype)
    return model._row_linear_ssq(lw, "o", attn, lw.wo, h, None, lw.fold_ffn)


def _yarn_multiplier(cfg) -> float:
    """Softmax-scale correction of YaRN-extended checkpoints: (0.1 * mscale_all_dim * ln(factor) + 1)^2."""
    import math

    sc = cfg.rope_scaling or {}
    m, f = float(sc.get("mscale_all_dim", 0.0) or 0.0), float(sc.get("factor", 1.0) or 1.0)
    if m == 0.0 or f <= 1.0:
        return 1.0
    return (0.1 * m * math.log(f) + 1.0) ** 2


def random_mla_state(cfg, p, mat, ones):
    H, heads = cfg.hidden_size, cfg.num_attention_heads
    qd = cfg.qk_nope_head_dim + cfg.qk_rope_head_dim
    a = p + "self_attn."
    if cfg.q_lora_rank:
        mat(a + "q_a_proj.weight", cfg.q_lora_rank, H)
        ones(a + "q_a_layernorm.weight", cfg.q_lora_rank)
        mat(a + "q_b_proj.weight", heads * qd, cfg.q_lora_rank)
    else:
        mat(a + "q_proj.weight", heads * qd, H)
    mat(a + "kv_a_proj_with_mqa.weight", cfg.kv_lora_rank + cfg.qk_rope_head_dim, H)
    ones(a + "kv_a_layernorm.weight", cfg.kv_lora_rank)
    mat(a + "kv_b_proj.weight", heads * (cfg.qk_nope_head_dim + cfg.v_head_dim), cfg.kv_lora_rank)
    mat(a + "o_proj.weight", H, heads * cfg.v_head_dim)
