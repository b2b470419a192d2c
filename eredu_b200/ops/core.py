"""Decoder-block operators.

Each operator has two implementations with identical semantics:

* ``*_ref`` - plain PyTorch, any device/dtype; the numerics oracle for tests and the execution path for
  CPU tensors (the fp32 CPU slice of the framework).
* the sm_100a kernel from ``liberedu_cuda.so`` for CUDA bf16 tensors. There is no fallback from the
  kernel to PyTorch on a GPU: a missing library raises.
"""
from __future__ import annotations

from os import environ as _environ

import math

import torch
import torch.nn.functional as F

from . import native
from .native import check, lib, ptr, status_word, stream_ptr

PAGE = 16


def _sm_count(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


# ------------------------------------------------------------------------------------------ linear
def linear_ref(x, w, bias=None, residual=None, out_dtype=None):
    y = F.linear(x.float(), w.float(), None if bias is None else bias.float())
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype or x.dtype)


def gated_linear_ref(x, w_gate_up, inter, bias=None, out_dtype=None):
    """silu(x Wg^T) * (x Wu^T) with Wg = w[:inter], Wu = w[inter:2*inter]."""
    y = F.linear(x.float(), w_gate_up.float(), None if bias is None else bias.float())
    return (F.silu(y[..., :inter]) * y[..., inter:]).to(out_dtype or x.dtype)


def _norm_args(x, row_ssq, norm_eps, want_ssq, n_out):
    """(ssq_in ptr, parts, eps, dim, ssq_out tensor) for the RMSNorm fusion of the GEMM epilogue."""
    ssq_out = None
    if want_ssq:
        ssq_out = torch.empty((x.shape[0], (n_out + 127) // 128), dtype=torch.float32, device=x.device)
    if row_ssq is None:
        return None, 0, 0.0, 0, ssq_out
    assert row_ssq.dtype == torch.float32 and row_ssq.is_contiguous() and row_ssq.shape[0] == x.shape[0]
    return row_ssq, row_ssq.shape[1], float(norm_eps), x.shape[1], ssq_out


def linear(x, w, bias=None, residual=None, out_dtype=None, out=None, force_split=0, row_ssq=None, norm_eps=0.0,
           want_ssq=False, dynamic_weight=False):
    """y = x @ w.T (+ bias) (+ residual). x: [M, K], w: [N, K].

    ``row_ssq`` ([M, parts] fp32 partial sums of squares of x's rows): the output rows are scaled by
    ``rsqrt(sum(row_ssq) / K + norm_eps)`` - an RMSNorm whose weight vector was folded into ``w``.
    ``want_ssq``: also return per-128-column-tile sums of squares of the stored output ([M, ceil(N/128)]).
    ``dynamic_weight``: ``w`` was written by a kernel enqueued just before this call (e.g. a dequantised scratch
    matrix); the kernel then does not fetch weight tiles ahead of its stream dependency."""
    if not x.is_cuda:
        if row_ssq is not None:
            x = x.float() * torch.rsqrt(row_ssq.sum(-1, keepdim=True) / x.shape[1] + norm_eps)
        y = linear_ref(x, w, bias, residual, out_dtype or w.dtype)
        return (y, y.float().pow(2).sum(-1, keepdim=True)) if want_ssq else y
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "CUDA linear is bf16"
    M, K = x.shape
    N = w.shape[0]
    out_dtype = out_dtype or torch.bfloat16
    assert out_dtype in (torch.bfloat16, torch.float32)
    assert x.stride(1) == 1 and w.stride(1) == 1
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    ssq_in, parts, eps, dim, ssq_out = _norm_args(x, row_ssq, norm_eps, want_ssq, N)
    if M == 0:
        return (out, ssq_out) if want_ssq else out
    code = lib().eredu_gemm_bf16(
        ptr(x), ptr(w), ptr(out), ptr(residual), ptr(bias), M, N, K, x.stride(0), w.stride(0), out.stride(0),
        residual.stride(0) if residual is not None else 0, w.shape[0], 0, 0, 1 if out_dtype == torch.float32 else 0,
        force_split, _sm_count(x.device), ptr(status_word(x.device)), ptr(ssq_in), parts, eps, dim, ptr(ssq_out),
        1 if dynamic_weight else 0, stream_ptr(x.device))
    check(code, "eredu_gemm_bf16")
    return (out, ssq_out) if want_ssq else out


def gated_linear(x, w_gate_up, inter, bias=None, out=None, force_split=0, row_ssq=None, norm_eps=0.0):
    """Fused SwiGLU up-projection: one GEMM kernel, activation applied in the epilogue (``row_ssq``: see linear)."""
    if not x.is_cuda:
        if row_ssq is not None:
            x = x.float() * torch.rsqrt(row_ssq.sum(-1, keepdim=True) / x.shape[1] + norm_eps)
        return gated_linear_ref(x, w_gate_up, inter, bias, w_gate_up.dtype)
    assert x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16
    M, K = x.shape
    if out is None:
        out = torch.empty((M, inter), dtype=torch.bfloat16, device=x.device)
    if M == 0:
        return out
    ssq_in, parts, eps, dim, _ = _norm_args(x, row_ssq, norm_eps, False, inter)
    code = lib().eredu_gemm_bf16(
        ptr(x), ptr(w_gate_up), ptr(out), None, ptr(bias), M, inter, K, x.stride(0), w_gate_up.stride(0),
        out.stride(0), 0, w_gate_up.shape[0], 1, inter, 0, force_split, _sm_count(x.device),
        ptr(status_word(x.device)), ptr(ssq_in), parts, eps, dim, None, 0, stream_ptr(x.device))
    check(code, "eredu_gemm_bf16(dual)")
    return out


# ------------------------------------------------------------------------------------------ norm
def rmsnorm_ref(x, weight, eps, residual=None, weight_offset=0.0):
    h = x.float()
    if residual is not None:
        h = (h + residual.float()).to(x.dtype).float()
    y = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * (weight.float() + weight_offset)
    return y.to(x.dtype), (h.to(x.dtype) if residual is not None else None)


def rmsnorm(x, weight, eps, residual=None, weight_offset=0.0):
    """Returns (normed, h) where h = x + residual (None when no residual was given)."""
    if not x.is_cuda:
        return rmsnorm_ref(x, weight, eps, residual, weight_offset)
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.float32 and x.is_contiguous()
    M, H = x.shape
    y = torch.empty_like(x)
    h = torch.empty_like(x) if residual is not None else None
    code = lib().eredu_rmsnorm(ptr(x), ptr(residual), ptr(weight), ptr(y), ptr(h), M, H, eps, weight_offset,
                               stream_ptr(x.device))
    check(code, "eredu_rmsnorm")
    return y, h


# ------------------------------------------------------------------------------------------ rope + kv append
def rope_kv_ref(qkv, positions, slots, inv_freq, k_cache, v_cache, n_q, n_kv, head_dim, rot=None, interleaved=False,
                attn_factor=1.0, q_norm_w=None, k_norm_w=None, norm_eps=1e-6, norm_w_off=0.0, mrope_section=None):
    """``positions`` [M], or [3, M] (temporal, height, width axes of multimodal prompts) with ``mrope_section``: frequency
    index f then takes its angle from axis f % 3 while f < 3 * section[axis] (interleaved T H W T H W ... layout), the
    temporal axis otherwise."""
    M = qkv.shape[0]
    D = head_dim
    rot = rot or D
    x = qkv.float().view(M, n_q + 2 * n_kv, D)
    q, k, v = x[:, :n_q], x[:, n_q:n_q + n_kv], x[:, n_q + n_kv:]

    def hnorm(t, w):
        if w is None:
            return t
        y = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + norm_eps) * (w.float() + norm_w_off)
        return y.to(qkv.dtype).float()

    q, k = hnorm(q, q_norm_w), hnorm(k, k_norm_w)
    if positions.dim() == 2:
        axes = positions.float()[:, :, None] * inv_freq.float()[None, None, :]          # [3, M, rot/2]
        ang = axes[0].clone()
        for axis, offset in ((1, 1), (2, 2)):
            idx = slice(offset, int(mrope_section[axis]) * 3, 3)
            ang[:, idx] = axes[axis][:, idx]
    else:
        ang = positions.float()[:, None] * inv_freq.float()[None, :]  # [M, rot/2]
    cos, sin = (ang.cos() * attn_factor)[:, None, :], (ang.sin() * attn_factor)[:, None, :]

    def rotate(t):
        tr, tp = t[..., :rot], t[..., rot:]
        if interleaved:
            a, b = tr[..., 0::2], tr[..., 1::2]
            out = torch.stack((a * cos - b * sin, b * cos + a * sin), dim=-1).flatten(-2)
        else:
            a, b = tr[..., : rot // 2], tr[..., rot // 2:]
            out = torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1)
        return torch.cat((out, tp), dim=-1)

    q, k = rotate(q), rotate(k)
    ok = slots >= 0
    page, off = (slots[ok] // PAGE), (slots[ok] % PAGE)
    k_cache[page, :, off] = k[ok].to(k_cache.dtype)
    v_cache[page, :, off] = v[ok].to(v_cache.dtype)
    return q.to(qkv.dtype).contiguous()


def rope_kv(qkv, positions, slots, inv_freq, k_cache, v_cache, n_q, n_kv, head_dim, rot=None, interleaved=False,
            attn_factor=1.0, q_norm_w=None, k_norm_w=None, norm_eps=1e-6, norm_w_off=0.0, q_out=None, mrope_section=None):
    """Per-head q/k norm (optional) + RoPE on q and k, K/V scattered into their cache pages. Returns q [M,n_q,D].
    Three-axis positions ([3, M], prompts with images) take the tensor-operation path on either device."""
    if not qkv.is_cuda or head_dim not in KERNEL_HEAD_DIMS or positions.dim() == 2:
        return rope_kv_ref(qkv, positions, slots, inv_freq, k_cache, v_cache, n_q, n_kv, head_dim, rot, interleaved,
                           attn_factor, q_norm_w, k_norm_w, norm_eps, norm_w_off, mrope_section)
    M = qkv.shape[0]
    rot = rot or head_dim
    assert positions.dtype == torch.int32 and slots.dtype == torch.int64 and inv_freq.dtype == torch.float32
    if q_out is None:
        q_out = torch.empty((M, n_q, head_dim), dtype=qkv.dtype, device=qkv.device)
    code = lib().eredu_rope_kv(ptr(qkv), ptr(q_out), ptr(k_cache), ptr(v_cache), ptr(positions), ptr(slots),
                               ptr(inv_freq), ptr(q_norm_w), ptr(k_norm_w), M, qkv.stride(0), n_q, n_kv, head_dim, rot,
                               1 if interleaved else 0, attn_factor, norm_eps, norm_w_off, stream_ptr(qkv.device))
    check(code, "eredu_rope_kv")
    return q_out


# Head sizes the attention and RoPE kernels are instantiated for; other sizes (256 in the Qwen3-Next family) run through
# the tensor-operation references on either device, which read lengths on the host: such models decode eagerly.
KERNEL_HEAD_DIMS = (64, 128)


# ------------------------------------------------------------------------------------------ attention
def _gather_kv(cache, block_table_row, kv_len):
    n_pages = (kv_len + PAGE - 1) // PAGE
    pages = cache[block_table_row[:n_pages].long()]  # [n_pages, n_kv, 16, D]
    return pages.permute(1, 0, 2, 3).reshape(cache.shape[1], n_pages * PAGE, cache.shape[3])[:, :kv_len]


def attention_ref(q, k_cache, v_cache, block_table, seq_lens, q_lens, scale, window=0, sinks=None, bidir=None):
    """q: [total_q, n_q, D]; the last q_lens[b] positions of sequence b are its queries (causal).
    ``bidir``: per sequence None or an int tensor [kv_len] of group ids (negative: none); positions of one group see each
    other in both directions, whatever the causal order and the window say (soft tokens of one image)."""
    total, n_q, D = q.shape
    n_kv = k_cache.shape[1]
    group = n_q // n_kv
    out = torch.empty_like(q)
    start = 0
    for b, (kv_len, ql) in enumerate(zip(seq_lens.tolist(), q_lens)):
        k = _gather_kv(k_cache, block_table[b], kv_len).float()  # [n_kv, T, D]
        v = _gather_kv(v_cache, block_table[b], kv_len).float()
        qb = q[start:start + ql].float().permute(1, 0, 2)  # [n_q, ql, D]
        k = k.repeat_interleave(group, dim=0)
        v = v.repeat_interleave(group, dim=0)
        s = torch.einsum("hqd,hkd->hqk", qb, k) * scale
        qpos = torch.arange(kv_len - ql, kv_len, device=q.device)[:, None]
        kpos = torch.arange(kv_len, device=q.device)[None, :]
        mask = kpos <= qpos
        if window > 0:
            mask = mask & (kpos > qpos - window)
        if bidir is not None and bidir[b] is not None:
            grp = bidir[b].to(q.device)
            mask = mask | ((grp[kv_len - ql:kv_len, None] == grp[None, :kv_len]) & (grp[kv_len - ql:kv_len, None] >= 0))
        s = s.masked_fill(~mask[None], float("-inf"))
        if sinks is not None:
            s = torch.cat((s, sinks.float()[:, None, None].expand(n_q, ql, 1)), dim=-1)
            p = torch.softmax(s, dim=-1)[..., :-1]
        else:
            p = torch.softmax(s, dim=-1)
        out[start:start + ql] = torch.einsum("hqk,hkd->hqd", p, v).permute(1, 0, 2).to(q.dtype)
        start += ql
    return out


TC_PREFILL = _environ.get("EREDU_TC_PREFILL", "1") != "0"      # head size 64 / 128: the tcgen05 kernel (else the mma.sync one)


def attention_prefill(q, k_cache, v_cache, block_table, seq_lens, cu_q, max_q_len, scale, window=0, sinks=None,
                      out=None):
    if not q.is_cuda or q.shape[2] not in KERNEL_HEAD_DIMS:
        q_lens = (cu_q[1:] - cu_q[:-1]).tolist()
        return attention_ref(q, k_cache, v_cache, block_table, seq_lens, q_lens, scale, window, sinks)
    assert q.dtype == torch.bfloat16 and q.is_contiguous()
    assert block_table.dtype == torch.int32 and seq_lens.dtype == torch.int32 and cu_q.dtype == torch.int32
    if out is None:
        out = torch.empty_like(q)
    B = seq_lens.shape[0]
    if (TC_PREFILL and q.shape[2] in (64, 128) and k_cache.is_contiguous() and v_cache.is_contiguous()
            and k_cache.shape[2] == 16 and k_cache.shape[3] == q.shape[2] and v_cache.shape == k_cache.shape and out.is_contiguous()
            and (sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous()))):
        # tcgen05 kernel (csrc/kernels/attention_tc.cu): QK^T and PV on the 5th-generation tensor cores, pages by TMA
        code = lib().eredu_attn_prefill_tc(ptr(q), ptr(k_cache), ptr(v_cache), ptr(out), ptr(block_table), ptr(seq_lens),
                                           ptr(cu_q), ptr(sinks), B, q.shape[0], max_q_len, block_table.stride(0),
                                           k_cache.shape[0], q.shape[1], k_cache.shape[1], q.shape[2], int(window), scale,
                                           ptr(status_word(q.device)), stream_ptr(q.device))
        check(code, "eredu_attn_prefill_tc")
        return out
    code = lib().eredu_attn_prefill(ptr(q), ptr(k_cache), ptr(v_cache), ptr(out), ptr(block_table), ptr(seq_lens),
                                    ptr(cu_q), ptr(sinks), B, max_q_len, block_table.stride(0), q.shape[1],
                                    k_cache.shape[1], q.shape[2], window, scale, stream_ptr(q.device))
    check(code, "eredu_attn_prefill")
    return out


import os as _os

_SPLIT_WAVES = int(_os.environ.get("EREDU_DECODE_SPLIT_WAVES", "2"))   # CTAs per SM the split-KV grid aims for


CLUSTER_SPLITS = 8      # splits the decode kernel combines through distributed shared memory (portable cluster size)
FUSED_ROPE_MAX_NEW = 8  # new tokens per sequence the fused RoPE + append decode path takes


def decode_splits(batch, n_kv, max_kv_len, sm_count=148):
    """Split-KV factor: enough CTAs to fill the GPU once (a second wave costs more than it returns: the CTAs of the
    following kernel are already resident under programmatic dependent launch), at least 8 pages per split."""
    ctas = max(1, batch * n_kv)
    pages = max(1, (max_kv_len + PAGE - 1) // PAGE)
    want = max(1, (_SPLIT_WAVES * sm_count) // ctas)
    splits = int(max(1, min(want, pages // 8 if pages >= 8 else 1, 32)))
    # up to CLUSTER_SPLITS splits combine inside a thread-block cluster (no scratch, no second pass over global memory):
    # prefer that form while a split then still has at most 32 pages (8 per warp)
    if splits > CLUSTER_SPLITS and pages <= 32 * CLUSTER_SPLITS:
        splits = CLUSTER_SPLITS
    return splits


def attention_decode(q, k_cache, v_cache, block_table, seq_lens, q_per_seq, scale, splits=1, window=0, sinks=None,
                     scratch=None, out=None):
    """q: [B * q_per_seq, n_q, D]. ``scratch`` = (part_o, part_ml, counters) from :func:`decode_scratch` when
    splits > 1 (fp32 partials and zeroed int32 arrival tickets)."""
    if not q.is_cuda or q.shape[2] not in KERNEL_HEAD_DIMS:
        return attention_ref(q, k_cache, v_cache, block_table, seq_lens, [q_per_seq] * seq_lens.shape[0], scale,
                             window, sinks)
    assert q.dtype == torch.bfloat16 and q.is_contiguous()
    B = seq_lens.shape[0]
    n_q, D = q.shape[1], q.shape[2]
    if out is None:
        out = torch.empty_like(q)
    part_o = part_ml = counters = None
    if splits > CLUSTER_SPLITS:
        if scratch is None:
            scratch = decode_scratch(B, q_per_seq, n_q, D, splits, q.device)
        part_o, part_ml, counters = scratch
        assert part_o.numel() >= B * q_per_seq * n_q * splits * D and part_ml.numel() >= B * q_per_seq * n_q * splits * 2
        assert counters.numel() >= B * k_cache.shape[1] and counters.dtype == torch.int32
    code = lib().eredu_attn_decode(ptr(q), ptr(k_cache), ptr(v_cache), ptr(out), ptr(block_table), ptr(seq_lens),
                                   ptr(sinks), ptr(part_o), ptr(part_ml), ptr(counters), B, q_per_seq, block_table.stride(0), n_q,
                                   k_cache.shape[1], D, splits, window, scale, stream_ptr(q.device))
    check(code, "eredu_attn_decode")
    return out


def attention_decode_rope(qkv, k_cache, v_cache, block_table, seq_lens, q_per_seq, scale, positions, slots, inv_freq,
                          n_q, n_kv, head_dim, rot=None, interleaved=False, attn_factor=1.0, q_norm_w=None, k_norm_w=None,
                          norm_eps=1e-6, norm_w_off=0.0, splits=1, window=0, sinks=None, scratch=None):
    """Decode attention straight from the qkv projection output [B * q_per_seq, >= (n_q + 2 n_kv) * D]: per-head
    q/k norm, RoPE and the KV append run inside the attention kernel (one launch instead of two). CPU tensors and
    head sizes without a kernel compose the two reference operators."""
    if not qkv.is_cuda or head_dim not in KERNEL_HEAD_DIMS or positions.dim() != 1 or q_per_seq > FUSED_ROPE_MAX_NEW:
        q = rope_kv(qkv, positions, slots, inv_freq, k_cache, v_cache, n_q, n_kv, head_dim, rot, interleaved, attn_factor,
                    q_norm_w, k_norm_w, norm_eps, norm_w_off)
        return attention_decode(q, k_cache, v_cache, block_table, seq_lens, q_per_seq, scale, splits, window, sinks, scratch)
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1
    assert positions.dtype == torch.int32 and slots.dtype == torch.int64 and inv_freq.dtype == torch.float32
    B = seq_lens.shape[0]
    out = torch.empty((qkv.shape[0], n_q, head_dim), dtype=qkv.dtype, device=qkv.device)
    part_o = part_ml = counters = None
    if splits > CLUSTER_SPLITS:
        if scratch is None:
            scratch = decode_scratch(B, q_per_seq, n_q, head_dim, splits, qkv.device)
        part_o, part_ml, counters = scratch
        assert part_o.numel() >= B * q_per_seq * n_q * splits * head_dim and counters.numel() >= B * n_kv
    code = lib().eredu_attn_decode_rope(ptr(qkv), qkv.stride(0), ptr(k_cache), ptr(v_cache), ptr(out), ptr(block_table),
                                        ptr(seq_lens), ptr(sinks), ptr(part_o), ptr(part_ml), ptr(counters), ptr(positions),
                                        ptr(slots), ptr(inv_freq), ptr(q_norm_w), ptr(k_norm_w), B, q_per_seq,
                                        block_table.stride(0), n_q, n_kv, head_dim, rot or head_dim, 1 if interleaved else 0,
                                        splits, window, scale, attn_factor, norm_eps, norm_w_off, stream_ptr(qkv.device))
    check(code, "eredu_attn_decode_rope")
    return out


def decode_scratch(batch, q_per_seq, n_q, head_dim, splits, device):
    rows = batch * q_per_seq * n_q
    return (torch.empty(rows * splits * head_dim, dtype=torch.float32, device=device),
            torch.empty(rows * splits * 2, dtype=torch.float32, device=device),
            torch.zeros(batch * n_q, dtype=torch.int32, device=device))


# ------------------------------------------------------------------------------------------ embedding / activation
def embedding(ids, table, vocab_start=0, scale=1.0, want_ssq=False):
    """Rows of ``table`` for ``ids`` (zero rows for ids outside this shard). ``want_ssq``: also the per-row sum of
    squares ([M, 1] fp32) consumed by a GEMM with a folded RMSNorm."""
    if not table.is_cuda:
        local = ids.long() - vocab_start
        ok = (local >= 0) & (local < table.shape[0])
        out = table[local.clamp(0, table.shape[0] - 1)] * ok[:, None].to(table.dtype)
        out = out * scale if scale != 1.0 else out
        return (out, out.float().pow(2).sum(-1, keepdim=True)) if want_ssq else out
    assert ids.dtype == torch.int32 and table.dtype == torch.bfloat16
    M, H = ids.shape[0], table.shape[1]
    out = torch.empty((M, H), dtype=table.dtype, device=table.device)
    ssq = torch.empty((M, 1), dtype=torch.float32, device=table.device) if want_ssq else None
    code = lib().eredu_embedding(ptr(ids), ptr(table), ptr(out), M, H, vocab_start, table.shape[0], scale, ptr(ssq),
                                 stream_ptr(table.device))
    check(code, "eredu_embedding")
    return (out, ssq) if want_ssq else out


def silu_mul(x, inter, limit=0.0):
    """x: [M, 2*inter] = [gate | up] -> silu(gate) * up."""
    if not x.is_cuda:
        g, u = x[..., :inter].float(), x[..., inter:].float()
        if limit > 0:
            g, u = g.clamp(max=limit), u.clamp(-limit, limit)
        return (F.silu(g) * u).to(x.dtype)
    M = x.shape[0]
    y = torch.empty((M, inter), dtype=x.dtype, device=x.device)
    code = lib().eredu_silu_mul(ptr(x), ptr(y), M, inter, x.stride(0), limit, stream_ptr(x.device))
    check(code, "eredu_silu_mul")
    return y
