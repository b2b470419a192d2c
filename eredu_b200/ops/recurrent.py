"""Recurrent scans of hybrid (linear-attention) layers.

``gated_delta_scan``: the gated delta rule (eredu/src/backend/mlx/nn/gated_delta.rs:135-183 step, :295-360 scan)::

    S <- S * exp(g_t);  m = S^T k_t;  S <- S + k_t (beta_t (v_t - m))^T;  o_t = S^T q_t

with the state ``S [B, H, Dk, Dv]`` in fp32. ``log_decay`` is ``[B, T, H]`` (one decay per head) or ``[B, T, H, Dk]`` (one
per key channel). Feeding a sequence in chunks with the returned state gives the same outputs as one scan.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import native
from .native import I, P, check, lib, ptr, stream_ptr

native.register("eredu_gated_delta_scan", I, [P, P, P, P, P, P, P, I, I, I, I, I, I, P])
native.register("eredu_mamba2_scan", I, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, P])


# From this many tokens per call the chunk-parallel Mamba-2 form takes over from the token-by-token kernel (measured on a
# B200, 64 heads x 64, state 128: 1.15x at 2048 tokens, 2.5x at 8192). The gated-delta form is exact but, as a chain of
# small library calls (triangular solve, three GEMMs per chunk), 2.5-5x slower than the kernel at those lengths: it is
# not dispatched to.
CHUNKED_SCAN_MIN_TOKENS = 2048


def gated_delta_scan_ref(q, k, v, log_decay, beta, state: Optional[torch.Tensor] = None):
    """PyTorch reference; returns (state fp32 [B, H, Dk, Dv], out [B, T, H, Dv] in q's dtype)."""
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("gated-delta query, key and value tensors must be rank 4")
    if q.shape[:3] != k.shape[:3] or q.shape[:3] != v.shape[:3] or q.shape[3] != k.shape[3]:
        raise ValueError("gated-delta query, key and value batch / sequence / head dimensions must match")
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    if log_decay.dim() not in (3, 4) or tuple(log_decay.shape[:3]) != (B, T, H) or (log_decay.dim() == 4 and log_decay.shape[3] != Dk):
        raise ValueError(f"gated-delta log decay shape {tuple(log_decay.shape)} is incompatible with query shape {tuple(q.shape)}")
    if tuple(beta.shape) != (B, T, H):
        raise ValueError(f"gated-delta beta shape {tuple(beta.shape)} must equal {(B, T, H)}")
    S = torch.zeros((B, H, Dk, Dv), dtype=torch.float32, device=q.device) if state is None else state.float().clone()
    if tuple(S.shape) != (B, H, Dk, Dv):
        raise ValueError(f"gated-delta state shape {tuple(S.shape)} must equal {(B, H, Dk, Dv)}")
    outs = []
    qf, kf, vf, bf = q.float(), k.float(), v.float(), beta.float()
    decay = torch.exp(log_decay.float())
    for t in range(T):
        d = decay[:, t]
        d = d[:, :, None, None] if d.dim() == 2 else d[:, :, :, None]
        S = S * d
        kt = kf[:, t][..., None]                                  # [B, H, Dk, 1]
        mem = (S * kt).sum(-2)                                    # [B, H, Dv]
        delta = (vf[:, t] - mem) * bf[:, t][..., None]
        S = S + kt * delta[:, :, None, :]
        outs.append((S * qf[:, t][..., None]).sum(-2))
    return S, torch.stack(outs, 1).to(q.dtype)


def gated_delta_scan_chunked(q, k, v, log_decay, beta, state: Optional[torch.Tensor] = None, chunk: int = 64, gemm_dtype=None):
    """The gated delta rule with one decay per head and step in its chunk-parallel form. With ``gamma_t`` the decay
    accumulated since the start of the chunk, the state inside a chunk is ``S_t = gamma_t S_0 + sum_{s <= t}
    (gamma_t / gamma_s) k_s u_s^T`` for pseudo-values ``u`` that solve a unit lower-triangular system
    ``(I + diag(beta) A) U = diag(beta) (V - diag(gamma) K S_0)``, ``A[t, s] = (gamma_t / gamma_s) k_t . k_s`` for
    ``s < t``. The inverse and its products with ``V`` and ``K`` are computed for all chunks at once; what stays
    sequential is one step per chunk with three GEMMs (``U``, the outputs, the state). Same arguments and results as
    :func:`gated_delta_scan_ref` (``log_decay`` of shape [B, T, H] only)."""
    if log_decay.dim() != 3:
        raise ValueError("the chunk-parallel form takes one decay per head and step")
    B_, T, H, Dk = q.shape
    Dv = v.shape[-1]
    dev = q.device
    gd = gemm_dtype or (torch.bfloat16 if q.is_cuda else torch.float32)
    S = torch.zeros((B_, H, Dk, Dv), dtype=torch.float32, device=dev) if state is None else state.float().clone()
    Qn = int(chunk)
    nc = (T + Qn - 1) // Qn
    pad = nc * Qn - T

    def prep(t, width=None):                   # [B, T, H, (W)] -> [B, H, nc, Q, (W)] fp32, zero padded
        t = t.float()
        if pad:
            t = torch.cat((t, t.new_zeros((B_, pad) + tuple(t.shape[2:]))), 1)
        t = t.view(B_, nc, Qn, *t.shape[2:])
        return t.permute(0, 3, 1, 2, 4) if t.dim() == 5 else t.permute(0, 3, 1, 2)

    qf, kf, vf = prep(q), prep(k), prep(v)
    bf, a = prep(beta), prep(log_decay)                                 # padded steps: beta 0, decay 1, key 0
    L = torch.cumsum(a, -1)                                             # log gamma_t, inclusive
    gamma = torch.exp(L)
    diff = L[..., :, None] - L[..., None, :]
    tri = torch.ones((Qn, Qn), dtype=torch.bool, device=dev).tril()
    ratio = torch.where(tri, torch.exp(diff.masked_fill(~tri, 0.0)), torch.zeros((), device=dev))          # gamma_t / gamma_s, s <= t
    kk = torch.matmul(kf.to(gd), kf.to(gd).transpose(-1, -2)).float()   # [B, H, nc, Q, Q]
    strict = torch.ones((Qn, Qn), dtype=torch.bool, device=dev).tril(-1)
    A = torch.where(strict, ratio * kk, torch.zeros((), device=dev)) * bf[..., None]
    eye = torch.eye(Qn, device=dev)
    Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False, unitriangular=True)
    Wv = torch.matmul(Tm, vf * bf[..., None])                           # [B, H, nc, Q, Dv]
    Wk = torch.matmul(Tm, kf * (bf * gamma)[..., None])                 # [B, H, nc, Q, Dk]
    qk = torch.matmul(qf.to(gd), kf.to(gd).transpose(-1, -2)).float() * ratio                               # s <= t
    to_end = torch.exp(L[..., -1:] - L)                                 # gamma_Q / gamma_s
    kend = kf * to_end[..., None]
    outs = []
    for c in range(nc):
        U = Wv[:, :, c] - torch.matmul(Wk[:, :, c].to(gd), S.to(gd)).float()                               # [B, H, Q, Dv]
        o = torch.matmul(qf[:, :, c].to(gd), S.to(gd)).float() * gamma[:, :, c, :, None] + torch.matmul(qk[:, :, c].to(gd), U.to(gd)).float()
        S = S * gamma[:, :, c, -1, None, None] + torch.matmul(kend[:, :, c].to(gd).transpose(-1, -2), U.to(gd)).float()
        outs.append(o)
    out = torch.stack(outs, 2).permute(0, 2, 3, 1, 4).reshape(B_, nc * Qn, H, Dv)[:, :T]
    return S, out.to(q.dtype)


def gated_delta_scan(q, k, v, log_decay, beta, state: Optional[torch.Tensor] = None):
    """CUDA: one kernel for the whole chunk (bf16 q / k / v, Dk of 64 or 128); otherwise the reference."""
    if not q.is_cuda or q.dtype != torch.bfloat16 or q.shape[-1] not in (64, 128):
        return gated_delta_scan_ref(q, k, v, log_decay, beta, state)
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    if tuple(beta.shape) != (B, T, H) or tuple(log_decay.shape[:3]) != (B, T, H):
        raise ValueError("gated-delta beta / log decay shapes do not match the query")
    S = torch.zeros((B, H, Dk, Dv), dtype=torch.float32, device=q.device) if state is None else state.float().contiguous().clone()
    out = torch.empty((B, T, H, Dv), dtype=q.dtype, device=q.device)
    # every operand is bound to a name until the launch is queued: a temporary made by ``.contiguous()`` / ``.float()``
    # would go back to the caching allocator at once and the next temporary could land on the same bytes
    g = log_decay.float().contiguous()
    qc, kc, vc, bc = q.contiguous(), k.to(q.dtype).contiguous(), v.to(q.dtype).contiguous(), beta.float().contiguous()
    code = lib().eredu_gated_delta_scan(ptr(qc), ptr(kc), ptr(vc), ptr(g), ptr(bc), ptr(S), ptr(out), B, T, H, Dk, Dv,
                                        1 if g.dim() == 4 else 0, stream_ptr(q.device))
    check(code, "eredu_gated_delta_scan")
    return S, out


def mamba2_scan_ref(x, B, C, dt, A, D, state: Optional[torch.Tensor] = None):
    """Mamba-2 selective state-space recurrence, token by token (eredu/src/backend/mlx/architectures/nemotron_h/
    model.rs:1929-1962): ``S <- S * exp(dt A) + x (dt B)^T;  y = S C + D x`` per head.

    x [Bt, T, H, P]; B, C [Bt, T, G, N] with G dividing H (one B / C per group of heads; G = H when already expanded);
    dt [Bt, T, H] (after softplus and floor); A [H] (negative); D [H]; state fp32 [Bt, H, P, N]. Returns (state,
    y [Bt, T, H, P] in x's dtype)."""
    Bt, T, H, P = x.shape
    N = B.shape[-1]
    if B.shape[2] != H:
        if H % B.shape[2]:
            raise ValueError("Mamba-2 group count must divide the head count")
        B, C = B.repeat_interleave(H // B.shape[2], 2), C.repeat_interleave(H // C.shape[2], 2)
    S = torch.zeros((Bt, H, P, N), dtype=torch.float32, device=x.device) if state is None else state.float().clone()
    xf, Bf, Cf, dtf = x.float(), B.float(), C.float(), dt.float()
    Af, Df = A.float().view(1, H, 1, 1), D.float().view(1, H, 1)
    ys = []
    for t in range(T):
        d = dtf[:, t]                                                     # [Bt, H]
        dA = torch.exp(d[:, :, None, None] * Af)
        dBx = xf[:, t][..., None] * (d[:, :, None] * Bf[:, t])[:, :, None, :]
        S = S * dA + dBx
        ys.append((S * Cf[:, t][:, :, None, :]).sum(-1) + xf[:, t] * Df)
    return S, torch.stack(ys, 1).to(x.dtype)


def mamba2_scan_chunked(x, B, C, dt, A, D, state: Optional[torch.Tensor] = None, chunk: int = 64, gemm_dtype=None):
    """The same recurrence in its chunk-parallel (state-space duality) form: the sequence is cut into chunks of ``chunk``
    tokens; inside a chunk the outputs are a masked, decay-weighted ``(C B^T) x`` product, every chunk contributes one
    state update ``sum_s decay(s -> end) x_s B_s^T``, the states are carried from chunk to chunk (the only sequential
    part: T / chunk steps on [P, N] matrices) and enter the outputs as ``decay(start -> t) C_t S``. All four products
    are batched GEMMs, so a long prefill runs on the tensor cores instead of token by token. Same arguments and results
    as :func:`mamba2_scan_ref`; ``gemm_dtype`` (default: fp32 on the CPU, bf16 on CUDA) is the operand type of the
    GEMMs, decays and accumulation stay fp32."""
    Bt, T, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    if H % G:
        raise ValueError("Mamba-2 group count must divide the head count")
    dev = x.device
    gd = gemm_dtype or (torch.bfloat16 if x.is_cuda else torch.float32)
    S = torch.zeros((Bt, H, P, N), dtype=torch.float32, device=dev) if state is None else state.float().clone()
    Q = int(chunk)
    nc = (T + Q - 1) // Q
    pad = nc * Q - T
    xf, dtf = x.float(), dt.float()
    if pad:                                   # padded steps have dt = 0: no decay, no input, outputs dropped
        xf = torch.cat((xf, xf.new_zeros(Bt, pad, H, P)), 1)
        dtf = torch.cat((dtf, dtf.new_zeros(Bt, pad, H)), 1)
        B = torch.cat((B, B.new_zeros(Bt, pad, G, N)), 1)
        C = torch.cat((C, C.new_zeros(Bt, pad, G, N)), 1)
    rep = H // G
    a = dtf * A.float().view(1, 1, H)                                   # log decay per step, <= 0
    a = a.view(Bt, nc, Q, H).permute(0, 3, 1, 2)                        # [Bt, H, nc, Q]
    L = torch.cumsum(a, -1)                                             # inclusive prefix inside the chunk
    xs = (xf * dtf[..., None]).view(Bt, nc, Q, H, P).permute(0, 3, 1, 2, 4)            # x * dt: [Bt, H, nc, Q, P]
    Bc = B.float().view(Bt, nc, Q, G, N).permute(0, 3, 1, 2, 4)         # [Bt, G, nc, Q, N]
    Cc = C.float().view(Bt, nc, Q, G, N).permute(0, 3, 1, 2, 4)
    # inside a chunk: y[t] = sum_{s <= t} exp(L_t - L_s) (C_t . B_s) xs[s]
    cb = torch.matmul(Cc.to(gd), Bc.to(gd).transpose(-1, -2)).float()   # [Bt, G, nc, Q, Q]
    cb = cb.repeat_interleave(rep, 1) if rep > 1 else cb                # [Bt, H, nc, Q, Q]
    diff = L[..., :, None] - L[..., None, :]                            # L_t - L_s
    tri = torch.ones((Q, Q), dtype=torch.bool, device=dev).tril()
    w = torch.where(tri, torch.exp(diff.masked_fill(~tri, 0.0)), torch.zeros((), device=dev)) * cb
    y = torch.matmul(w.to(gd), xs.to(gd)).float()                       # [Bt, H, nc, Q, P]
    # what every chunk adds to the state: sum_s exp(L_end - L_s) xs[s] B_s^T
    to_end = torch.exp(L[..., -1:] - L)                                 # [Bt, H, nc, Q]
    Bh = Bc.repeat_interleave(rep, 1) if rep > 1 else Bc                # [Bt, H, nc, Q, N]
    Ch = Cc.repeat_interleave(rep, 1) if rep > 1 else Cc
    upd = torch.matmul((xs * to_end[..., None]).to(gd).transpose(-1, -2), Bh.to(gd)).float()      # [Bt, H, nc, P, N]
    total = torch.exp(L[..., -1])                                       # decay over a whole chunk: [Bt, H, nc]
    # the sequential part: the state that enters every chunk
    entering = []
    for c in range(nc):
        entering.append(S)
        S = S * total[:, :, c, None, None] + upd[:, :, c]
    Sin = torch.stack(entering, 2)                                      # [Bt, H, nc, P, N]
    # contribution of the entering state: exp(L_t) C_t . S
    y = y + torch.matmul(Ch.to(gd), Sin.to(gd).transpose(-1, -2)).float() * torch.exp(L)[..., None]
    y = y.permute(0, 2, 3, 1, 4).reshape(Bt, nc * Q, H, P)[:, :T]
    y = y + xf[:, :T] * D.float().view(1, 1, H, 1)
    return S, y.to(x.dtype)


def mamba2_scan(x, B, C, dt, A, D, state: Optional[torch.Tensor] = None):
    """CUDA: one kernel for the whole chunk (bf16 x / B / C, state size 64, 128 or 256) for decode-sized calls, the
    chunk-parallel GEMM form for long prefills; otherwise the reference."""
    if x.is_cuda and x.shape[1] >= CHUNKED_SCAN_MIN_TOKENS:
        return mamba2_scan_chunked(x, B, C, dt, A, D, state)
    if not x.is_cuda or x.dtype != torch.bfloat16 or B.shape[-1] not in (64, 128, 256):
        return mamba2_scan_ref(x, B, C, dt, A, D, state)
    Bt, T, H, P_ = x.shape
    G, N = B.shape[2], B.shape[3]
    if tuple(C.shape) != tuple(B.shape) or tuple(B.shape[:2]) != (Bt, T) or H % G or tuple(dt.shape) != (Bt, T, H):
        raise ValueError("Mamba-2 B / C / dt shapes do not match x")
    S = torch.zeros((Bt, H, P_, N), dtype=torch.float32, device=x.device) if state is None else state.float().contiguous().clone()
    if tuple(S.shape) != (Bt, H, P_, N):
        raise ValueError(f"Mamba-2 state shape {tuple(S.shape)} must equal {(Bt, H, P_, N)}")
    out = torch.empty((Bt, T, H, P_), dtype=x.dtype, device=x.device)
    # operands stay bound to names until the launch is queued (see gated_delta_scan)
    xc, Bc, Cc = x.contiguous(), B.to(torch.bfloat16).contiguous(), C.to(torch.bfloat16).contiguous()
    dtc, Ac, Dc = dt.float().contiguous(), A.float().contiguous(), D.float().contiguous()
    code = lib().eredu_mamba2_scan(ptr(xc), ptr(Bc), ptr(Cc), ptr(dtc), ptr(Ac), ptr(Dc), ptr(S), ptr(out), Bt, T, H, G,
                                   P_, N, stream_ptr(x.device))
    check(code, "eredu_mamba2_scan")
    return S, out
