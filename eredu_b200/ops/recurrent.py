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


def mamba2_scan(x, B, C, dt, A, D, state: Optional[torch.Tensor] = None):
    """CUDA: one kernel for the whole chunk (bf16 x / B / C, state size 64, 128 or 256); otherwise the reference."""
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
