"""Gated causal short convolution with recurrent state (the operator of LFM2's "conv" layers).

``proj = in_proj(x) = [B | C | X]``; ``bx = B * X``; ``y[t] = sum_j w[:, j] * bx[t - (L-1) + j]`` (depthwise, causal);
``out = C * (y + bias)`` (eredu/src/backend/mlx/architectures/lfm2/model.rs:899-914; the rolling cache of the last
L-1 inputs is ``CausalConv1dCache``). The state pool ``[pages, L-1, C]`` is indexed by each sequence's first KV page
(column 0 of the block table), so chunked prefill, decode and mixed batches share one code path and a captured
decode graph needs no host-side indices.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import native
from .native import I, P, check, lib, ptr, stream_ptr

native.register("eredu_short_conv", I, [P, I, P, P, P, P, I, P, I, P, P, P, I, I, I, I, I, I, P])


def short_conv_ref(proj, w, bias, state, block_table, cu_q, q_per_seq, positions, slots, mode=0, x_off=0):
    """PyTorch reference (any device, fp32 maths, bx and the state rounded to the state's dtype like the kernel).
    mode 0: gated LFM2 form over proj = [B | C | X]; mode 1: silu(conv(proj[:, x_off : x_off + C]))."""
    M = proj.shape[0]
    C = w.shape[0]
    L = w.shape[1]
    out = torch.zeros((M, C), dtype=proj.dtype, device=proj.device)
    B = block_table.shape[0]
    bounds = cu_q.tolist() if cu_q is not None else [i * q_per_seq for i in range(B + 1)]
    wf = w.float()
    for b in range(B):
        r0, r1 = bounds[b], bounds[b + 1]
        if r1 <= r0 or int(slots[r0]) < 0:
            continue
        page = int(block_table[b, 0])
        pos0 = int(positions[r0])
        pj = proj[r0:r1].float()
        bx = (pj[:, x_off:x_off + C] if mode == 1 else (pj[:, :C] * pj[:, 2 * C:3 * C])).to(state.dtype).float()
        hist = state[page].float().clone()                         # [L-1, C]: positions pos0-(L-1) .. pos0-1
        for j in range(L - 1):
            if pos0 - (L - 1) + j < 0:
                hist[j] = 0
        full = torch.cat((hist, bx), 0)                            # [L-1+n, C]
        n = r1 - r0
        y = torch.zeros((n, C), dtype=torch.float32, device=proj.device)
        for j in range(L):
            y += wf[:, j][None, :] * full[j:j + n]
        if bias is not None:
            y += bias.float()[None, :]
        out[r0:r1] = (torch.nn.functional.silu(y) if mode == 1 else pj[:, C:2 * C] * y).to(proj.dtype)
        state[page] = full[n:n + L - 1].to(state.dtype)
    return out


def short_conv(proj: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
               block_table: torch.Tensor, cu_q: Optional[torch.Tensor], q_per_seq: int, positions: torch.Tensor,
               slots: torch.Tensor, max_q_len: int = 1, mode: int = 0, x_off: int = 0) -> torch.Tensor:
    """proj [M, 3C] (mode 0) or [M, >= x_off + C] (mode 1) -> out [M, C]; ``state`` [pages, L-1, C] is updated in place.
    w fp32 [C, L]; column 0 of ``block_table`` names each sequence's state row."""
    if not proj.is_cuda:
        return short_conv_ref(proj, w, bias, state, block_table, cu_q, q_per_seq, positions, slots, mode, x_off)
    M = proj.shape[0]
    C, L = w.shape
    assert proj.dtype == torch.bfloat16 and state.dtype == torch.bfloat16 and proj.stride(1) == 1
    assert w.dtype == torch.float32 and w.is_contiguous() and state.is_contiguous() and slots.dtype == torch.int64
    out = torch.empty((M, C), dtype=proj.dtype, device=proj.device)
    B = block_table.shape[0]
    code = lib().eredu_short_conv(ptr(proj), proj.stride(0), ptr(w), ptr(bias), ptr(state), ptr(block_table),
                                  block_table.stride(0), ptr(cu_q), q_per_seq, ptr(positions), ptr(slots), ptr(out), C, L,
                                  B, max_q_len, mode, x_off, stream_ptr(proj.device))
    check(code, "eredu_short_conv")
    return out
