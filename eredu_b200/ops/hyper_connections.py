"""Hyper-connections: several residual streams per token, mixed by a small doubly-stochastic matrix.

The numerical definition of eredu/src/backend/mlx/nn/hyper_connections.rs (DeepSeek-V4's residual scheme). A block keeps
``n`` residual streams ``R[t, n, H]``. Before a sub-layer, ``collapse`` derives three things from the RMS-normalised,
flattened streams through one small projection: ``pre[t, n]`` (sigmoid + eps; the sub-layer's input is the pre-weighted
sum of the streams), ``post[t, n]`` (2·sigmoid; how much of the sub-layer's output each stream receives) and
``comb[t, n, n]`` (softmax rows, then Sinkhorn-normalised to a doubly-stochastic matrix that mixes the old streams).
After the sub-layer, ``expand`` forms ``R'[t, i] = post[t, i] · y[t] + sum_j comb[t, j, i] · R[t, j]``. ``HyperHead``
collapses the streams once more before the final norm. All mixing arithmetic runs in fp32.

Tensors here are token-major ``[T, n, H]`` (the engine's flat token layout); the reference's ``[batch, tokens, n, H]`` is the
same thing with one more leading axis, and every function accepts extra leading axes.
"""
from __future__ import annotations

import torch


def weightless_rms_norm(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps)


def split_sinkhorn(mixes: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, streams: int, iterations: int, eps: float):
    """``mixes [..., (2 + n) n]`` -> (pre [..., n], post [..., n], comb [..., n, n]); ``scale [3]``, ``base [(2 + n) n]``."""
    n = int(streams)
    if n <= 0:
        raise ValueError("hyper-connection stream count must be positive")
    if iterations <= 0:
        raise ValueError("hyper-connection Sinkhorn iteration count must be positive")
    if not (eps > 0 and eps == eps and eps != float("inf")):
        raise ValueError("hyper-connection epsilon must be finite and positive")
    width = (2 + n) * n
    if mixes.dim() == 0 or mixes.shape[-1] != width:
        raise ValueError(f"hyper-connection mixes need final dimension {width}, got {tuple(mixes.shape)}")
    if tuple(scale.shape) != (3,) or tuple(base.shape) != (width,):
        raise ValueError(f"hyper-connection scale / base shapes must be [3] and [{width}]")
    lead = mixes.shape[:-1]
    m = mixes.float().reshape(-1, width)
    scale, base = scale.float(), base.float()
    pre = torch.sigmoid(m[:, :n] * scale[0] + base[:n]) + eps
    post = torch.sigmoid(m[:, n:2 * n] * scale[1] + base[n:2 * n]) * 2.0
    comb = torch.softmax((m[:, 2 * n:] * scale[2] + base[2 * n:]).reshape(-1, n, n), dim=-1) + eps
    comb = comb / (comb.sum(-2, keepdim=True) + eps)
    for _ in range(1, iterations):
        comb = comb / (comb.sum(-1, keepdim=True) + eps)
        comb = comb / (comb.sum(-2, keepdim=True) + eps)
    return pre.reshape(*lead, n), post.reshape(*lead, n), comb.reshape(*lead, n, n)


class HyperConnection:
    """``function [(2 + n) n, n H]``, ``base [(2 + n) n]`` and ``scale [3]`` are fp32 parameters."""

    def __init__(self, function: torch.Tensor, base: torch.Tensor, scale: torch.Tensor, streams: int, hidden_size: int,
                 iterations: int = 20, eps: float = 1e-6):
        width = (2 + streams) * streams
        if streams <= 0 or hidden_size <= 0:
            raise ValueError("hyper-connection streams and hidden size must be positive")
        if tuple(function.shape) != (width, streams * hidden_size):
            raise ValueError(f"hyper-connection function must be [{width}, {streams * hidden_size}], got {tuple(function.shape)}")
        self.function, self.base, self.scale = function.float(), base.float(), scale.float()
        self.streams, self.hidden_size, self.iterations, self.eps = streams, hidden_size, iterations, eps

    def collapse(self, residual: torch.Tensor, norm_eps: float):
        """``residual [..., n, H]`` -> (sub-layer input ``[..., H]`` in the residual's dtype, post ``[..., n]``, comb ``[..., n, n]``)."""
        if residual.dim() < 2 or residual.shape[-2] != self.streams or residual.shape[-1] != self.hidden_size:
            raise ValueError(f"hyper-connection needs [..., {self.streams}, {self.hidden_size}], got {tuple(residual.shape)}")
        r = residual.float()
        flat = r.reshape(*r.shape[:-2], self.streams * self.hidden_size)
        mixes = weightless_rms_norm(flat, norm_eps) @ self.function.t()
        pre, post, comb = split_sinkhorn(mixes, self.scale, self.base, self.streams, self.iterations, self.eps)
        collapsed = torch.einsum("...h,...hd->...d", pre, r).to(residual.dtype)
        return collapsed, post, comb


def expand(sublayer: torch.Tensor, residual: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    """``R'[.., i, :] = post[.., i] · y + sum_j comb[.., j, i] · R[.., j, :]`` in fp32, returned in the sub-layer's dtype."""
    injected = post[..., None] * sublayer.float()[..., None, :]
    mixed = torch.einsum("...ji,...jd->...id", comb, residual.float())
    return (injected + mixed).to(sublayer.dtype)


class HyperHead:
    """Final learned collapse of the streams: ``function [n, n H]``, ``base [n]``, ``scale [1]`` (fp32)."""

    def __init__(self, function: torch.Tensor, base: torch.Tensor, scale: torch.Tensor, streams: int, hidden_size: int,
                 norm_eps: float, eps: float = 1e-6):
        if tuple(function.shape) != (streams, streams * hidden_size) or tuple(base.shape) != (streams,) or scale.numel() != 1:
            raise ValueError("hyper-head parameter shapes must be [n, n H], [n] and [1]")
        self.function, self.base, self.scale = function.float(), base.float(), scale.float().reshape(())
        self.streams, self.hidden_size, self.norm_eps, self.eps = streams, hidden_size, norm_eps, eps

    def __call__(self, residual: torch.Tensor) -> torch.Tensor:
        r = residual.float()
        flat = r.reshape(*r.shape[:-2], self.streams * self.hidden_size)
        logits = weightless_rms_norm(flat, self.norm_eps) @ self.function.t()
        pre = torch.sigmoid(logits * self.scale + self.base) + self.eps
        return torch.einsum("...h,...hd->...d", pre, r).to(residual.dtype)
