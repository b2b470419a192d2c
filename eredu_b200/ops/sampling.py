"""Sampling operators: the fused sampler / speculative-verify kernels and their PyTorch oracle.

The chain and its defaults follow the reference (eredu/src/backend/mlx/runtime/generation/sampler.rs:607-619,
780-923): penalties -> top-k -> top-p (sorted, at temperature 1) -> min-p -> 1/T -> argmax | categorical.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .native import check, lib, ptr, stream_ptr

ROW_DTYPE = np.dtype([
    ("temperature", "<f4"), ("top_p", "<f4"), ("min_p", "<f4"), ("repeat_penalty", "<f4"),
    ("frequency_penalty", "<f4"), ("presence_penalty", "<f4"), ("top_k", "<i4"), ("repeat_last_n", "<i4"),
    ("hist_len", "<i4"), ("position", "<i4"), ("seed_lo", "<u4"), ("seed_hi", "<u4"), ("stream_id", "<u4"),
    ("pad", "<i4"),
])
assert ROW_DTYPE.itemsize == 56


@dataclass
class SamplingParams:
    """Per-request sampling settings. Defaults are the reference's no-checkpoint-config defaults."""
    temperature: float = 0.0
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.05
    repeat_penalty: float = 1.0
    repeat_last_n: int = 64
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


def pack_rows(params: list[SamplingParams], positions: list[int], hist_lens: list[int] | None = None,
              stream_ids: list[int] | None = None) -> np.ndarray:
    rows = np.zeros(len(params), dtype=ROW_DTYPE)
    for i, sp in enumerate(params):
        rows[i] = (sp.temperature, sp.top_p, sp.min_p, sp.repeat_penalty, sp.frequency_penalty, sp.presence_penalty,
                   sp.top_k, sp.repeat_last_n, 0 if hist_lens is None else hist_lens[i], positions[i],
                   sp.seed & 0xFFFFFFFF, (sp.seed >> 32) & 0xFFFFFFFF, 0 if stream_ids is None else stream_ids[i], 0)
    return rows


def rows_to_tensor(rows: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(rows.view(np.uint8).reshape(len(rows), ROW_DTYPE.itemsize).copy()).to(device)


# ------------------------------------------------------------------------------------------ Philox (host twin)
def philox_uniform(seed: int, stream: int, position: int, purpose: int) -> float:
    """Host twin of the kernel's position-addressed uniform (Philox4x32-10)."""
    M32 = 0xFFFFFFFF
    c = [position & M32, stream & M32, purpose & M32, 0x45524544]
    k0, k1 = seed & M32, (seed >> 32) & M32
    for _ in range(10):
        p0 = 0xD2511F53 * c[0]
        p1 = 0xCD9E8D57 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & M32, p1 & M32, ((p0 >> 32) ^ c[3] ^ k1) & M32, p0 & M32]
        k0 = (k0 + 0x9E3779B9) & M32
        k1 = (k1 + 0xBB67AE85) & M32
    return float(np.float32(c[0] >> 8) * np.float32(1.0 / 16777216.0))


# ------------------------------------------------------------------------------------------ oracle
def process_logits_ref(logits: torch.Tensor, sp: SamplingParams, history=None, allow=None) -> torch.Tensor:
    """Final distribution of one row (dense fp32 probabilities)."""
    x = logits.detach().float().cpu().clone()
    V = x.numel()
    if allow is not None:
        x[~allow] = float("-inf")
    if history is not None and len(history) and (
            sp.repeat_penalty != 1.0 or sp.frequency_penalty != 0.0 or sp.presence_penalty != 0.0):
        window = history if sp.repeat_last_n < 0 else history[max(0, len(history) - sp.repeat_last_n):]
        counts: dict[int, int] = {}
        for t in window:
            counts[int(t)] = counts.get(int(t), 0) + 1
        for t, c in counts.items():
            if 0 <= t < V:
                v = x[t]
                if sp.repeat_penalty != 1.0:
                    v = v / sp.repeat_penalty if v > 0 else v * sp.repeat_penalty
                x[t] = v - (sp.frequency_penalty * c + sp.presence_penalty)
    if sp.temperature == 0.0:
        p = torch.zeros(V)
        p[int(torch.argmax(x))] = 1.0
        return p
    if 0 < sp.top_k < V:
        thr = torch.topk(x, sp.top_k).values.min()
        x[x < thr] = float("-inf")
    if sp.top_p < 1.0:
        order = torch.argsort(-x, stable=True)
        sx = x[order]
        p = torch.softmax(sx, -1)
        before = torch.cumsum(p, -1) - p
        sx[before > max(sp.top_p, 0.0)] = float("-inf")
        x = torch.full_like(x, float("-inf"))
        x[order] = sx
    if sp.min_p > 0.0:
        p = torch.softmax(x, -1)
        x[p < p.max() * sp.min_p] = float("-inf")
    return torch.softmax(x / sp.temperature, -1)


def verify_ref(p_t: torch.Tensor, p_d: torch.Tensor, drafted: list[int], seed: int, stream: int, position: int):
    """(accepted, next_token) by the reference's accept / residual / bonus rule with the kernel's uniforms."""
    n = len(drafted)
    for i, tok in enumerate(drafted):
        t, d = float(p_t[i, tok]), float(p_d[i, tok])
        u = philox_uniform(seed, stream, position + i, 1)
        ok = (u * d < t) if d > 0 else (t > 0)
        if ok:
            continue
        resid = (p_t[i] - p_d[i]).clamp(min=0)
        tot = float(resid.sum())
        if tot <= 0:
            return i, int(torch.argmax(p_t[i]))
        u2 = philox_uniform(seed, stream, position + i, 2)
        cum = torch.cumsum(resid.double(), 0)
        idx = int(torch.searchsorted(cum, torch.tensor(u2 * tot, dtype=torch.float64), right=True))
        return i, min(idx, resid.numel() - 1)
    u3 = philox_uniform(seed, stream, position + n, 0)
    cum = torch.cumsum(p_t[n].double(), 0)
    idx = int(torch.searchsorted(cum, torch.tensor(u3 * float(cum[-1]), dtype=torch.float64), right=True))
    return n, min(idx, p_t.shape[1] - 1)


def sample_ref(logits: torch.Tensor, sp: SamplingParams, position: int, history=None, allow=None, stream: int = 0):
    """Oracle token for one row, using the kernel's candidate order (logit descending, index ascending)."""
    p = process_logits_ref(logits, sp, history, allow)
    if sp.temperature == 0.0:
        return int(torch.argmax(p)), p
    u = philox_uniform(sp.seed, stream, position, 0)
    V = p.numel()
    dense = not (0 < sp.top_k < V) and not (sp.top_p < 1.0)
    if dense:
        order = torch.arange(V)
    else:
        order = torch.argsort(-logits.detach().float().cpu(), stable=True)
    w = p[order].double()
    cum = torch.cumsum(w, 0)
    idx = int(torch.searchsorted(cum, torch.tensor(u * float(cum[-1]), dtype=torch.float64), right=True))
    idx = min(idx, V - 1)
    while w[idx] == 0 and idx > 0:
        idx -= 1
    return int(order[idx]), p


# ------------------------------------------------------------------------------------------ kernels
def _philox_uniform_t(seed_lo, seed_hi, stream, position, purpose: int) -> torch.Tensor:
    """Tensor twin of :func:`philox_uniform` (int64 arithmetic on the device, no host sync)."""
    M32 = 0xFFFFFFFF
    c0, c1 = position.long() & M32, stream.long() & M32
    c2 = torch.full_like(c0, purpose)
    c3 = torch.full_like(c0, 0x45524544)
    k0, k1 = seed_lo.long() & M32, seed_hi.long() & M32

    def mulhilo(a: int, b):
        # 32x32 -> (hi, lo) without overflowing int64: split b into 16-bit halves
        b_lo, b_hi = b & 0xFFFF, b >> 16
        p0 = a * b_lo                      # < 2^48
        p1 = a * b_hi                      # < 2^48
        lo = (p0 + ((p1 & 0xFFFF) << 16))
        hi = (p1 >> 16) + (lo >> 32)
        return hi & M32, lo & M32

    for _ in range(10):
        hi0, lo0 = mulhilo(0xD2511F53, c0)
        hi1, lo1 = mulhilo(0xCD9E8D57, c2)
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & M32, lo1, (hi0 ^ c3 ^ k1) & M32, lo0
        k0 = (k0 + 0x9E3779B9) & M32
        k1 = (k1 + 0xBB67AE85) & M32
    return (c0 >> 8).to(torch.float32) * (1.0 / 16777216.0)


def _rows_fields(rows: torch.Tensor):
    r32 = rows.view(torch.int32)
    f32 = rows.view(torch.float32)
    return {"temperature": f32[:, 0], "top_p": f32[:, 1], "min_p": f32[:, 2], "repeat_penalty": f32[:, 3],
            "frequency_penalty": f32[:, 4], "presence_penalty": f32[:, 5], "top_k": r32[:, 6],
            "repeat_last_n": r32[:, 7], "hist_len": r32[:, 8], "position": r32[:, 9], "seed_lo": r32[:, 10],
            "seed_hi": r32[:, 11], "stream_id": r32[:, 12]}


def sample_tensor_ops(logits, rows, history=None, allow=None, probs=None, out=None):
    """The sampler chain written with tensor operations only (sort based, no host synchronisation, CUDA-graph
    safe). Same semantics and the same position-addressed uniforms as the fused kernel; used for rows with
    temperature > 0 on the GPU."""
    R, V = logits.shape
    f = _rows_fields(rows)
    x = logits
    if allow is not None:
        words = allow.view(-1, allow.shape[-1]).long() & 0xFFFFFFFF
        bits = ((words[:, :, None] >> torch.arange(32, device=x.device)) & 1).reshape(words.shape[0], -1)[:, :V]
        x = x.masked_fill(bits.expand(R, V) == 0, float("-inf"))
    if history is not None:
        H = history.shape[1]
        idx = torch.arange(H, device=x.device)[None, :]
        hl, rl = f["hist_len"][:, None], f["repeat_last_n"][:, None]
        start = torch.where(rl < 0, torch.zeros_like(hl), (hl - rl).clamp(min=0))
        inwin = (idx >= start) & (idx < hl)
        toks = history.long().clamp(0, V - 1)
        counts = torch.zeros(R, V, device=x.device).scatter_add_(1, toks, inwin.float())
        seen = counts > 0
        rp = f["repeat_penalty"][:, None]
        pen = torch.where(x > 0, x / rp, x * rp)
        x = torch.where(seen, pen, x)
        x = x - torch.where(seen, f["frequency_penalty"][:, None] * counts + f["presence_penalty"][:, None],
                            torch.zeros_like(x))
    greedy = f["temperature"] == 0
    sx, order = torch.sort(x, dim=-1, descending=True, stable=True)
    rank = torch.arange(V, device=x.device)[None, :]
    k = f["top_k"][:, None]
    use_k = (k > 0) & (k < V)
    kth = sx.gather(1, (k.long() - 1).clamp(0, V - 1))
    keep = torch.where(use_k, sx >= kth, torch.ones_like(sx, dtype=torch.bool))
    xs = sx.masked_fill(~keep, float("-inf"))
    p1 = torch.softmax(xs, -1)
    before = torch.cumsum(p1, -1) - p1
    tp = f["top_p"][:, None]
    keep = keep & ((tp >= 1.0) | (before <= tp.clamp(min=0)))
    keep = keep & ((sx - sx[:, :1]) >= torch.log(f["min_p"].clamp(min=1e-38))[:, None]) | (rank == 0)
    temp = torch.where(greedy, torch.ones_like(f["temperature"]), f["temperature"])[:, None]
    w = torch.softmax(sx.masked_fill(~keep, float("-inf")) / temp, -1)
    onehot = (rank == 0).float()
    w = torch.where(greedy[:, None], onehot, w)
    u = _philox_uniform_t(f["seed_lo"], f["seed_hi"], f["stream_id"], f["position"], 0)
    cum = torch.cumsum(w, -1)
    hit = (cum > (u * cum[:, -1])[:, None]) & (w > 0)
    first = torch.where(hit.any(-1), hit.float().argmax(-1), (w > 0).float().cumsum(-1).argmax(-1))
    tok = order.gather(1, first[:, None]).squeeze(1).to(torch.int32)
    if out is None:
        out = tok
    else:
        out.copy_(tok)
    if probs is not None:
        probs.zero_().scatter_(1, order, w)
    return out


def sample(logits: torch.Tensor, rows: torch.Tensor, history: torch.Tensor | None = None,
           allow: torch.Tensor | None = None, probs: torch.Tensor | None = None,
           out: torch.Tensor | None = None, all_greedy: bool | None = None) -> torch.Tensor:
    """logits: [R, V] fp32 CUDA (modified in place by penalties); rows: packed SamplerRow bytes [R, 56].

    Greedy rows run in the fused kernel. The fused kernel's stochastic path is kept off the GPU: two constructions of
    it (radix select + sorting network; counting search + rank ordering) raised a misaligned-address fault on B200 on
    their first stochastic row although every access in the compiled code is a 4-byte scalar on an aligned base, and
    the cause has not been found. Batches that contain a row with temperature > 0 use :func:`sample_tensor_ops`, which
    has the same semantics and the same position-addressed random numbers."""
    assert logits.is_cuda and logits.dtype == torch.float32 and logits.is_contiguous()
    R, V = logits.shape
    if all_greedy is None:
        all_greedy = bool((_rows_fields(rows)["temperature"] == 0).all().item())
    if not all_greedy:
        return sample_tensor_ops(logits, rows, history, allow, probs, out)
    if out is None:
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
    allow_stride = 0
    if allow is not None:
        assert allow.dtype == torch.int32 and allow.shape[-1] == (V + 31) // 32
        allow_stride = allow.stride(0) if allow.dim() == 2 and allow.shape[0] > 1 else 0
    code = lib().eredu_sample(ptr(logits), ptr(allow), allow_stride, ptr(rows), ptr(history),
                              history.stride(0) if history is not None else 0, ptr(out), ptr(probs), R, V,
                              stream_ptr(logits.device))
    check(code, "eredu_sample")
    return out


def spec_verify(p_t: torch.Tensor, p_d: torch.Tensor, drafted: torch.Tensor, rows: torch.Tensor,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """p_t: [B, k+1, V], p_d: [B, k, V] dense fp32; drafted: [B, k] int32 -> [B, 2] (accepted, next token)."""
    B, k1, V = p_t.shape
    if out is None:
        out = torch.empty((B, 2), dtype=torch.int32, device=p_t.device)
    code = lib().eredu_spec_verify(ptr(p_t), ptr(p_d), ptr(drafted), ptr(rows), ptr(out), B, k1 - 1, V,
                                   stream_ptr(p_t.device))
    check(code, "eredu_spec_verify")
    return out


def pack_allow_mask(allowed: torch.Tensor) -> torch.Tensor:
    """bool [.., V] -> int32 bit words [.., ceil(V/32)] (bit i of word w = token 32*w + i)."""
    V = allowed.shape[-1]
    pad = (-V) % 32
    a = torch.nn.functional.pad(allowed.to(torch.int64), (0, pad)).reshape(*allowed.shape[:-1], -1, 32)
    weights = (1 << torch.arange(32, dtype=torch.int64, device=allowed.device))
    words = (a * weights).sum(-1)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)
    return words.to(torch.int32)
