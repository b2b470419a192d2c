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
def sample(logits: torch.Tensor, rows: torch.Tensor, history: torch.Tensor | None = None,
           allow: torch.Tensor | None = None, probs: torch.Tensor | None = None,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """logits: [R, V] fp32 CUDA (modified in place by penalties); rows: packed SamplerRow bytes [R, 56]."""
    assert logits.is_cuda and logits.dtype == torch.float32 and logits.is_contiguous()
    R, V = logits.shape
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
