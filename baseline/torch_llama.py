"""Stand-in baseline: the same Llama decode step written with stock PyTorch operators only - cuBLAS GEMMs
(``F.linear``), ``F.scaled_dot_product_attention``, ``torch`` element-wise ops for RMSNorm / RoPE / SwiGLU, NCCL
collectives through ``torch.distributed`` (all-reduce after the row-parallel projections, all-gather of the logits,
the reference's algorithm: eredu/src/backend/mlx/nn/parallel.rs:736-757,1382-1409) - captured in a CUDA graph like
the product's decode step. None of this repository's kernels or engine code is imported here.

The KV cache is a contiguous [B, kv_heads, T, D] tensor (the simplest layout for the library attention; a paged
gather would only slow this arm down). Weights are random with the product benchmark's shapes and sharding.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


class TorchLlamaTP:
    def __init__(self, cfg, device, rank: int = 0, world: int = 1, group=None, max_len: int = 4096, batch: int = 32, seed: int = 0):
        self.cfg, self.dev, self.rank, self.world, self.group = cfg, device, rank, world, group
        H, D = cfg.hidden_size, cfg.head_dim
        self.nq = cfg.num_attention_heads // world
        self.nkv = max(1, cfg.num_key_value_heads // world)
        inter = cfg.intermediate_size // world
        g = torch.Generator(device=device).manual_seed(seed + rank)

        def w(*shape):
            return (torch.randn(*shape, device=device, generator=g, dtype=torch.bfloat16) * 0.02)

        self.embed = w(cfg.vocab_size, H)
        self.layers = []
        for _ in range(cfg.num_hidden_layers):
            self.layers.append(dict(n1=torch.ones(H, device=device, dtype=torch.bfloat16), n2=torch.ones(H, device=device, dtype=torch.bfloat16),
                                    wqkv=w((self.nq + 2 * self.nkv) * D, H), wo=w(H, self.nq * D),
                                    wgu=w(2 * inter, H), wd=w(H, inter)))
        self.norm = torch.ones(H, device=device, dtype=torch.bfloat16)
        self.head = w(cfg.vocab_size // world, H)
        self.inter = inter
        self.k = torch.zeros(cfg.num_hidden_layers, batch, self.nkv, max_len, D, device=device, dtype=torch.bfloat16)
        self.v = torch.zeros_like(self.k)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, device=device, dtype=torch.float32) / D))
        t = torch.arange(max_len, device=device, dtype=torch.float32)
        ang = torch.outer(t, inv)
        self.cos, self.sin = ang.cos(), ang.sin()
        self.max_len = max_len

    def _rms(self, x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.rms_norm_eps)).to(x.dtype) * w

    def _rope(self, x, pos):
        # x: [B, heads, 1, D]; pos: [B]
        D = x.shape[-1]
        c = self.cos[pos][:, None, None, :]
        s = self.sin[pos][:, None, None, :]
        a, b = x[..., : D // 2].float(), x[..., D // 2:].float()
        return torch.cat((a * c - b * s, b * c + a * s), -1).to(x.dtype)

    def _all_reduce(self, y):
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(y, group=self.group)
        return y

    @torch.no_grad()
    def prefill_fill(self, length: int):
        """Fill the cache with random keys / values up to ``length`` (the baseline times decode only)."""
        g = torch.Generator(device=self.dev).manual_seed(1)
        self.k[:, :, :, :length].copy_(torch.randn(self.k[:, :, :, :length].shape, device=self.dev, generator=g, dtype=torch.bfloat16) * 0.3)
        self.v[:, :, :, :length].copy_(torch.randn(self.v[:, :, :, :length].shape, device=self.dev, generator=g, dtype=torch.bfloat16) * 0.3)

    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor, pos: torch.Tensor, kv_len: int) -> torch.Tensor:
        """tokens [B] int64, pos [B] int64 (all equal to kv_len - 1 here); attends to cache[:kv_len]. Returns argmax ids."""
        cfg = self.cfg
        B, D = tokens.shape[0], cfg.head_dim
        h = self.embed[tokens]
        bidx = torch.arange(B, device=self.dev)
        for li, lw in enumerate(self.layers):
            x = self._rms(h, lw["n1"])
            qkv = F.linear(x, lw["wqkv"])
            q, k, v = qkv.split((self.nq * D, self.nkv * D, self.nkv * D), -1)
            q = self._rope(q.view(B, self.nq, 1, D), pos)
            k = self._rope(k.view(B, self.nkv, 1, D), pos)
            self.k[li, bidx, :, pos] = k[:, :, 0]
            self.v[li, bidx, :, pos] = v.view(B, self.nkv, D)
            att = F.scaled_dot_product_attention(q, self.k[li, :, :, :kv_len], self.v[li, :, :, :kv_len], enable_gqa=True)
            h = h + self._all_reduce(F.linear(att.reshape(B, self.nq * D), lw["wo"]))
            x = self._rms(h, lw["n2"])
            gu = F.linear(x, lw["wgu"])
            h = h + self._all_reduce(F.linear(F.silu(gu[:, : self.inter]) * gu[:, self.inter:], lw["wd"]))
        logits = F.linear(self._rms(h, self.norm), self.head).float()
        if self.world > 1:
            import torch.distributed as dist

            parts = [torch.empty_like(logits) for _ in range(self.world)]
            dist.all_gather(parts, logits, group=self.group)
            logits = torch.cat(parts, -1)
        return logits.argmax(-1)
