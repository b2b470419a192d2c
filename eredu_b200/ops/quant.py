"""Quantised linear layers: affine group quantisation (MLX-LM checkpoints, load-time quantisation) and GGUF block
quants, executed by the tcgen05 dequant-GEMM (``csrc/kernels/qgemm_tcgen05.cu``).

Format contract (eredu/src/backend/mlx/runtime/checkpoint/quantization.rs:1-8,137-232): ``name.weight`` uint32
``[out, in*bits/32]`` little-endian bit stream, ``name.scales`` / ``name.biases`` ``[out, in/group]``,
``w ~ scale * q + bias``. GGUF types map to affine (bits, group) as in eredu-gguf/src/convert.rs:124-152.

In device memory the codes live in a *kernel layout* (made once at load, the checkpoint bytes are untouched):
4-bit codes as bytes ``[N, K/2]`` with the eight nibbles of each u32 interleaved (n0,n2,n4,n6,n1,n3,n5,n7); every
other width (2/3/5/6/8 bits) in an 8-bit container ``[N, K]``; scales and biases bf16, transposed to ``[K/group, N]``.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import native
from .core import _sm_count, linear
from .native import F, I, P, check, lib, ptr, status_word, stream_ptr

native.register("eredu_qgemm", I, [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, P])
native.register("eredu_dequant_affine", I, [P, P, P, P, I, I, I, I, P])
native.register("eredu_qgemv4", I, [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, I, I, I, P, P, P])
native.register("eredu_qgemm_fp8", I, [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, P])
native.register("eredu_dequant_fp8", I, [P, P, P, I, I, P])
native.register("eredu_fp8_quant_act", I, [P, I, P, P, I, I, I, P])
native.register("eredu_gemm_fp8_tc", I, [P, P, I, P, P, P, P, P, I, I, I, I, I, I, P, P])

_NIBBLE_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)  # kernel position p holds logical nibble _NIBBLE_ORDER[p]


def unpack_bitstream(packed: torch.Tensor, bits: int) -> torch.Tensor:
    """uint32/int32 words [N, K*bits/32] (little-endian bit stream) -> codes uint8 [N, K]."""
    N, W = packed.shape
    words = packed.to(torch.int64) & 0xFFFFFFFF
    K = W * 32 // bits
    idx = torch.arange(K, device=packed.device, dtype=torch.int64) * bits
    wi, sh = idx // 32, idx % 32
    lo = words[:, wi] >> sh
    nxt = words[:, (wi + 1).clamp(max=W - 1)]
    hi = torch.where((sh + bits) > 32, nxt << (32 - sh), torch.zeros_like(nxt))
    return ((lo | hi) & ((1 << bits) - 1)).to(torch.uint8)


def tile_kernel4(by: torch.Tensor) -> torch.Tensor:
    """Row-major packed bytes [N, K/2] -> kernel tiles [ceil(N/16), K/64, 512]: a tile holds 16 rows x 64 columns
    (16 x 32 bytes, row-major inside), rows are padded with zero codes to whole tiles."""
    N, B = by.shape
    pad = (-N) % 16
    if pad:
        by = torch.cat((by, by.new_zeros((pad, B))), 0)
    return by.view((N + pad) // 16, 16, B // 32, 32).permute(0, 2, 1, 3).contiguous().view((N + pad) // 16, B // 32, 512)


def untile_kernel4(wq: torch.Tensor, N: int) -> torch.Tensor:
    """Kernel tiles -> row-major packed bytes [N, K/2]."""
    T, KB, _ = wq.shape
    return wq.view(T, KB, 16, 32).permute(0, 2, 1, 3).reshape(T * 16, KB * 32)[:N]


def codes_to_kernel4(codes: torch.Tensor) -> torch.Tensor:
    """4-bit codes uint8 [N, K] -> kernel layout: nibbles interleaved inside each u32, 16 x 64 tiles (see tile_kernel4)."""
    N, K = codes.shape
    c = codes.view(N, K // 8, 8).to(torch.int32)
    order = torch.tensor(_NIBBLE_ORDER, device=codes.device)
    c = c[:, :, order]  # position p <- logical nibble order[p]
    by = c[:, :, 0::2] | (c[:, :, 1::2] << 4)
    return tile_kernel4(by.to(torch.uint8).reshape(N, K // 2))


def affine_quantize_tensor(w: torch.Tensor, bits: int, group: int):
    """Load-time affine quantisation on the weight's device (vectorised form of the host reference quantiser:
    edge-anchored scale, bias at the larger-magnitude extreme). Returns (codes uint8 [N,K], scales, biases bf16
    [N, K/group])."""
    N, K = w.shape
    n_bins = float((1 << bits) - 1)
    out_codes = torch.empty((N, K), dtype=torch.uint8, device=w.device)
    scales = torch.empty((N, K // group), dtype=torch.bfloat16, device=w.device)
    biases = torch.empty_like(scales)
    step = max(1, (1 << 24) // K)
    for r0 in range(0, N, step):
        x = w[r0:r0 + step].float().view(-1, K // group, group)
        lo, hi = x.amin(-1), x.amax(-1)
        mask = lo.abs() > hi.abs()
        scale = ((hi - lo) / n_bins).clamp(min=1e-7)
        scale = torch.where(mask, scale, -scale)
        edge = torch.where(mask, lo, hi)
        q0 = torch.round(edge / scale)
        scale = torch.where(q0 != 0, edge / torch.where(q0 != 0, q0, torch.ones_like(q0)), scale)
        bias = torch.where(q0 == 0, torch.zeros_like(edge), edge)
        scale = scale.bfloat16()
        bias = bias.bfloat16()
        q = torch.round((x - bias.float()[..., None]) / scale.float()[..., None]).clamp(0, n_bins)
        out_codes[r0:r0 + step] = q.to(torch.uint8).view(-1, K)
        scales[r0:r0 + step] = scale
        biases[r0:r0 + step] = bias
    return out_codes, scales, biases


class QuantLinear:
    """y = x @ dequant(Wq).T (+bias) (+residual)."""

    def __init__(self, codes: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, bits: int, group: int, device):
        """codes: uint8 [N, K] (one code per byte); scales / biases: [N, K/group] (any float dtype)."""
        N, K = codes.shape
        self.out_features, self.in_features = N, K
        self.bits = bits
        self.group = group
        self.kbits = 4 if bits == 4 else 8
        dev = torch.device(device)
        codes = codes.to(dev)
        self.wq = codes_to_kernel4(codes) if self.kbits == 4 else codes.contiguous()
        self.scales_t = scales.to(dev, torch.bfloat16).t().contiguous()
        self.biases_t = biases.to(dev, torch.bfloat16).t().contiguous()
        self.device = dev

    # ------------------------------------------------------------------ constructors
    @classmethod
    def from_dense(cls, w: torch.Tensor, bits: int = 4, group: int = 64):
        codes, s, b = affine_quantize_tensor(w, bits, group)
        return cls(codes, s, b, bits, group, w.device)

    @classmethod
    def from_packed(cls, packed: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, bits: int, group: int, device):
        return cls(unpack_bitstream(packed.to(device), bits), scales, biases, bits, group, device)

    @staticmethod
    def concat_rows(parts: list["QuantLinear"]) -> "QuantLinear":
        """Fuse row-wise (q|k|v, gate|up). Parts with different widths / groups meet in the 8-bit container at
        the smallest group size (scales repeated), which keeps every code and scale exact."""
        first = parts[0]
        same = all(p.kbits == first.kbits and p.group == first.group for p in parts)
        out = object.__new__(QuantLinear)
        out.in_features = first.in_features
        out.out_features = sum(p.out_features for p in parts)
        out.device = first.device
        if same:
            out.kbits, out.bits, out.group = first.kbits, first.bits, first.group
            if first.kbits == 4 and any(p.out_features % 16 for p in parts[:-1]):
                out.wq = tile_kernel4(torch.cat([untile_kernel4(p.wq, p.out_features) for p in parts], 0))
            else:
                out.wq = torch.cat([p.wq for p in parts], 0)      # whole row tiles (4-bit) or rows (8-bit) stack as they are
            out.scales_t = torch.cat([p.scales_t for p in parts], 1).contiguous()
            out.biases_t = torch.cat([p.biases_t for p in parts], 1).contiguous()
            return out
        g = min(p.group for p in parts)
        out.kbits, out.bits, out.group = 8, 8, g
        out.wq = torch.cat([p.codes() for p in parts], 0)
        out.scales_t = torch.cat([p.scales_t.repeat_interleave(p.group // g, 0) for p in parts], 1).contiguous()
        out.biases_t = torch.cat([p.biases_t.repeat_interleave(p.group // g, 0) for p in parts], 1).contiguous()
        return out

    def slice_rows(self, r0: int, r1: int) -> "QuantLinear":
        out = object.__new__(QuantLinear)
        out.__dict__.update(self.__dict__)
        out.__dict__.pop("_dq_t", None)
        out.out_features = r1 - r0
        if self.kbits == 4:
            if r0 % 16 == 0 and (r1 % 16 == 0 or r1 == self.out_features):
                out.wq = self.wq[r0 // 16:(r1 + 15) // 16].contiguous()
            else:
                out.wq = tile_kernel4(untile_kernel4(self.wq, self.out_features)[r0:r1])
        else:
            out.wq = self.wq[r0:r1].contiguous()
        out.scales_t = self.scales_t[:, r0:r1].contiguous()
        out.biases_t = self.biases_t[:, r0:r1].contiguous()
        return out

    def slice_cols(self, k0: int, k1: int) -> "QuantLinear":
        """Input-dimension slice (row-parallel shard); boundaries must fall on 64-element and group boundaries."""
        assert k0 % 64 == 0 and k1 % 64 == 0 and k0 % self.group == 0 and k1 % self.group == 0
        out = object.__new__(QuantLinear)
        out.__dict__.update(self.__dict__)
        out.__dict__.pop("_dq_t", None)
        out.in_features = k1 - k0
        out.wq = self.wq[:, k0 // 64:k1 // 64].contiguous() if self.kbits == 4 else self.wq[:, k0:k1].contiguous()
        out.scales_t = self.scales_t[k0 // self.group:k1 // self.group].contiguous()
        out.biases_t = self.biases_t[k0 // self.group:k1 // self.group].contiguous()
        return out

    # ------------------------------------------------------------------ views
    def tensors(self):
        return [self.wq, self.scales_t, self.biases_t]

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors())

    def codes(self) -> torch.Tensor:
        """uint8 [N, K], one code per byte (logical order)."""
        if self.kbits == 8:
            return self.wq
        N = self.out_features
        by = untile_kernel4(self.wq, N).reshape(N, -1, 4).to(torch.int32)  # 4 bytes = 8 kernel positions
        pos = torch.stack((by & 0xF, by >> 4), -1).reshape(N, -1, 8)  # kernel positions 0..7
        inv = torch.empty(8, dtype=torch.long)
        for p, logical in enumerate(_NIBBLE_ORDER):
            inv[logical] = p
        return pos[:, :, inv.to(pos.device)].reshape(N, self.in_features).to(torch.uint8)

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        c = self.codes().float().view(self.out_features, -1, self.group)
        s = self.scales_t.t().float()[..., None]
        b = self.biases_t.t().float()[..., None]
        return (c * s + b).view(self.out_features, self.in_features).to(dtype)

    # ------------------------------------------------------------------ forward
    DENSE_FALLBACK_TOKENS = 256
    GEMV_MAX_TOKENS = 8           # up to here the register-resident decode kernel runs (csrc/kernels/qgemv_mma.cu)

    def decode_table(self) -> Optional[torch.Tensor]:
        """int32 [ceil(N/16), K/group, 16] for the decode kernel: the bf16 scale in the low half, the bf16 bias in the high
        half of each word, tiled like the codes (the words of a row tile are contiguous along K). None where that kernel does not apply (8-bit container, group that is no power of two >= 16)."""
        if self.kbits != 4 or self.group < 16 or self.group > 128 or self.group & (self.group - 1):
            return None
        t = self.__dict__.get("_dq_t")
        if t is None or t.shape[1] != self.scales_t.shape[0] or t.device != self.scales_t.device:
            lo = self.scales_t.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
            hi = self.biases_t.contiguous().view(torch.int16).to(torch.int32) << 16
            w = lo | hi                                              # [K/group, N]
            G, N = w.shape
            pad = (-N) % 16
            if pad:
                w = torch.cat((w, w.new_zeros((G, pad))), 1)      # rows of the padding take scale 0, bias 0
            t = w.view(G, (N + pad) // 16, 16).permute(1, 0, 2).contiguous()
            self._dq_t = t
        return t

    def _gemv(self, x, bias, residual, out, out_dtype, gated: bool, limit: float = 0.0, comm=None):
        M, K = x.shape
        dev = x.device
        n_out = self.out_features // 2 if gated else self.out_features
        if out is None:
            out = torch.empty((M, n_out), dtype=out_dtype, device=dev)
        dq = self.decode_table()
        code = lib().eredu_qgemv4(ptr(x), ptr(self.wq), ptr(dq), ptr(out), ptr(residual), ptr(bias), M, self.out_features, K,
                                  x.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0, self.group,
                                  1 if out_dtype == torch.float32 else 0, 1 if gated else 0, float(limit), 0, 0, 0,
                                  _sm_count(dev), comm, ptr(status_word(dev)), stream_ptr(dev))
        check(code, "eredu_qgemv4")
        return out

    def _gemv_ok(self, x) -> bool:
        return (x.is_cuda and x.shape[0] <= self.GEMV_MAX_TOKENS and x.dtype == torch.bfloat16 and x.stride(1) == 1
                and x.stride(0) % 8 == 0 and self.in_features % 64 == 0 and self.decode_table() is not None)

    def row_parallel(self, x, comm, residual=None, bias=None):
        """This rank's K shard of a row-parallel projection with the sum over the group inside the kernel (``comm``: the
        peer-memory context of the group). None when the decode kernel does not take the call."""
        if not self._gemv_ok(x):
            return None
        return self._gemv(x, bias, residual, None, torch.bfloat16, False, comm=comm)

    def gated(self, x, bias=None, limit: float = 0.0):
        """silu(x Wgate^T) * (x Wup^T) for a weight that stacks gate rows over up rows: one kernel for decode-sized
        batches, the projection followed by the activation kernel otherwise."""
        inter = self.out_features // 2
        if self._gemv_ok(x) and self.out_features % 32 == 0:
            return self._gemv(x, bias, None, None, torch.bfloat16, True, limit or 0.0)
        from .core import silu_mul

        return silu_mul(self(x, bias=bias), inter, limit or 0.0)

    def __call__(self, x, bias=None, residual=None, out=None, out_dtype=None):
        if not x.is_cuda:
            y = torch.nn.functional.linear(x.float(), self.dequantize(), None if bias is None else bias.float())
            if residual is not None:
                y = y + residual.float()
            return y.to(out_dtype or x.dtype)
        M, K = x.shape
        N = self.out_features
        assert K == self.in_features and x.dtype == torch.bfloat16 and x.stride(1) == 1
        out_dtype = out_dtype or torch.bfloat16
        dev = x.device
        if self._gemv_ok(x) and (out is None or out.stride(1) == 1):
            return self._gemv(x, bias, residual, out, out_dtype, False)
        if M > self.DENSE_FALLBACK_TOKENS:
            w = torch.empty((N, K), dtype=torch.bfloat16, device=dev)
            check(lib().eredu_dequant_affine(ptr(self.wq), ptr(self.scales_t), ptr(self.biases_t), ptr(w), N, K,
                                             self.kbits, self.group, stream_ptr(dev)), "eredu_dequant_affine")
            return linear(x, w, bias=bias, residual=residual, out_dtype=out_dtype, out=out, dynamic_weight=True)
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=dev)
        code = lib().eredu_qgemm(ptr(x), ptr(self.wq), ptr(self.scales_t), ptr(self.biases_t), ptr(out), ptr(residual),
                                 ptr(bias), M, N, K, x.stride(0), out.stride(0),
                                 residual.stride(0) if residual is not None else 0, self.kbits, self.group,
                                 1 if out_dtype == torch.float32 else 0, 0, _sm_count(dev), ptr(status_word(dev)),
                                 stream_ptr(dev))
        check(code, "eredu_qgemm")
        return out


class Fp8Linear:
    """y = x @ (e4m3(Wq) * block_scale).T (+bias) (+residual): block-scaled FP8 weights (128 x 128 blocks) kept in
    E4M3 on the device and decoded inside the tcgen05 pipeline; activations stay bf16. The block scales are expanded
    along the output rows into an fp32 table [K/128, N], so row slices and row concatenations need no alignment."""

    DENSE_FALLBACK_TOKENS = 256      # above this many tokens the weight-streaming kernel gives way to a GEMM-shaped one
    TENSOR_CORE_FP8 = True           # ... which is the FP8 tensor-core kernel when the scale table is block-uniform
    TENSOR_CORE_FP8_MAX_TOKENS = 1024   # ... up to here (measured: 34 us against 45 at 512 tokens, 94 against 73 at 2048);
    #                                     beyond, decoding the weight to bf16 once and running the bf16 GEMM is faster
    bits, kbits, group = 8, 8, 128

    def __init__(self, w8: torch.Tensor, block_scale: torch.Tensor, device, row_scales_t: Optional[torch.Tensor] = None):
        """w8: E4M3 bytes (uint8 or float8_e4m3fn) [N, K]; block_scale fp32 [ceil(N/128), ceil(K/128)]
        (or ``row_scales_t`` [K/128, N] directly)."""
        N, K = w8.shape
        if K % 128 != 0:
            raise ValueError("block-FP8 weights need an input width that is a multiple of 128")
        dev = torch.device(device)
        self.out_features, self.in_features = N, K
        self.device = dev
        self.wq = (w8.view(torch.uint8) if w8.dtype != torch.uint8 else w8).to(dev).contiguous()
        if row_scales_t is None:
            row_scales_t = block_scale.to(torch.float32).repeat_interleave(128, 0)[:N].t()
        self.scales_t = row_scales_t.to(dev, torch.float32).contiguous()
        assert self.scales_t.shape == (K // 128, N)
        # The FP8 tensor-core kernel folds one weight scale per 128 x 128 tile: usable when every aligned run of 128 rows
        # of the (possibly sliced or concatenated) table carries one value per K block.
        self.block_scales = None
        if N % 128 == 0:
            tiles = self.scales_t.view(K // 128, N // 128, 128)
            if bool((tiles == tiles[..., :1]).all()):
                self.block_scales = tiles[..., 0].contiguous()

    @classmethod
    def from_dense(cls, w: torch.Tensor):
        """Quantise a dense weight: per 128 x 128 block, scale = amax / 448, codes = round-to-nearest E4M3."""
        N, K = w.shape
        wf = w.float()
        nb, kb = (N + 127) // 128, K // 128
        pad = torch.zeros((nb * 128, K), dtype=torch.float32, device=w.device)
        pad[:N] = wf
        blocks = pad.view(nb, 128, kb, 128)
        scale = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12) / 448.0
        codes = (blocks / scale[:, None, :, None]).view(nb * 128, K)[:N].to(torch.float8_e4m3fn)
        return cls(codes, scale, w.device)

    @staticmethod
    def concat_rows(parts: list["Fp8Linear"]) -> "Fp8Linear":
        return Fp8Linear(torch.cat([p.wq for p in parts], 0), None, parts[0].device,
                         row_scales_t=torch.cat([p.scales_t for p in parts], 1))

    def slice_rows(self, r0: int, r1: int) -> "Fp8Linear":
        return Fp8Linear(self.wq[r0:r1], None, self.device, row_scales_t=self.scales_t[:, r0:r1])

    def slice_cols(self, k0: int, k1: int) -> "Fp8Linear":
        assert k0 % 128 == 0 and k1 % 128 == 0
        return Fp8Linear(self.wq[:, k0:k1], None, self.device, row_scales_t=self.scales_t[k0 // 128:k1 // 128])

    def tensors(self):
        return [self.wq, self.scales_t]

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors())

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        s = self.scales_t.t().repeat_interleave(128, 1)
        return (self.wq.view(torch.float8_e4m3fn).to(torch.float32) * s).to(dtype)

    def __call__(self, x, bias=None, residual=None, out=None, out_dtype=None):
        if not x.is_cuda:
            y = torch.nn.functional.linear(x.float(), self.dequantize(), None if bias is None else bias.float())
            if residual is not None:
                y = y + residual.float()
            return y.to(out_dtype or x.dtype)
        M, K = x.shape
        N = self.out_features
        assert K == self.in_features and x.dtype == torch.bfloat16 and x.stride(1) == 1
        out_dtype = out_dtype or torch.bfloat16
        dev = x.device
        if (self.DENSE_FALLBACK_TOKENS < M <= self.TENSOR_CORE_FP8_MAX_TOKENS and self.TENSOR_CORE_FP8
                and self.block_scales is not None):
            return self.tensor_core(x, bias=bias, residual=residual, out=out, out_dtype=out_dtype)
        if M > self.DENSE_FALLBACK_TOKENS:
            w = torch.empty((N, K), dtype=torch.bfloat16, device=dev)
            check(lib().eredu_dequant_fp8(ptr(self.wq), ptr(self.scales_t), ptr(w), N, K, stream_ptr(dev)), "eredu_dequant_fp8")
            return linear(x, w, bias=bias, residual=residual, out_dtype=out_dtype, out=out, dynamic_weight=True)
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=dev)
        code = lib().eredu_qgemm_fp8(ptr(x), ptr(self.wq), ptr(self.scales_t), ptr(out), ptr(residual), ptr(bias), M, N, K,
                                     x.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0,
                                     1 if out_dtype == torch.float32 else 0, 0, _sm_count(dev), ptr(status_word(dev)),
                                     stream_ptr(dev))
        check(code, "eredu_qgemm_fp8")
        return out


def _fp8_tensor_core(self, x, bias=None, residual=None, out=None, out_dtype=None):
    """The GEMM-shaped path of :class:`Fp8Linear`: the activations are quantised to E4M3 with one scale per row per 128
    columns (``eredu_fp8_quant_act``) and multiplied on the FP8 tensor cores, the scale product folded in per K block
    (``eredu_gemm_fp8_tc``). Reference: eredu/src/backend/mlx/nn/fp8.rs:291-323 (activation quantisation), :664-742."""
    M, K = x.shape
    N = self.out_features
    dev = x.device
    out_dtype = out_dtype or torch.bfloat16
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=dev)
    xq = torch.empty((M, K), dtype=torch.uint8, device=dev)
    ld = (M + 127) // 128 * 128                  # the GEMM fetches a tile's 128 scales with one aligned bulk copy
    sx = torch.empty((K // 128, ld), dtype=torch.float32, device=dev)
    check(lib().eredu_fp8_quant_act(ptr(x), x.stride(0), ptr(xq), ptr(sx), ld, M, K, stream_ptr(dev)), "eredu_fp8_quant_act")
    code = lib().eredu_gemm_fp8_tc(ptr(xq), ptr(sx), ld, ptr(self.wq), ptr(self.block_scales), ptr(out), ptr(residual), ptr(bias),
                                   M, N, K, out.stride(0), residual.stride(0) if residual is not None else 0,
                                   1 if out_dtype == torch.float32 else 0, ptr(status_word(dev)), stream_ptr(dev))
    check(code, "eredu_gemm_fp8_tc")
    return out


Fp8Linear.tensor_core = _fp8_tensor_core


def make_quantizer(src, opt):
    """Hook for ``build_from_tensors``: replaces the dense projections of a layer by :class:`QuantLinear`.

    * ``opt.quantization`` set: load-time affine quantisation of the (already tensor-parallel sliced) dense weights;
    * GGUF source with block-quantised tensors and ``opt.native_gguf``: the file's own codes and scales are used
      (Q4_0 / Q4_1 / Q4_K as 4-bit group 32, Q8_0 as 8-bit group 32, Q2_K..Q6_K in the 8-bit container).
    Returns None when neither applies."""
    qopt = getattr(opt, "quantization", None)
    gguf_native = bool(getattr(opt, "native_gguf", False)) and hasattr(src, "to_affine") and any(
        src.quant_info(f"model.layers.0.{n}.weight") is not None
        for n in ("self_attn.q_proj", "mlp.down_proj", "mlp.gate_proj"))
    fp8_native = hasattr(src, "fp8_scale_name") and any(
        src.fp8_scale_name(f"model.layers.0.{n}.weight") is not None
        for n in ("self_attn.q_proj", "mlp.down_proj", "mlp.gate_proj"))
    if qopt is None and not gguf_native and not fp8_native:
        return None

    def from_source(model, name, rows=None, cols=None):
        if fp8_native and src.fp8_scale_name(name) is not None:
            w8, sc = src.to_fp8(name)
            N = w8.shape[0]
            rs = sc.repeat_interleave(128, 0)[:N].t()
            r0, r1 = rows if rows is not None else (0, N)
            c0, c1 = cols if cols is not None else (0, w8.shape[1])
            if c0 % 128 or c1 % 128:
                raise RuntimeError("column slice does not fall on FP8 block boundaries")
            return Fp8Linear(w8[r0:r1, c0:c1], None, model.device, row_scales_t=rs[c0 // 128:c1 // 128, r0:r1])
        packed, scales, biases, bits, group = src.to_affine(name)
        q = QuantLinear.from_packed(packed, scales.float(), biases.float(), bits, group, model.device)
        if rows is not None:
            q = q.slice_rows(*rows)
        if cols is not None:
            q = q.slice_cols(*cols)
        return q

    def hook(model, li, lw):
        par = model.par
        tp, r = par.tp_size, par.tp_rank
        cfg = model.cfg
        if qopt is not None:
            if qopt.mode == "fp8":
                for role, attr in (("qkv", "wqkv"), ("o", "wo"), ("gate_up", "w_gate_up"), ("down", "w_down")):
                    w = getattr(lw, attr)
                    if w is None or w.shape[1] % 128 != 0:
                        continue
                    lw.qlin[role] = Fp8Linear.from_dense(w)
                    setattr(lw, attr, None)
                return
            if qopt.mode != "affine":
                raise NotImplementedError("load-time quantisation mode " + qopt.mode)
            bits, group = qopt.bits, qopt.group_size
            for role, attr in (("qkv", "wqkv"), ("o", "wo"), ("gate_up", "w_gate_up"), ("down", "w_down"),
                               ("conv_in", "conv_in"), ("conv_out", "conv_out")):
                w = getattr(lw, attr)
                if w is None or w.shape[1] % group != 0 or w.shape[1] % 64 != 0:
                    continue  # ineligible: stays dense (quantization.rs:24-38)
                lw.qlin[role] = QuantLinear.from_dense(w, bits, group)
                setattr(lw, attr, None)
            return
        if lw.conv_w is not None:
            return  # short-convolution layers keep their dense projections
        p = f"model.layers.{li}."
        D = cfg.head_dim
        nq, nkv, rep = model.n_q_local, model.n_kv_local, model.kv_rep
        q0 = r * nq
        kv0 = (r // rep) * nkv if rep > 1 else r * nkv
        try:
            parts = [from_source(model, p + "self_attn.q_proj.weight", rows=(q0 * D, (q0 + nq) * D)),
                     from_source(model, p + "self_attn.k_proj.weight", rows=(kv0 * D, (kv0 + nkv) * D)),
                     from_source(model, p + "self_attn.v_proj.weight", rows=(kv0 * D, (kv0 + nkv) * D))]
            lw.qlin["qkv"] = type(parts[0]).concat_rows(parts)
            lw.wqkv = None
            lw.qlin["o"] = from_source(model, p + "self_attn.o_proj.weight", cols=(q0 * D, (q0 + nq) * D))
            lw.wo = None
            if lw.moe is None:
                I_ = cfg.intermediate_size
                lo, hi = r * (I_ // tp), (r + 1) * (I_ // tp)
                gu = [from_source(model, p + "mlp.gate_proj.weight", rows=(lo, hi)),
                      from_source(model, p + "mlp.up_proj.weight", rows=(lo, hi))]
                lw.qlin["gate_up"] = type(gu[0]).concat_rows(gu)
                lw.w_gate_up = None
                lw.qlin["down"] = from_source(model, p + "mlp.down_proj.weight", cols=(lo, hi))
                lw.w_down = None
        except (RuntimeError, AssertionError):
            pass  # a tensor without an affine form (dense / IQ): the dense weights already loaded stay in use

    return hook
