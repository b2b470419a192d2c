"""Tensor-parallel execution of the row-parallel projections and of the vocabulary-parallel head.

The reference runs ``matmul -> all_sum`` (eredu/src/backend/mlx/nn/parallel.rs:736-757,824-841) and
``all_gather`` of the logits (:1382-1409) as separate NCCL collectives. Here:

* up to 64 tokens (decode, speculative verify): ONE kernel does the tcgen05 GEMM and the all-reduce — partial
  tiles are pushed to every peer over NVLink as they leave TMEM, as 4-byte bf16x2 words into sentinel-initialised
  slots (a word is valid once it differs from the sentinel: no tag, flag or fence), each rank sums in rank order
  (``eredu_gemm_bf16_comm`` mode 1); the logits use the same kernel in all-gather mode (mode 2);
* more tokens (prefill): the GEMM writes its bf16 partial into symmetric memory and a two-shot peer-memory
  all-reduce (reduce-scatter by P2P loads, all-gather by P2P stores, residual/bias folded in) finishes it.

``NcclTPOps`` is the library baseline with the same interface (torch.distributed collectives).
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import native
from .comm import PeerGroup


class PeerTPOps:
    supports_ssq = True

    def __init__(self, par, device, hidden: int, vocab: int, max_tokens: int = 8192, max_logit_rows: int = 64):
        self.par = par
        self.device = torch.device(device)
        slot = 64 * max(hidden, 1) * 4
        out_bytes = max(max_tokens * hidden * 2, max_logit_rows * vocab * 4)
        x_bytes = max_tokens * hidden * 2
        self.pg = PeerGroup(par.tp_group, self.device, slot, out_bytes, x_bytes)
        self.max_tokens = max_tokens
        self.sm = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.lib = native.lib()

    # ---------------------------------------------------------------- row-parallel linear (+ all-reduce)
    def row_linear(self, x, w, residual=None, bias=None, want_ssq=False):
        M, K = x.shape
        N = w.shape[0]
        st = native.status_word(self.device)
        if M <= 64:
            y = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
            ssq = torch.empty((M, (N + 127) // 128), dtype=torch.float32, device=x.device) if want_ssq else None
            code = self.lib.eredu_gemm_bf16_comm(
                x.data_ptr(), w.data_ptr(), y.data_ptr(), native.ptr(residual), native.ptr(bias), M, N, K,
                x.stride(0), w.stride(0), y.stride(0), residual.stride(0) if residual is not None else 0, w.shape[0],
                0, 1, 0, self.pg.comm, 0, self.sm, st.data_ptr(), None, 0, 0.0, 0, native.ptr(ssq),
                native.stream_ptr(self.device))
            native.check(code, "eredu_gemm_bf16_comm(all-reduce)")
            return (y, ssq) if want_ssq else y
        assert not want_ssq
        assert M <= self.max_tokens, f"{M} tokens exceed the symmetric buffer ({self.max_tokens})"
        partial = self.pg.x_view((M, N), torch.bfloat16)
        ops.linear(x, w, out=partial)
        return self._twoshot(M, N, residual, bias)

    def _twoshot(self, M, N, residual, bias):
        st = native.status_word(self.device)
        y = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
        code = self.lib.eredu_allreduce_twoshot(self.pg.comm, self.pg.x_off, native.ptr(residual), native.ptr(bias),
                                                y.data_ptr(), M, N, residual.stride(0) if residual is not None else 0,
                                                self.sm, st.data_ptr(), native.stream_ptr(self.device))
        native.check(code, "eredu_allreduce_twoshot")
        return y

    def fused_comm(self, tokens: int, hidden: int):
        """The communication context for kernels that fold the group sum into their own epilogue (the expert
        combine), or None when the partials do not fit one staging slot."""
        return self.pg.comm if tokens * hidden * 4 <= self.pg.slot_bytes else None

    def row_qlinear(self, q, x, residual=None, bias=None):
        """Row-parallel projection with quantised weights: decode-sized calls sum over the group in the kernel's epilogue
        (the same one-shot words as the dense path), larger ones run the local kernel and the peer-memory all-reduce."""
        M = x.shape[0]
        if hasattr(q, "row_parallel") and ((M + 1) // 2) * q.out_features * 4 <= self.pg.lam_bytes:
            y = q.row_parallel(x, self.pg.comm, residual=residual, bias=bias)
            if y is not None:
                return y
        return self.all_reduce(q(x), residual=residual, bias=bias)

    def all_reduce(self, partial, residual=None, bias=None):
        """Sum a local bf16 partial over the group (used after quantised row-parallel GEMMs)."""
        M, N = partial.shape
        if M * N * 4 <= self.pg.slot_bytes and partial.stride(1) == 1:
            st = native.status_word(self.device)
            y = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
            code = self.lib.eredu_allreduce_ll(self.pg.comm, partial.data_ptr(), partial.stride(0), native.ptr(residual),
                                               residual.stride(0) if residual is not None else 0, native.ptr(bias),
                                               y.data_ptr(), y.stride(0), M, N, st.data_ptr(), native.stream_ptr(self.device))
            native.check(code, "eredu_allreduce_ll")
            return y
        self.pg.x_view((M, N), torch.bfloat16).copy_(partial)
        return self._twoshot(M, N, residual, bias)

    # ---------------------------------------------------------------- vocabulary-parallel head (+ all-gather)
    def gathered_logits(self, normed, lm_head_local, vocab: int, col_offset: int, row_ssq=None, norm_eps=0.0):
        M, K = normed.shape
        Nl = lm_head_local.shape[0]
        st = native.status_word(self.device)
        out = self.pg.out_view((M, vocab), torch.float32)
        if M <= 64:
            code = self.lib.eredu_gemm_bf16_comm(
                normed.data_ptr(), lm_head_local.data_ptr(), None, None, None, M, Nl, K, normed.stride(0),
                lm_head_local.stride(0), vocab, 0, Nl, 1, 2, col_offset, self.pg.comm, 0, self.sm, st.data_ptr(),
                native.ptr(row_ssq), 0 if row_ssq is None else row_ssq.shape[1], float(norm_eps),
                K if row_ssq is not None else 0, None, native.stream_ptr(self.device))
            native.check(code, "eredu_gemm_bf16_comm(all-gather)")
            return out.clone()
        raise ValueError("logits are computed for at most 64 rows per step")

    def all_gather_logits(self, local, vocab: int):
        raise NotImplementedError("use gathered_logits (fused GEMM + all-gather)")


class NcclTPOps:
    """Library baseline: cuBLAS-free local GEMM is still ours, the collective is NCCL (or gloo on CPU)."""

    def __init__(self, par, device):
        self.par = par
        self.device = torch.device(device)

    def row_linear(self, x, w, residual=None, bias=None, want_ssq=False):
        import torch.distributed as dist

        assert not want_ssq
        y = ops.linear(x, w)
        dist.all_reduce(y, group=self.par.tp_group)
        if bias is not None:
            y = y + bias
        if residual is not None:
            y = y + residual
        return y

    def all_reduce(self, partial, residual=None, bias=None):
        import torch.distributed as dist

        y = partial.clone()
        dist.all_reduce(y, group=self.par.tp_group)
        if bias is not None:
            y = y + bias
        if residual is not None:
            y = y + residual
        return y

    def gathered_logits(self, normed, lm_head_local, vocab: int, col_offset: int, row_ssq=None, norm_eps=0.0):
        import torch.distributed as dist

        local = ops.linear(normed, lm_head_local, out_dtype=torch.float32, row_ssq=row_ssq, norm_eps=norm_eps)
        parts = [torch.empty_like(local) for _ in range(self.par.tp_size)]
        dist.all_gather(parts, local.contiguous(), group=self.par.tp_group)
        return torch.cat(parts, dim=-1)


def attach(model, par, max_tokens: int = 8192, backend: str = "peer", ep_mode: str = "replicated"):
    """Give a tensor-parallel model shard its collective implementation. ``ep_mode``: how sparse blocks spread over the
    expert ranks - "replicated" (every rank routes all tokens, partial outputs are summed: the reference's production
    path) or "a2a" (token-sharded all-to-all dispatch and combine, see :mod:`eredu_b200.parallel.ep_a2a`)."""
    if par.tp_size == 1:
        return model
    if backend == "peer" and model.device.type == "cuda":
        model.tp_ops = PeerTPOps(par, model.device, model.cfg.hidden_size, model.cfg.vocab_size, max_tokens)
    else:
        model.tp_ops = NcclTPOps(par, model.device)
    if par.ep_size > 1 and par.ep_group is par.tp_group:
        # experts are spread over the same ranks as the attention heads: one collective context serves both
        from ..models.moe import attach_ep

        attach_ep(model, model.tp_ops)
        if ep_mode == "a2a":
            from .ep_a2a import attach_ep_a2a

            attach_ep_a2a(model, par, "peer" if (backend == "peer" and model.device.type == "cuda") else "collective", max_tokens)
    return model
