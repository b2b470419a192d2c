"""Decoder-only transformer of the Llama family: Llama / Mistral / Qwen2 / Qwen3 dense and, through a
pluggable MoE block, Qwen3-MoE / Mixtral-style sparse models.

Block semantics follow eredu-architectures/src/llama.rs:289-345,418-431,472-495 (pre-norm,
``h = x + o_proj(attn(rope(q), rope(k), v))``, ``y = h + down(silu(gate(n(h))) * up(n(h)))``, scale
1/sqrt(head_dim), RoPE before the cache append, logits of the last prompt position only) and
architectures/qwen/dense.rs:739-790 (per-head q/k RMSNorm before RoPE, qkv bias for Qwen2).

The execution plan is B200-specific: q/k/v and gate/up weights are fused at load so that a layer is
``rmsnorm -> qkv GEMM -> norm+rope+KV-append -> paged attention -> o_proj GEMM(+residual) -> rmsnorm ->
gate_up GEMM(+SwiGLU) -> down GEMM(+residual)`` - eight launches, residual adds and the activation living
in GEMM epilogues. Under tensor parallelism the two row-parallel GEMMs run through the fused
GEMM + all-reduce path of :mod:`eredu_b200.parallel.tp`.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from .. import ops
from ..utils import nvtx
from .config import ModelConfig
from .rope import rope_tables


# EREDU_FUSED_ROPE=0 keeps the separate RoPE + KV-append launch in front of decode attention (A/B measurements).
FUSED_DECODE_ROPE = os.environ.get("EREDU_FUSED_ROPE", "1") != "0"


@dataclass
class ForwardBatch:
    """Device-side description of one model step (prefill chunk(s) or decode tokens)."""
    token_ids: torch.Tensor            # [M] int32
    positions: torch.Tensor            # [M] int32
    slots: torch.Tensor                # [M] int64: page * 16 + offset into the KV pool, -1 = skip
    block_table: torch.Tensor          # [B, max_pages] int32
    seq_lens: torch.Tensor             # [B] int32, kv length after this step
    is_prefill: bool
    cu_q: Optional[torch.Tensor] = None        # prefill: [B+1] int32
    max_q_len: int = 1
    q_per_seq: int = 1                 # decode / verify: query tokens per sequence
    logit_rows: Optional[torch.Tensor] = None  # rows of the hidden state that need logits ([R] int64), None = all
    splits: int = 1                    # decode split-KV factor
    scratch: Optional[tuple] = None    # decode split-KV scratch
    hidden_in: Optional[torch.Tensor] = None   # pipeline stages > 0: incoming activations instead of token ids
    # multimodal prompts (vision-language models): rows whose embedding is replaced by tower features, the DeepStack
    # features added to those rows after the first decoder layers, and rotary positions that differ from the cache index
    embed_rows: Optional[torch.Tensor] = None       # [n_vis] int64 rows of this batch
    embed_values: Optional[torch.Tensor] = None     # [n_vis, H]
    deepstack: Optional[list] = None                # list of [n_vis, H]: added after layer 0, 1, ...
    rope_positions: Optional[torch.Tensor] = None   # [M] or [3, M]; None: ``positions``
    per_layer_inputs: Optional[torch.Tensor] = None  # Gemma 4: [M, layers, P], filled by the model
    bidir_groups: Optional[list] = None             # per sequence: int tensor [kv_len] of bidirectional-attention group ids
    # embedded prediction heads: keep the hidden state that enters the final norm (all rows) in ``hidden_out``
    capture_hidden: bool = False
    hidden_out: Optional[torch.Tensor] = None
    # block drafters that condition on intermediate activations: the outputs of these layers (all rows) land in ``layer_hidden``
    capture_layers: Optional[tuple] = None
    layer_hidden: Optional[dict] = None


@dataclass
class LayerWeights:
    attn_norm: torch.Tensor
    wqkv: Optional[torch.Tensor]
    wo: Optional[torch.Tensor]
    ffn_norm: Optional[torch.Tensor]
    w_gate_up: Optional[torch.Tensor] = None
    w_down: Optional[torch.Tensor] = None
    bqkv: Optional[torch.Tensor] = None
    bo: Optional[torch.Tensor] = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    sinks: Optional[torch.Tensor] = None
    moe: object = None       # MoE block (callable) for sparse layers
    fold_attn: bool = False  # attn_norm weights are folded into wqkv (RMSNorm fused into the GEMM)
    fold_ffn: bool = False   # ffn_norm weights are folded into w_gate_up
    qlin: dict = field(default_factory=dict)  # quantised linears by role: "qkv", "o", "gate_up", "down"
    # LFM2 "conv" layers: gated short convolution instead of attention (wqkv / wo are None); attn_norm is the
    # operator norm and fold_attn then refers to conv_in
    # Nemotron-H: the layer is one mixer ("mamba" | "attention_only" | "mlp_only" | "moe_only"); attn_norm is its norm
    block_kind: str = ""
    extra: Optional[dict] = None   # tensors of blocks that keep their own layout (Gemma 4)
    m_in: Optional[torch.Tensor] = None        # Mamba-2 input projection [z | x B C | dt]
    m_in_b: Optional[torch.Tensor] = None
    m_conv_w: Optional[torch.Tensor] = None
    m_conv_b: Optional[torch.Tensor] = None
    m_A_log: Optional[torch.Tensor] = None
    m_D: Optional[torch.Tensor] = None
    m_dt_bias: Optional[torch.Tensor] = None
    m_norm_w: Optional[torch.Tensor] = None
    m_out: Optional[torch.Tensor] = None
    m_out_b: Optional[torch.Tensor] = None
    # Kimi Delta Attention: kda_in = [q | k | v | f_a | b | g_a] rows; fold_attn then refers to kda_in
    kda_in: Optional[torch.Tensor] = None
    kda_conv_w: Optional[torch.Tensor] = None
    kda_f_b: Optional[torch.Tensor] = None
    kda_g_b: Optional[torch.Tensor] = None
    kda_A_log: Optional[torch.Tensor] = None
    kda_dt_bias: Optional[torch.Tensor] = None
    kda_o_norm: Optional[torch.Tensor] = None
    # DeepSeek latent attention: mla_in = [q_a (or q) | kv_a] rows; fold_attn then refers to mla_in
    mla_in: Optional[torch.Tensor] = None
    mla_q_norm: Optional[torch.Tensor] = None
    mla_q_b: Optional[torch.Tensor] = None
    mla_kv_norm: Optional[torch.Tensor] = None
    mla_w_uk: Optional[torch.Tensor] = None    # [heads_local, nope, kv_lora]
    mla_w_uv: Optional[torch.Tensor] = None    # [heads_local, v, kv_lora]
    attn_gate: bool = False   # wqkv carries a fourth block: the per-channel sigmoid gate of the attention output
    # Qwen3-Next "linear_attention" layers (gated delta network); fold_attn then refers to la_in
    la_in: Optional[torch.Tensor] = None       # [2 key + value + value + Hv + Hv, H]: qkv | z | b | a
    la_conv_w: Optional[torch.Tensor] = None   # [2 key + value, K] fp32
    la_dt_bias: Optional[torch.Tensor] = None
    la_A_log: Optional[torch.Tensor] = None
    la_norm_w: Optional[torch.Tensor] = None   # [dv] gated RMSNorm weight (not zero-centred)
    la_out: Optional[torch.Tensor] = None      # [H, value]
    conv_in: Optional[torch.Tensor] = None    # [3C, H]: B | C | X projections
    conv_w: Optional[torch.Tensor] = None     # [C, L] fp32 depthwise kernel
    conv_out: Optional[torch.Tensor] = None   # [H, C]
    conv_in_b: Optional[torch.Tensor] = None
    conv_b: Optional[torch.Tensor] = None
    conv_out_b: Optional[torch.Tensor] = None


class CausalLM:
    """Weights + forward of one model replica / shard. Not an nn.Module: inference only, explicit tensors."""

    def __init__(self, cfg: ModelConfig, device, dtype, parallel=None):
        from ..parallel.context import ParallelContext

        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype
        self.par = parallel or ParallelContext.single()
        tp = self.par.tp_size
        self.n_q_local, self.n_kv_local, self.kv_rep = self.par.attention_partition(cfg.num_attention_heads,
                                                                                    cfg.num_key_value_heads)
        if cfg.is_mla:
            self.n_kv_local = 1     # one latent row per token, replicated on every tensor rank
        self.inter_local = cfg.intermediate_size // tp if cfg.intermediate_size % tp == 0 else None
        self.layers: list[LayerWeights] = []
        self.first_layer, self.last_layer = self.par.layer_range(cfg.num_hidden_layers)
        self.embed: Optional[torch.Tensor] = None
        self.final_norm: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None  # [V_local, H]
        self.vocab_start = 0
        inv, factor = rope_tables(cfg)
        if not cfg.use_rope:
            inv = torch.zeros_like(inv)      # angle 0 everywhere: the RoPE step of the KV-append kernel is the identity
        self.inv_freq = inv.to(self.device)
        self.attn_factor = factor
        self.scale = 1.0 / math.sqrt(cfg.head_dim)
        self.tp_ops = None  # set by parallel.tp when tp_size > 1
        self.head_folded = False
        self.residency = None  # set by runtime.weight_residency when the layers live in host memory
        self.observer = None   # runtime.inspection.ActivationObserver for observed (eager) passes

    # ------------------------------------------------------------------------------------------ layer
    def _linear(self, lw: LayerWeights, role: str, x, w, bias=None, residual=None):
        q = lw.qlin.get(role)
        if q is not None:
            return q(x, bias=bias, residual=residual)
        return ops.linear(x, w, bias=bias, residual=residual)

    def _row_linear(self, lw: LayerWeights, role: str, x, w, residual, bias=None):
        """Row-parallel projection: local GEMM, sum over the TP group, residual added once."""
        if self.par.tp_size == 1:
            return self._linear(lw, role, x, w, bias=bias, residual=residual)
        q = lw.qlin.get(role)
        if q is not None:
            if hasattr(self.tp_ops, "row_qlinear"):
                return self.tp_ops.row_qlinear(q, x, residual=residual, bias=bias)
            partial = q(x)
            return self.tp_ops.all_reduce(partial, residual=residual, bias=bias)
        return self.tp_ops.row_linear(x, w, residual=residual, bias=bias)

    FUSED_NORM_MAX_TOKENS = 64

    def _normed_linear(self, h, ssq, folded: bool, norm_w, w, lw, role, bias=None, gated_inter=0):
        """RMSNorm followed by a column-parallel GEMM. With folded norm weights the scale is applied in the GEMM
        epilogue from the producer's partial sums of squares (decode) or by a weight-free normalisation kernel
        (prefill); otherwise the plain rmsnorm kernel runs first."""
        cfg = self.cfg
        q = lw.qlin.get(role)
        if folded and q is None:
            if ssq is not None and h.shape[0] <= self.FUSED_NORM_MAX_TOKENS:
                if gated_inter:
                    return ops.gated_linear(h, w, gated_inter, bias=bias, row_ssq=ssq, norm_eps=cfg.rms_norm_eps)
                return ops.linear(h, w, bias=bias, row_ssq=ssq, norm_eps=cfg.rms_norm_eps)
            normed, _ = ops.rmsnorm(h, self._ones(h.shape[1]), cfg.rms_norm_eps)
        else:
            normed, _ = ops.rmsnorm(h, norm_w, cfg.rms_norm_eps, weight_offset=cfg.norm_weight_offset)
        if q is not None:
            if gated_inter and hasattr(q, "gated"):
                return q.gated(normed, bias=bias, limit=cfg.swiglu_limit)
            y = q(normed, bias=bias)
            return ops.silu_mul(y, q.out_features // 2, cfg.swiglu_limit) if gated_inter else y
        if gated_inter:
            return ops.gated_linear(normed, w, gated_inter, bias=bias)
        return ops.linear(normed, w, bias=bias)

    def _ones(self, n):
        t = getattr(self, "_ones_cache", None)
        if t is None or t.shape[0] != n:
            t = torch.ones(n, dtype=torch.float32, device=self.device)
            self._ones_cache = t
        return t

    def _row_linear_ssq(self, lw, role, x, w, residual, bias, want_ssq):
        """Row-parallel projection that can also return the partial sums of squares of its output rows."""
        if (not want_ssq or lw.qlin.get(role) is not None or x.shape[0] > self.FUSED_NORM_MAX_TOKENS
                or (self.par.tp_size > 1 and not getattr(self.tp_ops, 'supports_ssq', False))):
            return self._row_linear(lw, role, x, w, residual=residual, bias=bias), None
        if self.par.tp_size == 1:
            return ops.linear(x, w, bias=bias, residual=residual, want_ssq=True)
        return self.tp_ops.row_linear(x, w, residual=residual, bias=bias, want_ssq=True)

    def layer_forward(self, li: int, lw: LayerWeights, h, batch: ForwardBatch, kv, ssq=None, next_folded=False):
        """One decoder block. ``ssq``: partial sums of squares of h's rows (or None); returns (h, ssq')."""
        cfg = self.cfg
        if lw.block_kind == "gemma4":
            from .gemma4 import block_forward as gemma4_block

            return gemma4_block(self, li, lw, h, batch, kv), None
        if lw.block_kind == "muse_glimmer":
            from .muse_glimmer import block_forward as muse_block

            return muse_block(self, li, lw, h, batch, kv), None
        if lw.block_kind:
            from .nemotron_h import block_forward

            return block_forward(self, li, lw, h, batch, kv), None
        if lw.conv_w is not None:
            proj = self._normed_linear(h, ssq, lw.fold_attn, lw.attn_norm, lw.conv_in, lw, "conv_in", bias=lw.conv_in_b)
            y = ops.short_conv(proj, lw.conv_w, lw.conv_b, kv.conv_layer(li), batch.block_table,
                               batch.cu_q if batch.is_prefill else None, batch.q_per_seq, batch.positions, batch.slots,
                               batch.max_q_len)
            h, ssq = self._row_linear_ssq(lw, "conv_out", y, lw.conv_out, h, lw.conv_out_b, lw.fold_ffn)
            return self._ffn(lw, h, ssq, next_folded)
        if lw.kda_in is not None:
            from .kimi_linear import kda_forward

            h, ssq = kda_forward(self, li, lw, h, ssq, batch, kv)
            return self._ffn(lw, h, ssq, next_folded)
        if lw.mla_in is not None:
            from .deepseek import mla_forward

            h, ssq = mla_forward(self, li, lw, h, ssq, batch, kv)
            return self._ffn(lw, h, ssq, next_folded)
        if lw.la_in is not None:
            from .qwen_next import linear_attention_forward

            h, ssq = linear_attention_forward(self, li, lw, h, ssq, batch, kv)
            return self._ffn(lw, h, ssq, next_folded)
        qkv = self._normed_linear(h, ssq, lw.fold_attn, lw.attn_norm, lw.wqkv, lw, "qkv", bias=lw.bqkv)
        gate = None
        if lw.attn_gate:
            width = (self.n_q_local + 2 * self.n_kv_local) * cfg.head_dim
            gate, qkv = qkv[:, width:], qkv[:, :width]
        k_cache, v_cache = kv.layer(li)
        rope_pos = batch.positions if batch.rope_positions is None else batch.rope_positions
        window = cfg.layer_window(li)
        if (not batch.is_prefill and rope_pos.dim() == 1 and qkv.is_cuda and cfg.head_dim in ops.KERNEL_HEAD_DIMS
                and FUSED_DECODE_ROPE):
            # decode / verify steps: q/k norm, RoPE and the KV append happen inside the attention kernel
            attn = ops.attention_decode_rope(qkv, k_cache, v_cache, batch.block_table, batch.seq_lens, batch.q_per_seq,
                                             self.scale, rope_pos, batch.slots, self.inv_freq, self.n_q_local,
                                             self.n_kv_local, cfg.head_dim, rot=cfg.rotary_dim,
                                             interleaved=cfg.rope_traditional, attn_factor=self.attn_factor,
                                             q_norm_w=lw.q_norm, k_norm_w=lw.k_norm, norm_eps=cfg.rms_norm_eps,
                                             norm_w_off=cfg.norm_weight_offset, splits=batch.splits, window=window,
                                             sinks=lw.sinks, scratch=batch.scratch)
            return self._attn_out(lw, attn, gate, h, next_folded)
        q = ops.rope_kv(qkv, rope_pos, batch.slots, self.inv_freq, k_cache, v_cache, self.n_q_local,
                        self.n_kv_local, cfg.head_dim, rot=cfg.rotary_dim, interleaved=cfg.rope_traditional,
                        attn_factor=self.attn_factor, q_norm_w=lw.q_norm, k_norm_w=lw.k_norm, norm_eps=cfg.rms_norm_eps,
                        norm_w_off=cfg.norm_weight_offset, mrope_section=(cfg.rope_scaling or {}).get("mrope_section"))
        if batch.is_prefill:
            attn = ops.attention_prefill(q, k_cache, v_cache, batch.block_table, batch.seq_lens, batch.cu_q,
                                         batch.max_q_len, self.scale, window=window, sinks=lw.sinks)
        else:
            attn = ops.attention_decode(q, k_cache, v_cache, batch.block_table, batch.seq_lens, batch.q_per_seq,
                                        self.scale, splits=batch.splits, window=window, sinks=lw.sinks,
                                        scratch=batch.scratch)
        return self._attn_out(lw, attn, gate, h, next_folded)

    def _attn_out(self, lw: LayerWeights, attn, gate, h, next_folded):
        """Output projection of an attention block (optional sigmoid gate first), then the feed-forward half."""
        attn = attn.view(attn.shape[0], -1)
        if gate is not None:
            attn = (attn.float() * torch.sigmoid(gate.float())).to(attn.dtype)
        h, ssq = self._row_linear_ssq(lw, "o", attn, lw.wo, h, lw.bo, lw.fold_ffn)
        return self._ffn(lw, h, ssq, next_folded)

    def _ffn(self, lw: LayerWeights, h, ssq, next_folded):
        """Second half of a block: norm -> dense SwiGLU or sparse experts -> residual."""
        cfg = self.cfg
        if lw.moe is not None:
            normed, _ = ops.rmsnorm(h, lw.ffn_norm, cfg.rms_norm_eps, weight_offset=cfg.norm_weight_offset)
            if self.observer is not None:
                return lw.moe.observed_call(normed, h, self.observer), None
            return lw.moe(normed, residual=h), None
        inter = (lw.qlin["gate_up"].out_features if "gate_up" in lw.qlin else lw.w_gate_up.shape[0]) // 2
        act = self._normed_linear(h, ssq, lw.fold_ffn, lw.ffn_norm, lw.w_gate_up, lw, "gate_up", gated_inter=inter)
        return self._row_linear_ssq(lw, "down", act, lw.w_down, h, None, next_folded)

    # ------------------------------------------------------------------------------------------ model
    def forward_hidden(self, batch: ForwardBatch, kv):
        """Runs this shard's layers. Returns (h, ssq) - ssq is None unless the next consumer folds its norm."""
        fused = bool(self.layers) and self.layers[0].fold_attn and batch.token_ids.shape[0] <= self.FUSED_NORM_MAX_TOKENS
        ssq = None
        if self.par.owns_embedding() and batch.hidden_in is None:
            if fused:
                h, ssq = ops.embedding(batch.token_ids, self.embed, 0, self.cfg.embedding_scale, want_ssq=True)
            else:
                h = ops.embedding(batch.token_ids, self.embed, 0, self.cfg.embedding_scale)
        else:
            h = batch.hidden_in
        if getattr(self, "mg", None) is not None and self.par.owns_embedding() and batch.hidden_in is None:
            from .muse_glimmer import _wrms

            # Muse-Glimmer normalises the token embeddings; tower rows arrive normalised and take their places after it
            h, ssq = _wrms(h, self.cfg.rms_norm_eps).to(h.dtype), None
        if batch.embed_rows is not None and self.par.owns_embedding():
            h = h.index_copy(0, batch.embed_rows, batch.embed_values.to(h.dtype))
            ssq = None                      # the embedding kernel's row sums no longer describe these rows
        if getattr(self, "g4", None) is not None:
            from .gemma4 import per_layer_inputs

            # the per-layer token table sees the ids as fed (padding at soft-token rows), the projected part sees the
            # activations after soft tokens took their rows
            batch.per_layer_inputs = per_layer_inputs(self, batch.token_ids, h)
        n = len(self.layers)
        obs = self.observer
        if obs is not None and self.par.owns_embedding():
            obs.observe("model.embed_tokens", h)
        for i, lw in enumerate(self.layers):
            nxt = self.layers[i + 1].fold_attn if i + 1 < n else (self.head_folded and self.par.owns_output_head())
            if self.residency is not None:
                self.residency.acquire(i)
            with nvtx.annotate(f"layer{self.first_layer + i}"):
                h, ssq = self.layer_forward(self.first_layer + i, lw, h, batch, kv, ssq, nxt)
            if self.residency is not None:
                self.residency.release(i)
            if batch.capture_layers is not None and self.first_layer + i in batch.capture_layers:
                if batch.layer_hidden is None:
                    batch.layer_hidden = {}
                batch.layer_hidden[self.first_layer + i] = h
            if batch.deepstack is not None and self.first_layer + i < len(batch.deepstack):
                h = h.index_add(0, batch.embed_rows, batch.deepstack[self.first_layer + i].to(h.dtype))
                ssq = None
            if obs is not None:
                name = f"model.layers.{self.first_layer + i}.output"
                repl = obs.intervene(name, h)
                if repl is not None:
                    h, ssq = repl.to(h.dtype), None     # the producer's row sums no longer describe the activation
                obs.observe(name, h)
        return h, ssq

    def logits(self, h, rows=None, ssq=None):
        if rows is not None:
            h = h.index_select(0, rows)
            ssq = ssq.index_select(0, rows) if ssq is not None else None
        h = h.contiguous()
        if self.head_folded:
            if ssq is None or h.shape[0] > self.FUSED_NORM_MAX_TOKENS:
                h, _ = ops.rmsnorm(h, self._ones(h.shape[1]), self.cfg.rms_norm_eps)
                ssq = None
        else:
            h, _ = ops.rmsnorm(h, self.final_norm, self.cfg.rms_norm_eps, weight_offset=self.cfg.norm_weight_offset)
            ssq = None
        eps = self.cfg.rms_norm_eps
        if self.par.tp_size > 1 and self.lm_head.shape[0] != self.cfg.vocab_size:
            out = self.tp_ops.gathered_logits(h, self.lm_head, self.cfg.vocab_size, self.vocab_start, row_ssq=ssq,
                                              norm_eps=eps)
        else:
            out = ops.linear(h, self.lm_head, out_dtype=torch.float32, row_ssq=ssq, norm_eps=eps)
        cap = (self.cfg.extra.get("gemma4") or {}).get("final_logit_softcapping")
        if cap:
            out = torch.tanh(out / float(cap)) * float(cap)
        mg = self.cfg.extra.get("muse_glimmer")
        if mg:
            cap, mult = float(mg["final_logit_softcapping"]), float(mg["output_multiplier"])
            out = torch.tanh(out * (mult / cap)) * cap
        return out

    def forward(self, batch: ForwardBatch, kv):
        """Returns fp32 logits [R, V] on the last pipeline stage, the hidden state otherwise."""
        h, ssq = self.forward_hidden(batch, kv)
        if batch.capture_hidden:
            batch.hidden_out = h
        if not self.par.owns_output_head():
            return h
        return self.logits(h, batch.logit_rows, ssq)

    def fold_norms(self) -> None:
        """Multiply the RMSNorm weight vectors into the K dimension of the GEMM that consumes the normalised
        activations (qkv, gate_up, lm_head), so that the normalisation reduces to a per-row scale applied in the
        GEMM epilogue. Dense bf16 weights on CUDA only; quantised and MoE consumers keep the explicit kernel."""
        off = self.cfg.norm_weight_offset
        for lw in self.layers:
            self.fold_layer_norms(lw)
        if self.lm_head is not None and self.final_norm is not None and not self.head_folded:
            folded = torch.empty_like(self.lm_head)
            step = 16384
            for r0 in range(0, self.lm_head.shape[0], step):
                folded[r0:r0 + step] = (self.lm_head[r0:r0 + step].float() * (self.final_norm + off)[None, :]).to(self.dtype)
            self.lm_head = folded  # a separate tensor even when the head was tied to the embedding
            self.head_folded = True

    def fold_layer_norms(self, lw) -> None:
        off = self.cfg.norm_weight_offset
        if lw.block_kind:
            return       # single-mixer blocks keep their explicit norm
        if "qkv" not in lw.qlin and not lw.fold_attn and lw.wqkv is not None:
            lw.wqkv = (lw.wqkv.float() * (lw.attn_norm + off)[None, :]).to(self.dtype).contiguous()
            lw.fold_attn = True
        if "kda_in" not in lw.qlin and not lw.fold_attn and lw.kda_in is not None:
            lw.kda_in = (lw.kda_in.float() * (lw.attn_norm + off)[None, :]).to(self.dtype).contiguous()
            lw.fold_attn = True
        if "mla_in" not in lw.qlin and not lw.fold_attn and lw.mla_in is not None:
            lw.mla_in = (lw.mla_in.float() * (lw.attn_norm + off)[None, :]).to(self.dtype).contiguous()
            lw.fold_attn = True
        if "la_in" not in lw.qlin and not lw.fold_attn and lw.la_in is not None:
            lw.la_in = (lw.la_in.float() * (lw.attn_norm + off)[None, :]).to(self.dtype).contiguous()
            lw.fold_attn = True
        if "conv_in" not in lw.qlin and not lw.fold_attn and lw.conv_in is not None:
            lw.conv_in = (lw.conv_in.float() * (lw.attn_norm + off)[None, :]).to(self.dtype).contiguous()
            lw.fold_attn = True
        if lw.moe is None and "gate_up" not in lw.qlin and lw.w_gate_up is not None and not lw.fold_ffn:
            lw.w_gate_up = (lw.w_gate_up.float() * (lw.ffn_norm + off)[None, :]).to(self.dtype).contiguous()
            lw.fold_ffn = True

    # ------------------------------------------------------------------------------------------ weights
    def num_local_layers(self) -> int:
        return self.last_layer - self.first_layer

    def weight_bytes(self) -> int:
        total = 0
        seen = set()

        def add(t):
            nonlocal total
            if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()

        for t in (self.embed, self.final_norm, self.lm_head):
            add(t)
        for lw in self.layers:
            for v in vars(lw).values():
                add(v)
            for v in (lw.extra or {}).values():
                add(v)
            for q in lw.qlin.values():
                for t in q.tensors():
                    add(t)
            if lw.moe is not None:
                for t in lw.moe.tensors():
                    add(t)
        return total


# ---------------------------------------------------------------------------------------------- builders
def _tp_rows(t: torch.Tensor, rank: int, size: int) -> torch.Tensor:
    n = t.shape[0] // size
    return t[rank * n:(rank + 1) * n]


def _tp_cols(t: torch.Tensor, rank: int, size: int) -> torch.Tensor:
    n = t.shape[1] // size
    return t[:, rank * n:(rank + 1) * n]


def shard_attention(cfg: ModelConfig, par, wq, wk, wv, wo, bq=None, bk=None, bv=None):
    """Tensor-parallel slices of the attention projections; a GQA group is the atomic unit and KV heads are
    replicated when there are fewer of them than ranks (nn/parallel.rs:104-183 defines the group rule; the
    replication extends it to tp > n_kv)."""
    from ..parallel.planner import ParallelPlan, attention_groups

    tp, r = par.tp_size, par.tp_rank
    # the typed plan owns the arithmetic: query-head group, key / value-head group (replicated over tp / n_kv consecutive
    # ranks when there are fewer heads than ranks), the output projection following the query heads on its inputs
    plan = ParallelPlan(tp)
    for g in attention_groups(cfg, tp, "", bias=bq is not None):
        plan.add(g)
    wq_l = plan.select("q_proj.weight", wq, r)
    wk_l = plan.select("k_proj.weight", wk, r)
    wv_l = plan.select("v_proj.weight", wv, r)
    wo_l = plan.select("o_proj.weight", wo, r)
    b = None
    if bq is not None:
        b = torch.cat((plan.select("q_proj.bias", bq, r), plan.select("k_proj.bias", bk, r), plan.select("v_proj.bias", bv, r)))
    return torch.cat((wq_l, wk_l, wv_l), 0), wo_l, b


def build_from_tensors(cfg: ModelConfig, get: Callable[[str], torch.Tensor], has: Callable[[str], bool], device, dtype,
                       parallel=None, moe_factory=None, quantizer=None, fold_norms: bool = True, on_layer=None) -> CausalLM:
    """Populate a model from HF-named tensors. ``get(name)`` returns a CPU (or device) tensor; slicing for
    tensor/pipeline parallelism happens here so that a rank only uploads what it owns."""
    model = CausalLM(cfg, device, dtype, parallel)
    par = model.par
    tp, r = par.tp_size, par.tp_rank

    def up(t, dt=None):
        return t.to(device=model.device, dtype=dt or dtype).contiguous()

    if par.owns_embedding() or (par.owns_output_head() and cfg.tie_word_embeddings):
        model.embed = up(get("model.embed_tokens.weight"))
    if par.owns_output_head():
        model.final_norm = up(get("model.norm.weight"), torch.float32)
        head = get("lm_head.weight") if (not cfg.tie_word_embeddings and has("lm_head.weight")) else None
        if head is None:
            head = get("model.embed_tokens.weight")
        if tp > 1 and cfg.vocab_size % tp == 0:
            head = _tp_rows(head, r, tp)
            model.vocab_start = r * (cfg.vocab_size // tp)
            model.lm_head = up(head)
        else:
            model.lm_head = model.embed if (head is None or (cfg.tie_word_embeddings and model.embed is not None
                                                             and not has("lm_head.weight"))) else up(head)
    if cfg.model_type == "gemma4":
        from .gemma4 import build as build_gemma4

        build_gemma4(model, cfg, get, has, up)
        return model
    if cfg.model_type == "muse_glimmer":
        from .muse_glimmer import build as build_muse

        build_muse(model, cfg, get, has, up)
        return model
    for li in range(model.first_layer, model.last_layer):
        p = f"model.layers.{li}."
        bq = bk = bv = None
        if cfg.model_type == "nemotron_h":
            from .nemotron_h import build_block

            lw = build_block(model, cfg, li, p, get, has, up, moe_factory)
            model.layers.append(lw)
            if on_layer is not None:
                on_layer(model, li, lw)
            continue
        if cfg.layer_is_conv(li) or cfg.layer_is_linear_attention(li) or cfg.is_mla or cfg.layer_is_kda(li):
            if cfg.layer_is_kda(li):
                from .kimi_linear import build_kda_layer

                lw = build_kda_layer(model, cfg, p, get, has, up)
            elif cfg.is_mla:
                from .deepseek import build_mla_layer

                lw = build_mla_layer(model, cfg, p, get, has, up)
            elif cfg.layer_is_conv(li):
                lw = _build_conv_layer(model, cfg, p, get, has, up)
            else:
                from .qwen_next import build_linear_attention_layer

                lw = build_linear_attention_layer(model, cfg, p, get, has, up)
            _build_ffn(model, cfg, li, p, lw, get, has, up, moe_factory)
            if quantizer is not None:
                quantizer(model, li, lw)
            model.layers.append(lw)
            if on_layer is not None:
                if model.device.type == "cuda" and dtype == torch.bfloat16 and fold_norms:
                    model.fold_layer_norms(lw)
                on_layer(model, li, lw)
            continue
        if has(p + "self_attn.qkv_proj.weight"):
            # Phi-3 style checkpoints store q, k and v as one matrix and gate / up as another
            qn, kn = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
            fused = get(p + "self_attn.qkv_proj.weight")
            wq, wk, wv = fused[:qn], fused[qn:qn + kn], fused[qn + kn:qn + 2 * kn]
            wo = get(p + "self_attn.o_proj.weight")
            if has(p + "self_attn.qkv_proj.bias"):
                fb = get(p + "self_attn.qkv_proj.bias")
                bq, bk, bv = fb[:qn], fb[qn:qn + kn], fb[qn + kn:qn + 2 * kn]
        else:
            wq, wk, wv, wo = (get(p + f"self_attn.{n}_proj.weight") for n in "qkvo")
        w_gate = None
        if cfg.attn_output_gate:
            # q_proj rows are [query (D) | gate (D)] per head: the gate block moves behind q, k and v
            two = wq.view(cfg.num_attention_heads, 2 * cfg.head_dim, wq.shape[1])
            wq = two[:, :cfg.head_dim].reshape(cfg.num_attention_heads * cfg.head_dim, -1)
            nq_l = model.n_q_local
            w_gate = two[r * nq_l:(r + 1) * nq_l, cfg.head_dim:].reshape(nq_l * cfg.head_dim, -1)   # this rank's heads
        if has(p + "self_attn.q_proj.bias"):
            bq, bk, bv = (get(p + f"self_attn.{n}_proj.bias") for n in "qkv")
        wqkv, wo_l, bqkv = shard_attention(cfg, par, wq, wk, wv, wo, bq, bk, bv)
        if w_gate is not None:
            wqkv = torch.cat((wqkv, w_gate), 0)
        lw = LayerWeights(
            attn_norm=up(get(p + "input_layernorm.weight"), torch.float32),
            wqkv=up(wqkv), wo=up(wo_l),
            ffn_norm=up(get(p + "post_attention_layernorm.weight"), torch.float32),
            bqkv=up(bqkv) if bqkv is not None else None,
        )
        lw.attn_gate = w_gate is not None
        if has(p + "self_attn.o_proj.bias"):
            lw.bo = up(get(p + "self_attn.o_proj.bias"))
        if cfg.qk_norm and has(p + "self_attn.q_norm.weight"):
            lw.q_norm = up(get(p + "self_attn.q_norm.weight"), torch.float32)
            lw.k_norm = up(get(p + "self_attn.k_norm.weight"), torch.float32)
        if has(p + "self_attn.sinks"):
            n_q_local = model.n_q_local
            lw.sinks = up(get(p + "self_attn.sinks")[r * n_q_local:(r + 1) * n_q_local], torch.float32)
        _build_ffn(model, cfg, li, p, lw, get, has, up, moe_factory)
        if quantizer is not None:
            quantizer(model, li, lw)
        model.layers.append(lw)
        if on_layer is not None:
            # the caller takes the layer away (host residency): fold its norms while it is still on the device
            if model.device.type == "cuda" and dtype == torch.bfloat16 and fold_norms:
                model.fold_layer_norms(lw)
            on_layer(model, li, lw)
    if model.device.type == "cuda" and dtype == torch.bfloat16 and fold_norms:
        model.fold_norms()
    return model


def _build_ffn(model, cfg, li, p, lw, get, has, up, moe_factory) -> None:
    par = model.par
    tp, r = par.tp_size, par.tp_rank
    if cfg.layer_is_moe(li):
        assert moe_factory is not None, "MoE layer needs a moe_factory"
        lw.moe = moe_factory(model, li, get, has)
        return
    if has(p + "mlp.gate_up_proj.weight"):
        fused = get(p + "mlp.gate_up_proj.weight")
        wg, wu = fused[: cfg.intermediate_size], fused[cfg.intermediate_size:]
        wd = get(p + "mlp.down_proj.weight")
    else:
        wg, wu, wd = (get(p + f"mlp.{n}_proj.weight") for n in ("gate", "up", "down"))
    if tp > 1:
        from ..parallel.planner import ParallelPlan, feed_forward_group

        plan = ParallelPlan(tp)
        plan.add(feed_forward_group(cfg, "", intermediate=wg.shape[0]))
        wg, wu, wd = (plan.select("gate_proj.weight", wg, r), plan.select("up_proj.weight", wu, r),
                      plan.select("down_proj.weight", wd, r))
    lw.w_gate_up = up(torch.cat((wg, wu), 0))
    lw.w_down = up(wd)


def _build_conv_layer(model, cfg, p, get, has, up) -> LayerWeights:
    """LFM2 short-convolution layer. Tensor parallelism slices the channels: the B, C and X blocks of ``in_proj``
    row-wise, the depthwise kernel by channel and ``out_proj`` column-wise (row-parallel, summed over the group)."""
    par = model.par
    tp, r = par.tp_size, par.tp_rank
    C = cfg.hidden_size
    w_in, w_conv, w_out = get(p + "conv.in_proj.weight"), get(p + "conv.conv.weight"), get(p + "conv.out_proj.weight")
    w_conv = w_conv.reshape(C, -1)
    lo, hi = (r * (C // tp), (r + 1) * (C // tp)) if tp > 1 else (0, C)
    blocks = [w_in[i * C + lo:i * C + hi] for i in range(3)]
    lw = LayerWeights(attn_norm=up(get(p + "input_layernorm.weight"), torch.float32), wqkv=None, wo=None,
                      ffn_norm=up(get(p + "post_attention_layernorm.weight"), torch.float32))
    lw.conv_in = up(torch.cat(blocks, 0))
    lw.conv_w = up(w_conv[lo:hi], torch.float32)
    lw.conv_out = up(w_out[:, lo:hi])
    if has(p + "conv.in_proj.bias"):
        b_in = get(p + "conv.in_proj.bias")
        lw.conv_in_b = up(torch.cat([b_in[i * C + lo:i * C + hi] for i in range(3)], 0))
        lw.conv_b = up(get(p + "conv.conv.bias")[lo:hi], torch.float32)
        lw.conv_out_b = up(get(p + "conv.out_proj.bias"))
    return lw


def random_state(cfg: ModelConfig, seed: int = 0, std: float = 0.02, dtype=torch.float32, device="cpu") -> dict:
    """Seeded HF-named random checkpoint: N(0, std) matrices, unit norms. Deterministic per tensor name, so
    any subset (a pipeline stage, a TP slice source) can be generated independently."""
    import zlib

    out: dict[str, torch.Tensor] = {}

    def mat(name, *shape):
        g = torch.Generator(device="cpu")
        g.manual_seed((seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFF)
        out[name] = (torch.randn(*shape, generator=g, dtype=torch.float32) * std).to(dtype=dtype, device=device)

    def ones(name, n):
        out[name] = torch.ones(n, dtype=dtype, device=device)

    H, D = cfg.hidden_size, cfg.head_dim
    mat("model.embed_tokens.weight", cfg.vocab_size, H)
    ones("model.norm.weight", H)
    if not cfg.tie_word_embeddings:
        mat("lm_head.weight", cfg.vocab_size, H)
    for li in range(cfg.num_hidden_layers):
        p = f"model.layers.{li}."
        if cfg.model_type == "nemotron_h":
            from .nemotron_h import random_block_state

            random_block_state(cfg, li, p, mat, out, std)
            continue
        ones(p + "input_layernorm.weight", H)
        ones(p + "post_attention_layernorm.weight", H)
        if cfg.layer_is_linear_attention(li):
            from .qwen_next import random_linear_attention_state

            random_linear_attention_state(cfg, p, mat, out, std)
            _random_ffn(cfg, li, p, mat)
            continue
        if cfg.layer_is_conv(li):
            mat(p + "conv.in_proj.weight", 3 * H, H)
            mat(p + "conv.conv.weight", H, 1, cfg.conv_l_cache)
            out[p + "conv.conv.weight"] = out[p + "conv.conv.weight"] * (0.5 / std)
            mat(p + "conv.out_proj.weight", H, H)
            if cfg.conv_bias:
                mat(p + "conv.in_proj.bias", 3 * H)
                mat(p + "conv.conv.bias", H)
                mat(p + "conv.out_proj.bias", H)
            _random_ffn(cfg, li, p, mat)
            continue
        if cfg.layer_is_kda(li):
            from .kimi_linear import random_kda_state

            random_kda_state(cfg, p, mat, ones, out, std)
            _random_ffn(cfg, li, p, mat)
            continue
        if cfg.is_mla:
            from .deepseek import random_mla_state

            random_mla_state(cfg, p, mat, ones)
            _random_ffn(cfg, li, p, mat)
            continue
        mat(p + "self_attn.q_proj.weight", cfg.num_attention_heads * D * (2 if cfg.attn_output_gate else 1), H)
        mat(p + "self_attn.k_proj.weight", cfg.num_key_value_heads * D, H)
        mat(p + "self_attn.v_proj.weight", cfg.num_key_value_heads * D, H)
        mat(p + "self_attn.o_proj.weight", H, cfg.num_attention_heads * D)
        if cfg.attention_bias:
            mat(p + "self_attn.q_proj.bias", cfg.num_attention_heads * D)
            mat(p + "self_attn.k_proj.bias", cfg.num_key_value_heads * D)
            mat(p + "self_attn.v_proj.bias", cfg.num_key_value_heads * D)
        if cfg.qk_norm:
            ones(p + "self_attn.q_norm.weight", D)
            ones(p + "self_attn.k_norm.weight", D)
        _random_ffn(cfg, li, p, mat)
    return out


def _random_ffn(cfg, li, p, mat) -> None:
    H = cfg.hidden_size
    if cfg.layer_is_moe(li):
        mat(p + "mlp.gate.weight", cfg.num_experts, H)
        if cfg.shared_expert_intermediate_size > 0:
            shared = "shared_experts" if cfg.model_type in ("deepseek_v3", "kimi_linear") else "shared_expert"
            for n, shape in (("gate", (cfg.shared_expert_intermediate_size, H)), ("up", (cfg.shared_expert_intermediate_size, H)),
                             ("down", (H, cfg.shared_expert_intermediate_size))):
                mat(p + f"mlp.{shared}.{n}_proj.weight", *shape)
            if cfg.model_type in ("deepseek_v3", "kimi_linear"):
                mat(p + "mlp.gate.e_score_correction_bias", cfg.num_experts)
            if cfg.shared_expert_gate:
                mat(p + "mlp.shared_expert_gate.weight", 1, H)
        if cfg.extra.get("use_expert_bias"):
            mat(p + "mlp.expert_bias", cfg.num_experts)
        for e in range(cfg.num_experts):
            mat(p + f"mlp.experts.{e}.gate_proj.weight", cfg.moe_intermediate_size, H)
            mat(p + f"mlp.experts.{e}.up_proj.weight", cfg.moe_intermediate_size, H)
            mat(p + f"mlp.experts.{e}.down_proj.weight", H, cfg.moe_intermediate_size)
    else:
        mat(p + "mlp.gate_proj.weight", cfg.intermediate_size, H)
        mat(p + "mlp.up_proj.weight", cfg.intermediate_size, H)
        mat(p + "mlp.down_proj.weight", H, cfg.intermediate_size)


def build_random(cfg: ModelConfig, device, dtype, seed: int = 0, parallel=None, moe_factory=None, quantizer=None,
                 std: float = 0.02) -> CausalLM:
    """Random-init model of the given shape, generated tensor by tensor on the target device (used by the
    benchmarks: no checkpoint on disk, no full fp32 copy on the host)."""
    import zlib

    dev = torch.device(device)

    def get(name: str) -> torch.Tensor:
        shape = _shape_of(cfg, name)
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            return torch.ones(shape, dtype=torch.float32, device=dev)
        g = torch.Generator(device=dev)
        g.manual_seed((seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFF)
        t = torch.randn(shape, generator=g, dtype=torch.float32 if dev.type == "cpu" else torch.bfloat16, device=dev)
        return (t * std).to(dtype)

    def has(name: str) -> bool:
        return _shape_of(cfg, name) is not None

    return build_from_tensors(cfg, get, has, device, dtype, parallel, moe_factory, quantizer)


def _shape_of(cfg: ModelConfig, name: str):
    H, D = cfg.hidden_size, cfg.head_dim
    if name == "model.embed_tokens.weight":
        return (cfg.vocab_size, H)
    if name == "lm_head.weight":
        return None if cfg.tie_word_embeddings else (cfg.vocab_size, H)
    if name == "model.norm.weight":
        return (H,)
    parts = name.split(".")
    if parts[:2] != ["model", "layers"]:
        return None
    li = int(parts[2])
    rest = ".".join(parts[3:])
    if cfg.layer_is_conv(li):
        conv = {"input_layernorm.weight": (H,), "post_attention_layernorm.weight": (H,),
                "conv.in_proj.weight": (3 * H, H), "conv.conv.weight": (H, 1, cfg.conv_l_cache),
                "conv.out_proj.weight": (H, H)}
        if cfg.conv_bias:
            conv.update({"conv.in_proj.bias": (3 * H,), "conv.conv.bias": (H,), "conv.out_proj.bias": (H,)})
        if rest in conv:
            return conv[rest]
        if rest.startswith("self_attn.") or rest.startswith("conv."):
            return None
    elif rest.startswith("conv."):
        return None
    table = {
        "input_layernorm.weight": (H,), "post_attention_layernorm.weight": (H,),
        "self_attn.q_proj.weight": (cfg.num_attention_heads * D, H),
        "self_attn.k_proj.weight": (cfg.num_key_value_heads * D, H),
        "self_attn.v_proj.weight": (cfg.num_key_value_heads * D, H),
        "self_attn.o_proj.weight": (H, cfg.num_attention_heads * D),
    }
    if cfg.attention_bias:
        table.update({"self_attn.q_proj.bias": (cfg.num_attention_heads * D,),
                      "self_attn.k_proj.bias": (cfg.num_key_value_heads * D,),
                      "self_attn.v_proj.bias": (cfg.num_key_value_heads * D,)})
    if cfg.qk_norm:
        table.update({"self_attn.q_norm.weight": (D,), "self_attn.k_norm.weight": (D,)})
    if cfg.layer_is_moe(li):
        table["mlp.gate.weight"] = (cfg.num_experts, H)
        if rest.startswith("mlp.experts."):
            kind = parts[-2]
            I = cfg.moe_intermediate_size
            return {"gate_proj": (I, H), "up_proj": (I, H), "down_proj": (H, I)}.get(kind)
    else:
        I = cfg.intermediate_size
        table.update({"mlp.gate_proj.weight": (I, H), "mlp.up_proj.weight": (I, H), "mlp.down_proj.weight": (H, I)})
    return table.get(rest)
