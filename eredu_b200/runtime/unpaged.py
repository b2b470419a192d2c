"""A small engine for model families whose cache is not a paged K / V pool.

Some decoders keep per-layer state that the paged pool cannot express (DeepSeek-V4: token keys, pooled streams and their
open windows). They implement ``new_cache()`` and ``forward(token_ids, cache, all_rows=False)``; this engine gives them the
part of :class:`runtime.engine.Engine`'s surface that text generation needs - ``generate`` with the position-addressed
sampler, ``prefill_logits``, ``step_logits``, sequences with ``release`` - one sequence at a time, eagerly. Continuous
batching, CUDA graphs, prefix reuse, speculative decoding and parking are the paged engine's and are refused here.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import ops
from ..ops.sampling import SamplingParams


@dataclass
class UnpagedSequence:
    seq_id: int
    prompt: list
    sampling: SamplingParams
    max_new_tokens: int
    eos_ids: tuple
    cache: object
    kv_len: int = 0
    output: list = field(default_factory=list)


class UnpagedEngine:
    paged = False

    def __init__(self, model, max_batch: int = 1, max_seq_len: int = 4096):
        self.model, self.cfg = model, model.cfg
        self.device = model.device
        self.cuda = self.device.type == "cuda"
        self.max_batch, self.max_seq_len = max_batch, max_seq_len
        self._next_id = 0
        self.last_finish_reasons: list = []

    # ------------------------------------------------------------------ sequences
    def new_sequence(self, prompt, sampling: Optional[SamplingParams] = None, max_new_tokens: int = 64, eos_ids=()):
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        if len(prompt) + max_new_tokens > self.max_seq_len:
            raise ValueError(f"prompt of {len(prompt)} tokens plus {max_new_tokens} new ones exceeds max_seq_len {self.max_seq_len}")
        self._next_id += 1
        return UnpagedSequence(self._next_id, list(prompt), sampling or SamplingParams(), max_new_tokens, tuple(eos_ids),
                               self.model.new_cache())

    def release(self, seq) -> None:
        seq.cache = None

    # ------------------------------------------------------------------ logits
    @torch.no_grad()
    def prefill_logits(self, seqs):
        """Feeds every sequence's prompt; returns one fp32 logits row per sequence."""
        rows = []
        for s in seqs:
            rows.append(self.model.forward(s.prompt, s.cache))
            s.kv_len = len(s.prompt)
        return rows

    @torch.no_grad()
    def feed_logits(self, seq, token_ids, multimodal=None):
        """Feeds ``token_ids`` with soft tokens at some rows (``multimodal``: (rows, values), the family's media ingress);
        returns the logits after the last one."""
        out = self.model.forward(list(token_ids), seq.cache) if multimodal is None else \
            self.model.forward(list(token_ids), seq.cache, embeds=multimodal)
        seq.kv_len += len(token_ids)
        return out

    @torch.no_grad()
    def step_logits(self, seq, token: int):
        out = self.model.forward([int(token)], seq.cache)
        seq.kv_len += 1
        return out

    # ------------------------------------------------------------------ generation
    def _sample(self, logits, sp: SamplingParams, position: int, stream_id: int) -> int:
        tok, _ = ops.sample_ref(logits.float().cpu(), sp, position, stream=stream_id)
        return int(tok)

    @torch.no_grad()
    def generate(self, prompts, sampling: Optional[SamplingParams] = None, max_new_tokens: int = 64, eos_ids=(), on_token=None):
        """Same contract as ``Engine.generate``: ``on_token(i, token)`` sees every token in order; a truthy return ends
        sequence i and is kept in ``last_finish_reasons``."""
        sp = sampling or SamplingParams()
        outs = []
        self.last_finish_reasons = [None] * len(prompts)
        for i, prompt in enumerate(prompts):
            seq = self.new_sequence(prompt, sp, max_new_tokens, eos_ids)
            try:
                logits = self.prefill_logits([seq])[0]
                out = []
                while len(out) < max_new_tokens:
                    tok = self._sample(logits, sp, seq.kv_len, seq.seq_id if sp.seed is None else i)
                    out.append(tok)
                    why = on_token(i, tok) if on_token is not None else None
                    if why:
                        self.last_finish_reasons[i] = why
                        break
                    if tok in eos_ids or len(out) >= max_new_tokens:
                        break
                    logits = self.step_logits(seq, tok)
                outs.append(out)
            finally:
                self.release(seq)
        return outs
