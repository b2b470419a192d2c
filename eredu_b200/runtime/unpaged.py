"""A small engine for model families whose cache is not a paged K / V pool.

Some decoders keep per-layer state that the paged pool cannot express (DeepSeek-V4: token keys, pooled streams and their
open windows). They implement ``new_cache()`` and ``forward(token_ids, cache, all_rows=False)``; this engine gives them the
part of :class:`runtime.engine.Engine`'s surface that text generation needs - ``generate`` with the position-addressed
sampler, ``prefill_logits``, ``step_logits``, sequences with ``release`` - one sequence at a time, eagerly - and a
draft-and-verify decoder that rolls such caches back by value (:class:`UnpagedSpeculativeDecoder`). Continuous batching,
CUDA graphs, prefix reuse, the speculative request scheduler and parking are the paged engine's and are refused here.
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


class UnpagedSpeculativeDecoder:
    """Draft-and-verify decoding for a target on :class:`UnpagedEngine` (families whose cache cannot be truncated: pooled
    streams, convolution states). The sampler is addressed by position, so the token the target would emit at a position
    does not depend on how the position was reached: a round feeds ``[last, d1 .. dk]`` to the target in one pass,
    samples every row with the position-addressed sampler and keeps the drafted tokens up to the first that differs,
    plus the target's own token there. The output is token for token what ``UnpagedEngine.generate`` produces, at any
    temperature. A cache that cannot forget is rolled back by value: the round starts from a copy (``cache.clone()``) and a
    partly rejected round re-feeds the accepted prefix to that copy.

    The draft is any engine with ``new_sequence / feed_logits / release``: another unpaged model, or a paged
    ``runtime.engine.Engine`` without recurrent state (its sequence is rolled back by length)."""

    def __init__(self, target: "UnpagedEngine", draft, k: int = 4):
        from .speculative import SpecStats

        if getattr(target, "paged", True):
            raise ValueError("the target of this decoder is an unpaged engine")
        if int(draft.cfg.vocab_size) != int(target.cfg.vocab_size):
            raise ValueError(f"draft vocabulary {draft.cfg.vocab_size} differs from the target's {target.cfg.vocab_size}")
        self.draft_paged = bool(getattr(draft, "paged", True))
        if self.draft_paged and getattr(getattr(draft, "kv", None), "recurrent_tensors", None) is not None \
                and list(draft.kv.recurrent_tensors()):
            raise NotImplementedError("a paged draft with recurrent state cannot be rolled back by length")
        self.target, self.draft, self.k = target, draft, int(k)
        self.stats = SpecStats()
        self.last_finish_reasons: list = []

    # the draft's state is "every committed token except the pending one"; it is restored to that point after each round
    def _draft_mark(self, dseq):
        return dseq.kv_len if self.draft_paged else (dseq.cache.clone(), dseq.kv_len)

    def _draft_restore(self, dseq, mark):
        if self.draft_paged:
            dseq.kv_len = mark
        else:
            dseq.cache, dseq.kv_len = mark[0].clone(), mark[1]

    @torch.no_grad()
    def generate(self, prompts, sampling: Optional[SamplingParams] = None, max_new_tokens: int = 64, eos_ids=(), on_token=None):
        sp = sampling or SamplingParams()
        tgt, outs = self.target, []
        self.last_finish_reasons = [None] * len(prompts)
        for i, prompt in enumerate(prompts):
            tseq = tgt.new_sequence(prompt, sp, max_new_tokens, eos_ids)
            dseq = self.draft.new_sequence(list(prompt), sp, max_new_tokens + self.k + 1, tuple(eos_ids))
            stream = tseq.seq_id if sp.seed is None else i
            out: list = []

            def emit(tok) -> bool:
                out.append(tok)
                why = on_token(i, tok) if on_token is not None else None
                if why:
                    self.last_finish_reasons[i] = why
                return bool(why) or tok in eos_ids or len(out) >= max_new_tokens

            try:
                logits = tgt.prefill_logits([tseq])[0]
                last = tgt._sample(logits, sp, tseq.kv_len, stream)
                done = emit(last)
                self.draft.feed_logits(dseq, list(prompt))              # the draft follows the target's context
                while not done:
                    k = min(self.k, max_new_tokens - len(out))
                    base = tseq.kv_len                                   # position of ``last``; row j samples position base + j + 1
                    mark = self._draft_mark(dseq)
                    drafted, feed = [], last
                    for j in range(k):
                        dl = self.draft.feed_logits(dseq, [feed])
                        feed = tgt._sample(dl, sp, base + j + 1, stream)
                        drafted.append(feed)
                    snapshot = tseq.cache.clone()
                    rows = tgt.model.forward([last] + drafted, tseq.cache, all_rows=True)
                    want = [tgt._sample(rows[j], sp, base + j + 1, stream) for j in range(k + 1)]
                    a = 0
                    while a < k and drafted[a] == want[a]:
                        a += 1
                    self.stats.rounds += 1
                    self.stats.proposed += k
                    self.stats.accepted += a
                    self.stats.emitted += a + 1
                    self.stats.full_accept_rounds += int(a == k)
                    if a == k:
                        tseq.kv_len = base + k + 1
                    else:                                                # roll back by value, keep the accepted prefix
                        tseq.cache = snapshot
                        tgt.model.forward([last] + drafted[:a], tseq.cache)
                        tseq.kv_len = base + a + 1
                    self._draft_restore(dseq, mark)
                    self.draft.feed_logits(dseq, [last] + drafted[:a])
                    for tok in want[:a + 1]:
                        done = emit(tok)
                        if done:
                            break
                    last = want[a]
                outs.append(out)
            finally:
                tgt.release(tseq)
                self.draft.release(dseq)
        return outs
