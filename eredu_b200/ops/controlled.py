"""Stateful samplers that wrap the stateless chain of :mod:`ops.sampling`: Mirostat v2 and grammar-constrained
sampling.

* ``MirostatV2``: the adaptive-surprise sampler of eredu/src/backend/mlx/runtime/generation/sampler.rs:356-545:
  penalties -> temperature-scaled probabilities -> keep tokens whose surprise ``-log2 p`` is at most ``mu`` (only
  the argmax when none qualifies) -> sample -> ``mu -= eta * (surprise of the sampled token - tau)`` with the
  probability taken AFTER truncation and renormalisation; ``mu`` starts at ``2 * tau``. One sequence per sampler;
  under speculative decoding only committed target tokens advance ``mu``.
* ``GrammarConstraint``: JSON-schema / Lark / regex constraints compiled by llguidance into per-step token masks
  (eredu/src/backend/mlx/runtime/chat/constraints.rs: schema -> grammar -> token masks, fork / rollback for
  speculation). The mask is a packed allow-bitmask consumed by the sampler kernels; ``is_complete`` ends a request
  with the ``grammar_complete`` reason.
"""
from __future__ import annotations

import json
import math
from typing import Optional

import numpy as np
import torch

from .sampling import SamplingParams, philox_uniform, process_logits_ref


class MirostatV2:
    def __init__(self, tau: float = 5.0, eta: float = 0.1, temperature: float = 1.0, seed: int = 0,
                 repeat_penalty: float = 1.0, repeat_last_n: int = 64, frequency_penalty: float = 0.0,
                 presence_penalty: float = 0.0):
        for name, v in (("tau", tau), ("eta", eta)):
            if not (math.isfinite(v) and v > 0):
                raise ValueError(f"Mirostat V2 {name} must be finite and greater than zero")
        if not (math.isfinite(temperature) and temperature > 0):
            raise ValueError("Mirostat V2 requires a finite temperature greater than zero")
        self.tau, self.eta, self.mu = float(tau), float(eta), 2.0 * float(tau)
        # penalties only: top-k / top-p / min-p are replaced by the surprise cut-off
        self.params = SamplingParams(temperature=temperature, top_k=0, top_p=1.0, min_p=0.0, seed=seed,
                                     repeat_penalty=repeat_penalty, repeat_last_n=repeat_last_n,
                                     frequency_penalty=frequency_penalty, presence_penalty=presence_penalty)
        self.history: list[int] = []

    def reset(self):
        self.mu = 2.0 * self.tau
        self.history.clear()

    def distribution(self, logits: torch.Tensor, allow: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Truncated, renormalised distribution for the next token (fp32, on the logits' device)."""
        p = process_logits_ref(logits, self.params, self.history, allow).to(torch.float32)
        cutoff = 2.0 ** (-self.mu)
        keep = p >= cutoff
        if not bool(keep.any()):
            keep = torch.zeros_like(keep)
            keep[int(torch.argmax(p))] = True
        q = torch.where(keep, p, torch.zeros_like(p))
        return q / q.sum()

    def accept(self, token: int, probability: float):
        """Record a committed token and move ``mu`` toward the target surprise."""
        if not (math.isfinite(probability) and 0.0 < probability <= 1.0):
            raise ValueError("accepted Mirostat V2 token probability must be finite and in (0, 1]")
        self.mu -= self.eta * (-math.log2(probability) - self.tau)
        self.history.append(int(token))

    def sample(self, logits: torch.Tensor, position: int, stream: int = 0, allow: Optional[torch.Tensor] = None) -> int:
        q = self.distribution(logits, allow)
        u = philox_uniform(self.params.seed, stream, position, 0)
        cum = torch.cumsum(q.double().cpu(), 0)
        idx = int(torch.searchsorted(cum, torch.tensor(u * float(cum[-1]), dtype=torch.float64), right=True))
        idx = min(idx, q.numel() - 1)
        while float(q[idx]) == 0.0 and idx > 0:
            idx -= 1
        self.accept(idx, float(q[idx]))
        return idx


class GrammarConstraint:
    """Token-level constraint for one request. ``kind``: "json_schema" (a dict or JSON text), "lark", "regex"."""

    def __init__(self, tokenizer_bundle, kind: str, spec, max_tokens_lookahead: int = 0):
        import llguidance
        import llguidance.hf

        tok = getattr(tokenizer_bundle, "tokenizer", tokenizer_bundle)
        self._lltok = _ll_tokenizer(tok)
        if kind == "json_schema":
            text = spec if isinstance(spec, str) else json.dumps(spec)
            grammar = llguidance.LLMatcher.grammar_from_json_schema(text)
        elif kind == "lark":
            grammar = llguidance.LLMatcher.grammar_from_lark(spec)
        elif kind == "regex":
            grammar = llguidance.LLMatcher.grammar_from_regex(spec)
        else:
            raise ValueError(f"unknown constraint kind {kind!r}")
        err = llguidance.LLMatcher.validate_grammar(grammar, self._lltok)
        if err:
            raise ValueError(f"invalid grammar: {err}")
        self.matcher = llguidance.LLMatcher(self._lltok, grammar)
        self.vocab_size = self._lltok.vocab_size
        self._consumed = 0

    # ---- masks
    def allow_bits(self) -> np.ndarray:
        """Packed little-endian allow mask (uint32 words, bit t of word t // 32 = token t allowed)."""
        raw = self.matcher.compute_bitmask()
        self._check()
        words = np.frombuffer(raw, dtype=np.uint8)
        pad = (-len(words)) % 4
        if pad:
            words = np.concatenate((words, np.zeros(pad, dtype=np.uint8)))
        return words.view("<u4").copy()

    def allow_mask(self, vocab_size: Optional[int] = None) -> torch.Tensor:
        """Dense boolean mask [vocab] (the reference path of the samplers)."""
        bits = self.allow_bits()
        n = vocab_size or self.vocab_size
        dense = np.unpackbits(bits.view(np.uint8), bitorder="little")[:n].astype(bool)
        if dense.shape[0] < n:
            dense = np.concatenate((dense, np.zeros(n - dense.shape[0], dtype=bool)))
        return torch.from_numpy(dense)

    # ---- state
    def commit(self, token: int) -> None:
        bits = self.allow_bits()   # checked against the mask first: a refused token must not poison the matcher
        t = int(token)
        if t < 0 or (t >> 5) >= len(bits) or not (int(bits[t >> 5]) >> (t & 31)) & 1:
            raise ValueError(f"token {token} violates the grammar")
        if not self.matcher.consume_token(int(token)):
            self._check()
            raise ValueError(f"token {token} violates the grammar")
        self._consumed += 1

    def rollback(self, n_tokens: int) -> None:
        """Undo the last n committed tokens (rejected speculative proposals)."""
        if n_tokens:
            if not self.matcher.rollback(int(n_tokens)):
                self._check()
            self._consumed -= n_tokens

    def fork(self) -> "GrammarConstraint":
        other = object.__new__(GrammarConstraint)
        other._lltok, other.vocab_size, other._consumed = self._lltok, self.vocab_size, self._consumed
        other.matcher = self.matcher.deep_copy()
        return other

    def is_complete(self) -> bool:
        """The grammar cannot take another token (generation ends with reason ``grammar_complete``)."""
        return bool(self.matcher.is_stopped())

    def is_accepting(self) -> bool:
        return bool(self.matcher.is_accepting())

    def forced_tokens(self) -> list[int]:
        """Tokens the grammar forces next (can be appended without sampling)."""
        return list(self.matcher.compute_ff_tokens())

    def _check(self):
        if self.matcher.is_error():
            raise RuntimeError(f"constraint engine error: {self.matcher.get_error()}")


_LL_CACHE: dict = {}


def _ll_tokenizer(tok):
    """llguidance tokenizer for a ``tokenizers.Tokenizer`` (cached per object: building it walks the vocabulary)."""
    import llguidance

    key = id(tok)
    if key not in _LL_CACHE:
        _LL_CACHE[key] = llguidance.LLTokenizer(tok.to_str()) if hasattr(tok, "to_str") else llguidance.LLTokenizer(tok)
    return _LL_CACHE[key]


def controlled_generate(engine, prompt: list[int], sampling: Optional[SamplingParams] = None, max_new_tokens: int = 256,
                        eos_ids=(), constraint: Optional[GrammarConstraint] = None, mirostat: Optional[MirostatV2] = None,
                        on_token=None):
    """Single-sequence generation with a stateful sampler: a grammar, Mirostat, or both. Every step's logits go
    through the constraint's mask before sampling; the grammar's own end stops the request. ``on_token(token)`` may
    return a finish reason to stop early (stop strings, cancellation). Returns (tokens, finish_reason).
    Runs the model through ``engine`` one decode step at a time (host-driven: the mask depends on the last token)."""
    from .sampling import sample_ref

    sp = sampling or SamplingParams(temperature=0.0)
    seq = engine.new_sequence(prompt, sp, max_new_tokens, eos_ids)
    out: list[int] = []
    reason = "max_tokens"
    try:
        logits = engine.prefill_logits([seq])[0]
        for step in range(max_new_tokens):
            allow = None
            if constraint is not None:
                allow = constraint.allow_mask(logits.shape[-1])
                for e in eos_ids:                     # EOS is legal exactly where the grammar accepts an end
                    allow[e] = constraint.is_accepting()
            pos = len(prompt) + step
            if mirostat is not None:
                tok = mirostat.sample(logits, pos, seq.seq_id, allow)
            else:
                tok, _ = sample_ref(logits.float().cpu(), sp, pos, history=out, allow=allow, stream=seq.seq_id)
            if tok in eos_ids:
                reason = "eos"
                break
            if constraint is not None:
                constraint.commit(tok)
            out.append(tok)
            if on_token is not None:
                early = on_token(tok)
                if early:
                    reason = early
                    break
            if constraint is not None and constraint.is_complete():
                reason = "grammar_complete"
                break
            if step + 1 == max_new_tokens:
                break
            logits = engine.step_logits(seq, tok)
    finally:
        engine.release(seq)
    return out, reason


def constrained_generate(engine, prompt: list[int], constraint: GrammarConstraint, sampling: Optional[SamplingParams] = None,
                         max_new_tokens: int = 256, eos_ids=(), mirostat: Optional[MirostatV2] = None):
    """:func:`controlled_generate` with a mandatory grammar."""
    return controlled_generate(engine, prompt, sampling, max_new_tokens, eos_ids, constraint, mirostat)
