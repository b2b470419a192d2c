"""Speculative decoding with an external draft model: propose k tokens, verify them in one target pass, accept /
resample with the exact rejection rule, roll back both KV caches by length.

Round structure and bookkeeping follow eredu-core/src/speculative.rs:1038-1216 (propose_block / resolve_round) and
doc/speculative-decoding.md:58-62: the target cache only holds tokens already fed as target inputs; the token that
ends a round (a resampled token or the bonus token after full acceptance) is emitted but stays the leading
*uncached* input of the next verify pass; a rejection truncates the target KV and discards the draft branch.
Acceptance follows eredu/src/backend/mlx/speculative.rs:520-574 (greedy: argmax == proposed; stochastic: accept with
min(1, p_t/p_d), else resample from norm(max(p_t - p_d, 0))) - here evaluated by one kernel launch per round
(``spec_verify``) with position-addressed uniforms instead of four host synchronisations per proposal.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from .. import ops
from ..models.llama import ForwardBatch
from ..ops.sampling import ROW_DTYPE, SamplingParams, pack_rows
from .engine import Engine, Sequence
from .kv_cache import PAGE


@dataclass
class SpecStats:
    rounds: int = 0
    proposed: int = 0
    accepted: int = 0
    emitted: int = 0
    full_accept_rounds: int = 0
    verify_ms: list = field(default_factory=list)
    draft_ms: list = field(default_factory=list)

    def summary(self) -> dict:
        r = max(1, self.rounds)
        return {"rounds": self.rounds, "proposed": self.proposed, "accepted": self.accepted, "emitted": self.emitted,
                "accepted_per_step": self.accepted / r, "tokens_per_step": self.emitted / r,
                "acceptance_rate": self.accepted / max(1, self.proposed), "full_accept_rounds": self.full_accept_rounds,
                "verify_ms_p50": float(np.median(self.verify_ms)) if self.verify_ms else None,
                "draft_ms_p50": float(np.median(self.draft_ms)) if self.draft_ms else None}


class SpeculativeDecoder:
    """Drives a target :class:`Engine` and a draft :class:`Engine` (same vocabulary). Default k follows the
    reference's ``MtpConfig`` (4 draft tokens, eredu-core/src/generation.rs:339-360)."""

    def __init__(self, target: Engine, draft: Engine, k: int = 4):
        assert target.cfg.vocab_size == draft.cfg.vocab_size, "draft and target must share the vocabulary"
        self.t, self.d, self.k = target, draft, k
        self.stats = SpecStats()
        self.cuda = target.cuda

    # ------------------------------------------------------------------------------------------ forward helpers
    @staticmethod
    def _slots(seq: Sequence, positions: np.ndarray) -> np.ndarray:
        pages = np.asarray(seq.pages, dtype=np.int64)
        return pages[positions // PAGE] * PAGE + (positions % PAGE)

    def _multi_token_step(self, eng: Engine, seqs, tokens: list[list[int]], all_rows: bool, uniform: bool):
        """Feed ``tokens[i]`` to sequence i starting at its kv_len. Returns logits of every fed row (all_rows) or
        of the last row of each sequence. Uniform token counts use the split-KV decode kernel, ragged counts the
        prefill kernel (both attend to the cached prefix)."""
        lens = [len(t) for t in tokens]
        pos = [np.arange(s.kv_len, s.kv_len + n) for s, n in zip(seqs, lens)]
        cu = np.concatenate(([0], np.cumsum(lens)))
        flat = np.concatenate([np.asarray(t, dtype=np.int32) for t in tokens])
        kv_after = np.asarray([s.kv_len + n for s, n in zip(seqs, lens)], dtype=np.int32)
        rows = None if all_rows else eng._t(cu[1:].astype(np.int64) - 1, torch.int64)
        common = dict(token_ids=eng._t(flat, torch.int32),
                      positions=eng._t(np.concatenate(pos).astype(np.int32), torch.int32),
                      slots=eng._t(np.concatenate([self._slots(s, p) for s, p in zip(seqs, pos)]), torch.int64),
                      block_table=eng._block_table(seqs), seq_lens=eng._t(kv_after, torch.int32), logit_rows=rows)
        if uniform and len(set(lens)) == 1:
            splits = ops.decode_splits(len(seqs), eng.model.n_kv_local, int(kv_after.max()), eng.sm_count) if eng.cuda else 1
            batch = ForwardBatch(is_prefill=False, q_per_seq=lens[0], splits=splits, **common)
        else:
            batch = ForwardBatch(is_prefill=True, cu_q=eng._t(cu.astype(np.int32), torch.int32), max_q_len=max(lens),
                                 **common)
        return eng.model.forward(batch, eng.kv)

    def _probs_and_tokens(self, eng: Engine, logits, sps, positions, stream_ids, want_tokens=True):
        """Final distributions (dense fp32) and sampled tokens for a set of rows."""
        R, V = logits.shape
        if self.cuda:
            rows = pack_rows(sps, positions, stream_ids=stream_ids)
            rows_t = eng._t(rows.view(np.uint8).reshape(R, ROW_DTYPE.itemsize), torch.uint8)
            probs = torch.empty((R, V), dtype=torch.float32, device=logits.device)
            toks = ops.sample(logits.contiguous(), rows_t, probs=probs, all_greedy=all(sp.greedy for sp in sps))
            return probs, toks
        probs, toks = [], []
        for i in range(R):
            t, p = ops.sample_ref(logits[i], sps[i], positions[i], stream=stream_ids[i])
            probs.append(p)
            toks.append(t)
        return torch.stack(probs), torch.tensor(toks, dtype=torch.int32)

    # ------------------------------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(self, prompts: list[list[int]], sampling: Optional[SamplingParams] = None, max_new_tokens: int = 64,
                 eos_ids=()) -> list[list[int]]:
        sp = sampling or SamplingParams()
        k = self.k
        tseqs = [self.t.new_sequence(p, sp, max_new_tokens + k + 2, eos_ids) for p in prompts]
        dseqs = [self.d.new_sequence(p, sp, max_new_tokens + k + 2, eos_ids) for p in prompts]
        try:
            first = self.t.prefill(tseqs).tolist()
            self.d.prefill(dseqs)  # the draft's own first sample is discarded: the target decides
            outs: list[list[int]] = [[int(t)] for t in first]
            pending = [[int(t)] for t in first]       # committed tokens missing from the draft cache
            last = [int(t) for t in first]            # leading uncached target input
            done = [int(t) in eos_ids or max_new_tokens <= 1 for t in first]
            while not all(done):
                live = [i for i, f in enumerate(done) if not f]
                self._round([tseqs[i] for i in live], [dseqs[i] for i in live], live, outs, pending, last, sp)
                for i in live:
                    if len(outs[i]) >= max_new_tokens:
                        outs[i] = outs[i][:max_new_tokens]
                        done[i] = True
                    for j, tok in enumerate(outs[i]):
                        if tok in eos_ids:
                            outs[i] = outs[i][: j + 1]
                            done[i] = True
                            break
            if self.cuda:
                ops.native.check_status(self.t.device)
            return outs
        finally:
            for s in tseqs:
                self.t.release(s)
            for s in dseqs:
                self.d.release(s)

    def _round(self, tseqs, dseqs, live, outs, pending, last, sp):
        k = self.k
        B = len(tseqs)
        V = self.t.cfg.vocab_size
        dev = self.t.device
        sync = (lambda: torch.cuda.synchronize(dev)) if self.cuda else (lambda: None)
        t0 = time.perf_counter()
        # ---- draft: k proposals per sequence
        drafted = [[] for _ in range(B)]
        p_d = []
        base = [s.kv_len + 1 for s in tseqs]  # position of the first drafted token (target kv_len = position of `last`)
        for j in range(k):
            if j == 0:
                feed = [pending[i] for i in live]
                logits = self._multi_token_step(self.d, dseqs, feed, all_rows=False, uniform=False)
                for s, f in zip(dseqs, feed):
                    s.kv_len += len(f)
            else:
                feed = [[drafted[b][-1]] for b in range(B)]
                logits = self._multi_token_step(self.d, dseqs, feed, all_rows=False, uniform=True)
                for s in dseqs:
                    s.kv_len += 1
            probs, toks = self._probs_and_tokens(self.d, logits, [sp] * B, [base[b] + j for b in range(B)],
                                                 [s.seq_id for s in tseqs])
            p_d.append(probs)
            for b, t in enumerate(toks.tolist()):
                drafted[b].append(int(t))
        sync()
        t1 = time.perf_counter()
        # ---- target: one pass over [last, d_1 .. d_k]
        feed = [[last[i]] + drafted[b] for b, i in enumerate(live)]
        logits = self._multi_token_step(self.t, tseqs, feed, all_rows=True, uniform=True)  # [B*(k+1), V]
        pos_rows = [base[b] + j for b in range(B) for j in range(k + 1)]
        sid_rows = [tseqs[b].seq_id for b in range(B) for _ in range(k + 1)]
        p_t, t_toks = self._probs_and_tokens(self.t, logits, [sp] * (B * (k + 1)), pos_rows, sid_rows)
        p_t = p_t.view(B, k + 1, V)
        t_toks = t_toks.view(B, k + 1)
        p_d3 = torch.stack(p_d, dim=1)  # [B, k, V]
        if self.cuda:
            rows = pack_rows([sp] * B, base, stream_ids=[s.seq_id for s in tseqs])
            rows_t = self.t._t(rows.view(np.uint8).reshape(B, ROW_DTYPE.itemsize), torch.uint8)
            dr = self.t._t(np.asarray(drafted, dtype=np.int32), torch.int32)
            res = ops.spec_verify(p_t.contiguous(), p_d3.contiguous(), dr, rows_t).tolist()
        else:
            res = [ops.verify_ref(p_t[b], p_d3[b], drafted[b], sp.seed, tseqs[b].seq_id, base[b]) for b in range(B)]
        bonus = t_toks[:, k].tolist()  # what plain sampling draws at that position: scheduling stays invisible
        sync()
        t2 = time.perf_counter()
        # ---- commit: accepted drafts + the token that ends the round
        for b, i in enumerate(live):
            a, nxt = int(res[b][0]), int(res[b][1])
            if a == k:
                nxt = int(bonus[b])
            outs[i].extend(drafted[b][:a] + [nxt])
            tseqs[b].kv_len += 1 + a                      # `last` and the accepted drafts are now cached
            d_valid = dseqs[b].kv_len - (k - 1) + min(a, k - 1)   # draft cache holds last, d_1..d_{k-1}
            dseqs[b].kv_len = d_valid
            pending[i] = ([drafted[b][k - 1]] if a == k else []) + [nxt]
            last[i] = nxt
            self.stats.accepted += a
            self.stats.emitted += a + 1
            self.stats.full_accept_rounds += 1 if a == k else 0
        self.stats.rounds += B  # one verify step per live sequence
        self.stats.proposed += k * B
        self.stats.draft_ms.append((t1 - t0) * 1e3)
        self.stats.verify_ms.append((t2 - t1) * 1e3)
