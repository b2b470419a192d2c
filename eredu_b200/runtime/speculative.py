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
    prefill_ms: float = 0.0

    def summary(self) -> dict:
        r = max(1, self.rounds)
        return {"rounds": self.rounds, "proposed": self.proposed, "accepted": self.accepted, "emitted": self.emitted,
                "accepted_per_step": self.accepted / r, "tokens_per_step": self.emitted / r,
                "acceptance_rate": self.accepted / max(1, self.proposed), "full_accept_rounds": self.full_accept_rounds,
                "verify_ms_p50": float(np.median(self.verify_ms)) if self.verify_ms else None,
                "draft_ms_p50": float(np.median(self.draft_ms)) if self.draft_ms else None,
                "prefill_ms": self.prefill_ms}


class SpeculativeDecoder:
    """Drives a target :class:`Engine` and a draft :class:`Engine` (same vocabulary). Default k follows the
    reference's ``MtpConfig`` (4 draft tokens, eredu-core/src/generation.rs:339-360)."""

    def __init__(self, target: Engine, draft: Engine, k: int = 4):
        assert target.cfg.vocab_size == draft.cfg.vocab_size, "draft and target must share the vocabulary"
        self.t, self.d, self.k = target, draft, k
        # Hybrid models: rejected proposals also have to leave the recurrent states. The draft keeps a snapshot after every
        # draft step and goes back to the one that matches the accepted prefix; the target keeps one snapshot per round
        # and, after a partial acceptance, re-feeds the accepted tokens from it (one extra pass in that case only).
        self.t_hybrid, self.d_hybrid = target.kv.has_recurrent_state(), draft.kv.has_recurrent_state()
        self.stats = SpecStats()
        self.cuda = target.cuda

    # ------------------------------------------------------------------------------------------ forward helpers
    @staticmethod
    def _slots(seq: Sequence, positions: np.ndarray) -> np.ndarray:
        pages = np.asarray(seq.pages, dtype=np.int64)
        return pages[positions // PAGE] * PAGE + (positions % PAGE)

    def _multi_token_step(self, eng: Engine, seqs, tokens: list[list[int]], all_rows: bool, uniform: bool, prepare=None):
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
        if prepare is not None:
            prepare(batch)             # embedded heads: activations instead of token embeddings, hidden-state capture
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
                 eos_ids=(), on_token=None) -> list[list[int]]:
        """``on_token(i, token)`` sees every committed token of sequence i in order (a round commits several at once);
        a truthy return value ends that sequence after the token and is kept in ``last_finish_reasons``."""
        sp = sampling or SamplingParams()
        k = self.k
        self.last_finish_reasons = [None] * len(prompts)
        seen = [0] * len(prompts)

        def publish(i, outs, done):
            if on_token is None:
                return
            while seen[i] < len(outs[i]):
                why = on_token(i, outs[i][seen[i]])
                seen[i] += 1
                if why:
                    outs[i] = outs[i][:seen[i]]
                    done[i] = True
                    self.last_finish_reasons[i] = why
                    return

        tseqs = [self.t.new_sequence(p, sp, max_new_tokens + k + 2, eos_ids) for p in prompts]
        dseqs = [self.d.new_sequence(p, sp, max_new_tokens + k + 2, eos_ids) for p in prompts]
        try:
            first = self._prefill(tseqs, dseqs)
            outs: list[list[int]] = [[int(t)] for t in first]
            pending = [[int(t)] for t in first]       # committed tokens missing from the draft cache
            last = [int(t) for t in first]            # leading uncached target input
            done = [int(t) in eos_ids or max_new_tokens <= 1 for t in first]
            for i in range(len(prompts)):
                publish(i, outs, done)
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
                    publish(i, outs, done)
            if self.cuda:
                ops.native.check_status(self.t.device)
            return outs
        finally:
            for s in tseqs:
                self.t.release(s)
            for s in dseqs:
                self.d.release(s)

    # ------------------------------------------------------------------------------------------ grammar-constrained
    @torch.no_grad()
    def generate_constrained(self, prompt: list[int], constraint, sampling: Optional[SamplingParams] = None,
                             max_new_tokens: int = 64, eos_ids=(), on_token=None):
        """One sequence under a grammar (``ops.controlled.GrammarConstraint``): proposals are drawn from the draft's masked
        distributions while a fork of the grammar state runs ahead, and the target's rows are masked with
        the states along the proposed path before the usual accept / resample rule; only accepted tokens (and the one that
        ends the round) are committed to the grammar (constraints.rs: fork / rollback for speculation). Returns
        (tokens, finish_reason)."""
        from ..ops.sampling import sample_ref

        if self.t_hybrid or self.d_hybrid:
            raise NotImplementedError("grammar-constrained speculation covers attention-only target and draft models")
        sp = sampling or SamplingParams(temperature=0.0)
        k = self.k
        V = self.t.cfg.vocab_size
        tseq = self.t.new_sequence(prompt, sp, max_new_tokens + k + 2, eos_ids)
        dseq = self.d.new_sequence(prompt, sp, max_new_tokens + k + 2, eos_ids)
        out: list[int] = []
        reason = "max_tokens"

        def masked(logits_row, position):
            allow = constraint.allow_mask(V)
            for e in eos_ids:
                allow[e] = constraint.is_accepting()
            return sample_ref(logits_row.float().cpu(), sp, position, allow=allow, stream=tseq.seq_id)

        def emit(tok) -> bool:
            """Commit one token everywhere; True when generation ends with it."""
            nonlocal reason
            if tok in eos_ids:
                reason = "eos"
                return True
            constraint.commit(tok)
            out.append(tok)
            early = on_token(tok) if on_token is not None else None
            if early:
                reason = early
                return True
            if constraint.is_complete():
                reason = "grammar_complete"
                return True
            return len(out) >= max_new_tokens

        try:
            logits = self.t.prefill_logits([tseq])[0]
            self.d.prefill_logits([dseq])
            tok, _ = masked(logits, len(prompt))
            done = emit(tok)
            pending = [tok]                       # committed tokens the draft has not seen
            while not done:
                base = tseq.kv_len + 1            # position of the first proposal; `out[-1]` is the target's next input
                drafted, q_rows, masks = [], [], []
                feed = pending
                draft_len = dseq.kv_len
                ahead = constraint.fork()         # the proposals advance a copy: a finished or refused path costs nothing

                def ahead_mask():
                    allow = ahead.allow_mask(V)
                    for e in eos_ids:
                        allow[e] = ahead.is_accepting()
                    return allow

                for j in range(k):
                    lg = self._multi_token_step(self.d, [dseq], [feed], all_rows=False, uniform=False)[0]
                    dseq.kv_len += len(feed)
                    allow = ahead_mask()
                    d_tok, q = sample_ref(lg.float().cpu(), sp, base + j, allow=allow, stream=tseq.seq_id)
                    if d_tok in eos_ids:
                        break                     # the draft wants to stop: let the target decide at this row
                    masks.append(allow)
                    drafted.append(d_tok)
                    q_rows.append(q)
                    ahead.commit(d_tok)
                    feed = [d_tok]
                    if ahead.is_complete():
                        break
                n = len(drafted)
                # state after every proposal: masks the bonus row (nothing but the end is legal after a finished grammar)
                tail = ahead_mask() if not (n and ahead.is_complete()) else masks[-1].new_zeros(V)
                lg_t = self._multi_token_step(self.t, [tseq], [[out[-1]] + drafted], all_rows=True, uniform=False)
                p_rows = [sample_ref(lg_t[j].float().cpu(), sp, base + j, allow=(masks + [tail])[j], stream=tseq.seq_id)[1]
                          for j in range(n + 1)]
                if n:
                    a, nxt = ops.verify_ref(torch.stack(p_rows), torch.stack(q_rows), drafted, sp.seed, tseq.seq_id, base)
                else:
                    a, nxt = 0, sample_ref(lg_t[0].float().cpu(), sp, base, allow=tail, stream=tseq.seq_id)[0]
                if a == n and n:
                    nxt = sample_ref(lg_t[n].float().cpu(), sp, base + n, allow=tail, stream=tseq.seq_id)[0]
                tseq.kv_len += 1 + a
                fed = dseq.kv_len - draft_len - len(pending)              # proposals the draft itself has consumed
                keep = min(a, fed)
                dseq.kv_len = draft_len + len(pending) + keep
                pending = drafted[keep:a] + [nxt]
                self.stats.rounds += 1
                self.stats.proposed += n
                self.stats.accepted += a
                self.stats.emitted += a + 1
                for tok in drafted[:a] + [nxt]:
                    done = emit(tok)
                    if done:
                        break
            return out, reason
        finally:
            self.t.release(tseq)
            self.d.release(dseq)

    # ---- the three places where an embedded prediction head differs from an external draft model
    def _prefill(self, tseqs, dseqs) -> list:
        first = self.t.prefill(tseqs).tolist()
        self.d.prefill(dseqs)  # the draft's own first sample is discarded: the target decides
        return first

    def _propose(self, tseqs, dseqs, live, pending, sp, base):
        """k proposals per sequence. Returns (drafted [B][k], draft distributions [k] of [B, V], context for _settle)."""
        k, B = self.k, len(tseqs)
        drafted = [[] for _ in range(B)]
        p_d = []
        d_snaps = []                          # hybrid draft: state after each draft step
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
            if self.d_hybrid:
                d_snaps.append([self.d.snapshot_state(s) for s in dseqs])
            probs, toks = self._probs_and_tokens(self.d, logits, [sp] * B, [base[b] + j for b in range(B)],
                                                 [s.seq_id for s in tseqs])
            p_d.append(probs)
            for b, t in enumerate(toks.tolist()):
                drafted[b].append(int(t))
        return drafted, p_d, d_snaps

    def _verify_forward(self, tseqs, feed):
        return self._multi_token_step(self.t, tseqs, feed, all_rows=True, uniform=True)  # [B*(k+1), V]

    def _settle(self, b, i, a, nxt, dseqs, drafted, pending, ctx):
        """Draft-side bookkeeping of sequence b (request i) after ``a`` proposals were accepted and ``nxt`` ended the round."""
        k = self.k
        if self.d_hybrid:
            self.d.restore_state(dseqs[b], ctx[min(a, k - 1)][b])
        d_valid = dseqs[b].kv_len - (k - 1) + min(a, k - 1)   # draft cache holds last, d_1..d_{k-1}
        dseqs[b].kv_len = d_valid
        pending[i] = ([drafted[b][k - 1]] if a == k else []) + [nxt]

    def _round(self, tseqs, dseqs, live, outs, pending, last, sp):
        k = self.k
        B = len(tseqs)
        V = self.t.cfg.vocab_size
        dev = self.t.device
        sync = (lambda: torch.cuda.synchronize(dev)) if self.cuda else (lambda: None)
        t0 = time.perf_counter()
        # ---- draft: k proposals per sequence
        base = [s.kv_len + 1 for s in tseqs]  # position of the first drafted token (target kv_len = position of `last`)
        drafted, p_d, dctx = self._propose(tseqs, dseqs, live, pending, sp, base)
        sync()
        t1 = time.perf_counter()
        # ---- target: one pass over [last, d_1 .. d_k]
        feed = [[last[i]] + drafted[b] for b, i in enumerate(live)]
        t_snaps = [self.t.snapshot_state(s) for s in tseqs] if self.t_hybrid else None
        logits = self._verify_forward(tseqs, feed)
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
        if self.t_hybrid:
            # the verify pass pushed all k+1 tokens through the recurrent layers: where fewer were accepted, go back and
            # feed only those (their K/V rows are rewritten with the same values)
            redo = [b for b in range(B) if int(res[b][0]) < k]
            if redo:
                for b in redo:
                    self.t.restore_state(tseqs[b], t_snaps[b])
                self._multi_token_step(self.t, [tseqs[b] for b in redo], [feed[b][:1 + int(res[b][0])] for b in redo],
                                       all_rows=False, uniform=False)
        for b, i in enumerate(live):
            a, nxt = int(res[b][0]), int(res[b][1])
            if a == k:
                nxt = int(bonus[b])
            outs[i].extend(drafted[b][:a] + [nxt])
            tseqs[b].kv_len += 1 + a                      # `last` and the accepted drafts are now cached
            self._settle(b, i, a, nxt, dseqs, drafted, pending, dctx)
            last[i] = nxt
            self.stats.accepted += a
            self.stats.emitted += a + 1
            self.stats.full_accept_rounds += 1 if a == k else 0
        self.stats.rounds += B  # one verify step per live sequence
        self.stats.proposed += k * B
        self.stats.draft_ms.append((t1 - t0) * 1e3)
        self.stats.verify_ms.append((t2 - t1) * 1e3)


class EmbeddedMtpDecoder(SpeculativeDecoder):
    """Speculative decoding with the checkpoint's own prediction layer as the drafter (``generate_prepared_chat_mtp``,
    eredu/src/api/loaded.rs:238; executor eredu/src/backend/mlx/speculative/embedded.rs). The head model is a one-layer
    engine next to the target; every draft row pairs a token with the hidden state of the position before it:

    * prefill: the target keeps the hidden states of the prompt; the head's cache is filled from ``(h_i, t_{i+1})``;
    * a round's first draft step feeds the accepted tokens of the previous round with the TARGET's hidden states from
      the verify pass (the head's cache holds exact rows only), further steps chain the head's own output;
    * the verify pass keeps its hidden states for the next round.

    The head's cache entry for ``(h_i, t_{i+1})`` sits at position i, one behind the target's position of the token."""

    def __init__(self, target: Engine, mtp, k: int = 3):
        draft = Engine(mtp.model, max_batch=target.max_batch, max_seq_len=target.max_seq_len, use_cuda_graph=False)
        super().__init__(target, draft, k)
        self.mtp = mtp
        self._pending_hidden: dict = {}      # target seq_id -> [len(pending), H] hidden rows that pair with `pending`
        self._verify_hidden = None

    def _capture(self, store: dict):
        def prepare(batch):
            batch.capture_hidden = True
            store["batch"] = batch
        return prepare

    def _head_step(self, dseqs, tokens, hidden_rows, store, uniform):
        """One pass of the head over ``tokens`` paired with ``hidden_rows`` (flat, same order). Logits of the last row of
        every sequence; the head's output hidden states land in ``store``."""
        def prepare(batch):
            batch.hidden_in = self.mtp.fuse(batch.token_ids, hidden_rows)
            batch.capture_hidden = True
            store["batch"] = batch
        return self._multi_token_step(self.d, dseqs, tokens, all_rows=False, uniform=uniform, prepare=prepare)

    def _prefill(self, tseqs, dseqs) -> list:
        prompts = [list(s.prompt) for s in tseqs]
        cap: dict = {}
        logits = self._multi_token_step(self.t, tseqs, prompts, all_rows=False, uniform=False, prepare=self._capture(cap))
        hidden = cap["batch"].hidden_out
        for s, p in zip(tseqs, prompts):
            s.kv_len = len(p)
        sps = [s.sampling for s in tseqs]
        _, toks = self._probs_and_tokens(self.t, logits, sps, [len(p) for p in prompts], [s.seq_id for s in tseqs])
        first = [int(t) for t in toks.tolist()]
        # head cache: rows (h_i, t_{i+1}) for i < n - 1; the row (h_{n-1}, first) opens the first round
        off, feed, rows = 0, [], []
        for p in prompts:
            feed.append(p[1:])
            rows.append(hidden[off:off + len(p) - 1])
            off += len(p)
        if any(feed):
            live = [i for i, f in enumerate(feed) if f]
            self._head_step([dseqs[i] for i in live], [feed[i] for i in live], torch.cat([rows[i] for i in live]), {}, False)
            for i in live:
                dseqs[i].kv_len += len(feed[i])
        off = 0
        for s, p in zip(tseqs, prompts):
            off += len(p)
            self._pending_hidden[s.seq_id] = hidden[off - 1:off].clone()
        return first

    def _propose(self, tseqs, dseqs, live, pending, sp, base):
        k, B = self.k, len(tseqs)
        drafted = [[] for _ in range(B)]
        p_d = []
        chain = None
        for j in range(k):
            store: dict = {}
            if j == 0:
                feed = [pending[i] for i in live]
                rows = torch.cat([self._pending_hidden[s.seq_id] for s in tseqs])
                logits = self._head_step(dseqs, feed, rows, store, uniform=False)
                for s, f in zip(dseqs, feed):
                    s.kv_len += len(f)
                ends = np.cumsum([len(f) for f in feed]) - 1
                chain = store["batch"].hidden_out.index_select(0, self.d._t(ends.astype(np.int64), torch.int64))
            else:
                feed = [[drafted[b][-1]] for b in range(B)]
                logits = self._head_step(dseqs, feed, chain, store, uniform=True)
                for s in dseqs:
                    s.kv_len += 1
                chain = store["batch"].hidden_out
            probs, toks = self._probs_and_tokens(self.d, logits, [sp] * B, [base[b] + j for b in range(B)],
                                                 [s.seq_id for s in tseqs])
            p_d.append(probs)
            for b, t in enumerate(toks.tolist()):
                drafted[b].append(int(t))
        self._last_chain = chain              # pairs with d_k: where an optimistic continuation picks up
        # the head's cache is exact up to the row that paired with the newest committed token; later rows were made from
        # chained hidden states and are rewritten from the target's after the verify pass
        return drafted, p_d, [s.kv_len - (k - 1) for s in dseqs]

    def _verify_forward(self, tseqs, feed):
        cap: dict = {}
        logits = self._multi_token_step(self.t, tseqs, feed, all_rows=True, uniform=True, prepare=self._capture(cap))
        self._verify_hidden = cap["batch"].hidden_out.view(len(tseqs), self.k + 1, -1)
        return logits

    def _settle(self, b, i, a, nxt, dseqs, drafted, pending, ctx):
        dseqs[b].kv_len = ctx[b]
        pending[i] = drafted[b][:a] + [nxt]
        # row j of the verify pass is the hidden state behind its (j+1)-th output: d_1 pairs with row 0, ..., nxt with row a
        self._pending_hidden[self._seq_ids[b]] = self._verify_hidden[b, :a + 1].clone()

    def _round(self, tseqs, dseqs, live, outs, pending, last, sp):
        self._seq_ids = [s.seq_id for s in tseqs]
        super()._round(tseqs, dseqs, live, outs, pending, last, sp)


class _NoDraftEngine:
    """Stands where a draft engine would for drafters that keep no cache of their own."""

    class _Seq:
        kv_len = 0

    class _Kv:
        @staticmethod
        def has_recurrent_state():
            return False

    def __init__(self, cfg):
        self.cfg, self.kv = cfg, self._Kv()

    def new_sequence(self, *a, **k):
        return self._Seq()

    def release(self, seq):
        pass


class Gemma4AssistantDecoder(SpeculativeDecoder):
    """Speculative decoding with a Gemma 4 assistant (eredu/src/backend/mlx/architectures/gemma4/mtp.rs): the drafter has
    no cache, it reads the K / V the target committed. Per request the decoder keeps the target's pre-norm hidden state of
    the newest cached token; a round's first draft step pairs it with the newest token, later steps chain the drafter's
    own projection. The verify pass keeps its hidden states, and row ``accepted`` becomes the next round's state."""

    carries_verify_hidden = True
    supports_lookahead = False

    def __init__(self, target: Engine, assistant, k: Optional[int] = None):
        k = min(k or assistant.max_proposals, assistant.max_proposals)
        super().__init__(target, _NoDraftEngine(target.cfg), k)
        self.assistant = assistant
        self._pending_hidden: dict = {}
        self._verify_hidden = None
        self._last_chain = None

    def _capture(self, store: dict):
        def prepare(batch):
            batch.capture_hidden = True
            store["batch"] = batch
        return prepare

    def _prefill(self, tseqs, dseqs) -> list:
        prompts = [list(s.prompt) for s in tseqs]
        cap: dict = {}
        logits = self._multi_token_step(self.t, tseqs, prompts, all_rows=False, uniform=False, prepare=self._capture(cap))
        hidden = cap["batch"].hidden_out
        ends = np.cumsum([len(p) for p in prompts]) - 1
        for s, p, e in zip(tseqs, prompts, ends):
            s.kv_len = len(p)
            self._pending_hidden[s.seq_id] = hidden[int(e):int(e) + 1].clone()
        _, toks = self._probs_and_tokens(self.t, logits, [s.sampling for s in tseqs], [len(p) for p in prompts],
                                         [s.seq_id for s in tseqs])
        return [int(t) for t in toks.tolist()]

    def _propose(self, tseqs, dseqs, live, pending, sp, base):
        k, B = self.k, len(tseqs)
        eng = self.t
        drafted = [[] for _ in range(B)]
        p_d = []
        hidden = torch.cat([self._pending_hidden[s.seq_id] for s in tseqs])
        tokens = eng._t(np.asarray([pending[i][-1] for i in live], dtype=np.int64), torch.int64)
        block_table = eng._block_table(tseqs)
        cache_lens = eng._t(np.asarray([s.kv_len for s in tseqs], dtype=np.int64), torch.int64)
        for j in range(k):
            logits, hidden = self.assistant.draft_step(tokens, hidden, eng.kv, block_table, cache_lens, j)
            probs, toks = self._probs_and_tokens(eng, logits, [sp] * B, [base[b] + j for b in range(B)],
                                                 [s.seq_id for s in tseqs])
            p_d.append(probs)
            tokens = toks.to(torch.int64)
            for b, t in enumerate(toks.tolist()):
                drafted[b].append(int(t))
        return drafted, p_d, None

    def _verify_forward(self, tseqs, feed):
        cap: dict = {}
        logits = self._multi_token_step(self.t, tseqs, feed, all_rows=True, uniform=True, prepare=self._capture(cap))
        self._verify_hidden = cap["batch"].hidden_out.view(len(tseqs), self.k + 1, -1)
        return logits

    def _settle(self, b, i, a, nxt, dseqs, drafted, pending, ctx):
        pending[i] = [nxt]
        # row j of the verify pass belongs to its j-th input: `last`, d_1 .. d_k; the newest cached token is input `a`
        self._pending_hidden[self._seq_ids[b]] = self._verify_hidden[b, a:a + 1].clone()

    def _round(self, tseqs, dseqs, live, outs, pending, last, sp):
        self._seq_ids = [s.seq_id for s in tseqs]
        super()._round(tseqs, dseqs, live, outs, pending, last, sp)


class DFlashDecoder(SpeculativeDecoder):
    """Speculative decoding with a DFlash block drafter (eredu/src/backend/mlx/architectures/muse_glimmer/mtp.rs): the
    target's passes keep the outputs of the drafter's ``target_layer_ids`` for every token they feed; per request the
    decoder holds the drafter's encoded context and the states of tokens that were committed since it was last extended.
    A round extends the context, runs ONE drafter pass over ``[newest token, mask x k]`` and reads all k proposal
    distributions from it through the target's head; the verify pass is the usual one."""

    carries_verify_hidden = True
    supports_lookahead = False

    def __init__(self, target: Engine, dflash, k: Optional[int] = None):
        k = min(k or dflash.max_proposals, dflash.max_proposals)
        super().__init__(target, _NoDraftEngine(target.cfg), k)
        if dflash.cfg.hidden_size != target.cfg.hidden_size:
            raise ValueError("the drafter's width differs from the target's")
        if max(dflash.cfg.target_layer_ids) >= target.cfg.num_hidden_layers:
            raise ValueError("the drafter conditions on layers the target does not have")
        self.dflash = dflash
        self.ids = tuple(dflash.cfg.target_layer_ids)
        self._ctx: dict = {}                 # seq_id -> DFlashContext
        self._pending_hidden: dict = {}      # seq_id -> [n, H * layers] states of committed tokens not yet in the context
        self._verify_hidden = None
        self._last_chain = None

    def _capture(self, store: dict):
        def prepare(batch):
            batch.capture_layers = self.ids
            store["batch"] = batch
        return prepare

    def _states(self, batch):
        return torch.cat([batch.layer_hidden[i] for i in self.ids], -1)

    def _prefill(self, tseqs, dseqs) -> list:
        from ..models.dflash import DFlashContext

        prompts = [list(s.prompt) for s in tseqs]
        cap: dict = {}
        logits = self._multi_token_step(self.t, tseqs, prompts, all_rows=False, uniform=False, prepare=self._capture(cap))
        states = self._states(cap["batch"])
        off = 0
        for s, p in zip(tseqs, prompts):
            s.kv_len = len(p)
            self._ctx[s.seq_id] = DFlashContext()
            self._pending_hidden[s.seq_id] = states[off:off + len(p)].clone()
            off += len(p)
        _, toks = self._probs_and_tokens(self.t, logits, [s.sampling for s in tseqs], [len(p) for p in prompts],
                                         [s.seq_id for s in tseqs])
        return [int(t) for t in toks.tolist()]

    def _propose(self, tseqs, dseqs, live, pending, sp, base):
        k, B = self.k, len(tseqs)
        eng = self.t
        model = eng.model
        rows = []
        for b, s in enumerate(tseqs):
            ctx = self.dflash.extend_context(self._ctx[s.seq_id], self._pending_hidden[s.seq_id], s.kv_len)
            self._ctx[s.seq_id] = ctx
            self._pending_hidden[s.seq_id] = self._pending_hidden[s.seq_id][:0]
            ids = torch.tensor([pending[live[b]][-1]] + [self.dflash.cfg.mask_token_id] * k, device=eng.device)
            rows.append(self.dflash.propose(model.embed[ids.long()], ctx))            # [k, H]
        # the proposal states carry the drafter's own final norm: they go through the target's output head and logit
        # scaling only, not through the target's final norm
        logits = ops.linear(torch.cat(rows).to(model.dtype).contiguous(), model.lm_head, out_dtype=torch.float32)
        mg = eng.cfg.extra.get("muse_glimmer")
        if mg:
            cap, mult = float(mg["final_logit_softcapping"]), float(mg["output_multiplier"])
            logits = torch.tanh(logits * (mult / cap)) * cap
        logits = logits.view(B, k, -1)
        drafted = [[] for _ in range(B)]
        p_d = []
        for j in range(k):
            probs, toks = self._probs_and_tokens(eng, logits[:, j].contiguous(), [sp] * B, [base[b] + j for b in range(B)],
                                                 [s.seq_id for s in tseqs])
            p_d.append(probs)
            for b, t in enumerate(toks.tolist()):
                drafted[b].append(int(t))
        return drafted, p_d, None

    def _verify_forward(self, tseqs, feed):
        cap: dict = {}
        logits = self._multi_token_step(self.t, tseqs, feed, all_rows=True, uniform=True, prepare=self._capture(cap))
        self._verify_hidden = self._states(cap["batch"]).view(len(tseqs), self.k + 1, -1)
        return logits

    def _settle(self, b, i, a, nxt, dseqs, drafted, pending, ctx):
        pending[i] = [nxt]
        # the verify pass fed `last`, d_1 .. d_k: inputs 0 .. a are now cached, their states join the context next round
        self._pending_hidden[self._seq_ids[b]] = self._verify_hidden[b, :a + 1].clone()

    def _round(self, tseqs, dseqs, live, outs, pending, last, sp):
        self._seq_ids = [s.seq_id for s in tseqs]
        super()._round(tseqs, dseqs, live, outs, pending, last, sp)


class GraphSpeculativeDecoder(SpeculativeDecoder):
    """The speculative round as ONE CUDA graph (GPU only, fixed batch): k draft steps, the target's verify pass over
    k+1 tokens, both samplers and the accept / resample kernel are captured once; a round is a few small
    host-to-device copies (positions, the two newest tokens, sampler rows), one replay and one read-back.

    Uniform shapes come from always feeding the draft TWO tokens in its first step - the token before ``last`` and
    ``last`` itself. Whatever the previous round accepted, the draft cache is valid up to the token before that, so
    the first of the two is at worst recomputed into the slot it already occupies; no ragged catch-up pass exists.
    Sequences that finish early stay in the batch (their slots keep cycling over reserved pages) and are ignored.
    """

    def __init__(self, target: Engine, draft: Engine, k: int = 4):
        if target.cfg.is_hybrid or draft.cfg.is_hybrid:
            # rejected proposals would have to be rolled out of the recurrent convolution state as well
            raise NotImplementedError("speculative decoding is not available for hybrid (convolution-state) models")
        super().__init__(target, draft, k)
        if not self.cuda:
            raise RuntimeError("GraphSpeculativeDecoder needs CUDA engines; use SpeculativeDecoder on the CPU")
        self._state = None

    @staticmethod
    def _slots_dev(bt: torch.Tensor, pos: torch.Tensor, per: int) -> torch.Tensor:
        """KV slot of every (sequence, position): bt [B, max_pages] int32, pos [B * per] int32 -> int64 [B * per]."""
        B = bt.shape[0]
        p = pos.view(B, per).long()
        page = bt.long().gather(1, p // PAGE)
        return (page * PAGE + p % PAGE).view(-1)

    def _build(self, tseqs, dseqs, sp):
        t, d, k = self.t, self.d, self.k
        B, V, dev = len(tseqs), t.cfg.vocab_size, t.device
        max_len = max(len(s.prompt) + s.max_new_tokens for s in tseqs)
        i32 = dict(dtype=torch.int32, device=dev)
        st = {
            "B": B, "P": torch.zeros(B, **i32), "prev": torch.zeros(B, **i32), "last": torch.zeros(B, **i32),
            "t_bt": t._block_table(tseqs), "d_bt": d._block_table(dseqs),
            "d_rows": torch.zeros((k, B, ROW_DTYPE.itemsize), dtype=torch.uint8, device=dev),
            "t_rows": torch.zeros((B * (k + 1), ROW_DTYPE.itemsize), dtype=torch.uint8, device=dev),
            "v_rows": torch.zeros((B, ROW_DTYPE.itemsize), dtype=torch.uint8, device=dev),
            "p_d": torch.empty((k, B, V), dtype=torch.float32, device=dev),
            "p_t": torch.empty((B * (k + 1), V), dtype=torch.float32, device=dev),
            "res": torch.zeros((B, 2), **i32), "drafted": torch.zeros((B, k), **i32), "bonus": torch.zeros(B, **i32),
            "rows2": torch.arange(B, device=dev, dtype=torch.int64) * 2 + 1,
            "ar": torch.arange(k + 1, **i32),
            "all_greedy": sp.greedy, "graph": None,
        }
        for name, eng, q in (("d2", d, 2), ("d1", d, 1), ("tv", t, k + 1)):
            splits = ops.decode_splits(B, eng.model.n_kv_local, max_len + k + 2, eng.sm_count)
            st[name + "_splits"] = splits
            st[name + "_scratch"] = (ops.decode_scratch(B, q, eng.model.n_q_local, eng.cfg.head_dim, splits, dev)
                                     if splits > 1 else None)
        st["host"] = {n: torch.zeros(B, dtype=torch.int32).pin_memory() for n in ("P", "prev", "last")}
        st["host_res"] = torch.zeros((B, 2), dtype=torch.int32).pin_memory()
        st["host_drafted"] = torch.zeros((B, k), dtype=torch.int32).pin_memory()
        st["host_bonus"] = torch.zeros(B, dtype=torch.int32).pin_memory()
        return st

    def _device_round(self, st):
        t, d, k, B = self.t, self.d, self.k, st["B"]
        V = t.cfg.vocab_size
        P, prev, last = st["P"], st["prev"], st["last"]
        greedy = st["all_greedy"]
        # ---- draft step 0: [token before last, last] at positions [P-1, P]
        tok = torch.stack((prev, last), 1).reshape(-1)
        pos = torch.stack((P - 1, P), 1).reshape(-1)
        batch = ForwardBatch(token_ids=tok, positions=pos, slots=self._slots_dev(st["d_bt"], pos, 2), block_table=st["d_bt"],
                             seq_lens=P + 1, is_prefill=False, q_per_seq=2, splits=st["d2_splits"],
                             scratch=st["d2_scratch"], logit_rows=st["rows2"])
        logits = d.model.forward(batch, d.kv)
        cur = ops.sample(logits.contiguous(), st["d_rows"][0], probs=st["p_d"][0], all_greedy=greedy)
        toks = [cur]
        for j in range(1, k):
            pos = P + j
            batch = ForwardBatch(token_ids=cur, positions=pos, slots=self._slots_dev(st["d_bt"], pos, 1),
                                 block_table=st["d_bt"], seq_lens=P + 1 + j, is_prefill=False, q_per_seq=1,
                                 splits=st["d1_splits"], scratch=st["d1_scratch"])
            logits = d.model.forward(batch, d.kv)
            cur = ops.sample(logits.contiguous(), st["d_rows"][j], probs=st["p_d"][j], all_greedy=greedy)
            toks.append(cur)
        drafted = torch.stack(toks, 1).to(torch.int32)
        st["drafted"].copy_(drafted)
        # ---- target: one pass over [last, d_1 .. d_k] at positions P .. P+k
        tok = torch.cat((last[:, None], drafted), 1).reshape(-1)
        pos = (P[:, None] + st["ar"][None, :]).reshape(-1)
        batch = ForwardBatch(token_ids=tok, positions=pos, slots=self._slots_dev(st["t_bt"], pos, k + 1), block_table=st["t_bt"],
                             seq_lens=P + k + 1, is_prefill=False, q_per_seq=k + 1, splits=st["tv_splits"],
                             scratch=st["tv_scratch"])
        logits = t.model.forward(batch, t.kv)
        t_toks = ops.sample(logits.contiguous(), st["t_rows"], probs=st["p_t"], all_greedy=greedy)
        st["bonus"].copy_(t_toks.view(B, k + 1)[:, k])
        p_d3 = st["p_d"].permute(1, 0, 2).contiguous()
        ops.spec_verify(st["p_t"].view(B, k + 1, V), p_d3, st["drafted"], st["v_rows"], out=st["res"])

    @torch.no_grad()
    def generate(self, prompts, sampling: Optional[SamplingParams] = None, max_new_tokens: int = 64, eos_ids=()):
        sp = sampling or SamplingParams()
        k, t, d = self.k, self.t, self.d
        B = len(prompts)
        tseqs = [t.new_sequence(p, sp, max_new_tokens + k + 2, eos_ids) for p in prompts]
        dseqs = [d.new_sequence(p, sp, max_new_tokens + k + 2, eos_ids) for p in prompts]
        try:
            t_start = time.perf_counter()
            first = [int(x) for x in t.prefill(tseqs).tolist()]
            d.prefill(dseqs)
            torch.cuda.synchronize(t.device)
            self.stats.prefill_ms = (time.perf_counter() - t_start) * 1e3
            outs = [[x] for x in first]
            last = list(first)
            prev = [int(p[-1]) for p in prompts]
            P = [len(p) for p in prompts]             # position of `last`; the target cache holds 0 .. P-1
            done = [x in eos_ids or max_new_tokens <= 1 for x in first]
            st = self._build(tseqs, dseqs, sp)
            dev = t.device
            sids = [s.seq_id for s in tseqs]
            while not all(done):
                t0 = time.perf_counter()
                base = [p + 1 for p in P]
                for name, vals in (("P", P), ("prev", prev), ("last", last)):
                    st["host"][name].copy_(torch.as_tensor(vals, dtype=torch.int32))
                    st[name].copy_(st["host"][name], non_blocking=True)
                d_rows = np.stack([pack_rows([sp] * B, [b + j for b in base], stream_ids=sids).view(np.uint8)
                                   .reshape(B, ROW_DTYPE.itemsize) for j in range(k)])
                st["d_rows"].copy_(t._t(d_rows, torch.uint8))
                t_rows = pack_rows([sp] * (B * (k + 1)), [b + j for b in base for j in range(k + 1)],
                                   stream_ids=[s for s in sids for _ in range(k + 1)])
                st["t_rows"].copy_(t._t(t_rows.view(np.uint8).reshape(B * (k + 1), ROW_DTYPE.itemsize), torch.uint8))
                v_rows = pack_rows([sp] * B, base, stream_ids=sids)
                st["v_rows"].copy_(t._t(v_rows.view(np.uint8).reshape(B, ROW_DTYPE.itemsize), torch.uint8))
                if st["graph"] is None:
                    # eager warm-up (kernel attribute setup; it rewrites the same KV slots the replay will), then capture
                    side = torch.cuda.Stream(device=dev)
                    side.wait_stream(torch.cuda.current_stream(dev))
                    with torch.cuda.stream(side):
                        self._device_round(st)
                    torch.cuda.current_stream(dev).wait_stream(side)
                    torch.cuda.synchronize(dev)
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        self._device_round(st)
                    st["graph"] = g
                st["graph"].replay()
                st["host_res"].copy_(st["res"], non_blocking=True)
                st["host_drafted"].copy_(st["drafted"], non_blocking=True)
                st["host_bonus"].copy_(st["bonus"], non_blocking=True)
                torch.cuda.current_stream(dev).synchronize()
                res, drafted, bonus = st["host_res"].tolist(), st["host_drafted"].tolist(), st["host_bonus"].tolist()
                live = 0
                for b in range(B):
                    if done[b]:
                        continue
                    live += 1
                    a, nxt = int(res[b][0]), int(res[b][1])
                    if a == k:
                        nxt = int(bonus[b])
                    new = drafted[b][:a] + [nxt]
                    outs[b].extend(new)
                    seq_tokens = [last[b]] + new
                    prev[b] = seq_tokens[-2]
                    last[b] = nxt
                    P[b] += a + 1
                    self.stats.accepted += a
                    self.stats.emitted += a + 1
                    self.stats.full_accept_rounds += 1 if a == k else 0
                    if len(outs[b]) >= max_new_tokens:
                        outs[b] = outs[b][:max_new_tokens]
                        done[b] = True
                    for j, tok in enumerate(outs[b]):
                        if tok in eos_ids:
                            outs[b] = outs[b][: j + 1]
                            done[b] = True
                            break
                self.stats.rounds += live
                self.stats.proposed += k * live
                self.stats.verify_ms.append((time.perf_counter() - t0) * 1e3)   # the whole captured round
            ops.native.check_status(dev)
            return outs
        finally:
            for s in tseqs:
                t.release(s)
            for s in dseqs:
                d.release(s)
