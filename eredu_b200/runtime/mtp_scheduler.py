"""Fair scheduler for speculative (multi-token-prediction) requests with optimistic lookahead.

The counterpart of ``MlxMtpScheduler`` (eredu/src/backend/mlx/speculative/scheduler.rs:240-487) with the portable
options and counters of eredu-core/src/generation.rs:376-470 and eredu-core/src/speculative.rs:194-289. Requests
progress independently through explicit phases; one scheduler operation advances one request by one phase, visiting
the requests round-robin:

    Prefill -> ReadyToDraft -> ReadyToSubmitVerification -> TargetVerificationInFlight
            -> (OptimisticDraftInProgress -> OptimisticDraftReady) -> VerificationResolution -> ReadyToDraft | Completed

* The target's verification pass is *submitted*, not awaited: its kernels (forward, sampling, the accept / reject kernel)
  are enqueued on the target stream and an event marks their end. The host reads the few result integers only at
  ``VerificationResolution``. Until then the scheduler drafts for other requests (``cross_request_draft_opportunities``)
  on the draft stream, so the two models overlap on the GPU.
* Optimistic lookahead: while a request's own verification is in flight, its drafter assumes that every proposal is
  accepted, guesses the target's bonus token (one more draft step) and drafts the next block behind that guess. When
  the target accepts all proposals and its bonus equals the guess, the block is promoted: the next verification is
  submitted without a drafting phase in between. Otherwise the branch is discarded and the draft cache rolls back by
  length. Outputs never depend on the lookahead: draws are addressed by position, so a promoted block holds exactly
  the tokens that drafting after the resolution would have produced.
* Adaptive lookahead: once ``adaptive_lookahead_min_blocks`` optimistic blocks have been drafted for a request, lookahead
  is switched off for it when nothing was reused or when more optimistic tokens were discarded than reused.

Capacity: at most ``max_in_flight_verifications`` submitted verifications and ``max_optimistic_branches`` retained
optimistic branches exist at any time; a request that finds no capacity waits in its phase.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Optional

import numpy as np
import torch

from .. import ops
from ..ops.sampling import ROW_DTYPE, SamplingParams, pack_rows
from .speculative import EmbeddedMtpDecoder, SpeculativeDecoder
from .streaming import FinishReason


class Phase:
    PREFILL = "prefill"
    READY_TO_DRAFT = "ready_to_draft"
    READY_TO_SUBMIT = "ready_to_submit_verification"
    IN_FLIGHT = "target_verification_in_flight"
    OPTIMISTIC_IN_PROGRESS = "optimistic_draft_in_progress"
    OPTIMISTIC_READY = "optimistic_draft_ready"
    RESOLUTION = "verification_resolution"
    COMPLETED = "completed"
    CANCELLED = "cancelled"


@dataclass(frozen=True)
class MtpSchedulerOptions:
    max_in_flight_verifications: int = 1
    max_optimistic_branches: int = 1
    lookahead_blocks: int = 1            # proposal blocks drafted ahead per request: zero or one
    adaptive_lookahead: bool = True
    adaptive_lookahead_min_blocks: int = 4

    def with_lookahead(self, enabled: bool) -> "MtpSchedulerOptions":
        return MtpSchedulerOptions(self.max_in_flight_verifications, max(self.max_optimistic_branches, 1) if enabled
                                   else self.max_optimistic_branches, int(enabled), self.adaptive_lookahead,
                                   self.adaptive_lookahead_min_blocks)

    def validate(self) -> "MtpSchedulerOptions":
        if self.max_in_flight_verifications < 1:
            raise ValueError("MTP max_in_flight_verifications must be positive")
        if self.lookahead_blocks not in (0, 1):
            raise ValueError("MTP lookahead_blocks must be zero or one")
        if self.lookahead_blocks and self.max_optimistic_branches < 1:
            raise ValueError("MTP lookahead needs optimistic branch capacity")
        if self.lookahead_blocks and self.adaptive_lookahead and self.adaptive_lookahead_min_blocks < 1:
            raise ValueError("MTP adaptive_lookahead_min_blocks must be positive")
        return self


@dataclass
class MtpStats:
    target_tokens: int = 0
    draft_tokens: int = 0
    accepted_tokens: int = 0
    rounds: int = 0
    accept_lens: list = field(default_factory=list)
    emitted_tokens: int = 0
    optimistic_draft_tokens: int = 0
    optimistic_draft_blocks: int = 0
    reused_optimistic_tokens: int = 0
    reused_optimistic_blocks: int = 0
    consumed_optimistic_tokens: int = 0
    discarded_optimistic_tokens: int = 0
    discarded_optimistic_blocks: int = 0
    optimistic_target_bonus_tokens: int = 0
    optimistic_bonus_matches: int = 0
    optimistic_bonus_mismatches: int = 0
    adaptive_lookahead_disabled: bool = False
    optimistic_draft_time: float = 0.0
    verification_in_flight_time: float = 0.0
    scheduler_turns: int = 0
    cross_request_draft_opportunities: int = 0
    elapsed: float = 0.0

    def accept_rate(self) -> float:
        return self.accepted_tokens / self.draft_tokens if self.draft_tokens else 0.0

    def update_adaptive_lookahead(self, options: MtpSchedulerOptions):
        if (not options.adaptive_lookahead or self.adaptive_lookahead_disabled
                or self.optimistic_draft_blocks < options.adaptive_lookahead_min_blocks):
            return
        self.adaptive_lookahead_disabled = (self.reused_optimistic_tokens == 0
                                            or self.reused_optimistic_tokens < self.discarded_optimistic_tokens)


@dataclass
class MtpSchedulerStats:
    turns: int = 0
    cross_request_draft_opportunities: int = 0
    peak_in_flight_verifications: int = 0
    peak_optimistic_branches: int = 0


@dataclass
class MtpRequestOutput:
    id: int
    token_ids: list
    stats: MtpStats
    finish_reason: Optional[str]
    cancelled: bool = False


@dataclass
class MtpScheduleOutput:
    requests: list
    scheduler: MtpSchedulerStats


class _Request:
    def __init__(self, rid, prompt, sampling, max_tokens, eos_ids, on_token, should_cancel):
        self.id = rid
        self.prompt = list(prompt)
        self.sp = sampling
        self.max_tokens = max_tokens
        self.eos = set(int(e) for e in eos_ids)
        self.on_token = on_token
        self.should_cancel = should_cancel
        self.phase = Phase.PREFILL
        self.stats = MtpStats()
        self.tseq = self.dseq = None
        self.out: list = []
        self.published = 0
        self.pending: list = []          # committed tokens that the draft cache misses
        self.last = None                 # leading uncached target input
        self.block = None                # dict(drafted, p_d, ctx, base): proposals ready for submission
        self.flight = None               # dict(res, bonus, event, t0, block): the submitted verification
        self.branch = None               # dict(tokens, p_d, kv_before, ...): the optimistic continuation
        self.carry = None                # embedded heads: tokens / hidden rows behind the head's exact cache prefix
        self.finish_reason = None
        self.cancel_requested = False
        self.t_start = time.perf_counter()


class MtpScheduler:
    """Single-threaded: every method runs on the caller's thread; device work is asynchronous on two CUDA streams."""

    def __init__(self, decoder: SpeculativeDecoder, options: Optional[MtpSchedulerOptions] = None, streams=None):
        self.dec = decoder
        self.options = (options or MtpSchedulerOptions()).validate()
        self.k = decoder.k
        self.cuda = decoder.cuda
        self.embedded = isinstance(decoder, EmbeddedMtpDecoder)
        # decoders whose next round starts from hidden states of the verify pass (embedded heads, cache-less assistants)
        self.keeps_hidden = self.embedded or bool(getattr(decoder, "carries_verify_hidden", False))
        # recurrent drafters would need a state snapshot per optimistic step: their lookahead stays off; so does that of
        # drafters that say they cannot continue past an unverified block
        self.lookahead_possible = (bool(self.options.lookahead_blocks) and not decoder.d_hybrid
                                   and bool(getattr(decoder, "supports_lookahead", True)))
        if self.cuda:
            dev = decoder.t.device
            self.target_stream, self.draft_stream = streams or (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
        else:
            self.target_stream = self.draft_stream = None
        self.requests: list[_Request] = []
        self.stats = MtpSchedulerStats()
        self._cursor = 0

    # ------------------------------------------------------------------------------------------ request table
    def submit(self, prompt, sampling: Optional[SamplingParams] = None, max_tokens: int = 256, eos_ids=(),
               on_token: Optional[Callable[[int], Optional[str]]] = None,
               should_cancel: Optional[Callable[[], bool]] = None) -> int:
        """Registers a request; returns its id (the insertion index). ``on_token(token)`` sees every committed token in
        order; a truthy return value ends the request after that token (kept as its finish reason)."""
        if max_tokens < 1:
            raise ValueError("max_tokens must be positive")
        if not prompt:
            raise ValueError("empty prompt")
        req = _Request(len(self.requests), prompt, sampling or SamplingParams(), max_tokens, eos_ids, on_token, should_cancel)
        extra = 2 * self.k + 4
        req.tseq = self.dec.t.new_sequence(req.prompt, req.sp, max_tokens + extra, eos_ids)
        req.dseq = self.dec.d.new_sequence(req.prompt, req.sp, max_tokens + extra, eos_ids)
        self.requests.append(req)
        return req.id

    def phase(self, rid: int) -> Optional[str]:
        return self.requests[rid].phase if 0 <= rid < len(self.requests) else None

    def cancel(self, rid: int) -> str:
        """"already_terminal", "cancel_now", or "cancel_at_boundary" when a submitted verification has to resolve first
        (its cache effects are rolled back at the resolution; nothing of it is published)."""
        req = self.requests[rid]
        if req.phase in (Phase.COMPLETED, Phase.CANCELLED):
            return "already_terminal"
        if req.flight is None:
            self._finish(req, FinishReason.CANCELLED, cancelled=True)
            return "cancel_now"
        req.cancel_requested = True
        return "cancel_at_boundary"

    def is_finished(self) -> bool:
        return all(r.phase in (Phase.COMPLETED, Phase.CANCELLED) for r in self.requests)

    # ------------------------------------------------------------------------------------------ scheduling
    def _in_flight(self) -> int:
        return sum(1 for r in self.requests if r.flight is not None)

    def _branches(self) -> int:
        return sum(1 for r in self.requests if r.branch is not None)

    def _lookahead_wanted(self, req: _Request) -> bool:
        return (self.lookahead_possible and not req.stats.adaptive_lookahead_disabled and req.branch is None
                and not req.cancel_requested and self._branches() < self.options.max_optimistic_branches
                # a block behind the bonus only matters if the request can still emit it
                and len(req.out) + self.k + 1 < req.max_tokens)

    def step(self) -> bool:
        """One scheduler operation on the next request that can progress. False when every request is terminal."""
        n = len(self.requests)
        if n == 0 or self.is_finished():
            return False
        # round-robin, but a request that only waits for its verification yields to requests with draftable work
        order = [self.requests[(self._cursor + i) % n] for i in range(n)]
        draftable = [r for r in order if r.phase in (Phase.PREFILL, Phase.READY_TO_DRAFT)
                     or (r.phase == Phase.READY_TO_SUBMIT and self._in_flight() < self.options.max_in_flight_verifications)
                     or (r.phase == Phase.IN_FLIGHT and self._lookahead_wanted(r))
                     or r.phase == Phase.OPTIMISTIC_IN_PROGRESS]
        waiting = [r for r in order if r.phase in (Phase.IN_FLIGHT, Phase.OPTIMISTIC_READY, Phase.RESOLUTION)]
        req = draftable[0] if draftable else (waiting[0] if waiting else None)
        if req is None:
            return False
        self._cursor = (req.id + 1) % n
        self.stats.turns += 1
        req.stats.scheduler_turns += 1
        if req.should_cancel is not None and not req.cancel_requested and req.should_cancel():
            if self.cancel(req.id) != "cancel_at_boundary":
                return not self.is_finished()
        self._advance(req)
        self.stats.peak_in_flight_verifications = max(self.stats.peak_in_flight_verifications, self._in_flight())
        self.stats.peak_optimistic_branches = max(self.stats.peak_optimistic_branches, self._branches())
        return not self.is_finished()

    def run(self):
        while self.step():
            pass

    def finish(self) -> MtpScheduleOutput:
        """Drives every request to a terminal phase, releases the caches and returns outputs in submission order."""
        try:
            self.run()
            if self.cuda:
                ops.native.check_status(self.dec.t.device)
        finally:
            for r in self.requests:
                self._release(r)
        return MtpScheduleOutput([MtpRequestOutput(r.id, r.out, r.stats, r.finish_reason, r.phase == Phase.CANCELLED)
                                  for r in self.requests], self.stats)

    # ------------------------------------------------------------------------------------------ phases
    def _advance(self, req: _Request):
        p = req.phase
        if p == Phase.PREFILL:
            self._prefill(req)
        elif p == Phase.READY_TO_DRAFT:
            if any(r.flight is not None for r in self.requests if r is not req):
                self.stats.cross_request_draft_opportunities += 1
                req.stats.cross_request_draft_opportunities += 1
            self._draft(req)
        elif p == Phase.READY_TO_SUBMIT:
            self._submit_verification(req)
        elif p == Phase.IN_FLIGHT:
            if self._lookahead_wanted(req):
                req.phase = Phase.OPTIMISTIC_IN_PROGRESS
                self._optimistic(req)
            else:
                req.phase = Phase.RESOLUTION
                self._resolve(req)
        elif p == Phase.OPTIMISTIC_IN_PROGRESS:
            self._optimistic(req)
        elif p in (Phase.OPTIMISTIC_READY, Phase.RESOLUTION):
            req.phase = Phase.RESOLUTION
            self._resolve(req)

    def _on(self, stream):
        return torch.cuda.stream(stream) if self.cuda else _Null()

    def _prefill(self, req: _Request):
        with torch.no_grad(), self._on(self.target_stream):
            t0 = time.perf_counter()
            first = int(self.dec._prefill([req.tseq], [req.dseq])[0])
            if self.cuda:
                torch.cuda.current_stream().synchronize()
            self.dec.stats.prefill_ms += (time.perf_counter() - t0) * 1e3
        req.stats.target_tokens += len(req.prompt)
        req.pending = [first]
        req.last = first
        self._commit(req, [first])
        if req.phase == Phase.PREFILL:
            req.phase = Phase.READY_TO_DRAFT

    def _draft(self, req: _Request):
        base = req.tseq.kv_len + 1
        with torch.no_grad(), self._on(self.draft_stream):
            if self.keeps_hidden:
                self.dec._seq_ids = [req.tseq.seq_id]
            pend = {0: req.pending}
            drafted, p_d, ctx = self.dec._propose([req.tseq], [req.dseq], [0], pend, req.sp, [base])
            done = torch.cuda.Event() if self.cuda else None
            if done is not None:
                done.record()
        req.block = {"drafted": drafted[0], "p_d": p_d, "ctx": ctx, "base": base, "done": done,
                     "chain": self.dec._last_chain if self.embedded else None}
        req.stats.draft_tokens += self.k
        req.phase = Phase.READY_TO_SUBMIT

    def _submit_verification(self, req: _Request):
        """Enqueue the target pass over [last, d_1 .. d_k], the sampling of its k + 1 rows and the accept / reject kernel.
        Nothing is read back here."""
        k, blk = self.k, req.block
        dec, V = self.dec, self.dec.t.cfg.vocab_size
        with torch.no_grad(), self._on(self.target_stream):
            if blk["done"] is not None:
                torch.cuda.current_stream().wait_event(blk["done"])      # the draft distributions come from the other stream
            if self.keeps_hidden:
                dec._seq_ids = [req.tseq.seq_id]
            feed = [[req.last] + blk["drafted"]]
            snap = dec.t.snapshot_state(req.tseq) if dec.t_hybrid else None
            logits = dec._verify_forward([req.tseq], feed)
            hidden = dec._verify_hidden if self.keeps_hidden else None
            pos = [blk["base"] + j for j in range(k + 1)]
            p_t, t_toks = dec._probs_and_tokens(dec.t, logits, [req.sp] * (k + 1), pos, [req.tseq.seq_id] * (k + 1))
            p_t = p_t.view(1, k + 1, V)
            if self.cuda:
                for pd in blk["p_d"]:
                    pd.record_stream(torch.cuda.current_stream())       # allocated on the draft stream, read here
            p_d3 = torch.stack(blk["p_d"], dim=1)
            if self.cuda:
                rows = pack_rows([req.sp], [blk["base"]], stream_ids=[req.tseq.seq_id])
                rows_t = dec.t._t(rows.view(np.uint8).reshape(1, ROW_DTYPE.itemsize), torch.uint8)
                dr = dec.t._t(np.asarray([blk["drafted"]], dtype=np.int32), torch.int32)
                res = ops.spec_verify(p_t.contiguous(), p_d3.contiguous(), dr, rows_t)
                ev = torch.cuda.Event()
                ev.record()
            else:
                res = [ops.verify_ref(p_t[0], p_d3[0], blk["drafted"], req.sp.seed, req.tseq.seq_id, blk["base"])]
                ev = None
        req.flight = {"res": res, "toks": t_toks.view(1, k + 1), "event": ev, "t0": time.perf_counter(), "block": blk,
                      "feed": feed, "snap": snap, "hidden": hidden, "keep": (p_t, p_d3, logits)}
        req.block = None
        req.stats.target_tokens += k + 1
        req.phase = Phase.IN_FLIGHT

    def _optimistic(self, req: _Request):
        """k + 1 draft steps behind the in-flight block: the guess of the target's bonus, then the next k proposals."""
        k, dec, blk = self.k, self.dec, req.flight["block"]
        t0 = time.perf_counter()
        base2 = blk["base"] + k               # position of the bonus token
        kv_before = req.dseq.kv_len
        toks, p_d = [], []
        with torch.no_grad(), self._on(self.draft_stream):
            feed_tok = blk["drafted"][-1]
            chain = blk["chain"]
            for j in range(k + 1):
                if self.embedded:
                    store: dict = {}
                    logits = dec._head_step([req.dseq], [[feed_tok]], chain, store, uniform=True)
                    chain = store["batch"].hidden_out
                else:
                    logits = dec._multi_token_step(dec.d, [req.dseq], [[feed_tok]], all_rows=False, uniform=True)
                req.dseq.kv_len += 1
                probs, t = dec._probs_and_tokens(dec.d, logits, [req.sp], [base2 + j], [req.tseq.seq_id])
                feed_tok = int(t.tolist()[0])
                toks.append(feed_tok)
                if j > 0:
                    p_d.append(probs)
            done = torch.cuda.Event() if self.cuda else None
            if done is not None:
                done.record()
        # the last optimistic step fed o_{k-1} and produced o_k: the cache holds [.., o_0 .. o_{k-1}], the invariant of a
        # freshly drafted block whose leading uncached target input is o_0
        req.branch = {"tokens": toks, "p_d": p_d, "kv_before": kv_before, "done": done, "chain": chain}
        req.stats.optimistic_draft_blocks += 1
        req.stats.optimistic_draft_tokens += k + 1
        req.stats.optimistic_draft_time += time.perf_counter() - t0
        req.phase = Phase.OPTIMISTIC_READY

    def _resolve(self, req: _Request):
        k, dec, fl = self.k, self.dec, req.flight
        blk = fl["block"]
        if fl["event"] is not None:
            fl["event"].synchronize()
        req.stats.verification_in_flight_time += time.perf_counter() - fl["t0"]
        res = fl["res"].tolist() if self.cuda else fl["res"]
        a, nxt = int(res[0][0]), int(res[0][1])
        if a == k:
            nxt = int(fl["toks"][0, k])      # the bonus: what plain sampling draws at that position
        req.flight = None
        if req.cancel_requested:
            # roll both caches back to the committed prefix: nothing of this block is published
            if dec.t_hybrid:
                dec.t.restore_state(req.tseq, fl["snap"])
            self._drop_branch(req, count=True)
            self._finish(req, FinishReason.CANCELLED, cancelled=True)
            return
        with torch.no_grad(), self._on(self.target_stream):
            if dec.t_hybrid and a < k:
                dec.t.restore_state(req.tseq, fl["snap"])
                dec._multi_token_step(dec.t, [req.tseq], [fl["feed"][0][:1 + a]], all_rows=False, uniform=False)
        drafted = blk["drafted"]
        req.tseq.kv_len += 1 + a
        st = req.stats
        st.rounds += 1
        st.accepted_tokens += a
        st.accept_lens.append(a)
        dec.stats.rounds += 1
        dec.stats.proposed += k
        dec.stats.accepted += a
        dec.stats.emitted += a + 1
        dec.stats.full_accept_rounds += 1 if a == k else 0
        # ---- the optimistic branch: promote or discard
        promoted = False
        br = req.branch
        if br is not None:
            st.optimistic_target_bonus_tokens += 1 if a == k else 0
            terminal = nxt in req.eos or len(req.out) + a + 1 >= req.max_tokens
            if a == k and not terminal:
                if br["tokens"][0] == nxt:
                    st.optimistic_bonus_matches += 1
                    promoted = True
                else:
                    st.optimistic_bonus_mismatches += 1
        if self.keeps_hidden:
            dec._seq_ids = [req.tseq.seq_id]
            dec._verify_hidden = fl["hidden"]
            if self.cuda:
                fl["hidden"].record_stream(self.draft_stream)            # copied below on the draft stream
        with torch.no_grad(), self._on(self.draft_stream):
            promoted = self._settle(req, fl, a, nxt, promoted)
        req.last = nxt
        self._commit(req, blk["drafted"][:a] + [nxt])
        st.update_adaptive_lookahead(self.options)
        if req.phase not in (Phase.COMPLETED, Phase.CANCELLED):
            req.phase = Phase.READY_TO_SUBMIT if promoted else Phase.READY_TO_DRAFT
        elif promoted:
            # finished by a callback right after promoting: the block is never submitted
            st.discarded_optimistic_tokens += k
            req.block = None

    def _settle(self, req: _Request, fl, a: int, nxt: int, promoted: bool) -> bool:
        """Draft-side bookkeeping of a resolved block (tensor copies run on the draft stream, which consumes them)."""
        k, dec, st = self.k, self.dec, req.stats
        blk, br = fl["block"], req.branch
        drafted = blk["drafted"]
        if promoted:
            st.consumed_optimistic_tokens += 1
            st.reused_optimistic_tokens += k
            st.reused_optimistic_blocks += 1
            new_carry = None
            if self.embedded:
                # the head rows behind its exact prefix were made from chained states: remember what to re-feed (with the
                # target's hidden states) when a later round rolls the head back
                prev = req.carry or {"ctx": blk["ctx"][0], "tokens": [], "hidden": []}
                prev["tokens"] += drafted[:k] + [nxt]
                prev["hidden"].append(fl["hidden"][0, :k + 1].clone())
                new_carry = prev
            req.carry = new_carry
            req.block = {"drafted": br["tokens"][1:], "p_d": br["p_d"], "ctx": blk["ctx"], "base": blk["base"] + k + 1,
                         "done": br["done"], "chain": br["chain"]}
            st.draft_tokens += k
            req.branch = None
            req.pending = []
        else:
            self._drop_branch(req, count=True)
            pend = {0: req.pending}
            ctx = blk["ctx"]
            dec._settle(0, 0, a, nxt, [req.dseq], [drafted], pend, ctx)
            req.pending = pend[0]
            if self.embedded and req.carry is not None:
                c = req.carry
                req.dseq.kv_len = c["ctx"]
                req.pending = c["tokens"] + req.pending
                sid = req.tseq.seq_id
                dec._pending_hidden[sid] = torch.cat(c["hidden"] + [dec._pending_hidden[sid]])
                req.carry = None
        return promoted

    def _drop_branch(self, req: _Request, count: bool):
        br = req.branch
        if br is None:
            return
        if br["done"] is not None:
            br["done"].synchronize()
        req.dseq.kv_len = br["kv_before"]
        if count:
            req.stats.discarded_optimistic_tokens += len(br["tokens"])
            req.stats.discarded_optimistic_blocks += 1
        req.branch = None

    # ------------------------------------------------------------------------------------------ commit / finish
    def _commit(self, req: _Request, tokens: list):
        for tok in tokens:
            if len(req.out) >= req.max_tokens:
                break
            req.out.append(int(tok))
            req.stats.emitted_tokens += 1
            why = req.on_token(int(tok)) if req.on_token is not None else None
            if why:
                self._finish(req, why)
                return
            if int(tok) in req.eos:
                self._finish(req, FinishReason.EOS)
                return
            if len(req.out) >= req.max_tokens:
                self._finish(req, FinishReason.MAX_TOKENS)
                return

    def _finish(self, req: _Request, reason, cancelled: bool = False):
        self._drop_branch(req, count=True)
        req.block = None
        req.finish_reason = reason
        req.stats.elapsed = time.perf_counter() - req.t_start
        req.phase = Phase.CANCELLED if cancelled else Phase.COMPLETED
        self._release(req)

    def _release(self, req: _Request):
        if req.flight is not None and req.flight["event"] is not None:
            req.flight["event"].synchronize()
        req.flight = None
        if req.tseq is not None:
            if self.cuda:
                torch.cuda.synchronize(self.dec.t.device)
            self.dec.t.release(req.tseq)
            self.dec.d.release(req.dseq)
            if self.keeps_hidden:
                self.dec._pending_hidden.pop(req.tseq.seq_id, None)
            req.tseq = req.dseq = None


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def generate_mtp_batch(decoder: SpeculativeDecoder, prompts, sampling: Optional[SamplingParams] = None,
                       max_tokens: int = 256, eos_ids=(), options: Optional[MtpSchedulerOptions] = None,
                       on_token: Optional[Callable[[int, int], Optional[str]]] = None) -> MtpScheduleOutput:
    """Independently progressing lanes over shared weights (``MtpBatchOutput``, eredu-core/src/speculative.rs:291-300):
    one request per prompt, outputs in lane order. ``on_token(lane, token)``."""
    sched = MtpScheduler(decoder, options)
    for i, p in enumerate(prompts):
        cb = (lambda tok, i=i: on_token(i, tok)) if on_token is not None else None
        sched.submit(p, sampling, max_tokens, eos_ids, cb)
    return sched.finish()
