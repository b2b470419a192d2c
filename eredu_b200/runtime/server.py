"""Continuous-batching serving loop: scheduler-planned steps over one engine, with cross-rank consensus.

The step protocol follows the reference's distributed serving path (eredu-core/src/scheduler.rs:15-1410,
eredu-core/src/consensus.rs:122-244, eredu/src/backend/mlx/distributed.rs:216-241,383-399):

1. every rank plans the same step from the same request stream (fair round-robin, token and batch budgets, bounded
   admission - the C++ ``Scheduler``);
2. the plan is encoded as integer words and all-gathered; any rank whose plan differs poisons the scheduler and
   every later call fails closed (no rank ever runs a collective the others do not run);
3. the step executes: chunked prefills, then ONE decode step for all running requests (slot-based decode state:
   requests join and leave the captured CUDA graph's static buffers between steps);
4. completions are resolved the same way (complete / failed on any rank -> failed everywhere).

A transport is anything with ``all_gather_words(list[int]) -> list[int]`` (concatenation in rank order) and
``size``; ``TorchTransport`` carries the words over a ``torch.distributed`` group, ``None`` means single rank.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from ..lib import _eredu_host as H
from ..ops.sampling import SamplingParams
from .engine import Engine, Sequence

PROTOCOL_VERSION = 1


class ConsensusError(RuntimeError):
    pass


class TorchTransport:
    """Word frames over a torch.distributed process group (gloo on CPU ranks, NCCL on GPUs)."""

    def __init__(self, group=None, device="cpu"):
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.size = dist.get_world_size(group)
        self.device = torch.device(device)

    def all_gather_varlen(self, words: list[int]) -> list[list[int]]:
        """Every rank's word list (lengths may differ), in rank order."""
        n = torch.tensor([len(words)], dtype=torch.int64, device=self.device)
        lens = [torch.zeros_like(n) for _ in range(self.size)]
        self.dist.all_gather(lens, n, group=self.group)
        lens = [int(x.item()) for x in lens]
        width = max(lens + [1])
        t = torch.zeros(width, dtype=torch.int64, device=self.device)
        if words:
            t[:len(words)] = torch.tensor(words, dtype=torch.int64, device=self.device)
        out = [torch.zeros_like(t) for _ in range(self.size)]
        self.dist.all_gather(out, t, group=self.group)
        return [o[:k].tolist() for o, k in zip(out, lens)]

    def all_gather_words(self, words: list[int]) -> list[int]:
        # lengths first: a rank with a different plan may also have a different frame length
        n = torch.tensor([len(words)], dtype=torch.int64, device=self.device)
        lens = [torch.zeros_like(n) for _ in range(self.size)]
        self.dist.all_gather(lens, n, group=self.group)
        lens = [int(x.item()) for x in lens]
        if len(set(lens)) != 1:
            raise ConsensusError(f"consensus frames differ in length across ranks: {lens}")
        t = torch.tensor(words, dtype=torch.int64, device=self.device)
        out = [torch.zeros_like(t) for _ in range(self.size)]
        self.dist.all_gather(out, t, group=self.group)
        return [int(v) for part in out for v in part.tolist()]


@dataclass
class ServedRequest:
    request_id: int
    seq: Sequence
    on_token: Optional[Callable[[int, int], Optional[str]]] = None
    tokens: list = field(default_factory=list)
    finish_reason: Optional[str] = None
    first_token_time: Optional[float] = None
    submit_time: float = 0.0
    failed: bool = False


class Server:
    def __init__(self, engine: Engine, transport=None, max_step_tokens: int = 8192, max_waiting: int = 1024,
                 prefill_chunk: int = 2048, penalties: bool = False, fault_hook: Optional[Callable[[str, int], bool]] = None,
                 kv_tier=None):
        if not getattr(engine, "paged", True):
            raise NotImplementedError("continuous batching needs the paged engine; this model family runs one sequence at a time")
        self.engine = engine
        self.transport = transport
        self.kv_tier = kv_tier   # KVHostTier: running requests are parked in host memory when the page pool runs out
        self.sched = H.Scheduler(engine.max_batch, max_step_tokens, max_waiting, prefill_chunk)
        self.requests: dict[int, ServedRequest] = {}
        self.drain_cycle = 0
        self._pending_cancels: set = set()
        self.fault_hook = fault_hook  # (kind, request_id) -> True injects a request-local failure on this rank
        engine.open_decode(penalties=penalties)

    # ------------------------------------------------------------------------------------------ requests
    def submit(self, prompt: list[int], sampling: Optional[SamplingParams] = None, max_new_tokens: int = 256, eos_ids=(),
               on_token=None, deadline: float = 0.0) -> int:
        rid = int(self.sched.submit(len(prompt), max_new_tokens, deadline))
        try:
            seq = self._new_sequence_under_pressure(prompt, sampling, max_new_tokens, eos_ids)
        except Exception:
            self.sched.cancel(rid)
            raise
        self.requests[rid] = ServedRequest(rid, seq, on_token, submit_time=time.perf_counter())
        return rid

    def _new_sequence_under_pressure(self, prompt, sampling, max_new_tokens, eos_ids):
        """Reserve pages for a new request; when the pool is exhausted and a host tier exists, park running
        requests (policy: the tier's eviction order) until the reservation succeeds."""
        while True:
            try:
                return self.engine.new_sequence(prompt, sampling, max_new_tokens, eos_ids)
            except (MemoryError, RuntimeError) as e:
                if self.kv_tier is None or (isinstance(e, RuntimeError) and "exhausted" not in str(e)):
                    raise
                running = [r.seq for r in self.requests.values() if r.seq.slot >= 0 and not r.seq.finished]
                victim = self.kv_tier.victim(running)
                if victim is None:
                    raise
                self.engine.leave(victim)
                if not self.kv_tier.park(victim):
                    raise

    def cancel(self, request_id: int) -> None:
        """Cooperative cancellation. Single rank: takes effect now (or when the request's in-flight work completes).
        With a transport the request is only recorded; at the next step boundary every rank learns the union of all
        ranks' cancellations and applies it before planning, so the plans keep agreeing
        (eredu/src/backend/mlx/distributed.rs:216-241)."""
        if self.transport is None:
            self.sched.cancel(request_id)
            self._retire_terminal()
        else:
            self._pending_cancels.add(int(request_id))

    def _exchange_cancels(self) -> None:
        if self.transport is None:
            return
        try:
            everyone = self.transport.all_gather_varlen(sorted(self._pending_cancels))
        except Exception as e:
            self.sched.poison(f"cancellation exchange failed: {e}")
            raise ConsensusError(str(e)) from e
        self._pending_cancels.clear()
        for rid in sorted({r for ranks in everyone for r in ranks}):
            if rid in self.requests:
                self.sched.cancel(rid)
        self._retire_terminal()

    def pending(self) -> bool:
        rep = self.sched.report()
        return (rep["waiting"] + rep["running"]) > 0

    def result(self, request_id: int) -> ServedRequest:
        return self.requests[request_id]

    # ------------------------------------------------------------------------------------------ consensus
    def _agree(self, words: list[int], what: str) -> list[int]:
        if self.transport is None:
            return words
        try:
            gathered = self.transport.all_gather_words(words)
            bad = H.validate_gathered(words, gathered, self.transport.size)
        except Exception as e:
            self.sched.poison(f"{what} consensus failed: {e}")
            raise ConsensusError(str(e)) from e
        if bad >= 0:
            self.sched.poison(f"{what} differs on rank {bad}")
            raise ConsensusError(f"{what} differs on rank {bad}")
        return gathered

    # ------------------------------------------------------------------------------------------ one step
    def step(self, now: Optional[float] = None) -> int:
        """Plan, agree, execute and complete one step. Returns the number of work items executed."""
        self._exchange_cancels()
        plan = self.sched.plan_step(time.monotonic() if now is None else now)
        self._retire_terminal()  # deadline cancellations decided while planning
        if not plan:
            return 0
        frame = H.encode_schedule([(int(w.request_id), [int(w.work_id), 0 if w.kind == "prefill" else 1, int(w.tokens)])
                                   for w in plan], self.drain_cycle, PROTOCOL_VERSION)
        self._agree([int(x) for x in frame], "schedule")
        self.drain_cycle += 1
        status = {}  # work_id -> (tokens, generated, stop, failed)
        eng = self.engine
        prefills = [w for w in plan if w.kind == "prefill"]
        decodes = [w for w in plan if w.kind == "decode"]
        # ---- chunked prefill
        if prefills:
            reqs = [self.requests[int(w.request_id)] for w in prefills]
            try:
                toks = eng.prefill([r.seq for r in reqs], limits=[int(w.tokens) for w in prefills])
                toks = toks.tolist() if toks is not None else [0] * len(reqs)
                for w, r, t in zip(prefills, reqs, toks):
                    failed = bool(self.fault_hook and self.fault_hook("prefill", r.request_id))
                    if failed:
                        status[int(w.work_id)] = (int(w.tokens), 0, False, True)
                        continue
                    if r.seq.kv_len >= len(r.seq.prompt):  # the prompt is complete: t is the first generated token
                        stop = self._emit(r, int(t))
                        if not stop:
                            eng.join(r.seq, int(t))
                        status[int(w.work_id)] = (int(w.tokens), 1, stop, False)
                    else:
                        status[int(w.work_id)] = (int(w.tokens), 0, False, False)
            except Exception:
                for w in prefills:
                    status[int(w.work_id)] = (int(w.tokens), 0, False, True)
        # ---- one decode step for every planned running request
        if decodes:
            planned = {int(w.request_id): w for w in decodes}
            if self.kv_tier is not None:
                # parked requests come back when pages and a slot are free; otherwise they make no progress this step
                for rid in list(planned):
                    r = self.requests[rid]
                    if r.seq.seq_id in self.kv_tier.parked:
                        if eng.free_slots() and self.kv_tier.resume(r.seq):
                            eng.join(r.seq, r.tokens[-1])
                        else:
                            status[int(planned[rid].work_id)] = (0, 0, False, False)
                            del planned[rid]
                for rid in planned:
                    self.kv_tier.touch(self.requests[rid].seq)
            st = eng._decode_state
            mask = [s is not None and any(r.seq is s for r in (self.requests[i] for i in planned)) for s in st["seqs"]]
            eng.set_step_mask(mask)
            st["stepped"] = mask
            try:
                toks = eng.decode_step()
                host = toks.tolist()
                eng.commit(host)
                for rid, w in planned.items():
                    r = self.requests[rid]
                    failed = bool(self.fault_hook and self.fault_hook("decode", rid))
                    if failed:
                        status[int(w.work_id)] = (1, 0, False, True)
                        continue
                    tok = r.seq.output[-1]
                    stop = self._emit(r, tok, already_committed=True)
                    status[int(w.work_id)] = (1, 1, stop, False)
            except Exception:
                for w in decodes:
                    status[int(w.work_id)] = (1, 0, False, True)
        # ---- completion consensus: 1 complete, 2 failed (a failure on any rank fails the request everywhere)
        order = [int(w.work_id) for w in plan]
        local = [2 if status[i][3] else 1 for i in order]
        if self.transport is not None:
            gathered = self.transport.all_gather_words(local)
            resolved = H.resolve_completions([int(x) for x in gathered], self.transport.size, len(order))
        else:
            resolved = H.resolve_completions(local, 1, len(order))
        for i, res in zip(order, resolved):
            tokens, generated, stop, _ = status[i]
            self.sched.complete(i, tokens, generated, stop, res in (2, 3))
        self._retire_terminal()
        return len(plan)

    def _emit(self, r: ServedRequest, tok: int, already_committed: bool = False) -> bool:
        """Record a generated token; returns True when the request stops here (EOS, budget or callback)."""
        if r.first_token_time is None:
            r.first_token_time = time.perf_counter()
        s = r.seq
        if not already_committed:
            s.output.append(tok)
        r.tokens.append(tok)
        stop = False
        if r.on_token is not None:
            why = r.on_token(r.request_id, tok)
            if why:
                r.finish_reason = str(why)
                stop = True
        if not stop and tok in s.eos_ids:
            r.finish_reason, stop = "eos", True
        if not stop and len(s.output) >= s.max_new_tokens:
            r.finish_reason, stop = "max_tokens", True
        if stop:
            s.finished = True
        return stop

    def _retire_terminal(self) -> None:
        """Free the slot and the pages of every request the scheduler has finished, cancelled or failed."""
        for rid, r in self.requests.items():
            parked = self.kv_tier is not None and r.seq.seq_id in self.kv_tier.parked
            if (r.seq.pages or parked) and self.sched.request(rid)["state"] in ("finished", "cancelled", "failed"):
                if parked:
                    self.kv_tier.drop(r.seq)
                state = self.sched.request(rid)
                if r.finish_reason is None:
                    r.finish_reason = state["finish_reason"] or state["state"]
                r.failed = state["state"] == "failed"
                self.engine.leave(r.seq)
                self.engine.release(r.seq)

    def run_until_idle(self, max_steps: int = 1 << 30) -> int:
        steps = 0
        while self.pending() and steps < max_steps:
            if self.step() == 0 and not self.pending():
                break
            steps += 1
        return steps
