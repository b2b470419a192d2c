"""Realtime speech sessions: frame-synchronous stepping of a temporal + depth model, stream delays, a fair scheduler.

Counterpart of the reference's realtime contracts (eredu-core/src/realtime.rs:16-131 ``RealtimeSpeechConfig`` with its
codebook partition and per-codebook delays, :171-250 ``RealtimeSampling``, :392-456 sessions, :525-830 ``RealtimeScheduler``
with per-request queues, deadlines, cancellation and a report) and of the Moshi / PersonaPlex backend
(eredu/src/backend/mlx/realtime.rs). One step consumes the codes of one heard frame and produces one text token and the
codes of one spoken frame.

Delays. Every audio codebook k runs ``audio_delays[k]`` frames behind the text stream inside the model (the first, semantic
codebook 0, the acoustic ones usually 1). The session keeps rows in the model's delayed coordinates: row t holds, for every
stream, the token the model sees for step t+1. A heard frame c enters row ``c + delay_k`` of codebook k (earlier rows hold
the padding token); the spoken frame c is complete once row ``c + max_delay`` exists, so output starts ``max_delay`` steps
after input.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch


class RealtimeConfigError(ValueError):
    pass


@dataclass(frozen=True)
class RealtimeSpeechConfig:
    total_audio_codebooks: int
    input_audio_codebooks: int
    generated_audio_codebooks: int
    depth_audio_codebooks: int
    text_padding_token: int
    audio_padding_token: int
    audio_delays: tuple

    def __post_init__(self):
        t, i, g, d = (self.total_audio_codebooks, self.input_audio_codebooks, self.generated_audio_codebooks,
                      self.depth_audio_codebooks)
        if min(t, i, g, d) <= 0:
            raise RealtimeConfigError("codebook counts must be positive")
        if i + g != t:
            raise RealtimeConfigError(f"input ({i}) + generated ({g}) codebooks must equal the total ({t})")
        if len(self.audio_delays) != t:
            raise RealtimeConfigError(f"{len(self.audio_delays)} delays given for {t} codebooks")
        if d > g:
            raise RealtimeConfigError("the depth transformer cannot produce more codebooks than are generated")
        if any(int(x) < 0 for x in self.audio_delays):
            raise RealtimeConfigError("delays are non-negative")
        object.__setattr__(self, "audio_delays", tuple(int(x) for x in self.audio_delays))

    @property
    def max_audio_delay(self) -> int:
        return max(self.audio_delays)

    @classmethod
    def for_moshi(cls, cfg, delays=None) -> "RealtimeSpeechConfig":
        """Generated codebooks first, heard ones after (the order of the embedding tables); semantic codebooks undelayed,
        acoustic ones one frame behind."""
        K = cfg.num_codebooks
        per = [0] + [1] * (K - 1)
        return cls(2 * K, K, K, K, cfg.vocab_size, cfg.audio_vocab_size, tuple(delays) if delays is not None else tuple(per + per))


@dataclass(frozen=True)
class RealtimeSampling:
    text_temperature: float = 0.7
    audio_temperature: float = 0.8
    seed: int = 0
    text_top_k: int = 25
    audio_top_k: int = 250

    def __post_init__(self):
        for name in ("text_temperature", "audio_temperature"):
            v = getattr(self, name)
            if not (v == v and v >= 0.0 and v != float("inf")):
                raise RealtimeConfigError(f"{name} must be finite and non-negative")
        if self.text_top_k < 0 or self.audio_top_k < 0:
            raise RealtimeConfigError("top-k must be non-negative")


def _pick(logits: torch.Tensor, temperature: float, top_k: int, gen: torch.Generator) -> torch.Tensor:
    if temperature <= 0.0:
        return logits.argmax(-1)
    x = logits.float() / temperature
    if top_k and top_k < x.shape[-1]:
        kth = torch.topk(x, top_k, dim=-1).values[..., -1:]
        x = x.masked_fill(x < kth, float("-inf"))
    p = torch.softmax(x, -1)
    return torch.multinomial(p.cpu(), 1, generator=gen).squeeze(-1).to(logits.device)


@dataclass
class RealtimeStep:
    index: int
    text_token: torch.Tensor                       # [B]
    spoken_codes: Optional[torch.Tensor]           # [B, generated] of frame index - max_delay, None while delays fill
    seconds: float = 0.0


class RealtimeSession:
    """State of one conversation (batch B, usually 1): the temporal transformer's cache and the last rows of every stream."""

    def __init__(self, lm, speech: Optional[RealtimeSpeechConfig] = None, sampling: Optional[RealtimeSampling] = None,
                 batch: int = 1):
        self.lm = lm
        self.speech = speech or RealtimeSpeechConfig.for_moshi(lm.cfg)
        self.sampling = sampling or RealtimeSampling()
        self.batch = batch
        self.gen = torch.Generator().manual_seed(self.sampling.seed)
        self.state: dict = {}
        self.index = 0
        sp = self.speech
        G, I = sp.generated_audio_codebooks, sp.input_audio_codebooks
        dev = lm.device
        self._text_row = torch.full((batch,), sp.text_padding_token, dtype=torch.long, device=dev)
        self._spoken_row = torch.full((batch, G), sp.audio_padding_token, dtype=torch.long, device=dev)
        self._heard_row = torch.full((batch, I), sp.audio_padding_token, dtype=torch.long, device=dev)
        hist = sp.max_audio_delay + 1
        self._heard_frames: deque = deque(maxlen=hist)      # content frames, newest last
        self._spoken_rows: deque = deque(maxlen=hist)       # generated rows (delayed coordinates), newest last

    def set_sampling(self, sampling: RealtimeSampling) -> None:
        self.sampling = sampling
        self.gen = torch.Generator().manual_seed(sampling.seed + self.index)

    def _delayed_heard_row(self) -> torch.Tensor:
        """Row of the newest step: codebook k shows the frame from ``delay_k`` steps ago (padding before the stream began)."""
        sp = self.speech
        G = sp.generated_audio_codebooks
        row = torch.full_like(self._heard_row, sp.audio_padding_token)
        n = len(self._heard_frames)
        for k in range(sp.input_audio_codebooks):
            d = sp.audio_delays[G + k]
            if d < n:
                row[:, k] = self._heard_frames[n - 1 - d][:, k]
        return row

    @torch.no_grad()
    def step(self, heard_codes: Optional[torch.Tensor]) -> RealtimeStep:
        """``heard_codes`` [B, input codebooks] of the frame that just arrived (None: silence / no input stream)."""
        t0 = time.perf_counter()
        sp, lm, smp = self.speech, self.lm, self.sampling
        G = sp.generated_audio_codebooks
        # the model reads the previous rows of all streams
        x = lm.embed_frame(self._text_row[:, None], self._spoken_row[:, :, None], self._heard_row[:, :, None])
        text_logits, hidden = lm.temporal(x, self.state)
        text = _pick(text_logits[:, -1], smp.text_temperature, smp.text_top_k, self.gen)
        spoken = lm.depth_generate(hidden[:, -1], text,
                                   choose=lambda k, lg: _pick(lg, smp.audio_temperature, smp.audio_top_k, self.gen))
        if heard_codes is None:
            heard_codes = torch.full((self.batch, sp.input_audio_codebooks), sp.audio_padding_token, dtype=torch.long)
        if tuple(heard_codes.shape) != (self.batch, sp.input_audio_codebooks):
            raise ValueError(f"heard codes must be [{self.batch}, {sp.input_audio_codebooks}]")
        self._heard_frames.append(heard_codes.to(lm.device, torch.long))
        self._text_row, self._spoken_row, self._heard_row = text, spoken, self._delayed_heard_row()
        self._spoken_rows.append(spoken)
        out = None
        D = sp.max_audio_delay
        if self.index >= D:
            # content frame (index - D): codebook k sits in the row generated delay_k steps after it
            n = len(self._spoken_rows)
            out = torch.stack([self._spoken_rows[n - 1 - (D - sp.audio_delays[k])][:, k] for k in range(G)], 1)
        step = RealtimeStep(self.index, text, out, time.perf_counter() - t0)
        self.index += 1
        return step


class SpeechPipeline:
    """PCM in, PCM out: the codec's streaming encoder in front of a session and its streaming decoder behind it."""

    def __init__(self, session: RealtimeSession, codec):
        self.session, self.codec = session, codec
        if codec.cfg.num_quantizers < session.speech.input_audio_codebooks:
            raise RealtimeConfigError("the codec has fewer codebooks than the model hears")
        codec.reset_encode_state()
        codec.reset_decode_state()
        self.text_tokens: list = []

    def feed(self, pcm: torch.Tensor) -> Optional[torch.Tensor]:
        """Any amount of PCM [B, channels, samples]; returns the PCM spoken during the frames this input completed."""
        codes = self.codec.encode_step(pcm, self.session.speech.input_audio_codebooks)
        if codes is None:
            return None
        out = []
        for f in range(codes.shape[-1]):
            step = self.session.step(codes[:, :, f])
            self.text_tokens.append(step.text_token)
            if step.spoken_codes is not None:
                out.append(self.codec.decode_step(step.spoken_codes[:, :, None].clamp_max(self.codec.cfg.codebook_size - 1)))
        return torch.cat(out, -1) if out else None


# ---------------------------------------------------------------------------------------------------------------
class RealtimeError(RuntimeError):
    pass


@dataclass
class _Request:
    session: object
    queue: deque = field(default_factory=deque)        # (work id, input, deadline or None)
    status: str = "running"                            # running | finished | cancelled
    completed: int = 0
    missed_deadlines: int = 0


@dataclass
class RealtimeCompletedStep:
    work_id: int
    request_id: int
    output: object
    late: bool = False


class RealtimeScheduler:
    """Frame steps of several sessions, one step per request and round (round-robin in registration order), so that no
    conversation starves another. A queued step may carry a deadline (``time.monotonic`` seconds): a step that starts after
    its deadline still runs (the session's state must advance frame by frame) but is reported late."""

    def __init__(self, step_fn: Optional[Callable] = None, max_queue_per_request: int = 64, clock: Callable = time.monotonic):
        self.step_fn = step_fn or (lambda session, inp: session.step(inp))
        self.max_queue = max_queue_per_request
        self.clock = clock
        self.requests: dict[int, _Request] = {}
        self._next_request, self._next_work = 0, 0
        self._cursor = 0
        self.steps_run = 0

    def register_request(self, session) -> int:
        rid = self._next_request
        self._next_request += 1
        self.requests[rid] = _Request(session)
        return rid

    def _live(self, rid: int) -> _Request:
        r = self.requests.get(rid)
        if r is None:
            raise RealtimeError(f"unknown request {rid}")
        if r.status != "running":
            raise RealtimeError(f"request {rid} is {r.status}")
        return r

    def enqueue(self, rid: int, inp, deadline: Optional[float] = None) -> int:
        r = self._live(rid)
        if len(r.queue) >= self.max_queue:
            raise RealtimeError(f"request {rid} has {len(r.queue)} queued steps (limit {self.max_queue})")
        wid = self._next_work
        self._next_work += 1
        r.queue.append((wid, inp, deadline))
        return wid

    def enqueue_batch(self, items) -> list:
        """``[(request id, input[, deadline])]``: all or nothing."""
        for it in items:
            r = self._live(it[0])
            pending = sum(1 for j in items if j[0] == it[0])
            if len(r.queue) + pending > self.max_queue:
                raise RealtimeError(f"request {it[0]} would exceed its queue limit")
        return [self.enqueue(*it) for it in items]

    def queued_for_request(self, rid: int) -> int:
        return len(self.requests[rid].queue) if rid in self.requests else 0

    def run_bounded(self, max_steps: Optional[int] = None) -> list:
        """Run queued steps fairly until the queues are empty or ``max_steps`` ran. Returns the completions in order."""
        done = []
        order = sorted(self.requests)
        if not order:
            return done
        idle = 0
        while (max_steps is None or len(done) < max_steps) and idle < len(order):
            rid = order[self._cursor % len(order)]
            self._cursor += 1
            r = self.requests[rid]
            if r.status != "running" or not r.queue:
                idle += 1
                continue
            idle = 0
            wid, inp, deadline = r.queue.popleft()
            late = deadline is not None and self.clock() > deadline
            out = self.step_fn(r.session, inp)
            r.completed += 1
            r.missed_deadlines += 1 if late else 0
            self.steps_run += 1
            done.append(RealtimeCompletedStep(wid, rid, out, late))
        return done

    def run_queued(self) -> list:
        return self.run_bounded(None)

    def finish_request(self, rid: int) -> None:
        r = self._live(rid)
        if r.queue:
            raise RealtimeError(f"request {rid} still has {len(r.queue)} queued steps")
        r.status = "finished"

    def cancel_request(self, rid: int) -> None:
        r = self._live(rid)
        r.queue.clear()
        r.status = "cancelled"

    def forget_terminal_request(self, rid: int) -> None:
        r = self.requests.get(rid)
        if r is None or r.status == "running":
            raise RealtimeError(f"request {rid} is not terminal")
        del self.requests[rid]

    def request_status(self, rid: int) -> Optional[str]:
        r = self.requests.get(rid)
        return r.status if r else None

    def set_request_sampling(self, rid: int, sampling: RealtimeSampling) -> None:
        self._live(rid).session.set_sampling(sampling)

    def report(self) -> dict:
        return {"requests": {rid: {"status": r.status, "queued": len(r.queue), "completed": r.completed,
                                   "missed_deadlines": r.missed_deadlines} for rid, r in self.requests.items()},
                "steps_run": self.steps_run}
