"""Committed-token pipeline: incremental detokenisation -> stop-sequence look-behind -> reasoning / tool-call
parsing -> semantic events, plus finish-reason resolution and cooperative cancellation.

Counterpart of eredu/src/runtime/generation/streaming.rs:825-1025 (``RawTokenDecoder``, ``PartialPatternBuffer``,
``JsonFragmentBuffer``, ``SemanticEventSink``, ``CommittedTokenPipeline``) and eredu-core/src/generation.rs:12-48,802
(``FinishReason``, ``GenerationCancellationToken``, ``SemanticEvent``). Finish precedence is stop sequence > grammar
complete > EOS > max tokens (doc/tool-calling.md:97-100); cancellation is cooperative and never pre-empts submitted
work (doc/cancellation.md:1-30).
"""
from __future__ import annotations

import json
import threading
from dataclasses import dataclass, field
from typing import Callable, Optional


class FinishReason:
    EOS = "eos"
    STOP_SEQUENCE = "stop_sequence"
    GRAMMAR_COMPLETE = "grammar_complete"
    MAX_TOKENS = "max_tokens"
    CANCELLED = "cancelled"

    _RANK = {STOP_SEQUENCE: 0, GRAMMAR_COMPLETE: 1, EOS: 2, MAX_TOKENS: 3}

    @classmethod
    def resolve(cls, candidates) -> Optional[str]:
        """The reason that wins when several end conditions hold on the same token."""
        c = [x for x in candidates if x]
        if not c:
            return None
        if cls.CANCELLED in c and len(c) == 1:
            return cls.CANCELLED
        ranked = [x for x in c if x in cls._RANK]
        return min(ranked, key=cls._RANK.get) if ranked else c[0]


class CancellationToken:
    def __init__(self):
        self._flag = threading.Event()

    def cancel(self):
        self._flag.set()

    def is_cancelled(self) -> bool:
        return self._flag.is_set()


@dataclass
class SemanticEvent:
    kind: str                 # text | reasoning | tool_call_start | tool_call_arguments | tool_call_end | finished
    text: str = ""
    tool_name: Optional[str] = None
    tool_index: Optional[int] = None
    arguments: Optional[dict] = None
    finish_reason: Optional[str] = None


class PartialPatternBuffer:
    """Holds back the tail of the stream that could still turn into one of the patterns (stop sequences or
    structural tags). ``push`` returns (text safe to release, matched pattern or None)."""

    def __init__(self, patterns):
        self.patterns = [p for p in patterns if p]
        self.buf = ""

    def push(self, text: str):
        self.buf += text
        best = None
        for p in self.patterns:
            i = self.buf.find(p)
            if i >= 0 and (best is None or i < best[0]):
                best = (i, p)
        if best is not None:
            i, p = best
            out, self.buf = self.buf[:i], self.buf[i + len(p):]
            return out, p
        hold = 0
        for p in self.patterns:
            for n in range(min(len(p) - 1, len(self.buf)), 0, -1):
                if self.buf.endswith(p[:n]):
                    hold = max(hold, n)
                    break
        out = self.buf[:len(self.buf) - hold] if hold else self.buf
        self.buf = self.buf[len(out):]
        return out, None

    def flush(self) -> str:
        out, self.buf = self.buf, ""
        return out


class JsonFragmentBuffer:
    """Accumulates the text of one JSON value and reports when it is syntactically complete."""

    def __init__(self):
        self.text = ""

    def push(self, fragment: str) -> Optional[object]:
        self.text += fragment
        s = self.text.strip()
        if not s or s[0] not in "{[":
            return None
        depth, in_str, esc = 0, False, False
        for ch in s:
            if in_str:
                if esc:
                    esc = False
                elif ch == "\\":
                    esc = True
                elif ch == '"':
                    in_str = False
            elif ch == '"':
                in_str = True
            elif ch in "{[":
                depth += 1
            elif ch in "}]":
                depth -= 1
        if depth == 0 and not in_str:
            try:
                return json.loads(s)
            except json.JSONDecodeError:
                return None
        return None


class CommittedTokenPipeline:
    """push(token id) -> list of SemanticEvents. States: text, reasoning, tool call body."""

    def __init__(self, decoder, plan=None, stop=(), on_event: Optional[Callable[[SemanticEvent], None]] = None,
                 max_parallel_tool_calls: Optional[int] = None):
        self.decoder = decoder
        self.plan = plan
        self.on_event = on_event
        self.stop = [s for s in stop if s]
        self.state = "reasoning" if (plan and plan.starts_in_reasoning) else "text"
        self.tool_json = None
        self.tool_count = 0
        self.max_tools = max_parallel_tool_calls
        self.finished: Optional[str] = None
        self.text_out: list[str] = []
        self.reasoning_out: list[str] = []
        self.tool_calls: list[dict] = []
        self._bare_decided = False
        self._bare_hold = ""
        self._retarget()

    def _retarget(self):
        pats = list(self.stop)
        p = self.plan
        if p is not None:
            if self.state == "text":
                pats += [p.reasoning_open, p.tool_open]
            elif self.state == "reasoning":
                pats += [p.reasoning_close]
            elif self.state == "tool":
                pats += [p.tool_close]
        held = self.matcher.flush() if hasattr(self, "matcher") else ""
        self.matcher = PartialPatternBuffer(pats)
        self._carry = held

    def _emit(self, ev: SemanticEvent, out: list):
        out.append(ev)
        if self.on_event:
            self.on_event(ev)

    def _content(self, text: str, out: list):
        if not text:
            return
        if self.state == "text":
            self.text_out.append(text)
            self._emit(SemanticEvent("text", text), out)
        elif self.state == "reasoning":
            self.reasoning_out.append(text)
            self._emit(SemanticEvent("reasoning", text), out)
        else:
            self._tool_fragment(text, out)

    def _tool_fragment(self, text: str, out: list):
        if self.tool_json.text.lstrip().startswith("<") or (not self.tool_json.text.strip() and text.lstrip().startswith("<")):
            self.tool_json.text += text        # tagged syntax: not JSON, collected verbatim until the closing tag
            self._emit(SemanticEvent("tool_call_arguments", text, tool_index=self.tool_count - 1), out)
            return
        value = self.tool_json.push(text)
        self._emit(SemanticEvent("tool_call_arguments", text, tool_index=self.tool_count - 1), out)
        if value is not None and self.plan.tool_close is None:
            self._close_tool(out)

    def _close_tool(self, out: list):
        raw = self.tool_json.text.strip()
        name, args = None, None
        if raw.startswith("<function="):
            # Qwen tagged-parameter syntax: <function=NAME><parameter=KEY>VALUE</parameter>...</function>
            from ..text.dialects import parse_tagged_call

            try:
                call = parse_tagged_call(raw, getattr(self, "tools", None))[0]
                name, args = call["name"], call["arguments"]
            except ValueError:
                pass
            self.tool_calls.append({"name": name, "arguments": args, "raw": raw})
            self._emit(SemanticEvent("tool_call_end", tool_name=name, tool_index=self.tool_count - 1, arguments=args), out)
            self.state = "text"
            self._retarget()
            return
        try:
            obj = json.loads(raw)
            if isinstance(obj, list) and obj:
                obj = obj[0]
            name = obj.get("name")
            args = obj.get("arguments", obj.get("parameters"))
            if isinstance(args, str):
                args = json.loads(args)
        except Exception:
            pass
        self.tool_calls.append({"name": name, "arguments": args, "raw": raw})
        self._emit(SemanticEvent("tool_call_end", tool_name=name, tool_index=self.tool_count - 1, arguments=args), out)
        self.state = "text"
        self._bare_decided = False
        self._retarget()

    def _bare_json_gate(self, text: str, out: list) -> str:
        """Bare-JSON tool calls (Llama-3 style ``{"name": ..., "parameters": ...}`` with no tags): the reply is a call
        exactly when its first visible character is ``{`` (the activation rule of runtime/chat/dialect.rs:464-495).
        Returns the text that the ordinary path still has to see."""
        if self.state != "text" or self._bare_decided:
            return text
        text = self._bare_hold + text
        self._bare_hold = ""
        body = text.lstrip()
        if not body:
            self._bare_hold = text           # only white space so far: undecided
            return ""
        self._bare_decided = True
        if not body.startswith("{") or (self.max_tools is not None and self.tool_count >= self.max_tools):
            return text
        self.state = "tool"
        self.tool_json = JsonFragmentBuffer()
        self.tool_count += 1
        self._emit(SemanticEvent("tool_call_start", tool_index=self.tool_count - 1), out)
        self._retarget()
        return body

    def _feed(self, text: str, out: list):
        text = self._carry + text
        self._carry = ""
        if self.plan is not None and getattr(self.plan, "bare_json_tools", False):
            text = self._bare_json_gate(text, out)
        while text or False:
            released, hit = self.matcher.push(text)
            text = ""
            self._content(released, out)
            if hit is None:
                return
            p = self.plan
            if hit in self.stop:
                self.finished = FinishReason.STOP_SEQUENCE
                return
            if p is not None and hit == p.reasoning_open and self.state == "text":
                self.state = "reasoning"
            elif p is not None and hit == p.reasoning_close and self.state == "reasoning":
                self.state = "text"
            elif p is not None and hit == p.tool_open and self.state == "text":
                if self.max_tools is not None and self.tool_count >= self.max_tools:
                    self.finished = FinishReason.GRAMMAR_COMPLETE
                    return
                self.state = "tool"
                self.tool_json = JsonFragmentBuffer()
                self.tool_count += 1
                self._emit(SemanticEvent("tool_call_start", tool_index=self.tool_count - 1), out)
            elif p is not None and hit == p.tool_close and self.state == "tool":
                rest = self.matcher.flush()
                self._close_tool(out)
                text = rest
                continue
            rest = self.matcher.flush()
            self._retarget()
            text = self._carry + rest
            self._carry = ""

    def push(self, token_id: int) -> list:
        out: list = []
        if self.finished:
            return out
        self._feed(self.decoder.push(token_id), out)
        return out

    def finish(self, reason: str) -> list:
        """Flush held-back text and emit the final event. A stop sequence seen earlier wins over ``reason``."""
        out: list = []
        if not self.finished:
            tail = self.decoder.flush()
            if tail:
                self._feed(tail, out)
        if not self.finished or self.finished != FinishReason.STOP_SEQUENCE:
            held = self._bare_hold + self._carry + self.matcher.flush()
            self._carry = self._bare_hold = ""
            if self.state == "tool" and held:
                self._tool_fragment(held, out)
            else:
                self._content(held, out)
        final = FinishReason.resolve([self.finished, reason]) if reason != FinishReason.CANCELLED else (self.finished or reason)
        self.finished = final
        self._emit(SemanticEvent("finished", finish_reason=final), out)
        return out
