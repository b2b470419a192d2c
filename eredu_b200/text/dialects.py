"""Checkpoint-specific chat surface syntaxes on top of the committed-token pipeline.

* LFM2: tool calls are a Python-style call list between ``<|tool_call_start|>`` and ``<|tool_call_end|>``, e.g.
  ``[get_weather(city="Paris", days=3), now()]`` (eredu/src/runtime/chat/lfm2.rs:1-40: structural tokens, stops; the
  module's incremental normaliser turns the calls into name + JSON arguments).
* Harmony (GPT-OSS): a message is ``<|start|>ROLE[ to=RECIPIENT]<|channel|>CHANNEL[ to=RECIPIENT][ <|constrain|>TYPE]
  <|message|>BODY`` closed by ``<|end|>`` (more messages follow), ``<|return|>`` (final answer done) or ``<|call|>``
  (tool call issued). The ``analysis`` channel is reasoning, ``final`` is the reply, ``commentary`` addressed to
  ``functions.NAME`` is a tool call whose body is the JSON arguments (eredu/src/runtime/chat/harmony.rs).

Both parsers keep the interface of :class:`eredu_b200.runtime.streaming.CommittedTokenPipeline` (``push`` /
``finish`` / ``text_out`` / ``reasoning_out`` / ``tool_calls`` / ``finished``) and need the detokeniser to render
special tokens.
"""
from __future__ import annotations

import ast
import json
import re
from typing import Callable, Optional

from ..runtime.streaming import (CommittedTokenPipeline, FinishReason, JsonFragmentBuffer, PartialPatternBuffer,
                                 SemanticEvent)

LFM2_TOOL_OPEN, LFM2_TOOL_CLOSE = "<|tool_call_start|>", "<|tool_call_end|>"
_JSON_NAMES = {"true": True, "false": False, "null": None, "True": True, "False": False, "None": None}


def _literal(node):
    """Value of an argument expression: Python / JSON literals, nested lists and dicts, negative numbers."""
    if isinstance(node, ast.Name) and node.id in _JSON_NAMES:
        return _JSON_NAMES[node.id]
    if isinstance(node, (ast.List, ast.Tuple)):
        return [_literal(e) for e in node.elts]
    if isinstance(node, ast.Dict):
        return {str(_literal(k)): _literal(v) for k, v in zip(node.keys, node.values)}
    return ast.literal_eval(node)


def parse_python_calls(text: str) -> list[dict]:
    """``[f(a=1, b="x"), g()]`` (or a single call) -> ``[{"name": "f", "arguments": {...}}, ...]``.
    Raises ValueError for anything that is not a list of calls with keyword arguments."""
    src = text.strip()
    try:
        tree = ast.parse(src, mode="eval").body
    except SyntaxError as e:
        raise ValueError(f"not a Python call list: {e}") from None
    nodes = tree.elts if isinstance(tree, (ast.List, ast.Tuple)) else [tree]
    calls = []
    for n in nodes:
        if not isinstance(n, ast.Call):
            raise ValueError("tool call block must contain function calls only")
        f = n.func
        parts = []
        while isinstance(f, ast.Attribute):
            parts.append(f.attr)
            f = f.value
        if not isinstance(f, ast.Name):
            raise ValueError("unsupported callee expression")
        parts.append(f.id)
        if n.args:
            raise ValueError("tool arguments must be passed by keyword")
        try:
            args = {kw.arg: _literal(kw.value) for kw in n.keywords if kw.arg is not None}
        except (ValueError, SyntaxError) as e:
            raise ValueError(f"unsupported argument expression: {e}") from None
        calls.append({"name": ".".join(reversed(parts)), "arguments": args})
    return calls


_FUNCTION = re.compile(r"<function=([^>\s]+)>(.*?)(?:</function>|\Z)", re.S)
_PARAMETER = re.compile(r"<parameter=([^>\s]+)>\n?(.*?)\n?</parameter>", re.S)


def parse_tagged_call(raw: str, tools=None) -> list[dict]:
    """Qwen tagged-parameter syntax inside a tool-call block::

        <function=NAME>
        <parameter=KEY>
        VALUE
        </parameter>
        </function>

    Values are text; a declared parameter of type integer / number / boolean / object / array / null (or a value
    that only parses as JSON when no schema is known) is converted, strings stay as written."""
    schemas = {}
    for t in tools or []:
        f = t.get("function", t)
        schemas[f.get("name")] = (f.get("parameters") or {}).get("properties", {})
    calls = []
    for name, body in _FUNCTION.findall(raw):
        props = schemas.get(name, {})
        args = {}
        for key, val in _PARAMETER.findall(body):
            kind = (props.get(key) or {}).get("type")
            if kind == "string":
                args[key] = val
                continue
            try:
                parsed = json.loads(val)
            except json.JSONDecodeError:
                parsed = val
            args[key] = val if (kind is None and isinstance(parsed, str)) else parsed
        calls.append({"name": name, "arguments": args})
    if not calls:
        raise ValueError("no <function=...> block found")
    return calls


class Lfm2Pipeline(CommittedTokenPipeline):
    """Generic pipeline with the tool body parsed as a Python call list: every call of the block becomes one tool
    call (the first one was announced when the block opened, the others are announced when it closes)."""

    def _tool_fragment(self, text: str, out: list):
        self.tool_json.text += text
        self._emit(SemanticEvent("tool_call_arguments", text, tool_index=self.tool_count - 1), out)

    def _close_tool(self, out: list):
        raw = self.tool_json.text.strip()
        try:
            calls = parse_python_calls(raw)
        except ValueError:
            calls = [{"name": None, "arguments": None}]
        first = self.tool_count - 1
        for j, c in enumerate(calls):
            if self.max_tools is not None and first + j >= self.max_tools:
                break
            if j > 0:
                self.tool_count += 1
                self._emit(SemanticEvent("tool_call_start", tool_index=first + j), out)
            self.tool_calls.append({"name": c["name"], "arguments": c["arguments"], "raw": raw})
            self._emit(SemanticEvent("tool_call_end", tool_name=c["name"], tool_index=first + j, arguments=c["arguments"]), out)
        self.state = "text"
        self._retarget()


_HARMONY_END = ("<|end|>", "<|return|>", "<|call|>")
_RECIPIENT = re.compile(r"to=([^\s<]+)")


class HarmonyPipeline:
    """Streaming parser of the Harmony message format. The prompt ends inside a header (``<|start|>assistant``), so
    the parser starts in the header state."""

    def __init__(self, decoder, plan=None, stop=(), on_event: Optional[Callable[[SemanticEvent], None]] = None,
                 max_parallel_tool_calls: Optional[int] = None):
        self.decoder = decoder
        self.plan = plan
        self.on_event = on_event
        self.stop = [s for s in stop if s]
        self.max_tools = max_parallel_tool_calls
        self.finished: Optional[str] = None
        self.text_out: list[str] = []
        self.reasoning_out: list[str] = []
        self.tool_calls: list[dict] = []
        self.tool_count = 0
        self.state = "header"
        self.header = ""
        self.channel = None
        self.recipient = None
        self.body: Optional[JsonFragmentBuffer] = None
        self.matcher = PartialPatternBuffer(["<|message|>"])

    # ---- helpers
    def _emit(self, ev: SemanticEvent, out: list):
        out.append(ev)
        if self.on_event:
            self.on_event(ev)

    def _set_state(self, state: str):
        held = self.matcher.flush()
        self.state = state
        if state == "header":
            pats = ["<|message|>"]
        elif state == "body":
            pats = list(_HARMONY_END) + ["<|start|>"] + (self.stop if self.channel == "final" else [])
        else:  # between messages
            pats = ["<|start|>"]
        self.matcher = PartialPatternBuffer(pats)
        return held

    def _open_body(self, out: list):
        h = self.header.replace("<|constrain|>", " ")
        m = _RECIPIENT.search(h)
        self.recipient = m.group(1) if m else None
        chan = h.split("<|channel|>", 1)[1] if "<|channel|>" in h else ""
        self.channel = (chan.split() or ["final"])[0]
        self.header = ""
        if self.recipient and self.recipient.startswith("functions."):
            if self.max_tools is not None and self.tool_count >= self.max_tools:
                self.finished = FinishReason.GRAMMAR_COMPLETE
                return
            self.channel = "tool"
            self.body = JsonFragmentBuffer()
            self.tool_count += 1
            self._emit(SemanticEvent("tool_call_start", tool_name=self.recipient[len("functions."):],
                                     tool_index=self.tool_count - 1), out)

    def _content(self, text: str, out: list):
        if not text:
            return
        if self.state == "header":
            self.header += text
        elif self.state == "body":
            if self.channel == "tool":
                self.body.text += text
                self._emit(SemanticEvent("tool_call_arguments", text, tool_index=self.tool_count - 1), out)
            elif self.channel == "final":
                self.text_out.append(text)
                self._emit(SemanticEvent("text", text), out)
            else:  # analysis and commentary preambles are shown as reasoning
                self.reasoning_out.append(text)
                self._emit(SemanticEvent("reasoning", text), out)

    def _close_body(self, out: list):
        if self.channel == "tool" and self.body is not None:
            raw = self.body.text.strip()
            try:
                args = json.loads(raw) if raw else {}
            except json.JSONDecodeError:
                args = None
            name = self.recipient[len("functions."):]
            self.tool_calls.append({"name": name, "arguments": args, "raw": raw})
            self._emit(SemanticEvent("tool_call_end", tool_name=name, tool_index=self.tool_count - 1, arguments=args), out)
            self.body = None

    def _feed(self, text: str, out: list):
        while text and not self.finished:
            released, hit = self.matcher.push(text)
            text = ""
            self._content(released, out)
            if hit is None:
                return
            if hit in self.stop and self.state == "body":
                self.finished = FinishReason.STOP_SEQUENCE
                return
            if hit == "<|message|>":
                self._open_body(out)
                text = self._set_state("body")
            elif hit in _HARMONY_END:
                was_tool = self.channel == "tool"
                self._close_body(out)
                if hit == "<|return|>":
                    self.finished = FinishReason.EOS
                    return
                if hit == "<|call|>" or was_tool:
                    self.finished = FinishReason.GRAMMAR_COMPLETE if hit != "<|call|>" else FinishReason.EOS
                    return
                text = self._set_state("between")
            elif hit == "<|start|>":
                if self.state == "body":
                    self._close_body(out)
                text = self._set_state("header")

    # ---- pipeline interface
    def push(self, token_id: int) -> list:
        out: list = []
        if not self.finished:
            self._feed(self.decoder.push(token_id), out)
        return out

    def finish(self, reason: str) -> list:
        out: list = []
        if not self.finished:
            tail = self.decoder.flush()
            if tail:
                self._feed(tail, out)
        if not self.finished:
            held = self.matcher.flush()
            if held and self.state == "body":
                self._content(held, out)
            if self.state == "body":
                self._close_body(out)    # the end token was the EOS id and never reached the text stream
        final = FinishReason.resolve([self.finished, reason]) if reason != FinishReason.CANCELLED else (self.finished or reason)
        self.finished = final
        self._emit(SemanticEvent("finished", finish_reason=final), out)
        return out


def pipeline_for(plan) -> type:
    """Pipeline class for a parser plan's dialect."""
    dialect = getattr(plan, "dialect", "generic") if plan is not None else "generic"
    return {"lfm2": Lfm2Pipeline, "harmony": HarmonyPipeline}.get(dialect, CommittedTokenPipeline)
