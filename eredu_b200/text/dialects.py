"""Checkpoint-specific chat surface syntaxes on top of the committed-token pipeline.

* LFM2: tool calls are a Python-style call list between ``<|tool_call_start|>`` and ``<|tool_call_end|>``, e.g.
  ``[get_weather(city="Paris", days=3), now()]`` (eredu/src/runtime/chat/lfm2.rs:1-40: structural tokens, stops; the
  module's incremental normaliser turns the calls into name + JSON arguments).
* Harmony (GPT-OSS): a message is ``<|start|>ROLE[ to=RECIPIENT]<|channel|>CHANNEL[ to=RECIPIENT][ <|constrain|>TYPE]
  <|message|>BODY`` closed by ``<|end|>`` (more messages follow), ``<|return|>`` (final answer done) or ``<|call|>``
  (tool call issued). The ``analysis`` channel is reasoning, ``final`` is the reply, ``commentary`` addressed to
  ``functions.NAME`` is a tool call whose body is the JSON arguments (eredu/src/runtime/chat/harmony.rs).

* Gemma 4: reasoning travels in ``<|channel>thought\n ... <channel|>``, a tool call is ``<|tool_call>call:NAME{key:value,
  ...}<tool_call|>`` - an object with bare keys whose strings are delimited by the ``<|"|>`` token; ``<|tool_response>`` and
  ``<turn|>`` end the turn (eredu/src/runtime/chat/gemma.rs:14-20, eredu/src/runtime/chat/mod.rs:982-1022).

* Inkling: every model message is ``<|message_model|>`` + a content marker + body + ``<|end_message|>``; the marker is
  ``<|content_thinking|>`` (reasoning), ``<|content_text|>`` (reply) or, after the tool's name,
  ``<|content_invoke_tool_json|>`` with a ``{"name", "args"}`` object; ``<|content_model_end_sampling|>`` ends the turn
  (eredu/src/runtime/chat/inkling.rs:17-22).
* ATEM (Muse-Glimmer): messages are ``<|start|>HEADER<|message|>BODY`` closed by ``<|eom|>`` (more follow) or ``<|eot|>``
  (turn over); the header's ``to=`` names the recipient: ``self`` is reasoning, ``user`` the reply, anything else a tool
  whose body is ``<atem:function_calls><atem:invoke name=".."><atem:parameter name="..">VALUE</atem:parameter>..``
  (eredu/src/runtime/chat/atem.rs:15-18).

All parsers keep the interface of :class:`eredu_b200.runtime.streaming.CommittedTokenPipeline` (``push`` /
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


GEMMA_CHANNEL_OPEN, GEMMA_CHANNEL_CLOSE = "<|channel>", "<channel|>"
GEMMA_TOOL_OPEN, GEMMA_TOOL_CLOSE = "<|tool_call>", "<tool_call|>"
GEMMA_STRING = '<|"|>'
GEMMA_STOPS = ("<|tool_response>", "<turn|>")


def parse_structural_object(text: str, string_delimiter: str = GEMMA_STRING):
    """``{count:2,enabled:true,place:<|"|>Bogota<|"|>,tags:[<|"|>a<|"|>]}`` -> Python value. Keys are bare (up to the
    colon), strings sit between two delimiter tokens and are taken verbatim, scalars are JSON scalars; duplicate keys and
    trailing text are errors."""
    pos = 0
    n = len(text)

    def ws():
        nonlocal pos
        while pos < n and text[pos].isspace():
            pos += 1

    def value():
        nonlocal pos
        ws()
        if text.startswith(string_delimiter, pos):
            end = text.find(string_delimiter, pos + len(string_delimiter))
            if end < 0:
                raise ValueError("unterminated string")
            out = text[pos + len(string_delimiter):end]
            pos = end + len(string_delimiter)
            return out
        if pos < n and text[pos] == "{":
            return obj()
        if pos < n and text[pos] == "[":
            pos += 1
            items = []
            ws()
            if pos < n and text[pos] == "]":
                pos += 1
                return items
            while True:
                items.append(value())
                ws()
                if pos < n and text[pos] == ",":
                    pos += 1
                    continue
                if pos < n and text[pos] == "]":
                    pos += 1
                    return items
                raise ValueError("expected ',' or ']' in array")
        start = pos
        while pos < n and text[pos] not in ",}]" and not text[pos].isspace():
            pos += 1
        raw = text[start:pos]
        try:
            val = json.loads(raw)
        except json.JSONDecodeError:
            raise ValueError(f"invalid scalar {raw!r}") from None
        if isinstance(val, (dict, list, str)):
            raise ValueError(f"invalid scalar {raw!r}")
        return val

    def obj():
        nonlocal pos
        ws()
        if pos >= n or text[pos] != "{":
            raise ValueError("expected '{'")
        pos += 1
        out: dict = {}
        ws()
        if pos < n and text[pos] == "}":
            pos += 1
            return out
        while True:
            ws()
            colon = text.find(":", pos)
            if colon < 0:
                raise ValueError("expected ':' after a key")
            key = text[pos:colon].strip()
            if not key or any(c in key for c in "{}[],") or string_delimiter in key:
                raise ValueError(f"invalid key {key!r}")
            if key in out:
                raise ValueError(f"duplicate key {key!r}")
            pos = colon + 1
            out[key] = value()
            ws()
            if pos < n and text[pos] == ",":
                pos += 1
                continue
            if pos < n and text[pos] == "}":
                pos += 1
                return out
            raise ValueError("expected ',' or '}' in object")

    result = obj()
    ws()
    if pos != n:
        raise ValueError("text after the object")
    return result


def parse_gemma_call(raw: str) -> dict:
    """``call:NAME{...}`` -> ``{"name": NAME, "arguments": {...}}``."""
    body = raw.strip()
    if not body.startswith("call:"):
        raise ValueError("a Gemma tool call starts with 'call:'")
    brace = body.find("{")
    if brace < 0:
        raise ValueError("a Gemma tool call needs an argument object")
    name = body[len("call:"):brace].strip()
    if not name:
        raise ValueError("a Gemma tool call needs a name")
    return {"name": name, "arguments": parse_structural_object(body[brace:])}


class GemmaPipeline(CommittedTokenPipeline):
    """Generic pipeline (reasoning channel and call envelope come from the plan's tags) with the call payload in the
    structural-object syntax. A channel other than ``thought`` is shown as written."""

    def _tool_fragment(self, text: str, out: list):
        self.tool_json.text += text
        self._emit(SemanticEvent("tool_call_arguments", text, tool_index=self.tool_count - 1), out)

    def _close_tool(self, out: list):
        raw = self.tool_json.text.strip()
        try:
            call = parse_gemma_call(raw)
        except ValueError:
            call = {"name": None, "arguments": None}
        self.tool_calls.append({"name": call["name"], "arguments": call["arguments"], "raw": raw})
        self._emit(SemanticEvent("tool_call_end", tool_name=call["name"], tool_index=self.tool_count - 1,
                                 arguments=call["arguments"]), out)
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


class _MarkerPipeline:
    """Shared plumbing of the marker-driven dialects: the generated text is cut at a fixed set of marker strings;
    subclasses decide what a marker means (``_marker``) and where text goes (``_content``)."""

    MARKERS: tuple = ()

    def __init__(self, decoder, plan=None, stop=(), on_event: Optional[Callable[[SemanticEvent], None]] = None,
                 max_parallel_tool_calls: Optional[int] = None):
        self.decoder, self.plan, self.on_event = decoder, plan, on_event
        self.stop = [s for s in stop if s]
        self.max_tools = max_parallel_tool_calls
        self.finished: Optional[str] = None
        self.text_out: list[str] = []
        self.reasoning_out: list[str] = []
        self.tool_calls: list[dict] = []
        self.tool_count = 0
        self.tools = None
        self.matcher = PartialPatternBuffer(list(self.MARKERS) + self.stop)

    def _emit(self, ev: SemanticEvent, out: list):
        out.append(ev)
        if self.on_event:
            self.on_event(ev)

    def _say(self, kind: str, text: str, out: list):
        if not text:
            return
        (self.text_out if kind == "text" else self.reasoning_out).append(text)
        self._emit(SemanticEvent(kind, text), out)

    def _open_tool(self, name, out: list) -> bool:
        if self.max_tools is not None and self.tool_count >= self.max_tools:
            self.finished = FinishReason.GRAMMAR_COMPLETE
            return False
        self.tool_count += 1
        self._emit(SemanticEvent("tool_call_start", tool_name=name, tool_index=self.tool_count - 1), out)
        return True

    def _end_tool(self, name, args, raw: str, out: list):
        self.tool_calls.append({"name": name, "arguments": args, "raw": raw})
        self._emit(SemanticEvent("tool_call_end", tool_name=name, tool_index=self.tool_count - 1, arguments=args), out)

    def _feed(self, text: str, out: list):
        while text and not self.finished:
            released, hit = self.matcher.push(text)
            text = ""
            self._content(released, out)
            if hit is None:
                return
            if hit in self.stop and hit not in self.MARKERS:
                if self._stop_allowed():
                    self.finished = FinishReason.STOP_SEQUENCE
                    return
                self._content(hit, out)
            else:
                self._marker(hit, out)
            text = self.matcher.flush()

    def _stop_allowed(self) -> bool:
        return True

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
            self._content(self.matcher.flush(), out)
            self._close(out)
        final = FinishReason.resolve([self.finished, reason]) if reason != FinishReason.CANCELLED else (self.finished or reason)
        self.finished = final
        self._emit(SemanticEvent("finished", finish_reason=final), out)
        return out

    def _close(self, out: list):
        pass


INK_MESSAGE, INK_TEXT, INK_THINKING = "<|message_model|>", "<|content_text|>", "<|content_thinking|>"
INK_TOOL, INK_END, INK_END_SAMPLING = "<|content_invoke_tool_json|>", "<|end_message|>", "<|content_model_end_sampling|>"


class InklingPipeline(_MarkerPipeline):
    """The prompt ends with ``<|message_model|>``, so parsing starts in a message header (where a tool's name may stand)."""

    MARKERS = (INK_MESSAGE, INK_TEXT, INK_THINKING, INK_TOOL, INK_END, INK_END_SAMPLING)

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.state = "header"          # header | text | thinking | tool | between
        self.header = ""
        self.body = ""

    def _content(self, text: str, out: list):
        if not text:
            return
        if self.state == "header":
            self.header += text
        elif self.state == "text":
            self._say("text", text, out)
        elif self.state == "thinking":
            self._say("reasoning", text, out)
        elif self.state == "tool":
            self.body += text
            self._emit(SemanticEvent("tool_call_arguments", text, tool_index=self.tool_count - 1), out)

    def _marker(self, m: str, out: list):
        if m == INK_MESSAGE and self.state == "between":
            self.state, self.header = "header", ""
        elif m in (INK_TEXT, INK_THINKING) and self.state == "header":
            self.state = "text" if m == INK_TEXT else "thinking"
        elif m == INK_TOOL and self.state == "header":
            if self._open_tool(self.header.strip() or None, out):
                self.state, self.body = "tool", ""
        elif m == INK_END and self.state in ("text", "thinking", "tool"):
            if self.state == "tool":
                self._finish_call(out)
            self.state = "between"
        elif m == INK_END_SAMPLING and self.state == "between":
            self.finished = FinishReason.STOP_SEQUENCE
        else:                           # a marker where the protocol has none: shown as written, never a state change
            self._content(m, out)

    def _finish_call(self, out: list):
        raw = self.body.strip()
        name, args = self.header.strip() or None, None
        try:
            obj = json.loads(raw)
            if isinstance(obj, dict):
                name = obj.get("name", name)
                args = obj.get("args", obj.get("arguments"))
        except json.JSONDecodeError:
            pass
        self._end_tool(name, args, raw, out)

    def _close(self, out: list):
        if self.state == "tool":
            self._finish_call(out)


ATEM_START, ATEM_MESSAGE, ATEM_EOM, ATEM_EOT = "<|start|>", "<|message|>", "<|eom|>", "<|eot|>"
_ATEM_INVOKE = re.compile(r'<atem:invoke\s+name="([^"]*)"\s*>(.*?)</atem:invoke>', re.S)
_ATEM_PARAM = re.compile(r'<atem:parameter\s+name="([^"]*)"\s*>(.*?)</atem:parameter>', re.S)


def parse_atem_calls(body: str, tools=None) -> list[dict]:
    """``<atem:function_calls>`` envelope -> calls. Values are XML-escaped text; a value becomes a JSON scalar / array /
    object when it parses as one, unless the tool declares the parameter as a string."""
    from xml.sax.saxutils import unescape

    schemas = {}
    for t in tools or []:
        f = t.get("function", t)
        schemas[f.get("name")] = (f.get("parameters") or {}).get("properties", {})
    calls = []
    for name, inner in _ATEM_INVOKE.findall(body):
        name = unescape(name, {"&quot;": '"'})
        props = schemas.get(name, {})
        args = {}
        for key, val in _ATEM_PARAM.findall(inner):
            key, val = unescape(key, {"&quot;": '"'}), unescape(val, {"&quot;": '"', "&apos;": "'"})
            if (props.get(key) or {}).get("type") == "string":
                args[key] = val
                continue
            try:
                args[key] = json.loads(val)
            except json.JSONDecodeError:
                args[key] = val
        calls.append({"name": name, "arguments": args})
    if not calls:
        raise ValueError("no <atem:invoke> element found")
    return calls


class AtemPipeline(_MarkerPipeline):
    """The prompt ends inside the assistant's header (after ``<|start|>assistant`` or just ``<|start|>``)."""

    MARKERS = (ATEM_START, ATEM_MESSAGE, ATEM_EOM, ATEM_EOT)

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.state = "header"          # header | body | between
        self.header = ""
        self.recipient = None
        self.body = ""

    def _content(self, text: str, out: list):
        if not text:
            return
        if self.state == "header":
            self.header += text
        elif self.state == "body":
            if self.recipient == "self":
                self._say("reasoning", text, out)
            elif self.recipient in (None, "user"):
                self._say("text", text, out)
            else:
                self.body += text
                self._emit(SemanticEvent("tool_call_arguments", text, tool_index=self.tool_count - 1), out)

    def _marker(self, m: str, out: list):
        if m == ATEM_MESSAGE and self.state == "header":
            found = _RECIPIENT.search(self.header)
            self.recipient = found.group(1) if found else None
            self.state, self.body = "body", ""
            if self.recipient not in (None, "self", "user") and not self._open_tool(self.recipient, out):
                return
        elif m in (ATEM_EOM, ATEM_EOT) and self.state == "body":
            self._close(out)
            self.state = "between"
            if m == ATEM_EOT:
                self.finished = FinishReason.EOS
        elif m == ATEM_START and self.state == "between":
            self.state, self.header = "header", ""
        else:
            self._content(m, out)

    def _close(self, out: list):
        if self.state != "body" or self.recipient in (None, "self", "user"):
            return
        raw = self.body.strip()
        try:
            calls = parse_atem_calls(raw, self.tools)
        except ValueError:
            calls = [{"name": self.recipient, "arguments": None}]
        for j, c in enumerate(calls):
            if j > 0 and not self._open_tool(c["name"], out):
                break
            self._end_tool(c["name"], c["arguments"], raw, out)


def pipeline_for(plan) -> type:
    """Pipeline class for a parser plan's dialect."""
    dialect = getattr(plan, "dialect", "generic") if plan is not None else "generic"
    return {"lfm2": Lfm2Pipeline, "harmony": HarmonyPipeline, "gemma": GemmaPipeline, "inkling": InklingPipeline,
            "atem": AtemPipeline}.get(dialect, CommittedTokenPipeline)
