"""Grammar constraints for tool calls: the declared tools become a JSON schema, the schema a grammar, the grammar
per-step token masks (llguidance), so that a generated call always names a declared tool and carries arguments that
satisfy its parameter schema.

Counterpart of eredu/src/runtime/chat/constraints.rs (``parse_tools`` :897, ``tool_call_bounds`` :813-843,
``tool_call_schema`` :845-895, trigger matching :346-420, ``compile_tool_plan`` :615): with ``tool_choice = required``
the grammar is active from the first token and demands between one and the parallel-call limit of calls; with ``auto``
generation is free until the call-opening tag has been produced, then the call body is constrained until its closing
tag, then generation is free again (until the call limit is reached).
"""
from __future__ import annotations

import json
from typing import Optional

import torch

from ..ops.controlled import GrammarConstraint
from ..runtime.streaming import PartialPatternBuffer


def parse_tools(tools: list) -> list[tuple[str, dict]]:
    """(name, parameter schema) of every declared tool; accepts the OpenAI wrapper ``{"type": "function", "function":
    {...}}`` and the bare ``{"name", "parameters"}`` form."""
    out = []
    for i, t in enumerate(tools or []):
        f = t.get("function", t) if isinstance(t, dict) else None
        if not isinstance(f, dict) or not isinstance(f.get("name"), str) or not f["name"]:
            raise ValueError(f"tool {i} has no function name")
        params = f.get("parameters") or {"type": "object", "properties": {}}
        if not isinstance(params, dict):
            raise ValueError(f"tool {f['name']!r}: parameters must be a JSON schema object")
        out.append((f["name"], params))
    names = [n for n, _ in out]
    if len(set(names)) != len(names):
        raise ValueError("tool names must be unique")
    return out


def tool_call_bounds(mode: str, max_parallel_calls: Optional[int], tools: list) -> tuple[int, Optional[int]]:
    """(minimum, maximum) number of calls a reply may contain; maximum None = unbounded."""
    if mode == "required" and not tools:
        raise ValueError("tool_choice is required but no tools were supplied")
    if mode == "none":
        return 0, 0
    lo = 1 if mode == "required" else 0
    hi = max_parallel_calls
    if hi is not None and hi < lo:
        raise ValueError("parallel tool-call limit cannot satisfy tool_choice")
    return lo, hi


def tool_call_schema(tools: list, name_field: str = "name", arguments_field: str = "arguments") -> dict:
    """JSON schema of one call object: any of the declared tools with its own argument schema."""
    items = [{"type": "object",
              "properties": {name_field: {"const": name}, arguments_field: params},
              "required": [name_field, arguments_field], "additionalProperties": False}
             for name, params in parse_tools(tools)]
    if not items:
        return {"type": "null"}
    return items[0] if len(items) == 1 else {"anyOf": items}


def _tag(tokenizer, text: str) -> str:
    """Grammar spelling of a structural tag: the special token itself when the vocabulary has one, else its text."""
    tok = getattr(tokenizer, "tokenizer", tokenizer)
    tid = tok.token_to_id(text) if hasattr(tok, "token_to_id") else None
    if tid is not None and len(tok.encode(text, add_special_tokens=False).ids) == 1:
        return f"<[{tid}]>"
    return json.dumps(text)


def call_body_grammar(tokenizer, tools: list, close: Optional[str]) -> str:
    """Grammar of what follows the opening tag: optional newline, the call object, optional newline, the closing tag."""
    schema = json.dumps(tool_call_schema(tools))
    tail = f' {_tag(tokenizer, close)}' if close else ""
    return f'start: NL? call NL?{tail}\ncall: %json {schema}\nNL: "\\n"\n'


def required_calls_grammar(tokenizer, tools: list, open_tag: str, close: Optional[str], lo: int, hi: Optional[int]) -> str:
    schema = json.dumps(tool_call_schema(tools))
    tail = f' {_tag(tokenizer, close)}' if close else ""
    rep = f"{{{lo},{hi}}}" if hi is not None else (f"{{{lo},}}" if lo != 1 else "+")
    return (f'start: (block NL?){rep}\nblock: {_tag(tokenizer, open_tag)} NL? call NL?{tail}\n'
            f'call: %json {schema}\nNL: "\\n"\n')


class TriggeredToolConstraint:
    """``tool_choice = auto``: unconstrained until the opening tag appears in the committed text, constrained to one
    call body (up to the closing tag) after it. Same interface as :class:`GrammarConstraint`."""

    def __init__(self, tokenizer_bundle, tools: list, open_tag: str, close_tag: Optional[str], max_calls: Optional[int] = None):
        self.bundle = tokenizer_bundle
        self.tools, self.open_tag, self.close_tag = tools, open_tag, close_tag
        self.max_calls = max_calls
        self.calls = 0
        self.active: Optional[GrammarConstraint] = None
        self._body = call_body_grammar(tokenizer_bundle, tools, close_tag)
        self._watch = PartialPatternBuffer([open_tag])
        from .tokenizer import TextDecoder

        self._decoder = TextDecoder(tokenizer_bundle, skip_special_tokens=False)
        self.vocab_size = None

    def allow_mask(self, vocab_size: Optional[int] = None) -> torch.Tensor:
        if self.active is not None:
            return self.active.allow_mask(vocab_size)
        return torch.ones(vocab_size or self.bundle.vocab_size(), dtype=torch.bool)

    def commit(self, token: int) -> None:
        if self.active is not None:
            self.active.commit(token)
            if self.active.is_complete():
                self.active = None
                self.calls += 1
                self._watch = PartialPatternBuffer([self.open_tag])
            return
        _, hit = self._watch.push(self._decoder.push(token))
        if hit is not None and (self.max_calls is None or self.calls < self.max_calls):
            self.active = GrammarConstraint(self.bundle, "lark", self._body)

    def is_complete(self) -> bool:
        """The reply must end: the call limit has been reached and the last call is closed."""
        return self.active is None and self.max_calls is not None and self.calls >= self.max_calls and self.calls > 0

    def is_accepting(self) -> bool:
        return self.active is None


def constraint_for_tools(tokenizer_bundle, tools: list, mode: str, max_parallel_calls: Optional[int], open_tag: str,
                         close_tag: Optional[str]):
    """Constraint object for a prepared chat's tool policy, or None when nothing has to be enforced."""
    lo, hi = tool_call_bounds(mode, max_parallel_calls, tools)
    if not tools or hi == 0:
        return None
    if mode == "required":
        return GrammarConstraint(tokenizer_bundle, "lark", required_calls_grammar(tokenizer_bundle, tools, open_tag, close_tag, lo, hi))
    return TriggeredToolConstraint(tokenizer_bundle, tools, open_tag, close_tag, hi)
