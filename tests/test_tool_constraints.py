"""Tool-call constraints: schema of the declared tools, call bounds, required and triggered (auto) enforcement."""
import dataclasses
import json

import pytest
import torch

pytest.importorskip("llguidance")

from eredu_b200.ops.controlled import GrammarConstraint
from eredu_b200.text.tool_constraints import (TriggeredToolConstraint, constraint_for_tools, parse_tools, required_calls_grammar,
                                              tool_call_bounds, tool_call_schema)
from test_text_streaming import make_bundle

TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {
    "type": "object", "properties": {"city": {"type": "string", "enum": ["Paris", "Rome"]},
                                     "days": {"type": "integer", "minimum": 1, "maximum": 3}},
    "required": ["city"], "additionalProperties": False}}},
    {"name": "now", "parameters": {"type": "object", "properties": {}, "additionalProperties": False}}]


def test_tool_parsing_bounds_and_schema():
    assert [n for n, _ in parse_tools(TOOLS)] == ["get_weather", "now"]
    with pytest.raises(ValueError):
        parse_tools([{"function": {}}])
    with pytest.raises(ValueError):
        parse_tools([{"name": "a"}, {"name": "a"}])
    assert tool_call_bounds("none", None, TOOLS) == (0, 0) and tool_call_bounds("auto", None, TOOLS) == (0, None)
    assert tool_call_bounds("required", 2, TOOLS) == (1, 2)
    with pytest.raises(ValueError):
        tool_call_bounds("required", None, [])
    with pytest.raises(ValueError):
        tool_call_bounds("required", 0, TOOLS)
    schema = tool_call_schema(TOOLS)
    assert [s["properties"]["name"]["const"] for s in schema["anyOf"]] == ["get_weather", "now"]
    assert tool_call_schema([]) == {"type": "null"}


def accepts(b, grammar, text):
    c = GrammarConstraint(b, "lark", grammar)
    try:
        for t in b.encode(text):
            c.commit(t)
    except ValueError:
        return False
    return c.is_accepting()


def test_required_grammar_accepts_only_declared_calls():
    b = make_bundle()
    g = required_calls_grammar(b, TOOLS, "<tool_call>", "</tool_call>", 1, 2)
    ok = '<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris", "days": 2}}\n</tool_call>'
    assert accepts(b, g, ok)
    assert accepts(b, g, ok + '\n<tool_call>{"name": "now", "arguments": {}}</tool_call>')
    assert not accepts(b, g, ok + ok + ok)                                              # at most two calls
    assert not accepts(b, g, '<tool_call>{"name": "launch", "arguments": {}}</tool_call>')
    assert not accepts(b, g, '<tool_call>{"name": "get_weather", "arguments": {"city": "Oslo"}}</tool_call>')
    assert not accepts(b, g, '<tool_call>{"name": "get_weather", "arguments": {"city": "Rome", "days": 9}}</tool_call>')
    assert not accepts(b, g, 'Sure! <tool_call>{"name": "now", "arguments": {}}</tool_call>')   # required: no free text first
    assert constraint_for_tools(b, TOOLS, "none", None, "<tool_call>", "</tool_call>") is None
    assert constraint_for_tools(b, [], "auto", None, "<tool_call>", "</tool_call>") is None


def test_triggered_constraint_only_binds_inside_a_call():
    b = make_bundle()
    c = constraint_for_tools(b, TOOLS, "auto", 1, "<tool_call>", "</tool_call>")
    assert isinstance(c, TriggeredToolConstraint)
    V = b.vocab_size()
    for t in b.encode("Let me look that up. <tool_call>"):
        assert bool(c.allow_mask(V).all()) and c.is_accepting()
        c.commit(t)
    assert c.active is not None and not c.is_accepting()
    mask = c.allow_mask(V)
    assert not bool(mask.all()) and bool(mask[b.encode("{")[0]]) and not bool(mask[b.encode("x")[0]])
    with pytest.raises(ValueError):
        c.commit(b.encode("x")[0])
    for t in b.encode('{"name": "now", "arguments": {}}</tool_call>'):
        c.commit(t)
    assert c.active is None and c.calls == 1 and c.is_complete()          # the single allowed call has been made


def test_required_tool_choice_end_to_end(tmp_path):
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models import config as C
    from eredu_b200.models.llama import random_state
    from eredu_b200.ops import SamplingParams
    from eredu_b200.text.chat import ToolChoice

    b = make_bundle(tmp_path)
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=b.vocab_size(), eos_token_id=b.eos_ids[0])
    ck.save_safetensors_checkpoint(tmp_path, cfg, random_state(cfg, seed=0, std=0.05), torch.float32)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=512))
    chat = lm.prepare_chat([{"role": "user", "content": "weather?"}], tools=TOOLS, tool_choice=ToolChoice("required", 1))
    res = lm.generate_prepared_chat(chat, SamplingParams(temperature=0.8, seed=3), max_new_tokens=200)
    assert res["finish_reason"] in ("grammar_complete", "eos") and len(res["tool_calls"]) == 1, res
    call = res["tool_calls"][0]
    assert call["name"] in ("get_weather", "now") and isinstance(call["arguments"], dict)
    if call["name"] == "get_weather":
        assert call["arguments"]["city"] in ("Paris", "Rome")
    json.loads(call["raw"])
