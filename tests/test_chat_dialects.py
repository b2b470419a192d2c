"""LFM2 Python-call tool syntax and Harmony channels on the streaming pipeline."""
import pytest

from eredu_b200.runtime.streaming import FinishReason
from eredu_b200.text.chat import ParserPlan, detect_plan
from eredu_b200.text.dialects import HarmonyPipeline, Lfm2Pipeline, parse_python_calls, pipeline_for


class PieceDecoder:
    """Stands in for the detokeniser: token i is the i-th text piece."""

    def __init__(self, pieces):
        self.pieces = pieces

    def push(self, i):
        return self.pieces[i]

    def flush(self):
        return ""


def run(cls, plan, text, chunk=3, stop=(), max_tools=None, reason=FinishReason.EOS):
    pieces = [text[i:i + chunk] for i in range(0, len(text), chunk)]     # tags get split across tokens
    pipe = cls(PieceDecoder(pieces), plan, stop, None, max_tools)
    events = []
    for i in range(len(pieces)):
        events += pipe.push(i)
        if pipe.finished:
            break
    events += pipe.finish(reason)
    return pipe, events


def test_python_call_parser():
    calls = parse_python_calls('[get_weather(city="Paris", days=3, units=None), now()]')
    assert calls == [{"name": "get_weather", "arguments": {"city": "Paris", "days": 3, "units": None}},
                     {"name": "now", "arguments": {}}]
    assert parse_python_calls('f(x=[1, -2.5, {"a": true}], y=false, z=null)')[0]["arguments"] == \
        {"x": [1, -2.5, {"a": True}], "y": False, "z": None}
    assert parse_python_calls("ns.tool(a='b')")[0]["name"] == "ns.tool"
    for bad in ("[1, 2]", "f(1)", "f(x=open('a'))", "import os", "f(x=__import__('os'))"):
        with pytest.raises(ValueError):
            parse_python_calls(bad)


def test_lfm2_tool_block_streams_as_tool_calls():
    plan = detect_plan("...<|tool_call_start|>...", "", tools=[{"name": "get_weather"}])
    assert plan.dialect == "lfm2" and plan.render_special_tokens and pipeline_for(plan) is Lfm2Pipeline
    text = 'Let me check.<|tool_call_start|>[get_weather(city="Paris"), get_time(tz="CET")]<|tool_call_end|>Done.'
    pipe, events = run(Lfm2Pipeline, plan, text)
    assert "".join(pipe.text_out) == "Let me check.Done."
    assert [(c["name"], c["arguments"]) for c in pipe.tool_calls] == [("get_weather", {"city": "Paris"}), ("get_time", {"tz": "CET"})]
    kinds = [e.kind for e in events if e.kind.startswith("tool_call") and e.kind != "tool_call_arguments"]
    assert kinds == ["tool_call_start", "tool_call_end", "tool_call_start", "tool_call_end"]
    assert [e.tool_index for e in events if e.kind == "tool_call_end"] == [0, 1]
    # the parallel-call limit drops the calls beyond it
    pipe, _ = run(Lfm2Pipeline, plan, text, max_tools=1)
    assert len(pipe.tool_calls) == 1
    # a malformed block is reported without a name instead of raising
    pipe, _ = run(Lfm2Pipeline, plan, "<|tool_call_start|>not python(<|tool_call_end|>")
    assert pipe.tool_calls[0]["name"] is None and pipe.tool_calls[0]["raw"] == "not python("


def test_harmony_channels():
    plan = detect_plan("<|start|>{{ role }}<|channel|>final<|message|>", "", tools=None)
    assert plan.dialect == "harmony" and pipeline_for(plan) is HarmonyPipeline
    # the prompt ended with "<|start|>assistant": generation continues inside the header
    text = ("<|channel|>analysis<|message|>User wants 2+2.<|end|>"
            "<|start|>assistant<|channel|>final<|message|>It is 4.<|return|>ignored")
    pipe, events = run(HarmonyPipeline, plan, text)
    assert "".join(pipe.reasoning_out) == "User wants 2+2." and "".join(pipe.text_out) == "It is 4."
    assert pipe.finished == FinishReason.EOS and events[-1].kind == "finished"
    # tool call on the commentary channel; <|call|> is usually the EOS id and never reaches the text stream
    for tail in ("<|call|>", ""):
        text = ("<|channel|>analysis<|message|>Need the weather.<|end|><|start|>assistant<|channel|>commentary "
                'to=functions.get_weather <|constrain|>json<|message|>{"city": "Paris"}' + tail)
        pipe, events = run(HarmonyPipeline, plan, text, chunk=5)
        assert pipe.tool_calls == [{"name": "get_weather", "arguments": {"city": "Paris"}, "raw": '{"city": "Paris"}'}]
        assert [e.kind for e in events if e.kind in ("tool_call_start", "tool_call_end")] == ["tool_call_start", "tool_call_end"]
        assert "".join(pipe.text_out) == ""
    # recipient in the role part of the header
    text = '<|channel|>commentary<|message|>preamble<|end|><|start|>assistant to=functions.f<|channel|>commentary json<|message|>{}<|call|>'
    pipe, _ = run(HarmonyPipeline, plan, text)
    assert pipe.tool_calls[0]["name"] == "f" and pipe.tool_calls[0]["arguments"] == {} and "".join(pipe.reasoning_out) == "preamble"
    # stop sequences apply to the final channel only
    pipe, _ = run(HarmonyPipeline, plan, "<|channel|>analysis<|message|>a STOP b<|end|><|start|>assistant<|channel|>final<|message|>x STOP y",
                  stop=["STOP"], reason=FinishReason.MAX_TOKENS)
    assert "".join(pipe.text_out) == "x " and pipe.finished == FinishReason.STOP_SEQUENCE and "STOP" in "".join(pipe.reasoning_out)


def test_generic_plan_is_unchanged():
    plan = detect_plan("<tool_call>", "", tools=[{"name": "x"}])
    assert plan.dialect == "generic" and plan.tool_open == "<tool_call>" and not plan.render_special_tokens
    assert pipeline_for(None).__name__ == "CommittedTokenPipeline" and isinstance(ParserPlan().dialect, str)


def test_qwen_tagged_parameter_calls():
    from eredu_b200.runtime.streaming import CommittedTokenPipeline
    from eredu_b200.text.dialects import parse_tagged_call

    tools = [{"type": "function", "function": {"name": "write_file", "parameters": {"type": "object", "properties": {
        "path": {"type": "string"}, "mode": {"type": "integer"}, "content": {"type": "string"}, "force": {"type": "boolean"}}}}}]
    body = ("<function=write_file>\n<parameter=path>\n/tmp/a.txt\n</parameter>\n<parameter=mode>\n420\n</parameter>\n"
            "<parameter=content>\n{\"not\": \"parsed\"}\nline two\n</parameter>\n<parameter=force>\ntrue\n</parameter>\n</function>")
    call = parse_tagged_call(body, tools)[0]
    assert call == {"name": "write_file", "arguments": {"path": "/tmp/a.txt", "mode": 420,
                                                        "content": "{\"not\": \"parsed\"}\nline two", "force": True}}
    loose = parse_tagged_call("<function=f><parameter=n>3</parameter><parameter=s>abc</parameter></function>")[0]
    assert loose["arguments"] == {"n": 3, "s": "abc"}
    with pytest.raises(ValueError):
        parse_tagged_call("{}")
    plan = detect_plan("<tool_call>", "", tools=tools)
    pieces_text = "I will write it.<tool_call>\n" + body + "\n</tool_call>"
    pieces = [pieces_text[i:i + 4] for i in range(0, len(pieces_text), 4)]
    pipe = CommittedTokenPipeline(PieceDecoder(pieces), plan, (), None, None)
    pipe.tools = tools
    for i in range(len(pieces)):
        pipe.push(i)
    pipe.finish(FinishReason.EOS)
    assert "".join(pipe.text_out) == "I will write it."
    assert pipe.tool_calls[0]["name"] == "write_file" and pipe.tool_calls[0]["arguments"]["mode"] == 420
