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


def test_gemma_channels_and_structural_object_calls():
    from eredu_b200.text.chat import prepare_chat
    from eredu_b200.text.dialects import GemmaPipeline, parse_gemma_call, parse_structural_object

    assert parse_structural_object('{count:2,enabled:true,place:<|"|>Bogotá<|"|>,tags:[<|"|>東京<|"|>,<|"|>quote: " and slash \\\\<|"|>]}') == \
        {"count": 2, "enabled": True, "place": "Bogotá", "tags": ["東京", 'quote: " and slash \\\\']}
    assert parse_structural_object("{}") == {} and parse_structural_object('{ a : { b : [ ] , c : null } , d : -1.5e3 }') == \
        {"a": {"b": [], "c": None}, "d": -1500.0}
    for bad in ('{a:1,a:2}', '{a:<|"|>open}', '{a:1} x', '{a:one}', '{:1}', '[1]', '{a:1,}'):
        with pytest.raises(ValueError):
            parse_structural_object(bad)
    assert parse_gemma_call('call:lookup-place{count:1}') == {"name": "lookup-place", "arguments": {"count": 1}}
    for bad in ('lookup{a:1}', 'call:{a:1}', 'call:name'):
        with pytest.raises(ValueError):
            parse_gemma_call(bad)

    template = "{{ bos_token }}{% for m in messages %}<|turn>{{ m.role }}\n{{ m.content }}<turn|>{% endfor %}<|turn>model\n{# <|channel> <|tool_call> #}"
    tools = [{"type": "function", "function": {"name": "lookup-place", "parameters": {"type": "object", "properties": {}}}}]
    prepared = prepare_chat([{"role": "user", "content": "hi"}], template, tools=tools)
    plan = prepared.plan
    assert plan.dialect == "gemma" and plan.render_special_tokens and pipeline_for(plan) is GemmaPipeline
    assert plan.reasoning_open == "<|channel>thought\n" and plan.tool_open == "<|tool_call>" and "<turn|>" in prepared.stop
    text = ('<|channel>thought\nNeed 🦀 context<channel|>Checking.'
            '<|tool_call>call:lookup-place{count:2,enabled:true,place:<|"|>Bogotá<|"|>}<tool_call|>'
            '<|tool_call>call:lookup-place{count:1,enabled:false,place:<|"|>東京<|"|>}<tool_call|><|tool_response>ignored')
    for chunk in (1, 3, 7, 1000):
        pipe, events = run(GemmaPipeline, plan, text, chunk=chunk, stop=prepared.stop)
        assert "".join(pipe.reasoning_out) == "Need 🦀 context" and "".join(pipe.text_out) == "Checking."
        assert [(c["name"], c["arguments"]) for c in pipe.tool_calls] == [
            ("lookup-place", {"count": 2, "enabled": True, "place": "Bogotá"}),
            ("lookup-place", {"count": 1, "enabled": False, "place": "東京"})]
        assert pipe.finished == FinishReason.STOP_SEQUENCE
        assert [e.kind for e in events if e.kind.startswith("tool_call_")].count("tool_call_end") == 2
    # without tools the call tags are plain text; thinking off never starts inside the channel
    quiet = prepare_chat([{"role": "user", "content": "hi"}], template, thinking="off").plan
    assert quiet.dialect == "gemma" and quiet.tool_open is None and not quiet.starts_in_reasoning
    pipe, _ = run(GemmaPipeline, plan, "<|tool_call>call:broken{a:<tool_call|>")
    assert pipe.tool_calls[0]["name"] is None and pipe.tool_calls[0]["raw"] == "call:broken{a:"


def test_inkling_messages():
    from eredu_b200.text.dialects import InklingPipeline

    plan = detect_plan("...<|message_model|>...<|content_text|>...", "", tools=None)
    assert plan.dialect == "inkling" and pipeline_for(plan) is InklingPipeline and plan.render_special_tokens
    text = ("<|content_thinking|>check both values, literally<|end_message|><|message_model|><|content_text|>I'll look them up."
            "<|end_message|>"
            '<|message_model|>lookup<|content_invoke_tool_json|>{"name":"lookup","args":{"value":7}}<|end_message|>'
            '<|message_model|>lookup<|content_invoke_tool_json|>{"name":"lookup","args":{"value":11}}<|end_message|>'
            "<|content_model_end_sampling|>never shown")
    for chunk in (1, 4, 9, 1000):
        pipe, events = run(InklingPipeline, plan, text, chunk=chunk)
        assert "".join(pipe.reasoning_out) == "check both values, literally" and "".join(pipe.text_out) == "I'll look them up."
        assert [(c["name"], c["arguments"]) for c in pipe.tool_calls] == [("lookup", {"value": 7}), ("lookup", {"value": 11})]
        assert pipe.finished == FinishReason.STOP_SEQUENCE
        kinds = [e.kind for e in events]
        assert kinds.count("tool_call_start") == 2 and kinds[-1] == "finished"
    # a token limit inside the thinking message keeps what was produced
    pipe, _ = run(InklingPipeline, plan, "<|content_thinking|>partial thought", reason=FinishReason.MAX_TOKENS)
    assert "".join(pipe.reasoning_out) == "partial thought" and pipe.finished == FinishReason.MAX_TOKENS
    # a content marker inside a body is not a transition
    pipe, _ = run(InklingPipeline, plan, "<|content_thinking|>a<|content_text|>b<|end_message|>")
    assert "".join(pipe.reasoning_out) == "a<|content_text|>b"
    pipe, _ = run(InklingPipeline, plan, "<|content_text|>x<|end_message|>" + "<|message_model|>t<|content_invoke_tool_json|>{}<|end_message|>" * 3,
                  max_tools=2)
    assert len(pipe.tool_calls) == 2 and pipe.finished == FinishReason.GRAMMAR_COMPLETE


def test_atem_messages():
    from eredu_b200.text.dialects import AtemPipeline, parse_atem_calls

    plan = detect_plan("<|start|>..<|message|>..<|eom|>..<|eot|>", "", tools=None)
    assert plan.dialect == "atem" and pipeline_for(plan) is AtemPipeline
    envelope = ('<atem:function_calls>\n<atem:invoke name="weather.lookup">\n<atem:parameter name="days">3</atem:parameter>\n'
                '<atem:parameter name="units">metric &amp; SI</atem:parameter>\n</atem:invoke>\n</atem:function_calls>')
    assert parse_atem_calls(envelope) == [{"name": "weather.lookup", "arguments": {"days": 3, "units": "metric & SI"}}]
    typed = [{"function": {"name": "weather.lookup", "parameters": {"properties": {"days": {"type": "string"}}}}}]
    assert parse_atem_calls(envelope, typed)[0]["arguments"]["days"] == "3"
    with pytest.raises(ValueError):
        parse_atem_calls("<atem:function_calls></atem:function_calls>")
    text = " to=self<|message|>reason<|eom|><|start|>assistant to=weather.lookup<|message|>" + envelope + "<|eot|>trailing"
    for chunk in (1, 5, 1000):
        pipe, events = run(AtemPipeline, plan, text, chunk=chunk)
        assert "".join(pipe.reasoning_out) == "reason" and not pipe.text_out
        assert pipe.tool_calls == [{"name": "weather.lookup", "arguments": {"days": 3, "units": "metric & SI"}, "raw": envelope}]
        assert pipe.finished == FinishReason.EOS
    pipe, _ = run(AtemPipeline, plan, " to=user<|message|>direct answer<|eot|>")
    assert "".join(pipe.text_out) == "direct answer" and not pipe.tool_calls
    pipe, _ = run(AtemPipeline, plan, " to=self<|message|>think<|eom|><|start|>assistant to=user<|message|>hello", reason=FinishReason.MAX_TOKENS)
    assert "".join(pipe.reasoning_out) == "think" and "".join(pipe.text_out) == "hello" and pipe.finished == FinishReason.MAX_TOKENS
