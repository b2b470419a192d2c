"""Five real-world-shaped chat templates (Llama 3.x, Qwen3 with tools, Harmony, Gemma, LFM2) kept as fixtures: each is
rendered by ``prepare_chat``, its parser plan is detected from the template alone, and a reply in that model's own
syntax streams through the pipeline the plan selects (eredu/src/runtime/chat/mod.rs:471-560, chat/dialect.rs)."""
import json
import os

import pytest

from eredu_b200.runtime.streaming import CommittedTokenPipeline, FinishReason
from eredu_b200.text.chat import ToolChoice, prepare_chat
from eredu_b200.text.dialects import HarmonyPipeline, Lfm2Pipeline, pipeline_for

FIX = os.path.join(os.path.dirname(__file__), "fixtures", "chat_templates")
WEATHER = {"type": "function", "function": {
    "name": "get_weather", "description": "Current weather for a city.",
    "parameters": {"type": "object", "required": ["city"], "properties": {
        "city": {"type": "string", "description": "City name"}, "days": {"type": "integer"}}}}}
TALK = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Weather in Paris?"}]


def template(name):
    with open(os.path.join(FIX, name + ".jinja")) as f:
        return f.read()


class Pieces:
    def __init__(self, text, chunk):
        self.pieces = [text[i:i + chunk] for i in range(0, len(text), chunk)]

    def push(self, i):
        return self.pieces[i]

    def flush(self):
        return ""


def stream(prepared, reply, chunk=3, reason=FinishReason.EOS):
    dec = Pieces(reply, chunk)
    pipe = pipeline_for(prepared.plan)(dec, prepared.plan, prepared.stop, None, prepared.tool_choice.max_parallel_calls)
    pipe.tools = prepared.tools
    events = []
    for i in range(len(dec.pieces)):
        events += pipe.push(i)
        if pipe.finished:
            break
    events += pipe.finish(reason)
    return pipe, events


def test_llama3_bare_json_calls():
    t = template("llama3")
    plain = prepare_chat(TALK, t, bos_token="<|begin_of_text|>")
    assert plain.prompt.startswith("<|begin_of_text|><|start_header_id|>system<|end_header_id|>\n\nCutting Knowledge Date")
    assert "Be brief.<|eot_id|><|start_header_id|>user<|end_header_id|>\n\nWeather in Paris?<|eot_id|>" in plain.prompt
    assert plain.prompt.endswith("<|start_header_id|>assistant<|end_header_id|>\n\n")
    assert plain.plan.dialect == "generic" and not plain.plan.bare_json_tools and plain.plan.tool_open is None
    pipe, _ = stream(plain, '{"not": "a call"} just text')
    assert pipe.tool_calls == [] and "".join(pipe.text_out) == '{"not": "a call"} just text'

    tooled = prepare_chat(TALK, t, bos_token="<|begin_of_text|>", tools=[WEATHER])
    assert "Environment: ipython\n" in tooled.prompt and '"name": "get_weather"' in tooled.prompt
    assert tooled.plan.bare_json_tools and pipeline_for(tooled.plan) is CommittedTokenPipeline
    for lead in ("", "\n ", "<|python_tag|>"):
        pipe, events = stream(tooled, lead + '{"name": "get_weather", "parameters": {"city": "Paris", "days": 2}}')
        assert pipe.tool_calls[0]["name"] == "get_weather" and pipe.tool_calls[0]["arguments"] == {"city": "Paris", "days": 2}
        assert "".join(pipe.text_out).strip() == ""
        assert [e.kind for e in events if e.kind in ("tool_call_start", "tool_call_end")] == ["tool_call_start", "tool_call_end"]
    pipe, _ = stream(tooled, 'It is sunny. {"name": "x"}')
    assert pipe.tool_calls == [] and "".join(pipe.text_out) == 'It is sunny. {"name": "x"}'
    # a tool round trip renders: assistant call as JSON, result under the ipython role
    history = TALK + [{"role": "assistant", "content": "", "tool_calls": [{"type": "function", "function": {
        "name": "get_weather", "arguments": {"city": "Paris"}}}]}, {"role": "tool", "content": {"temp_c": 21}}]
    again = prepare_chat(history, t, tools=[WEATHER])
    assert '{"name": "get_weather", "parameters": {"city": "Paris"}}<|eot_id|><|start_header_id|>ipython<|end_header_id|>\n\n{"temp_c": 21}<|eot_id|>' in again.prompt


def test_qwen3_thinking_and_tagged_json_calls():
    t = template("qwen3")
    on = prepare_chat(TALK, t, tools=[WEATHER])
    assert on.prompt.startswith("<|im_start|>system\nBe brief.\n\n# Tools\n\n") and "<tools>\n" + json.dumps(WEATHER) + "\n</tools>" in on.prompt
    assert on.prompt.endswith("<|im_start|>assistant\n")
    plan = on.plan
    assert (plan.reasoning_open, plan.reasoning_close, plan.tool_open, plan.tool_close) == ("<think>", "</think>", "<tool_call>", "</tool_call>")
    assert not plan.starts_in_reasoning and plan.dialect == "generic"
    reply = ('<think>\nNeed the tool.\n</think>\n\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>\n'
             '<tool_call>\n{"name": "get_weather", "arguments": {"city": "Lyon"}}\n</tool_call>')
    pipe, events = stream(on, reply, chunk=4)
    assert "".join(pipe.reasoning_out).strip() == "Need the tool."
    assert [c["arguments"]["city"] for c in pipe.tool_calls] == ["Paris", "Lyon"]
    assert [e.tool_index for e in events if e.kind == "tool_call_end"] == [0, 1]
    off = prepare_chat(TALK, t, thinking="off")
    assert off.prompt.endswith("<|im_start|>assistant\n<think>\n\n</think>\n\n") and not off.plan.starts_in_reasoning
    # tool_choice none hides the tools from the template and from the parser
    none = prepare_chat(TALK, t, tools=[WEATHER], tool_choice=ToolChoice("none"))
    assert "# Tools" not in none.prompt and none.plan.tool_open is None
    # earlier reasoning is dropped from the history, the tool response is folded into a user turn
    history = TALK + [{"role": "assistant", "content": "<think>\nold thoughts\n</think>\n\nCalling.", "tool_calls": [
        {"function": {"name": "get_weather", "arguments": {"city": "Paris"}}}]}, {"role": "tool", "content": "21C"},
        {"role": "assistant", "content": "It is 21C."}, {"role": "user", "content": "And Lyon?"}]
    again = prepare_chat(history, t, tools=[WEATHER])
    assert "old thoughts" not in again.prompt
    assert '<|im_start|>user\n<tool_response>\n21C\n</tool_response><|im_end|>\n' in again.prompt


def test_harmony_channels_and_function_namespace():
    t = template("harmony")
    p = prepare_chat(TALK, t, tools=[WEATHER], reasoning_effort="high")
    assert p.prompt.startswith("<|start|>system<|message|>You are ChatGPT") and "Reasoning: high\n\n" in p.prompt
    assert "<|start|>developer<|message|># Instructions\n\nBe brief.\n\n# Tools\n\n## functions\n\nnamespace functions {\n\n" in p.prompt
    assert "// Current weather for a city.\ntype get_weather = (_: {\n// City name\ncity: string,\ndays?: number,\n}) => any;" in p.prompt
    assert p.prompt.endswith("<|start|>user<|message|>Weather in Paris?<|end|><|start|>assistant")
    assert p.plan.dialect == "harmony" and p.plan.render_special_tokens and pipeline_for(p.plan) is HarmonyPipeline
    reply = ("<|channel|>analysis<|message|>Look it up.<|end|><|start|>assistant to=functions.get_weather<|channel|>commentary json"
             '<|message|>{"city": "Paris"}<|call|>')
    pipe, _ = stream(p, reply, chunk=5)
    assert "".join(pipe.reasoning_out) == "Look it up." and pipe.tool_calls[0]["name"] == "get_weather"
    assert pipe.tool_calls[0]["arguments"] == {"city": "Paris"} and "".join(pipe.text_out) == ""
    history = TALK + [{"role": "assistant", "thinking": "Look it up.", "tool_calls": [{"function": {"name": "get_weather", "arguments": {"city": "Paris"}}}]},
                      {"role": "tool", "content": "21C"}]
    again = prepare_chat(history, t, tools=[WEATHER])
    assert ('<|start|>assistant<|channel|>analysis<|message|>Look it up.<|end|><|start|>assistant to=functions.get_weather<|channel|>commentary json'
            '<|message|>{"city": "Paris"}<|call|><|start|>functions.get_weather to=assistant<|channel|>commentary<|message|>"21C"<|end|>') in again.prompt
    with pytest.raises(ValueError, match="no previous assistant message"):
        prepare_chat(TALK + [{"role": "tool", "content": "x"}], t)


def test_gemma_turns_and_alternation():
    t = template("gemma")
    p = prepare_chat(TALK + [{"role": "assistant", "content": " Sunny. "}, {"role": "user", "content": [
        {"type": "image"}, {"type": "text", "text": "And this?"}]}], t, bos_token="<bos>")
    assert p.prompt == ("<bos><start_of_turn>user\nBe brief.\n\nWeather in Paris?<end_of_turn>\n<start_of_turn>model\nSunny.<end_of_turn>\n"
                        "<start_of_turn>user\n<start_of_image>And this?<end_of_turn>\n<start_of_turn>model\n")
    assert p.plan.dialect == "generic" and p.plan.reasoning_open is None and p.plan.tool_open is None
    pipe, _ = stream(p, "Cloudy.<end_of_turn>", reason=FinishReason.EOS)
    assert "".join(pipe.text_out) == "Cloudy.<end_of_turn>"          # the turn end is the EOS id and never reaches the text
    with pytest.raises(ValueError, match="alternate"):
        prepare_chat([{"role": "user", "content": "a"}, {"role": "user", "content": "b"}], t)


def test_lfm2_tool_list_and_python_calls():
    t = template("lfm2")
    p = prepare_chat(TALK, t, bos_token="<|startoftext|>", tools=[WEATHER])
    assert p.prompt == ("<|startoftext|><|im_start|>system\nBe brief.\nList of tools: <|tool_list_start|>[" + json.dumps(WEATHER) +
                        "]<|tool_list_end|><|im_end|>\n<|im_start|>user\nWeather in Paris?<|im_end|>\n<|im_start|>assistant\n")
    assert p.plan.dialect == "lfm2" and p.plan.render_special_tokens and pipeline_for(p.plan) is Lfm2Pipeline
    pipe, _ = stream(p, '<|tool_call_start|>[get_weather(city="Paris", days=2)]<|tool_call_end|>Checking.')
    assert pipe.tool_calls[0]["name"] == "get_weather" and pipe.tool_calls[0]["arguments"] == {"city": "Paris", "days": 2}
    assert "".join(pipe.text_out) == "Checking."
    again = prepare_chat(TALK + [{"role": "assistant", "content": '<|tool_call_start|>[get_weather(city="Paris")]<|tool_call_end|>'},
                                 {"role": "tool", "content": {"temp_c": 21}}], t)
    assert '<|im_start|>tool\n<|tool_response_start|>{"temp_c": 21}<|tool_response_end|><|im_end|>\n' in again.prompt
