"""Chat preparation: Jinja chat templates (Hugging Face conventions), tool schemas, reasoning controls, and the
parser plan that the streaming pipeline uses to turn generated text into semantic events.

Counterpart of eredu/src/runtime/chat/mod.rs:471-560 (``PreparedChat``: rendered prompt + parser / constraint plan),
eredu-text/src/tokenizer.rs (minijinja templates with Python-compat helpers) and the dialect recognisers of
runtime/chat/dialect.rs (JSON tool calls in ``<tool_call>`` tags, Qwen style; bare JSON objects; Harmony-like
channel markers are recognised by tag names only).
"""
from __future__ import annotations

import datetime
import json
from dataclasses import dataclass, field
from typing import Optional

DEFAULT_TEMPLATE = (
    "{% for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] }}<|im_end|>\n{% endfor %}"
    "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}"
)


@dataclass
class ToolChoice:
    mode: str = "auto"            # none | auto | required
    max_parallel_calls: Optional[int] = None


@dataclass
class ParserPlan:
    """What the streaming parser should look for in the generated text."""
    reasoning_open: Optional[str] = None     # e.g. "<think>"
    reasoning_close: Optional[str] = None
    starts_in_reasoning: bool = False        # the template already opened the reasoning block in the prompt
    tool_open: Optional[str] = None          # e.g. "<tool_call>"
    tool_close: Optional[str] = None
    allow_unparsed_reasoning: bool = False
    dialect: str = "generic"                 # generic | lfm2 | harmony | gemma | inkling | atem (text/dialects.py)
    render_special_tokens: bool = False      # the structural tags are special tokens: the detokeniser must show them
    bare_json_tools: bool = False            # a reply whose first visible character is "{" is one JSON tool call


@dataclass
class PreparedChat:
    prompt: str
    plan: ParserPlan
    stop: list = field(default_factory=list)
    tools: Optional[list] = None
    tool_choice: ToolChoice = field(default_factory=ToolChoice)
    template_signature: str = ""


def _raise(msg):
    raise ValueError(f"chat template error: {msg}")


def _environment():
    from jinja2 import StrictUndefined
    from jinja2.sandbox import ImmutableSandboxedEnvironment

    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, undefined=StrictUndefined,
                                        extensions=["jinja2.ext.loopcontrols"])
    env.globals["raise_exception"] = _raise
    env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
    env.filters["tojson"] = lambda v, indent=None, ensure_ascii=False: json.dumps(v, indent=indent, ensure_ascii=ensure_ascii)
    return env


def render_template(template: str, messages: list, tools=None, add_generation_prompt: bool = True, **kwargs) -> str:
    from jinja2 import ChainableUndefined

    env = _environment()
    env.undefined = ChainableUndefined  # HF templates probe optional keys (message.tool_calls, tools, ...)
    tpl = env.from_string(template)
    return tpl.render(messages=messages, tools=tools, add_generation_prompt=add_generation_prompt, **kwargs)


def detect_plan(template: str, rendered: str, tools, thinking: str = "auto", allow_unparsed_reasoning=False) -> ParserPlan:
    plan = ParserPlan(allow_unparsed_reasoning=allow_unparsed_reasoning)
    if "<think>" in template or "<think>" in rendered:
        plan.reasoning_open, plan.reasoning_close = "<think>", "</think>"
        tail = rendered[-64:]
        plan.starts_in_reasoning = tail.rstrip().endswith("<think>")
    if thinking == "off":
        plan.starts_in_reasoning = False
    if "<|message_model|>" in template and "<|content_text|>" in template:
        plan.dialect, plan.render_special_tokens = "inkling", True
        return plan
    if "<|eom|>" in template and "<|eot|>" in template and "<|message|>" in template:
        plan.dialect, plan.render_special_tokens = "atem", True
        return plan
    if "<|channel|>" in template and "<|message|>" in template:
        # Harmony (GPT-OSS): channels carry reasoning, reply and tool calls; the dialect parser owns all of it
        plan.dialect, plan.render_special_tokens = "harmony", True
        return plan
    if "<|channel>" in template or "<|tool_call>" in template:
        # Gemma 4: thought channel and structural-object tool calls, all tags are special tokens
        from .dialects import GEMMA_CHANNEL_CLOSE, GEMMA_CHANNEL_OPEN, GEMMA_TOOL_CLOSE, GEMMA_TOOL_OPEN

        plan.dialect, plan.render_special_tokens = "gemma", True
        plan.reasoning_open, plan.reasoning_close = GEMMA_CHANNEL_OPEN + "thought\n", GEMMA_CHANNEL_CLOSE
        plan.starts_in_reasoning = rendered.rstrip(" ").endswith(plan.reasoning_open) and thinking != "off"
        if tools:
            plan.tool_open, plan.tool_close = GEMMA_TOOL_OPEN, GEMMA_TOOL_CLOSE
        return plan
    if "<|tool_call_start|>" in template or "<|tool_list_start|>" in template:
        plan.dialect, plan.render_special_tokens = "lfm2", True
        plan.tool_open, plan.tool_close = "<|tool_call_start|>", "<|tool_call_end|>"
        return plan
    if tools:
        if "<tool_call>" in template:
            plan.tool_open, plan.tool_close = "<tool_call>", "</tool_call>"
        elif "[TOOL_CALLS]" in template:
            plan.tool_open, plan.tool_close = "[TOOL_CALLS]", None
        elif "<|start_header_id|>" in template and '"parameters"' in template:
            # Llama 3.x: the whole reply is {"name": ..., "parameters": {...}}; <|python_tag|> may precede it
            plan.bare_json_tools = True
            plan.tool_open, plan.tool_close = "<|python_tag|>", None
        else:
            plan.tool_open, plan.tool_close = "<tool_call>", "</tool_call>"
    return plan


def prepare_chat(messages: list, template: Optional[str] = None, bos_token: str = "", eos_token: str = "", tools=None,
                 tool_choice: Optional[ToolChoice] = None, thinking: str = "auto", stop: Optional[list] = None,
                 allow_unparsed_reasoning: bool = False, **template_kwargs) -> PreparedChat:
    """Render the conversation and derive the parser plan. ``thinking``: auto | on | off maps to the template's
    ``enable_thinking`` control when the template knows it."""
    import hashlib

    template = template or DEFAULT_TEMPLATE
    tool_choice = tool_choice or ToolChoice()
    use_tools = tools if (tools and tool_choice.mode != "none") else None
    kwargs = dict(template_kwargs)
    if thinking != "auto" and "enable_thinking" in template:
        kwargs["enable_thinking"] = thinking == "on"
    prompt = render_template(template, messages, tools=use_tools, add_generation_prompt=True, bos_token=bos_token or "",
                             eos_token=eos_token or "", **kwargs)
    plan = detect_plan(template, prompt, use_tools, thinking, allow_unparsed_reasoning)
    stops = list(stop or [])
    if plan.dialect == "gemma":
        from .dialects import GEMMA_STOPS

        stops += [s for s in GEMMA_STOPS if s not in stops]
    return PreparedChat(prompt=prompt, plan=plan, stop=stops, tools=use_tools, tool_choice=tool_choice,
                        template_signature=hashlib.sha256(template.encode()).hexdigest()[:16])
