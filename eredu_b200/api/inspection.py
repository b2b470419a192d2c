"""Text-side inspection: tokenizer, chat template, end-of-sequence ids, semantic streaming and native tool calling.

Counterpart of ``inspect_text_model`` (eredu/src/api/inspection.rs:29-140): it enriches a report made by
``runtime.plan.inspect_artifact`` (which looks at configuration and tensors only) with the readiness of everything a chat
request needs, found by behaviour: the tokenizer is loaded, the chat template is rendered with a probe conversation (and a
probe tool), the parser plan is derived from it and its structural markers are looked up in the vocabulary. No weights are read.

Readiness values: ``ready`` | ``missing`` | ``invalid`` | ``unverified`` (a prerequisite was missing).
"""
from __future__ import annotations

from pathlib import Path
from typing import Optional

from ..runtime.plan import InspectionIssue, ModelInspectionReport

READY, MISSING, INVALID, UNVERIFIED = "ready", "missing", "invalid", "unverified"

_PROBE_TOOL = {"type": "function", "function": {"name": "eredu_probe_tool", "description": "probe",
                                                "parameters": {"type": "object", "properties": {"value": {"type": "integer"}},
                                                               "required": ["value"]}}}

# markers a dialect's parser can only see when each of them is one vocabulary entry (they arrive as single special tokens)
_STRUCTURAL = {
    "harmony": ["<|start|>", "<|channel|>", "<|message|>", "<|end|>", "<|return|>", "<|call|>"],
    "gemma": ["<|channel>", "<channel|>", "<|tool_call>", "<tool_call|>", '<|"|>', "<|tool_response>", "<turn|>"],
    "lfm2": ["<|tool_call_start|>", "<|tool_call_end|>"],
    "inkling": ["<|message_model|>", "<|content_text|>", "<|content_thinking|>", "<|content_invoke_tool_json|>", "<|end_message|>",
                "<|content_model_end_sampling|>"],
    "atem": ["<|start|>", "<|message|>", "<|eom|>", "<|eot|>"],
}


def inspect_text_model(report: ModelInspectionReport, messages: Optional[list] = None, tools: Optional[list] = None) -> ModelInspectionReport:
    """``messages`` / ``tools``: the probe chat request (default: one user turn, one probe tool)."""
    from ..text.tokenizer import load_tokenizer

    text = {"tokenizer": UNVERIFIED, "chat_template": UNVERIFIED, "eos": UNVERIFIED, "semantic_streaming": UNVERIFIED,
            "native_tools": UNVERIFIED, "dialect": None}
    report.text = text

    def issue(code, severity, message):
        report.issues.append(InspectionIssue(code, severity, message))

    path = Path(report.path)
    source = None
    if report.format == "gguf":
        try:
            from ..formats.checkpoint import open_checkpoint

            source = open_checkpoint(path)
        except Exception as e:       # the header was readable a moment ago: report, do not raise
            text["tokenizer"] = INVALID
            issue("io", "error", f"could not reopen GGUF metadata for text inspection: {e}")
            return report
    try:
        tok = load_tokenizer(path, source)
        text["tokenizer"] = READY
        report.has_tokenizer = True
    except FileNotFoundError as e:
        tok = None
        text["tokenizer"] = MISSING
        issue("missing_tokenizer", "error", str(e) or "no tokenizer found")
    except Exception as e:
        tok = None
        text["tokenizer"] = INVALID
        issue("invalid_tokenizer", "error", f"tokenizer could not be loaded: {e}")
    if tok is None:
        text["chat_template"] = text["semantic_streaming"] = text["native_tools"] = MISSING
        return report
    eos = set(getattr(tok, "eos_ids", ()) or ())
    cfg_eos = report.config.eos_token_id if report.config is not None else None
    if cfg_eos is not None:
        eos |= set(cfg_eos if isinstance(cfg_eos, (list, tuple)) else [cfg_eos])
    text["eos"] = READY if eos else MISSING
    if not eos:
        issue("missing_eos", "warning", "no end-of-sequence token id in the configuration or the tokenizer sidecars")
    if not tok.chat_template:
        text["chat_template"] = MISSING
        text["semantic_streaming"] = text["native_tools"] = MISSING
        issue("missing_chat_template", "warning", "no tokenizer_config.json chat_template or chat_template.jinja is available")
        return report
    from ..text.chat import prepare_chat

    probe = messages or [{"role": "user", "content": "eredu inspection probe"}]
    try:
        plain = prepare_chat(probe, template=tok.chat_template, bos_token=tok.bos_token or "", eos_token=tok.eos_token or "")
        text["chat_template"] = READY
    except Exception as e:
        text["chat_template"] = INVALID
        text["semantic_streaming"] = text["native_tools"] = UNVERIFIED
        issue("invalid_chat_template", "warning", f"the chat template does not render a plain user turn: {e}")
        return report
    if "eredu inspection probe" not in plain.prompt and messages is None:
        issue("chat_template_drops_content", "warning", "the rendered prompt does not contain the user's text")
    # semantic streaming: the parser's structural markers must be single vocabulary entries
    dialect = plain.plan.dialect
    text["dialect"] = dialect
    missing = []
    for marker in _STRUCTURAL.get(dialect, []):
        ids = tok.encode(marker, add_special_tokens=False)
        if len(ids) != 1:
            missing.append(marker)
    if missing:
        text["semantic_streaming"] = INVALID
        issue("unresolved_structural_token", "warning",
              f"the {dialect} parser needs {missing} as single tokens; this tokenizer splits them")
    else:
        text["semantic_streaming"] = READY
    # native tools: the template must show a declared tool and the plan must know where calls appear
    try:
        with_tools = prepare_chat(probe, template=tok.chat_template, bos_token=tok.bos_token or "", eos_token=tok.eos_token or "",
                                  tools=tools or [_PROBE_TOOL])
    except Exception as e:
        text["native_tools"] = INVALID
        issue("invalid_tool_template", "warning", f"the chat template fails when tools are declared: {e}")
        return report
    name = (tools or [_PROBE_TOOL])[0].get("function", {}).get("name", "")
    shown = bool(name) and name in with_tools.prompt
    knows_calls = dialect in ("harmony", "inkling", "atem") or bool(with_tools.plan.tool_open)
    if shown and knows_calls and text["semantic_streaming"] == READY:
        text["native_tools"] = READY
    elif not shown:
        text["native_tools"] = MISSING
        issue("template_ignores_tools", "info", "the chat template does not render declared tools: tool calling is not available")
    else:
        text["native_tools"] = INVALID if text["semantic_streaming"] == INVALID else MISSING
    return report
