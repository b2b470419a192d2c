"""Tokenizer bundles, chat templates, the committed-token pipeline (stop sequences, reasoning, tool calls), finish
precedence and cancellation - CPU only, with a small synthetic tokenizer."""
import json

import pytest
import torch

from eredu_b200.runtime.streaming import (CancellationToken, CommittedTokenPipeline, FinishReason, JsonFragmentBuffer,
                                          PartialPatternBuffer)
from eredu_b200.text.chat import ToolChoice, prepare_chat
from eredu_b200.text.tokenizer import TextDecoder, TokenizerBundle, load_tokenizer


def make_bundle(tmp_path=None):
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers

    alphabet = pre_tokenizers.ByteLevel.alphabet()
    vocab = {ch: i for i, ch in enumerate(sorted(alphabet))}
    for w in ("<|im_start|>", "<|im_end|>", "<think>", "</think>"):
        vocab[w] = len(vocab)
    tok = Tokenizer(models.BPE(vocab=vocab, merges=[]))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)
    tok.decoder = decoders.ByteLevel()
    from tokenizers import AddedToken
    tok.add_special_tokens([AddedToken("<|im_start|>", special=True), AddedToken("<|im_end|>", special=True)])
    b = TokenizerBundle(tok, None, None, "<|im_end|>", (tok.token_to_id("<|im_end|>"),))
    if tmp_path is not None:
        tok.save(str(tmp_path / "tokenizer.json"))
        (tmp_path / "tokenizer_config.json").write_text(json.dumps({
            "eos_token": {"content": "<|im_end|>"}, "chat_template": "{% for m in messages %}[{{ m.role }}]{{ m.content }}{% endfor %}{% if add_generation_prompt %}[assistant]{% endif %}"}))
        (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [5, 7], "do_sample": True}))
    return b


def test_text_decoder_never_splits_utf8():
    b = make_bundle()
    text = "héllo → 世界 🙂 done"
    ids = b.encode(text)
    dec = TextDecoder(b)
    pieces = [dec.push(t) for t in ids]
    assert all("�" not in p for p in pieces)
    assert "".join(pieces) + dec.flush() == text


def test_hf_sidecars(tmp_path):
    make_bundle(tmp_path)
    b = load_tokenizer(tmp_path)
    assert b.chat_template.startswith("{% for m") and 5 in b.eos_ids and 7 in b.eos_ids
    assert b.generation_config["do_sample"] is True and len(b.fingerprint()) == 64


def test_partial_pattern_buffer_look_behind():
    m = PartialPatternBuffer(["STOP", "</s>"])
    out = ""
    hit = None
    for piece in ["hello S", "T", "O", "x ST", "OP tail"]:
        o, h = m.push(piece)
        out += o
        hit = hit or h
    assert out == "hello STOx " and hit == "STOP"


def test_json_fragment_buffer():
    j = JsonFragmentBuffer()
    assert j.push('{"name": "f", "arguments": {"x": "}') is None
    assert j.push('"}}') == {"name": "f", "arguments": {"x": "}"}}


def _run(pipe, b, text, chunk=3):
    ids = b.encode(text)
    evs = []
    for t in ids:
        evs += pipe.push(t)
        if pipe.finished:
            break
    return evs


def test_pipeline_reasoning_tools_and_stop():
    from eredu_b200.text.chat import ParserPlan

    b = make_bundle()
    plan = ParserPlan("<think>", "</think>", False, "<tool_call>", "</tool_call>")
    pipe = CommittedTokenPipeline(TextDecoder(b), plan, stop=["###"])
    text = 'Hi <think>plan it</think>ok <tool_call>{"name": "get", "arguments": {"q": 1}}</tool_call> bye ### never'
    evs = _run(pipe, b, text)
    evs += pipe.finish(FinishReason.MAX_TOKENS)
    kinds = [e.kind for e in evs]
    assert "".join(pipe.reasoning_out) == "plan it"
    assert "".join(pipe.text_out) == "Hi ok  bye "
    assert pipe.tool_calls == [{"name": "get", "arguments": {"q": 1}, "raw": '{"name": "get", "arguments": {"q": 1}}'}]
    assert kinds.count("tool_call_start") == 1 and kinds.count("tool_call_end") == 1 and kinds[-1] == "finished"
    assert evs[-1].finish_reason == FinishReason.STOP_SEQUENCE  # stop sequence beats max tokens


def test_finish_precedence_and_cancellation():
    R = FinishReason
    assert R.resolve([R.MAX_TOKENS, R.EOS]) == R.EOS
    assert R.resolve([R.EOS, R.GRAMMAR_COMPLETE, R.STOP_SEQUENCE]) == R.STOP_SEQUENCE
    assert R.resolve([R.MAX_TOKENS, R.GRAMMAR_COMPLETE]) == R.GRAMMAR_COMPLETE
    c = CancellationToken()
    assert not c.is_cancelled()
    c.cancel()
    assert c.is_cancelled()


def test_prepare_chat_templates_and_tools():
    tpl = ("{% if tools %}TOOLS:{{ tools | tojson }}\n<tool_call> format{% endif %}"
           "{% for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] }}<|im_end|>\n{% endfor %}"
           "{% if add_generation_prompt %}<|im_start|>assistant\n"
           "{% if enable_thinking is defined and enable_thinking %}<think>\n{% endif %}{% endif %}")
    msgs = [{"role": "user", "content": "2+2?"}]
    tools = [{"type": "function", "function": {"name": "calc", "parameters": {"type": "object"}}}]
    p = prepare_chat(msgs, tpl, tools=tools, thinking="on", stop=["\n\n"])
    assert "TOOLS:" in p.prompt and p.prompt.rstrip().endswith("<think>")
    assert p.plan.starts_in_reasoning and p.plan.tool_open == "<tool_call>"
    q = prepare_chat(msgs, tpl, tools=tools, tool_choice=ToolChoice("none"), thinking="off")
    assert "TOOLS:" not in q.prompt and q.plan.tool_open is None and not q.plan.starts_in_reasoning
    with pytest.raises(Exception):
        prepare_chat(msgs, "{{ raise_exception('nope') }}")


def test_generate_prepared_chat_end_to_end(tmp_path):
    """Tiny random model + synthetic tokenizer through the public chat API: events stream, stop sequences and
    cancellation end the generation with the right reason."""
    import dataclasses

    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models import config as C
    from eredu_b200.models.llama import random_state

    b = make_bundle(tmp_path)
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=b.vocab_size(), eos_token_id=b.eos_ids[0])
    ck.save_safetensors_checkpoint(tmp_path, cfg, random_state(cfg, seed=0, std=0.05), torch.float32)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=256))
    assert lm.tokenizer is not None
    prepared = lm.prepare_chat([{"role": "user", "content": "hello"}])
    events = []
    res = lm.generate_prepared_chat(prepared, max_new_tokens=12, on_event=events.append)
    assert res["finish_reason"] in (FinishReason.MAX_TOKENS, FinishReason.EOS) and events[-1].kind == "finished"
    assert res["prompt_tokens"] > 0 and res["timing"]["time_to_first_token"] > 0
    assert "".join(e.text for e in events if e.kind == "text") == res["text"]
    cancel = CancellationToken()
    seen = []

    def on_event(ev):
        seen.append(ev)
        if len(seen) == 3:
            cancel.cancel()

    res2 = lm.generate_prepared_chat(prepared, max_new_tokens=64, on_event=on_event, cancellation=cancel)
    assert res2["finish_reason"] == FinishReason.CANCELLED and len(res2["tokens"]) < 64
