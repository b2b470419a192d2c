"""Activation observer: named block outputs, interventions, MoE routing records; observed passes change nothing."""
import dataclasses

import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.models.moe import make_moe_factory
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.engine import Engine
from eredu_b200.runtime.inspection import ActivationObserver, RecordingObserver, observed


def test_observer_sees_block_outputs_and_can_intervene():
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=300, num_hidden_layers=3)
    sd = random_state(cfg, seed=0, std=0.05)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32)
    eng = Engine(model, max_batch=1, max_seq_len=64)
    prompt = list(range(5, 25))
    plain = eng.generate([prompt], SamplingParams(temperature=0.0), 6)[0]
    rec = RecordingObserver()
    with observed(model, rec):
        seen = eng.generate([prompt], SamplingParams(temperature=0.0), 6)[0]
    assert seen == plain and model.observer is None
    assert set(rec.tensors) == {"model.embed_tokens"} | {f"model.layers.{i}.output" for i in range(3)}
    assert rec.tensors["model.layers.2.output"].shape[-1] == cfg.hidden_size

    class ZeroLayer1(ActivationObserver):
        def intervene(self, name, value):
            return torch.zeros_like(value) if name == "model.layers.1.output" else None

    with observed(model, ZeroLayer1()):
        changed = eng.generate([prompt], SamplingParams(temperature=0.0), 6)[0]
    assert changed != plain
    assert eng.generate([prompt], SamplingParams(temperature=0.0), 6)[0] == plain       # nothing sticks


def test_moe_routing_observation():
    cfg = dataclasses.replace(C.tiny_llama(), model_type="qwen3_moe", qk_norm=True, vocab_size=300, num_experts=8,
                              num_experts_per_tok=2, moe_intermediate_size=64, norm_topk_prob=True, num_hidden_layers=2,
                              tie_word_embeddings=False)
    sd = random_state(cfg, seed=1, std=0.08)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    eng = Engine(model, max_batch=1, max_seq_len=64)
    prompt = list(range(9, 20))
    plain = eng.generate([prompt], SamplingParams(temperature=0.0), 4)[0]
    rec = RecordingObserver(names=[])
    with observed(model, rec):
        assert eng.generate([prompt], SamplingParams(temperature=0.0), 4)[0] == plain
    first = rec.routing[0]
    assert first.prefix == "model.layers.0.mlp" and first.num_experts == 8
    assert first.selected_experts.shape == (len(prompt), 2) and first.routing_weights.shape == (len(prompt), 2)
    assert torch.allclose(first.routing_weights.sum(-1), torch.ones(len(prompt)), atol=1e-5)
    assert bool((first.selected_scores <= 1).all()) and first.routed_output.shape == (len(prompt), cfg.hidden_size)
    assert first.shared_output is None and first.reduced_routed_output is None
    assert len(rec.routing) == 2 * (1 + 3)          # two sparse layers x (prefill + three decode steps)


def test_text_side_inspection(tmp_path):
    """Tokenizer, chat template, end-of-sequence ids, streaming markers and tool calling are probed by behaviour."""
    import dataclasses
    import json

    import torch
    from test_text_streaming import make_bundle

    from eredu_b200.api import inspect_text_model
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models import config as C
    from eredu_b200.models.llama import random_state
    from eredu_b200.runtime.plan import inspect_artifact

    b = make_bundle(tmp_path)
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=b.vocab_size(), eos_token_id=b.eos_ids[0])
    ck.save_safetensors_checkpoint(tmp_path, cfg, random_state(cfg, seed=0, std=0.05), torch.float32)
    rep = inspect_text_model(inspect_artifact(tmp_path))
    assert rep.text["tokenizer"] == "ready" and rep.text["chat_template"] == "ready" and rep.text["eos"] == "ready"
    assert rep.text["semantic_streaming"] == "ready" and rep.text["dialect"] == "generic"
    assert rep.text["native_tools"] == "missing" and "template_ignores_tools" in [i.code for i in rep.issues]   # the template never shows tools
    assert rep.is_loadable and "text" in rep.to_dict()
    # a template that renders tools and names the call tags
    tc = json.loads((tmp_path / "tokenizer_config.json").read_text())
    tc["chat_template"] = ("{% if tools %}{% for t in tools %}{{ t.function.name }}{% endfor %}<tool_call></tool_call>{% endif %}"
                           "{% for m in messages %}[{{ m.role }}]{{ m.content }}{% endfor %}[assistant]")
    (tmp_path / "tokenizer_config.json").write_text(json.dumps(tc))
    assert inspect_text_model(inspect_artifact(tmp_path)).text["native_tools"] == "ready"
    # a dialect whose markers this tokenizer splits: streaming (and with it tool calling) is not usable
    tc["chat_template"] = "{% for m in messages %}<|start|>{{ m.role }}<|message|>{{ m.content }}<|end|>{% endfor %}<|start|>assistant<|channel|>"
    (tmp_path / "tokenizer_config.json").write_text(json.dumps(tc))
    rep = inspect_text_model(inspect_artifact(tmp_path))
    assert rep.text["dialect"] == "harmony" and rep.text["semantic_streaming"] == "invalid" and rep.text["native_tools"] != "ready"
    assert "unresolved_structural_token" in [i.code for i in rep.issues]
    # broken and absent templates, absent tokenizer
    tc["chat_template"] = "{% for m in messages %}{{ m.content | no_such_filter }}{% endfor %}"
    (tmp_path / "tokenizer_config.json").write_text(json.dumps(tc))
    rep = inspect_text_model(inspect_artifact(tmp_path))
    assert rep.text["chat_template"] == "invalid" and rep.text["native_tools"] == "unverified"
    del tc["chat_template"]
    (tmp_path / "tokenizer_config.json").write_text(json.dumps(tc))
    assert inspect_text_model(inspect_artifact(tmp_path)).text["chat_template"] == "missing"
    (tmp_path / "tokenizer.json").unlink()
    rep = inspect_text_model(inspect_artifact(tmp_path))
    assert rep.text["tokenizer"] in ("missing", "invalid") and not rep.is_loadable
