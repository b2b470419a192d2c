"""CLI: flag parsing / validation, sampling default resolution, and one end-to-end run on CPU with telemetry."""
import dataclasses
import json

import pytest
import torch

from eredu_b200.cli.main import build_parser, main, resolve_sampling, validate_args
from test_text_streaming import make_bundle


def test_flag_validation():
    p = build_parser()
    a = p.parse_args(["-m", "x", "hi", "--quantize", "4", "--quantization-group-size", "64"])
    validate_args(a)
    for bad in (["--quantize", "7"], ["--quantization-group-size", "48"], ["-n", "0"], ["--device", "tpu"],
                ["--allow-mixed-revisions", "--require-same-revision"]):
        with pytest.raises(SystemExit):
            validate_args(p.parse_args(["-m", "x", "hi"] + bad))


def test_sampling_defaults_follow_checkpoint_config():
    p = build_parser()
    a = p.parse_args(["-m", "x", "hi"])
    s = resolve_sampling(a, {})
    assert s.temperature == 0.0 and s.top_k == 40 and s.top_p == 0.95 and abs(s.min_p - 0.05) < 1e-9
    s = resolve_sampling(a, {"do_sample": True, "temperature": 0.6})
    assert s.temperature == 0.6 and s.top_k == 50 and s.top_p == 1.0 and s.min_p == 0.0
    a = p.parse_args(["-m", "x", "hi", "-t", "0.8", "--top-p", "0.9", "--seed", "7"])
    s = resolve_sampling(a, {"do_sample": True, "temperature": 0.6, "top_p": 0.5})
    assert s.temperature == 0.8 and s.top_p == 0.9 and s.seed == 7


def test_cli_end_to_end_cpu(tmp_path, capsys):
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models import config as C
    from eredu_b200.models.llama import random_state

    b = make_bundle(tmp_path)
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=b.vocab_size(), eos_token_id=b.eos_ids[0])
    ck.save_safetensors_checkpoint(tmp_path, cfg, random_state(cfg, seed=0, std=0.05), torch.float32)
    tel = tmp_path / "tel.json"
    rc = main(["-m", str(tmp_path), "hello", "--device", "cpu", "-n", "8", "--timing", "--telemetry-json", str(tel)])
    assert rc == 0
    out = capsys.readouterr()
    assert "TTFT" in out.err
    t = json.loads(tel.read_text())
    assert t["generated_tokens"] <= 8 and t["prompt_tokens"] > 0 and t["stop_reason"] in ("max_tokens", "eos")
    assert t["weights_bytes"] > 0 and t["plan"]["device"] == "cpu" and "host" in t["hardware"]
    assert t["counters"]["memory"]["process"]["rss_bytes"] > 0 and "weight_store" in t["counters"]


def test_cli_automatic_plan_and_cache(tmp_path, capsys):
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models import config as C
    from eredu_b200.models.llama import random_state

    b = make_bundle(tmp_path)
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=b.vocab_size(), eos_token_id=b.eos_ids[0])
    ck.save_safetensors_checkpoint(tmp_path, cfg, random_state(cfg, seed=0, std=0.05), torch.float32)
    tel, cache = tmp_path / "tel.json", tmp_path / "auto.json"
    # --auto plan: the report goes to stdout, nothing is loaded or generated
    assert main(["-m", str(tmp_path), "hi", "--device", "cpu", "--auto", "plan"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["plan"]["schema_version"] == 2 and rep["plan"]["residency"]["mode"] == "fully_resident" and rep["explanation"]["summary"]
    # --auto quick (the default): plan, then run with it; the plan is cached and recorded in the telemetry
    args = ["-m", str(tmp_path), "hi", "--device", "cpu", "-n", "4", "--auto-cache", str(cache), "--telemetry-json", str(tel)]
    assert main(args) == 0
    assert "automatic plan:" in capsys.readouterr().err
    t = json.loads(tel.read_text())
    plan = t["plan"]["execution_plan"]
    assert plan["schema_version"] == 2 and plan["residency"]["mode"] == "fully_resident" and plan["topology"]["tensor"] == 1
    assert t["plan"]["model_type"] == "llama" and t["plan"]["tensor_bytes"] > 0
    assert len(json.loads(cache.read_text())) == 1
    assert main(args) == 0                                     # second run takes the cached plan
    capsys.readouterr()
    # --auto-feedback: earlier telemetry of this model decides; the faster plan (layer window, made up here) wins
    slow = dict(t, timing=dict(t["timing"], decode_token_rate=10.0))
    fast_plan = dict(plan, residency={"mode": "layerwise_host", "device_layer_window": 1})
    fast = dict(t, plan=dict(t["plan"], execution_plan=fast_plan), timing=dict(t["timing"], decode_token_rate=50.0))
    other = dict(fast, plan=dict(fast["plan"], model_type="qwen3"), timing=dict(t["timing"], decode_token_rate=500.0))
    fb = tmp_path / "fb.json"
    fb.write_text(json.dumps([slow, fast, fast, other]))
    assert main(["-m", str(tmp_path), "hi", "--device", "cpu", "--auto", "plan", "--auto-feedback", str(fb)]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["plan"]["residency"]["mode"] == "layerwise_host" and "2 matching runtime sample" in rep["explanation"]["summary"]
    with pytest.raises(SystemExit):
        main(["-m", str(tmp_path), "hi", "--device", "cpu", "--auto-feedback", str(tmp_path / "missing.json")])
    # an artifact that cannot be loaded is refused before any payload is read
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "config.json").write_text(json.dumps({"model_type": "deepseek_v3", "hidden_size": 64}))
    with pytest.raises(SystemExit):
        main(["-m", str(bad), "hi", "--device", "cpu"])


def test_cli_mirostat_and_regex_constraint(tmp_path, capsys):
    pytest.importorskip("llguidance")
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models import config as C
    from eredu_b200.models.llama import random_state

    b = make_bundle(tmp_path)
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=b.vocab_size(), eos_token_id=b.eos_ids[0])
    ck.save_safetensors_checkpoint(tmp_path, cfg, random_state(cfg, seed=0, std=0.05), torch.float32)
    base = ["-m", str(tmp_path), "hello", "--device", "cpu", "--no-auto", "--raw"]
    tel = tmp_path / "t.json"
    assert main(base + ["-n", "6", "--mirostat-v2", "-t", "0.9", "--seed", "3", "--telemetry-json", str(tel)]) == 0
    first = capsys.readouterr().out
    assert json.loads(tel.read_text())["generated_tokens"] <= 6
    assert main(base + ["-n", "6", "--mirostat-v2", "-t", "0.9", "--seed", "3"]) == 0
    assert capsys.readouterr().out == first                    # seeded: reproducible
    with pytest.raises(SystemExit):
        main(base + ["--mirostat-v2", "-t", "0"])
    # a regular expression bounds the reply: whatever the random model prefers, the text matches it
    assert main(base + ["-n", "12", "--regex", "(ab|ba){1,3}", "--telemetry-json", str(tel)]) == 0
    text = capsys.readouterr().out.strip()
    import re

    assert re.fullmatch("(ab|ba){1,3}", text), text
    assert json.loads(tel.read_text())["stop_reason"] in ("grammar_complete", "eos")


def test_cli_draft_model_gives_the_same_text(tmp_path, capsys):
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models import config as C
    from eredu_b200.models.llama import random_state

    tgt, drf = tmp_path / "target", tmp_path / "draft"
    for path, layers, seed in ((tgt, 2, 0), (drf, 1, 0)):
        path.mkdir()
        b = make_bundle(path)
        cfg = dataclasses.replace(C.tiny_llama(), vocab_size=b.vocab_size(), eos_token_id=b.eos_ids[0], num_hidden_layers=layers)
        ck.save_safetensors_checkpoint(path, cfg, random_state(cfg, seed=seed, std=0.05), torch.float32)
    base = ["-m", str(tgt), "hello there", "--device", "cpu", "--no-auto", "--raw", "-n", "12", "-t", "0"]
    assert main(base) == 0
    plain = capsys.readouterr().out
    tel = tmp_path / "t.json"
    assert main(base + ["--draft-model", str(drf), "--mtp-draft-tokens", "3", "--telemetry-json", str(tel)]) == 0
    assert capsys.readouterr().out == plain
    spec = json.loads(tel.read_text())["plan"]["speculative"]
    assert spec["rounds"] > 0 and spec["proposed"] >= spec["accepted"]
    with pytest.raises(SystemExit):
        main(base + ["--draft-model", str(drf), "--mirostat-v2", "-t", "0.7"])


def test_cli_profile_components(tmp_path, capsys):
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models import config as C
    from eredu_b200.models.llama import random_state

    b = make_bundle(tmp_path)
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=b.vocab_size(), eos_token_id=b.eos_ids[0], num_hidden_layers=3)
    ck.save_safetensors_checkpoint(tmp_path, cfg, random_state(cfg, seed=0, std=0.05), torch.float32)
    tel = tmp_path / "t.json"
    assert main(["-m", str(tmp_path), "hello", "--device", "cpu", "--no-auto", "-n", "3", "--profile-components",
                 "--telemetry-json", str(tel)]) == 0
    err = capsys.readouterr().err
    assert "model.layers.2.output" in err and "lm_head" in err
    comp = json.loads(tel.read_text())["counters"]["components"]
    names = [s["name"] for s in comp["stages"]]
    assert names == ["model.embed_tokens", "model.layers.0.output", "model.layers.1.output", "model.layers.2.output", "lm_head"]
    assert abs(sum(s["share"] for s in comp["stages"]) - 1.0) < 1e-6


def test_cli_automatic_benchmark(tmp_path, capsys):
    """--auto benchmark times each admitted residency form in a fresh process and reports the fastest."""
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models import config as C
    from eredu_b200.models.llama import random_state

    b = make_bundle(tmp_path)
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=b.vocab_size(), eos_token_id=-1)
    ck.save_safetensors_checkpoint(tmp_path, cfg, random_state(cfg, seed=0, std=0.05), torch.float32)
    cache = tmp_path / "auto.json"
    assert main(["-m", str(tmp_path), "--device", "cpu", "--auto", "benchmark", "--auto-benchmark-tokens", "6",
                 "--auto-cache", str(cache), "hello"]) == 0
    rep = json.loads(capsys.readouterr().out)
    modes = [c["plan"]["residency"]["mode"] for c in rep["candidates"]]
    assert modes[:3] == ["fully_resident", "layerwise_host", "dense_disk_stream"] and len(modes) == 3
    assert all(c["median_token_rate"] and not any("error" in t for t in c["trials"]) for c in rep["candidates"]), rep
    assert rep["selected"] == rep["candidates"][rep["selected_index"]]["plan"] and rep["selection_metric"] == "median_decode_token_rate"
    entry = next(iter(json.loads(cache.read_text()).values()))
    assert entry["plan"] == rep["selected"] and entry["benchmark_token_rate"] == rep["selected_median_token_rate"]


def test_cli_draft_model_with_a_grammar(tmp_path, capsys):
    """--draft-model and --regex together: speculation under the grammar gives the text constrained decoding gives."""
    pytest.importorskip("llguidance")
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models import config as C
    from eredu_b200.models.llama import random_state

    tgt, drf = tmp_path / "t", tmp_path / "d"
    for d, layers, seed in ((tgt, 2, 0), (drf, 1, 4)):
        d.mkdir()
        b = make_bundle(d)
        cfg = dataclasses.replace(C.tiny_llama(), vocab_size=b.vocab_size(), eos_token_id=b.eos_ids[0], num_hidden_layers=layers)
        ck.save_safetensors_checkpoint(d, cfg, random_state(cfg, seed=seed, std=0.05), torch.float32)
    base = ["-m", str(tgt), "answer:", "--device", "cpu", "--no-auto", "--raw", "-n", "16", "-t", "0", "--regex", "(ab|ba){2,4}!"]
    assert main(base) == 0
    plain = capsys.readouterr().out
    tel = tmp_path / "tel.json"
    assert main(base + ["--draft-model", str(drf), "--telemetry-json", str(tel)]) == 0
    assert capsys.readouterr().out == plain and plain.strip().endswith("!")
    spec = json.loads(tel.read_text())["plan"]["speculative"]
    assert spec["constrained"] and spec["rounds"] >= 1
    with pytest.raises(SystemExit):
        main(base + ["--draft-model", str(drf), "--mirostat-v2", "-t", "0.7"])
