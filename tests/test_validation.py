"""Validation harness: probes of this runtime and of Transformers, gates, command line."""
import json

import pytest
import torch

transformers = pytest.importorskip("transformers")

from eredu_b200.api import LoadedModel, ModelLoadOptions
from eredu_b200.validation import PROFILES, compare_probes, default_token_ids, probe_checkpoint, probe_reference
from eredu_b200.validation.__main__ import main


def tiny(tmp_path):
    cfg = transformers.Qwen3Config(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=32, max_position_embeddings=256)
    torch.manual_seed(0)
    m = transformers.Qwen3ForCausalLM(cfg).eval().float()
    m.save_pretrained(tmp_path, safe_serialization=True)
    return m


def test_probes_and_gates(tmp_path):
    m = tiny(tmp_path)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=128))
    ids = default_token_ids(320, 40)
    assert ids == default_token_ids(320, 40) and len(ids) == 40
    ours, ref = probe_checkpoint(lm, ids, decode_steps=8), probe_reference(m, ids, decode_steps=8)
    assert sorted(ours["prefill"]) == [0, 7, 31] and len(ours["decode"]) == 8 and sorted(ours["recompute"]) == [0, 7]
    v = compare_probes(ours, ref, PROFILES["fp32_exact"])
    assert v["passed"], v["failures"]
    assert any(r["row"].startswith("cached_vs_recompute") for r in v["rows"])
    # a damaged runtime result is caught by several gates at once
    bad = dict(ours, decode=[t + torch.randn_like(t) * 0.5 for t in ours["decode"]])
    v2 = compare_probes(bad, ref, PROFILES["bf16_reference"])
    assert not v2["passed"] and any("relative L2" in f for f in v2["failures"]) and any("cached_vs_recompute" in f for f in v2["failures"])
    # an argmax flip only counts where the reference's margin is above the profile's floor
    flip = {k: v_ for k, v_ in ours.items()}
    t = ours["prefill"][0].clone()
    top = torch.topk(ref["prefill"][0], 2).indices
    t[top[0]], t[top[1]] = ours["prefill"][0][top[1]], ours["prefill"][0][top[0]]
    flip["prefill"] = {**ours["prefill"], 0: t}
    loose = PROFILES["bf16_reference"].__class__(relative_l2_max=1.0, cosine_similarity_min=0.0, top_k_overlap_min=0,
                                                 argmax_margin_min=1e9, require_cached_vs_full_recompute=False)
    assert compare_probes(flip, ref, loose)["passed"]
    strict = loose.__class__(relative_l2_max=1.0, cosine_similarity_min=0.0, top_k_overlap_min=0, argmax_margin_min=0.0,
                             require_cached_vs_full_recompute=False)
    assert any("argmax" in f for f in compare_probes(flip, ref, strict)["failures"])
    with pytest.raises(ValueError):
        compare_probes(dict(ours, token_ids=[1]), ref, loose)


def test_command_line(tmp_path, capsys):
    tiny(tmp_path)
    rep = tmp_path / "report.json"
    rc = main(["--model", str(tmp_path), "--profile", "fp32_exact", "--device", "cpu", "--length", "40", "--decode-steps", "8",
               "--report", str(rep)])
    assert rc == 0 and "validated" in capsys.readouterr().out
    data = json.loads(rep.read_text())
    assert data["passed"] and data["profile"] == "fp32_exact" and len(data["rows"]) >= 11
