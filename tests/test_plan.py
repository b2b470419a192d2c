"""Inspection reports, resource estimates, admission and the automatic planner (CPU, no payload I/O)."""
import dataclasses
import json

import pytest
import torch

from eredu_b200.formats import checkpoint as ck
from eredu_b200.models import config as C
from eredu_b200.models.llama import random_state
from eredu_b200.runtime import plan as P


def test_inspection_reports(tmp_path):
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=512)
    sd = random_state(cfg, seed=0)
    ck.save_safetensors_checkpoint(tmp_path / "st", cfg, sd, torch.float32)
    rep = P.inspect_artifact(tmp_path / "st")
    assert rep.is_loadable and rep.format == "safetensors" and rep.model_type == "llama"
    assert rep.parameter_count == sum(v.numel() for v in sd.values()) and rep.dtypes == {"F32": rep.tensor_bytes}
    assert any(i.code == "no_tokenizer" for i in rep.issues)
    ck.save_gguf_checkpoint(tmp_path / "m.gguf", cfg, sd, "F32")
    g = P.inspect_artifact(tmp_path / "m.gguf")
    assert g.is_loadable and g.format == "gguf" and g.parameter_count == rep.parameter_count
    # unsupported family and missing tensors are errors, found without touching a payload
    bad = dataclasses.replace(cfg, model_type="some_future_family")
    ck.save_safetensors_checkpoint(tmp_path / "bad", bad, {k: v for k, v in sd.items() if "embed_tokens" not in k}, torch.float32)
    b = P.inspect_artifact(tmp_path / "bad")
    assert not b.is_loadable and {"unsupported_architecture", "missing_tensor"} <= {i.code for i in b.issues}
    assert not P.inspect_artifact(tmp_path / "nope").is_loadable
    json.dumps(rep.to_dict())


def test_estimates_and_admission():
    cfg = C.llama3_8b()
    prof = P.estimate_runtime_state(cfg)
    assert prof.kv_bytes_per_token == 2 * 8 * 128 * 2 * 32            # 128 KiB per token
    assert abs(prof.weight_bytes - 16.06e9) < 0.1e9
    ok = P.apply_admission_policy(prof, 180 * 10**9, context=8192, batch=32)
    assert ok.admitted and ok.max_context > 8192
    no = P.apply_admission_policy(prof, 24 * 10**9, context=65536, batch=32)
    assert not no.admitted and "KV cache" in no.reason
    moe = P.estimate_runtime_state(C.qwen3_30b_a3b())
    assert 55e9 < moe.weight_bytes < 65e9 and moe.expert_bytes > 0.9 * moe.weight_bytes * 0.9
    win = dataclasses.replace(cfg, sliding_window=1024, model_type="mistral")
    pw = P.estimate_runtime_state(win)
    assert P.kv_bytes_for(pw, 8192, 1) == 1024 * pw.kv_bytes_per_token


def test_planner_choices():
    hw8 = P.HardwareProfile(device_count=8)
    planner = P.AutomaticPlanner(hw8)
    p8b = planner.plan(C.llama3_8b(), P.estimate_runtime_state(C.llama3_8b()), context=4096, batch=32)
    assert p8b.topology["tensor"] == 1 and p8b.residency["mode"] == "fully_resident"
    assert p8b.weight_transformation["mode"] == "preserve_checkpoint" and p8b.schema_version == 2
    c70 = C.llama3_70b()
    p70 = planner.plan(c70, P.estimate_runtime_state(c70), context=8192, batch=32)
    assert p70.topology["tensor"] == 2 and p70.required_capabilities["collectives"]
    moe = C.qwen3_30b_a3b()
    pm = planner.plan(moe, P.estimate_runtime_state(moe), context=2048, batch=32, prefer_devices=8)
    assert pm.topology == {"data": 1, "pipeline": 1, "tensor": 8, "expert": 8, "expert_over_tensor": True}
    one = P.AutomaticPlanner(P.HardwareProfile(device_count=1, device_memory_bytes=80 * 10**9))
    q = one.plan(c70, P.estimate_runtime_state(c70), context=4096, batch=8)
    assert q.weight_transformation == {"mode": "affine", "bits": 4, "group_size": 64} and q.topology["tensor"] == 1
    small = P.AutomaticPlanner(P.HardwareProfile(device_count=1, device_memory_bytes=24 * 10**9))
    h = small.plan(c70, P.estimate_runtime_state(c70), context=2048, batch=1)
    assert h.residency["mode"] == "layerwise_host" and h.residency["device_layer_window"] >= 1
    d = planner.plan(C.llama3_8b(), P.estimate_runtime_state(C.llama3_8b()), draft_model="draft-16l")
    assert d.drafting["mode"] == "external" and d.drafting["max_draft_tokens"] == 4
    again = P.ExecutionPlan.from_json(p70.to_json())
    assert again.topology == p70.topology
    with pytest.raises(ValueError):
        P.ExecutionPlan.from_json(p70.to_json().replace('"schema_version": 2', '"schema_version": 1'))


def test_hybrid_models_are_inspectable_and_sized_by_their_attention_layers(tmp_path):
    import json

    from eredu_b200.models.config import ModelConfig
    from eredu_b200.runtime.plan import estimate_runtime_state, inspect_artifact, kv_bytes_for

    d = {"model_type": "qwen3_next", "vocab_size": 1000, "hidden_size": 256, "num_hidden_layers": 8, "num_attention_heads": 4,
         "num_key_value_heads": 2, "head_dim": 128, "linear_num_key_heads": 2, "linear_num_value_heads": 4,
         "linear_key_head_dim": 64, "linear_value_head_dim": 64, "num_experts": 8, "num_experts_per_tok": 2,
         "moe_intermediate_size": 64, "shared_expert_intermediate_size": 64}
    cfg = ModelConfig.from_hf_dict(d)
    prof = estimate_runtime_state(cfg)
    assert prof.kv_bytes_per_token == 2 * 2 * 128 * 2 * 2               # two full-attention layers of eight
    conv_dim = 2 * 2 * 64 + 4 * 64
    assert prof.state_bytes_per_sequence == 6 * (3 * conv_dim * 2 + 4 * 64 * 64 * 4)
    assert kv_bytes_for(prof, 100, 3) == 3 * (prof.kv_bytes_per_token * 100 + prof.state_bytes_per_sequence)
    (tmp_path / "config.json").write_text(json.dumps(d))
    rep = inspect_artifact(tmp_path)
    assert all(i.code != "unsupported_architecture" for i in rep.issues)
    lf = ModelConfig.from_hf_dict({"model_type": "lfm2", "vocab_size": 100, "hidden_size": 64, "intermediate_size": 128,
                                   "num_hidden_layers": 3, "num_attention_heads": 2, "num_key_value_heads": 2,
                                   "layer_types": ["conv", "full_attention", "conv"]})
    p2 = estimate_runtime_state(lf)
    assert p2.kv_bytes_per_token == 2 * 2 * 32 * 2 and p2.state_bytes_per_sequence == 2 * 2 * 64 * 2


def test_inspection_knows_every_family_layout(tmp_path):
    """A freshly written checkpoint of each family inspects as loadable; a malformed config is reported, not raised."""
    import json
    import sys
    from pathlib import Path

    import torch

    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models.llama import random_state
    from eredu_b200.runtime.plan import inspect_artifact

    sys.path.insert(0, str(Path(__file__).parent))
    from test_deepseek import ds_cfg
    from test_kimi_linear import kimi_cfg
    from test_lfm2 import lfm2_cfg
    from test_nemotron_h import nh_cfg
    from test_qwen_next import next_cfg

    from eredu_b200.models import lfm2, nemotron_h

    for name, cfg, rename in (("lfm2", lfm2_cfg(), lfm2.to_checkpoint_names), ("qnext", next_cfg(), None),
                              ("nemotron", nh_cfg(), nemotron_h.to_checkpoint_names), ("dsv3", ds_cfg(), None),
                              ("kimi", kimi_cfg(), None)):
        sd = random_state(cfg, seed=0, std=0.05)
        ck.save_safetensors_checkpoint(tmp_path / name, cfg, rename(sd) if rename else sd, torch.float32)
        rep = inspect_artifact(tmp_path / name)
        assert rep.is_loadable, (name, [(i.code, i.message) for i in rep.issues])
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "config.json").write_text(json.dumps({"model_type": "kimi_linear", "hidden_size": 64, "num_hidden_layers": 2}))
    rep = inspect_artifact(bad)
    assert not rep.is_loadable and rep.issues[0].code == "invalid_config"


def test_cache_formulas_of_families_with_mixed_layer_widths():
    """Gemma 4 (two head geometries, a KV-sharing tail), DeepSeek-V4 (windowed keys + pooled streams) and Inkling (sliding
    layers with their own heads, convolution tails): what grows with the context, what saturates at the window."""
    import sys
    from pathlib import Path

    sys.path.insert(0, str(Path(__file__).parent))
    from test_deepseek_v4 import v4_cfg
    from test_inkling import ink_cfg

    from eredu_b200.models.config import ModelConfig

    v4 = ModelConfig.from_hf_dict(dict(v4_cfg(), model_type="deepseek_v4"))
    prof = P.estimate_runtime_state(v4, weight_bytes=1000)
    # ratios [0, 3, 4, 4], head 16, index head 8, window 6, bf16 cache: 4 layers x 16 x 2 bytes inside the window;
    # pooled: 16/3 + 2 x (16 + 8)/4 values per token
    assert prof.windowed_bytes_per_token == 4 * 16 * 2 and prof.sliding_window == 6
    assert prof.kv_bytes_per_token == int((16 / 3 + 2 * 24 / 4) * 2)
    short, long = P.kv_bytes_for(prof, 6, 1), P.kv_bytes_for(prof, 6000, 1)
    assert long - short == prof.kv_bytes_per_token * (6000 - 6)             # only the pooled streams keep growing
    ink = ModelConfig.from_hf_dict(ink_cfg())
    prof = P.estimate_runtime_state(ink, weight_bytes=1000)
    # layers: sliding (1 kv head x 8), full (2 x 8), sliding; window 5; four convolution tails of 2 rows per layer
    assert prof.kv_bytes_per_token == 2 * 2 * 8 * 2 and prof.windowed_bytes_per_token == 2 * (2 * 1 * 8 * 2)
    assert prof.state_bytes_per_sequence == (2 * (2 * 1 * 8 + 2 * 40) * 4) * 2 + 2 * (2 * 2 * 8 + 2 * 40) * 4
    from test_hf_parity import G4
    import transformers

    g4 = ModelConfig.from_hf_dict(transformers.Gemma4TextConfig(**dict(G4, num_kv_shared_layers=3, hidden_size_per_layer_input=0,
                                                                       attention_k_eq_v=False, enable_moe_block=False)).to_dict())
    prof = P.estimate_runtime_state(g4, weight_bytes=1000)
    # six layers [s, s, f] x 2, the last three share: two sliding layers (2 kv x 16) and one global (2 kv x 32) own a cache
    assert prof.windowed_bytes_per_token == 2 * (2 * 2 * 16 * 2) and prof.kv_bytes_per_token == 2 * 2 * 32 * 2
