"""``plan_and_load`` / ``load_execution_plan``: the facade applies a plan's transformation, residency, expert cache and
drafting to the load, refuses plans whose topology the caller is not bound to, and keeps the plan on the result."""
import dataclasses

import pytest
import torch

from eredu_b200.api import LoadedModel, ModelLoadOptions
from eredu_b200.formats import checkpoint as ck
from eredu_b200.models import config as C
from eredu_b200.models.llama import random_state
from eredu_b200.runtime.plan import ExecutionPlan


def write_tiny(tmp_path):
    cfg = C.tiny_llama()
    ck.save_safetensors_checkpoint(tmp_path, cfg, random_state(cfg, seed=0, std=0.05), torch.float32)
    return cfg


def plan(**kw):
    base = dict(device={"backend": "cuda-sm100a", "device": "gpu:0"},
                topology={"data": 1, "pipeline": 1, "tensor": 1, "expert": 1, "expert_over_tensor": False},
                residency={"mode": "fully_resident"}, weight_transformation={"mode": "preserve_checkpoint"})
    base.update(kw)
    return ExecutionPlan(**base)


def test_plan_and_load_on_cpu(tmp_path):
    write_tiny(tmp_path)
    opt = ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64)
    lm = LoadedModel.plan_and_load(tmp_path, opt, context=64)
    assert lm.execution_plan.residency["mode"] == "fully_resident" and lm.execution_plan.topology["tensor"] == 1
    assert lm.execution_plan.weight_transformation["mode"] == "preserve_checkpoint" and lm.execution_plan.rationale
    ref = LoadedModel.load(tmp_path, opt)
    ids = [1, 5, 9, 2]
    assert torch.equal(lm.prefill_logits(ids), ref.prefill_logits(ids))
    assert opt.weight_residency == "device"                         # the caller's options object is left alone


def test_load_execution_plan_applies_and_refuses(tmp_path):
    write_tiny(tmp_path)
    opt = ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64)
    lw = LoadedModel.load_execution_plan(tmp_path, plan(residency={"mode": "layerwise_host", "device_layer_window": 1},
                                                        max_mapped_shards=2), opt)
    assert lw.model.residency is not None and lw.execution_plan.max_mapped_shards == 2
    ids = [1, 5, 9, 2]
    assert torch.allclose(lw.prefill_logits(ids), LoadedModel.load(tmp_path, opt).prefill_logits(ids), atol=1e-5)
    with pytest.raises(ValueError, match="topology"):
        LoadedModel.load_execution_plan(tmp_path, plan(topology={"data": 1, "pipeline": 1, "tensor": 2, "expert": 1,
                                                                  "expert_over_tensor": False}), opt)
    with pytest.raises(ValueError, match="data parallelism"):
        LoadedModel.load_execution_plan(tmp_path, plan(topology={"data": 2, "pipeline": 1, "tensor": 1, "expert": 1}), opt)
    bad = plan()
    bad.schema_version = 1
    with pytest.raises(ValueError, match="schema"):
        LoadedModel.load_execution_plan(tmp_path, bad, opt)
    # a serialized plan round-trips through the same entry point
    again = LoadedModel.load_execution_plan(tmp_path, ExecutionPlan.from_json(plan().to_json()), opt)
    assert dataclasses.asdict(again.execution_plan)["residency"] == {"mode": "fully_resident"}
