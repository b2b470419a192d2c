"""Layerwise host residency: identical tokens with the layers streamed through a device window; prefetch keeps
acquire() on the hit path; dense, quantised and sparse layers are units."""
import dataclasses

import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.engine import Engine
from eredu_b200.runtime.weight_residency import LayerwiseHostResidency


def _run(device, dtype, cfg, window, moe=False, prompts_n=2):
    from eredu_b200.models.moe import make_moe_factory

    sd = random_state(cfg, seed=0, std=0.05)
    kw = {"moe_factory": make_moe_factory()} if moe else {}
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 21)][:prompts_n]
    sp = SamplingParams(temperature=0.0)
    ref = Engine(build_from_tensors(cfg, sd.__getitem__, sd.__contains__, device, dtype, **kw), max_batch=2, max_seq_len=64)
    want = ref.generate(prompts, sp, 8)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, device, dtype, **kw)
    res = LayerwiseHostResidency(model, device_layer_window=window)
    got = Engine(model, max_batch=2, max_seq_len=64).generate(prompts, sp, 8)
    return want, got, res


@pytest.mark.parametrize("window", [1, 2, 5])
def test_layerwise_host_cpu(window):
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=512, num_hidden_layers=5)
    want, got, res = _run("cpu", torch.float32, cfg, window)
    assert got == want
    rep = res.report()
    assert rep["loads"] >= 5 and rep["host_bytes"] > 0 and rep["device_layer_window"] == min(window, 5)
    if window < 5:
        assert rep["hits"] > rep["stalls"]      # prefetch covered most acquisitions
    with pytest.raises(ValueError):
        LayerwiseHostResidency(res.model, 0)


def test_layerwise_host_moe_cpu():
    cfg = dataclasses.replace(C.tiny_llama(), model_type="qwen3_moe", qk_norm=True, vocab_size=512, num_experts=4,
                              num_experts_per_tok=2, moe_intermediate_size=64, tie_word_embeddings=False,
                              num_hidden_layers=3)
    want, got, _ = _run("cpu", torch.float32, cfg, 1, moe=True)
    assert got == want


@pytest.mark.gpu
@pytest.mark.parametrize("window", [1, 3])
def test_layerwise_host_gpu(window):
    cfg = dataclasses.replace(C.tiny_llama(), hidden_size=1024, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                              intermediate_size=2048, vocab_size=4096, num_hidden_layers=6, tie_word_embeddings=False)
    want, got, res = _run("cuda:0", torch.bfloat16, cfg, window)
    assert got == want
    assert res.report()["device_slot_bytes"] < res.report()["host_bytes"]


def test_layerwise_host_through_the_load_api(tmp_path):
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats import checkpoint as ck

    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=512, num_hidden_layers=4)
    ck.save_safetensors_checkpoint(tmp_path, cfg, random_state(cfg, seed=0, std=0.05), torch.float32)
    prompt = list(range(3, 20))
    want = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64)).generate([prompt], None, 6)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64,
                                                     weight_residency="layerwise_host", device_layer_window=2))
    assert lm.model.residency is not None and lm.generate([prompt], None, 6) == want
    assert lm.model.residency.report()["loads"] > 4


def test_dense_disk_stream_cpu(tmp_path):
    from eredu_b200.runtime.weight_residency import DiskStreamResidency

    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=512, num_hidden_layers=6)
    sd = random_state(cfg, seed=0, std=0.05)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 21)]
    sp = SamplingParams(temperature=0.0)
    want = Engine(build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32), max_batch=2,
                  max_seq_len=64).generate(prompts, sp, 8)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32)
    res = DiskStreamResidency(model, host_lookahead=2, background_queue=2, spill_dir=tmp_path)
    assert len(list(tmp_path.glob("layer-*.bin"))) == 6 and all(lw.wqkv is None for lw in model.layers)
    got = Engine(model, max_batch=2, max_seq_len=64).generate(prompts, sp, 8)
    assert got == want
    rep = res.report()
    assert rep["mode"] == "dense_disk_stream" and rep["max_host_layers"] <= 2 + 1 + 1   # window + one being published
    assert rep["host_layers_now"] <= 3 and rep["evictions"] > 0 and rep["bytes_read"] > 0
    assert rep["background_reads"] > rep["demand_reads"]          # the readers stayed ahead of the compute
    led = rep["ledger"]
    assert led["host"]["resident_units"] == rep["host_layers_now"] and led["device"]["resident_units"] <= 2
    assert led["transfers"]["disk_to_host"]["count"] == rep["background_reads"] + rep["demand_reads"]
    assert led["transfers"]["host_to_device"]["bytes"] == rep["bytes_loaded"] and led["disk"]["resident_units"] == 6
    res.close()
    with pytest.raises(ValueError):
        DiskStreamResidency(model, host_lookahead=0)


def test_dense_disk_stream_load_option(tmp_path):
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats import checkpoint as ck

    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=512, num_hidden_layers=4)
    ck.save_safetensors_checkpoint(tmp_path / "m", cfg, random_state(cfg, seed=1, std=0.05), torch.float32)
    a = LoadedModel.load(tmp_path / "m", ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    b = LoadedModel.load(tmp_path / "m", ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64,
                                                          weight_residency="dense_disk_stream", dense_host_lookahead=1,
                                                          dense_background_queue=1, dense_spill_dir=str(tmp_path / "spill")))
    prompt = list(range(4, 30))
    assert torch.equal(a.prefill_logits(prompt), b.prefill_logits(prompt))
    assert b.model.residency.report()["mode"] == "dense_disk_stream"
