"""Checkpoint-embedded prediction layers (Qwen3-Next ``mtp.*``, DeepSeek-V3 layer L) as the drafter of speculative decoding."""
import dataclasses

import pytest
import torch

from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.models.moe import make_moe_factory
from eredu_b200.models.mtp import build_embedded_mtp, head_config
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.engine import Engine
from eredu_b200.runtime.speculative import EmbeddedMtpDecoder


def with_mtp(family, seed=0):
    """Configuration and tensors of a tiny checkpoint that carries one prediction layer in its family's own naming."""
    if family == "qwen3_next":
        from test_qwen_next import next_cfg, state_for

        cfg = next_cfg(mtp_num_hidden_layers=1)
        sd = state_for(cfg, seed)
        head = state_for(head_config(cfg), seed + 100)
        for k, v in head.items():
            if k.startswith("model.layers.0."):
                sd["mtp.layers.0." + k[len("model.layers.0."):]] = v
        g = torch.Generator().manual_seed(seed + 7)
        H = cfg.hidden_size
        sd["mtp.norm.weight"] = torch.randn(H, generator=g) * 0.2
        sd["mtp.fc.weight"] = torch.randn(H, 2 * H, generator=g) * 0.08
        sd["mtp.pre_fc_norm_embedding.weight"] = torch.randn(H, generator=g) * 0.2
        sd["mtp.pre_fc_norm_hidden.weight"] = torch.randn(H, generator=g) * 0.2
    elif family == "nemotron_h":
        from test_nemotron_h import nh_cfg, state_for

        cfg = nh_cfg(num_nextn_predict_layers=1, mtp_hybrid_override_pattern="*E")
        sd = state_for(cfg, seed)
        hcfg = head_config(cfg, "*E")
        head = state_for(hcfg, seed + 100)
        for k, v in head.items():
            if k.startswith("model.layers."):
                sd["mtp.layers." + k[len("model.layers."):]] = v
        g = torch.Generator().manual_seed(seed + 7)
        H = cfg.hidden_size
        sd["mtp.layers.0.enorm.weight"] = torch.rand(H, generator=g) + 0.5
        sd["mtp.layers.0.hnorm.weight"] = torch.rand(H, generator=g) + 0.5
        sd["mtp.layers.0.eh_proj.weight"] = torch.randn(H, 2 * H, generator=g) * 0.1
        sd["mtp.layers.1.final_layernorm.weight"] = torch.rand(H, generator=g) + 0.5
    else:
        from test_deepseek import ds_cfg, state_for

        cfg = ds_cfg(num_nextn_predict_layers=1)
        sd = state_for(cfg, seed)
        L = cfg.num_hidden_layers
        head = state_for(head_config(cfg), seed + 100)
        for k, v in head.items():
            if k.startswith("model.layers.0."):
                sd[f"model.layers.{L}." + k[len("model.layers.0."):]] = v
        g = torch.Generator().manual_seed(seed + 7)
        H = cfg.hidden_size
        p = f"model.layers.{L}."
        sd[p + "shared_head.norm.weight"] = torch.rand(H, generator=g) + 0.5
        sd[p + "shared_head.head.weight"] = torch.randn(cfg.vocab_size, H, generator=g) * 0.1
        sd[p + "embed_tokens.weight"] = sd["model.embed_tokens.weight"].clone()
        sd[p + "eh_proj.weight"] = torch.randn(H, 2 * H, generator=g) * 0.1
        sd[p + "enorm.weight"] = torch.rand(H, generator=g) + 0.5
        sd[p + "hnorm.weight"] = torch.rand(H, generator=g) + 0.5
    return cfg, sd


def build(family, seed=0):
    cfg, sd = with_mtp(family, seed)
    target = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    mtp = build_embedded_mtp(cfg, sd.__getitem__, sd.__contains__, target, "cpu", torch.float32, moe_factory=make_moe_factory())
    return cfg, sd, target, mtp


def test_nemotron_h_prediction_step_has_its_own_block_pattern():
    cfg, sd, target, mtp = build("nemotron_h")
    assert cfg.mtp_layers == 1 and mtp is not None and mtp.model.cfg.layer_types == ["attention_only", "moe_only"]
    assert len(mtp.model.layers) == 2 and mtp.model.layers[1].moe is not None and mtp.model.layers[0].moe is None
    assert mtp.model.embed is target.embed and mtp.model.lm_head is target.lm_head
    assert not mtp.model.cfg.extra.get("mtp_hybrid_override_pattern")
    bad = dataclasses.replace(cfg, extra=dict(cfg.extra, mtp_hybrid_override_pattern="M*"))
    with pytest.raises(ValueError, match="made of"):
        build_embedded_mtp(bad, sd.__getitem__, sd.__contains__, target, "cpu", torch.float32, make_moe_factory())


@pytest.mark.parametrize("family", ["qwen3_next", "deepseek_v3"])
def test_head_binding(family):
    cfg, sd, target, mtp = build(family)
    assert cfg.mtp_layers == 1 and mtp is not None and len(mtp.model.layers) == 1 and mtp.model.cfg.mtp_layers == 0
    assert mtp.model.layers[0].moe is not None                       # the prediction block is sparse like the family's later layers
    assert mtp.model.embed is target.embed or family == "deepseek_v3"
    if family == "qwen3_next":
        assert mtp.model.lm_head is target.lm_head                    # the model's own vocabulary head
    else:
        assert mtp.model.lm_head is not target.lm_head                # shared_head.head is the layer's own
    # without the tensors (or without the configuration key) there is no drafter
    plain = {k: v for k, v in sd.items() if not (k.startswith("mtp.") or f"layers.{cfg.num_hidden_layers}." in k)}
    assert build_embedded_mtp(cfg, plain.__getitem__, plain.__contains__, target, "cpu", torch.float32, make_moe_factory()) is None
    x = mtp.fuse(torch.tensor([5, 9], dtype=torch.int32), torch.randn(2, cfg.hidden_size))
    assert x.shape == (2, cfg.hidden_size)


@pytest.mark.parametrize("family", ["qwen3_next", "deepseek_v3", "nemotron_h"])
@pytest.mark.parametrize("k,temperature", [(1, 0.0), (3, 0.0), (2, 0.8)])
def test_committed_tokens_are_the_targets_own(family, k, temperature):
    cfg, _, target, mtp = build(family)
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in (7, 18)]
    sp = SamplingParams(temperature=temperature, top_k=30, top_p=0.95, min_p=0.0, seed=5)
    plain = Engine(target, max_batch=2, max_seq_len=96).generate(prompts, sp, 18)
    dec = EmbeddedMtpDecoder(Engine(target, max_batch=2, max_seq_len=96, use_cuda_graph=False), mtp, k=k)
    spec = dec.generate(prompts, sp, 18)
    if temperature == 0.0:
        assert spec == plain
    else:       # rejection resampling keeps the distribution, not the draw: only the prefill sample is the same draw
        assert [len(o) for o in spec] == [18, 18] and [o[0] for o in spec] == [o[0] for o in plain]
    st = dec.stats.summary()
    assert st["proposed"] == k * st["rounds"] and st["emitted"] >= st["rounds"]


@pytest.mark.parametrize("family", ["qwen3_next", "deepseek_v3"])
def test_head_cache_rows_are_exact_after_every_round(family):
    """After each round the head's cache holds only rows made from the target's hidden states: its next proposal equals
    that of a head whose cache is rebuilt from scratch over the committed tokens."""
    cfg, _, target, mtp = build(family)
    prompt = list(range(5, 16))
    sp = SamplingParams(temperature=0.0)
    dec = EmbeddedMtpDecoder(Engine(target, max_batch=1, max_seq_len=96, use_cuda_graph=False), mtp, k=3)
    seen = []
    out = dec.generate([prompt], sp, 12, on_token=lambda i, t: seen.append(t))[0]
    assert seen == out
    # rebuild: target hidden states over prompt + committed tokens, head over (h_i, t_{i+1}); its last row predicts what
    # follows the committed text, and so does a decoder that continues from the committed text
    full = prompt + out
    eng = Engine(target, max_batch=1, max_seq_len=96, use_cuda_graph=False)
    d2 = EmbeddedMtpDecoder(eng, mtp, k=1)
    ts, ds = eng.new_sequence(full, sp, 4), d2.d.new_sequence(full, sp, 4)
    first = d2._prefill([ts], [ds])
    drafted, _, _ = d2._propose([ts], [ds], [0], [[first[0]]], sp, [len(full) + 1])
    cont = EmbeddedMtpDecoder(Engine(target, max_batch=1, max_seq_len=96, use_cuda_graph=False), mtp, k=1)
    log = []
    orig = cont._propose

    def spy(*a, **kw):
        r = orig(*a, **kw)
        log.append(r[0][0][0])
        return r

    cont._propose = spy
    cont.generate([full], sp, 3)
    assert log[0] == drafted[0][0]
    eng.release(ts)
    d2.d.release(ds)


def test_loaded_model_and_command_line_use_the_embedded_drafter(tmp_path, capsys):
    import dataclasses
    import json

    from test_cli import make_bundle

    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.cli.main import main
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.runtime.plan import AutomaticPlanner, HardwareProfile, estimate_runtime_state

    b = make_bundle(tmp_path)
    cfg, sd = with_mtp("qwen3_next")
    V = b.vocab_size()
    cfg = dataclasses.replace(cfg, vocab_size=V, eos_token_id=-1)
    g = torch.Generator().manual_seed(1)
    for name in ("model.embed_tokens.weight", "lm_head.weight"):
        if name in sd:
            sd[name] = torch.randn(V, cfg.hidden_size, generator=g) * 0.08
    ck.save_safetensors_checkpoint(tmp_path, cfg, sd, torch.float32)
    assert json.loads((tmp_path / "config.json").read_text())["mtp_num_hidden_layers"] == 1
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=128))
    assert lm.mtp is not None and lm.mtp_error is None
    off = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=128, embedded_mtp=False))
    assert off.mtp is None
    base = ["-m", str(tmp_path), "hello there", "--device", "cpu", "--no-auto", "--raw", "-n", "10", "-t", "0"]
    tel = tmp_path / "tel.json"
    assert main(base + ["--telemetry-json", str(tel)]) == 0
    with_head = capsys.readouterr().out
    spec = json.loads(tel.read_text())["plan"]["speculative"]
    assert spec["drafter"] == "embedded" and spec["proposed"] == 3 * spec["rounds"]
    assert main(base + ["--mtp-draft-tokens", "0"]) == 0
    assert capsys.readouterr().out == with_head                      # same text with and without drafting
    plan = AutomaticPlanner(HardwareProfile(device_count=1)).plan(cfg, estimate_runtime_state(cfg, 10**6))
    assert plan.drafting["mode"] == "embedded" and plan.drafting["max_draft_tokens"] == 3
