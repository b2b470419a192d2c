"""DFlash block drafter: attention mask and context bookkeeping against direct restatements, and the speculative loop's
exactness (greedy output equals plain decoding) on a Muse-Glimmer target and on a Llama target."""
import json

import pytest
import torch

from eredu_b200.api import LoadedModel, ModelLoadOptions
from eredu_b200.models.dflash import DFlash, DFlashConfig, DFlashContext
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.speculative import DFlashDecoder


def df_cfg(**over):
    d = dict(model_type="muse_glimmer_assistant", hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, max_position_embeddings=256, sliding_window=12, block_size=5,
             mask_token_id=199, target_layer_ids=[0, 2], layer_types=["sliding_attention"] * 2, hidden_act="silu",
             rope_parameters={"rope_theta": 10000.0})
    d.update(over)
    return d


def df_state(cfg: DFlashConfig, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, std=0.2: torch.randn(*s, generator=g) * std          # noqa: E731
    H, D, Hq, Hkv, I = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
    sd = {"encoder.fc.weight": r(H, H * len(cfg.target_layer_ids)), "encoder.output_norm_enc.weight": 1 + r(H, std=0.1),
          "norm.weight": 1 + r(H, std=0.1)}
    for li in range(cfg.num_hidden_layers):
        p = f"layers.{li}."
        sd[p + "self_attn.q_proj.weight"], sd[p + "self_attn.o_proj.weight"] = r(Hq * D, H), r(H, Hq * D)
        sd[p + "self_attn.k_proj.weight"], sd[p + "self_attn.v_proj.weight"] = r(Hkv * D, H), r(Hkv * D, H)
        sd[p + "self_attn.q_norm.weight"], sd[p + "self_attn.k_norm.weight"] = 1 + r(D, std=0.1), 1 + r(D, std=0.1)
        sd[p + "input_layernorm.weight"], sd[p + "post_attention_layernorm.weight"] = 1 + r(H, std=0.1), 1 + r(H, std=0.1)
        sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"], sd[p + "mlp.down_proj.weight"] = r(I, H), r(I, H), r(H, I)
    return sd


def test_context_is_windowed_and_incremental():
    cfg = DFlashConfig.from_dict(df_cfg())
    sd = df_state(cfg)
    d = DFlash(cfg, sd.__getitem__, sd.__contains__)
    states = torch.randn(20, 128, generator=torch.Generator().manual_seed(1))
    whole = d.extend_context(DFlashContext(), states, 20)
    assert (whole.start, whole.end) == (8, 20) and whole.keys[0].shape == (12, 2, 16)
    step = d.extend_context(DFlashContext(), states[:7], 7)
    step = d.extend_context(step, states[7:15], 15)
    step = d.extend_context(step, states[15:], 20)
    for a, b in zip(whole.keys + whole.values, step.keys + step.values):
        assert torch.allclose(a, b, atol=1e-5)
    with pytest.raises(ValueError, match="context ends"):
        d.extend_context(step, states[:3], 30)


def test_block_attention_is_causal_over_the_context_and_bidirectional_inside_the_block():
    cfg = DFlashConfig.from_dict(df_cfg(num_hidden_layers=1))
    sd = df_state(cfg)
    d = DFlash(cfg, sd.__getitem__, sd.__contains__)
    g = torch.Generator().manual_seed(2)
    ctx = d.extend_context(DFlashContext(), torch.randn(9, 128, generator=g), 9)
    block = torch.randn(4, 64, generator=g)
    out = d.propose(block, ctx)
    assert out.shape == (3, 64)
    # a later block token changes an earlier row's state (bidirectional inside the block) ...
    other = block.clone()
    other[3] += 1.0
    assert not torch.allclose(d.propose(other, ctx)[0], out[0])
    # ... and the window hides the oldest context position from the last block rows only
    far = d.extend_context(DFlashContext(), torch.randn(12, 128, generator=g), 12)     # positions 0 .. 11, block at 12 .. 15
    moved = far.clone()
    moved.values = [v.clone() for v in far.values]
    moved.values[0][0] += 5.0                     # context position 0: visible from position 11 at most (window 12)
    a, b = d.propose(block, far), d.propose(block, moved)
    assert torch.allclose(a, b, atol=1e-6)        # every block row stands at 12 or later
    # position 1 is visible from block row 0 (position 12) only: with two layers the change reaches rows 1.. through row 0
    cfg2 = DFlashConfig.from_dict(df_cfg())
    sd2 = df_state(cfg2)
    d2 = DFlash(cfg2, sd2.__getitem__, sd2.__contains__)
    far2 = d2.extend_context(DFlashContext(), torch.randn(12, 128, generator=g), 12)
    moved2 = far2.clone()
    moved2.values[0][1] += 5.0
    assert not torch.allclose(d2.propose(block, far2), d2.propose(block, moved2), atol=1e-6)
    moved.values[0][1] += 5.0
    assert torch.allclose(a, d.propose(block, moved), atol=1e-6)      # one layer: rows 1.. never read row 0's output
    with pytest.raises(ValueError, match="anchor"):
        d.propose(torch.randn(6, 64), ctx)


def _muse_target(tmp_path):
    from test_muse_glimmer import save, state

    sd = state()
    save(tmp_path / "target", sd) if (tmp_path / "target").mkdir() is None else None
    return LoadedModel.load(tmp_path / "target", ModelLoadOptions(device="cpu", max_batch=4, max_seq_len=96))


def test_speculative_generation_is_exact_on_a_muse_glimmer_target(tmp_path):
    from safetensors.torch import save_file

    lm = _muse_target(tmp_path)
    cfg = DFlashConfig.from_dict(df_cfg())
    sd = df_state(cfg)
    (tmp_path / "dflash").mkdir()
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "dflash" / "model.safetensors"))
    (tmp_path / "dflash" / "config.json").write_text(json.dumps(df_cfg()))
    lm.attach_dflash(tmp_path / "dflash")
    prompts = [list(range(3, 24)), list(range(50, 59))]
    sp = SamplingParams(temperature=0.0)
    plain = lm.engine.generate(prompts, sp, 18)
    dec = lm._mtp_decoder(None, 4)
    assert isinstance(dec, DFlashDecoder) and dec.k == 4
    assert dec.generate(prompts, sp, 18) == plain
    assert dec.stats.rounds > 0 and dec.stats.proposed == 4 * dec.stats.rounds
    # the context of a finished request covers every committed token but the newest, inside the window
    out = dec.generate(prompts[:1], SamplingParams(temperature=0.7, top_p=0.9, seed=3), 10)
    assert len(out[0]) == 10


def test_the_request_scheduler_drives_dflash(tmp_path):
    from eredu_b200.runtime.mtp_scheduler import MtpScheduler, MtpSchedulerOptions

    lm = _muse_target(tmp_path)
    cfg = DFlashConfig.from_dict(df_cfg())
    sd = df_state(cfg, seed=4)
    d = DFlash(cfg, sd.__getitem__, sd.__contains__)
    prompts = [list(range(3, 20)), list(range(40, 52)), list(range(100, 109))]
    sp = SamplingParams(temperature=0.0)
    plain = lm.engine.generate(prompts, sp, 12)
    sched = MtpScheduler(DFlashDecoder(lm.engine, d, k=3), MtpSchedulerOptions())
    for p in prompts:
        sched.submit(p, sp, 12)
    done = sched.finish()
    assert [r.token_ids for r in done.requests] == plain


def test_config_validation():
    with pytest.raises(ValueError, match="not a DFlash"):
        DFlashConfig.from_dict(df_cfg(model_type="llama"))
    with pytest.raises(ValueError, match="lacks"):
        DFlashConfig.from_dict({"model_type": "muse_glimmer_assistant", "hidden_size": 64})
    cfg = DFlashConfig.from_dict(df_cfg())
    assert cfg.rope_theta == 10000.0 and cfg.target_layer_ids == [0, 2]
