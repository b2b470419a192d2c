"""Muse-Glimmer text decoder on the paged engine. Oracle: a from-scratch dense restatement of the block in plain tensor
operations (whole sequence, explicit masks, no cache), written from the family's definition; plus the engine invariants
(chunked prefill + decode-shaped steps equal the full pass)."""
import json
import math

import pytest
import torch

from eredu_b200.api import LoadedModel, ModelLoadOptions
from eredu_b200.ops import SamplingParams

TEXT = dict(model_type="muse_glimmer_text", hidden_size=64, num_hidden_layers=4, intermediate_size=96, num_attention_heads=4,
            num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, post_norm_eps=1e-5, vocab_size=200, max_position_embeddings=256,
            rope_theta=10000.0, layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
            layer_rope_theta=[10000.0, 0.0, 10000.0, 10000.0], sliding_window=6, tie_word_embeddings=False, qk_scale_factor=1.7,
            output_multiplier=0.6, final_logit_softcapping=20.0)


def state(seed=0, D=16):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, std=0.2: torch.randn(*s, generator=g) * std          # noqa: E731
    H, I, Hq, Hkv = 64, 96, 4, 2
    root = "model.language_model."
    sd = {root + "embed_tokens.weight": r(200, H, std=1.0), root + "norm.weight": 1 + r(H, std=0.1), "lm_head.weight": r(200, H, std=0.5)}
    for li in range(4):
        p = f"{root}layers.{li}."
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
            sd[p + n + ".weight"] = r(H, std=0.2)                         # centered: the scale is 1 + this
        a = p + "self_attn."
        sd[a + "q_proj.weight"], sd[a + "gate_proj.weight"] = r(Hq * D, H), r(Hq * D, H, std=0.5)
        sd[a + "k_proj.weight"], sd[a + "v_proj.weight"], sd[a + "o_proj.weight"] = r(Hkv * D, H), r(Hkv * D, H), r(H, Hq * D)
        sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"], sd[p + "mlp.down_proj.weight"] = r(I, H), r(I, H), r(H, I)
    return sd


def dense_reference(sd, tokens, D=16):
    """The whole sequence at once, every step written out."""
    H, Hq, Hkv = 64, 4, 2
    root = "model.language_model."
    wrms = lambda z, eps: z * torch.rsqrt(z.square().mean(-1, keepdim=True) + eps)        # noqa: E731
    T = len(tokens)
    h = wrms(sd[root + "embed_tokens.weight"][tokens], 1e-6)
    pos = torch.arange(T, dtype=torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = pos[:, None] * inv[None, :]
    cos, sin = torch.cat((ang.cos(), ang.cos()), -1), torch.cat((ang.sin(), ang.sin()), -1)

    def rope(z):                                         # z [T, heads, D], half-split rotation
        rot = torch.cat((-z[..., D // 2:], z[..., :D // 2]), -1)
        return z * cos[:, None, :] + rot * sin[:, None, :]

    for li in range(4):
        p = f"{root}layers.{li}."
        x = wrms(h, 1e-6) * (1 + sd[p + "input_layernorm.weight"])
        q = wrms((x @ sd[p + "self_attn.q_proj.weight"].t()).view(T, Hq, D), 1e-6) * 1.7
        k = wrms((x @ sd[p + "self_attn.k_proj.weight"].t()).view(T, Hkv, D), 1e-6)
        v = (x @ sd[p + "self_attn.v_proj.weight"].t()).view(T, Hkv, D)
        if TEXT["layer_rope_theta"][li] != 0.0:
            q, k = rope(q), rope(k)
        k, v = k.repeat_interleave(Hq // Hkv, 1), v.repeat_interleave(Hq // Hkv, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(D)
        i = torch.arange(T)
        mask = i[None, :] <= i[:, None]
        if TEXT["layer_types"][li] == "sliding_attention":
            mask = mask & (i[:, None] - i[None, :] < 6)
        s = s.masked_fill(~mask[None], float("-inf"))
        att = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(T, Hq * D)
        att = att * torch.sigmoid(x @ sd[p + "self_attn.gate_proj.weight"].t())
        a = att @ sd[p + "self_attn.o_proj.weight"].t()
        h = h + wrms(a, 1e-5) * (1 + sd[p + "post_attention_layernorm.weight"])
        y = wrms(h, 1e-6) * (1 + sd[p + "pre_feedforward_layernorm.weight"])
        if p + "mlp.gate.weight" in sd:                  # routed experts: softmax over all, top-2, renormalised
            probs = torch.softmax(y @ sd[p + "mlp.gate.weight"].t(), -1)
            tw, ti = torch.topk(probs, 2)
            tw = tw / tw.sum(-1, keepdim=True)
            mix = torch.zeros_like(y)
            for t in range(T):
                for j in range(2):
                    e = int(ti[t, j])
                    u = y[t] @ sd[p + "mlp.experts.gate_up_proj"][e].t()
                    half = u.shape[0] // 2
                    mix[t] += (torch.nn.functional.silu(u[:half]) * u[half:]) @ sd[p + "mlp.experts.down_proj"][e].t() * tw[t, j]
            y = mix
        else:
            y = (torch.nn.functional.silu(y @ sd[p + "mlp.gate_proj.weight"].t()) * (y @ sd[p + "mlp.up_proj.weight"].t())) @ sd[p + "mlp.down_proj.weight"].t()
        h = h + wrms(y, 1e-5) * (1 + sd[p + "post_feedforward_layernorm.weight"])
    h = wrms(h, 1e-6) * sd[root + "norm.weight"]                          # the final norm stores its scale as is
    logits = h @ sd["lm_head.weight"].t()
    return torch.tanh(logits * (0.6 / 20.0)) * 20.0


def save(tmp_path, sd, text=TEXT):
    from safetensors.torch import save_file

    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "muse_glimmer", "architectures": ["MuseGlimmerForConditionalGeneration"],
                                                      "text_config": text, "eos_token_id": 3}))


def test_matches_the_dense_restatement_and_the_engine_invariants(tmp_path):
    from eredu_b200.runtime.plan import inspect_artifact

    sd = state()
    save(tmp_path, sd)
    report = inspect_artifact(tmp_path)
    assert report.is_loadable, [(i.code, i.message) for i in report.issues]
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=2, max_seq_len=64))
    tokens = torch.randint(0, 200, (21,), generator=torch.Generator().manual_seed(1)).tolist()      # 21 > window
    want = dense_reference(sd, tokens)
    got = lm.prefill_logits(tokens)
    assert float((got - want[-1]).abs().max()) < 2e-4
    # chunked prefill then decode-shaped steps through the paged cache
    seq = lm.engine.new_sequence(tokens[:9], max_new_tokens=16)
    first = lm.engine.prefill_logits([seq])
    assert float((first[0].float() - want[8]).abs().max()) < 2e-4
    for j, t in enumerate(tokens[9:]):
        row = lm.engine.step_logits(seq, t)
        assert float((row.float() - want[9 + j]).abs().max()) < 2e-4, j
    lm.engine.release(seq)
    # two sequences in one batch generate what they generate alone
    sp = SamplingParams(temperature=0.0)
    prompts = [tokens[:7], tokens[3:15]]
    both = lm.generate(prompts, sp, 6)
    assert both == [lm.generate([p], sp, 6)[0] for p in prompts]
    assert both[0][0] == int(want[6].argmax())                   # the first prompt is a prefix of the reference sequence


def test_routed_expert_variant_against_a_restatement(tmp_path):
    sd = state()
    g = torch.Generator().manual_seed(9)
    E, I, H = 6, 32, 64
    root = "model.language_model."
    for li in range(4):
        p = f"{root}layers.{li}.mlp."
        for n in ("gate_proj", "up_proj", "down_proj"):
            del sd[p + n + ".weight"]
        sd[p + "gate.weight"] = torch.randn(E, H, generator=g) * 0.5
        sd[p + "experts.gate_up_proj"] = torch.randn(E, 2 * I, H, generator=g) * 0.2
        sd[p + "experts.down_proj"] = torch.randn(E, H, I, generator=g) * 0.2
    text = dict(TEXT, num_experts=E, num_experts_per_tok=2, moe_intermediate_size=I, norm_topk_prob=True, num_hidden_layers=4)
    save(tmp_path, sd, text)
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=48))
    tokens = list(range(5, 30))
    want = dense_reference(sd, tokens)
    full = lm.prefill_logits(tokens)
    assert float((full - want[-1]).abs().max()) < 2e-4
    seq = lm.engine.new_sequence(tokens[:11], max_new_tokens=20)
    lm.engine.prefill_logits([seq])
    row = None
    for t in tokens[11:]:
        row = lm.engine.step_logits(seq, t)
    lm.engine.release(seq)
    assert float((row.float() - want[-1]).abs().max()) < 2e-4


def test_variants_that_are_not_built_say_so(tmp_path):
    sd = state()
    bad = {k: v for k, v in TEXT.items() if k != "qk_scale_factor"}
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "muse_glimmer", "text_config": bad}))
    from eredu_b200.runtime.plan import inspect_artifact

    report = inspect_artifact(tmp_path)
    assert not report.is_loadable and report.issues[0].code == "invalid_config"
