"""CPU fp32 slice: engine (paged cache, chunked prefill, decode loop, sampler) vs the dense full-recompute oracle."""
import dataclasses

import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.engine import Engine

from reference_model import forward_logits, greedy


def build(cfg, sd):
    return build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32)


def test_tiny_llama_greedy_matches_full_recompute():
    cfg = C.tiny_llama()
    sd = random_state(cfg, seed=0)
    model = build(cfg, sd)
    eng = Engine(model, max_batch=2, max_seq_len=128)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (32,), generator=g).tolist()
    out = eng.generate([prompt], SamplingParams(temperature=0.0), max_new_tokens=24)[0]
    assert out == greedy(cfg, sd, prompt, 24)


@pytest.mark.parametrize("variant", ["qwen3", "qwen2_bias", "interleaved_rope", "window", "partial_rotary", "llama3_rope"])
def test_family_variants(variant):
    cfg = C.tiny_llama()
    cfg = dataclasses.replace(cfg, num_hidden_layers=2, vocab_size=512)
    if variant == "qwen3":
        cfg = dataclasses.replace(cfg, model_type="qwen3", qk_norm=True, rms_norm_eps=1e-6, tie_word_embeddings=False)
    elif variant == "qwen2_bias":
        cfg = dataclasses.replace(cfg, model_type="qwen2", attention_bias=True)
    elif variant == "interleaved_rope":
        cfg = dataclasses.replace(cfg, rope_traditional=True)
    elif variant == "window":
        cfg = dataclasses.replace(cfg, model_type="mistral", sliding_window=8)
    elif variant == "partial_rotary":
        cfg = dataclasses.replace(cfg, partial_rotary_factor=0.5)
    elif variant == "llama3_rope":
        cfg = dataclasses.replace(cfg, rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                      "high_freq_factor": 4.0,
                                                      "original_max_position_embeddings": 64})
    sd = random_state(cfg, seed=1, std=0.08)
    if variant == "qwen3":
        for k in list(sd):
            if "q_norm" in k or "k_norm" in k:
                sd[k] = torch.rand_like(sd[k]) + 0.5
    model = build(cfg, sd)
    eng = Engine(model, max_batch=4, max_seq_len=96)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 17, 33)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=12)
    for p, o in zip(prompts, outs):
        assert o == greedy(cfg, sd, p, 12)


def test_prefill_logits_and_chunking():
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=300)
    sd = random_state(cfg, seed=2, std=0.05)
    model = build(cfg, sd)
    eng = Engine(model, max_batch=4, max_seq_len=64, prefill_chunk=20)  # forces several prefill groups
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 16, 31, 2)]
    seqs = [eng.new_sequence(p, max_new_tokens=4) for p in prompts]
    first = eng.prefill(seqs).tolist()
    for p, t in zip(prompts, first):
        assert t == int(torch.argmax(forward_logits(cfg, sd, p)[-1]))


def test_stochastic_sampling_is_position_addressed():
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=400)
    sd = random_state(cfg, seed=3, std=0.05)
    model = build(cfg, sd)
    sp = SamplingParams(temperature=0.9, top_k=20, top_p=0.9, min_p=0.0, seed=42)
    prompt = list(range(10))
    a = Engine(model, max_batch=1, max_seq_len=64).generate([prompt], sp, max_new_tokens=10)[0]
    b = Engine(model, max_batch=3, max_seq_len=64).generate([prompt, prompt[:5]], sp, max_new_tokens=10)[0]
    assert a == b  # batching does not change committed randomness
    c = Engine(model, max_batch=1, max_seq_len=64).generate([prompt], dataclasses.replace(sp, seed=43),
                                                            max_new_tokens=10)[0]
    assert a != c


def test_phi3_fused_projection_checkpoints():
    """Phi-3 stores q|k|v and gate|up as single matrices: same tokens as the split layout."""
    import dataclasses

    import torch

    from eredu_b200.models import config as C
    from eredu_b200.models.llama import build_from_tensors, random_state
    from eredu_b200.ops import SamplingParams
    from eredu_b200.runtime.engine import Engine

    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=512, model_type="phi3", tie_word_embeddings=False)
    sd = random_state(cfg, seed=0, std=0.05)
    fused = {}
    for k, v in sd.items():
        if ".self_attn.q_proj.weight" in k:
            base = k[: -len("q_proj.weight")]
            fused[base + "qkv_proj.weight"] = torch.cat((sd[base + "q_proj.weight"], sd[base + "k_proj.weight"], sd[base + "v_proj.weight"]), 0)
        elif ".mlp.gate_proj.weight" in k:
            base = k[: -len("gate_proj.weight")]
            fused[base + "gate_up_proj.weight"] = torch.cat((sd[base + "gate_proj.weight"], sd[base + "up_proj.weight"]), 0)
        elif any(t in k for t in (".k_proj.", ".v_proj.", ".up_proj.")):
            continue
        else:
            fused[k] = v
    prompt = list(range(5, 25))
    sp = SamplingParams(temperature=0.0)
    a = Engine(build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32), 1, 64).generate([prompt], sp, 6)
    b = Engine(build_from_tensors(cfg, fused.__getitem__, fused.__contains__, "cpu", torch.float32), 1, 64).generate([prompt], sp, 6)
    assert a == b


def test_vision_language_checkpoint_as_text_model(tmp_path):
    """Qwen3-VL style directory: nested text_config, decoder under model.language_model.*, a vision tower next to it."""
    import json

    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats import checkpoint as ck

    cfg = dataclasses.replace(C.tiny_llama(), model_type="qwen3", qk_norm=True, vocab_size=300, num_hidden_layers=2,
                              tie_word_embeddings=False, rms_norm_eps=1e-6)
    sd = random_state(cfg, seed=3, std=0.05)
    stored = {("model.language_model." + k[len("model."):] if k.startswith("model.") else k): v for k, v in sd.items()}
    stored["model.visual.patch_embed.proj.weight"] = torch.zeros(8, 3, 2, 2, 2)
    ck.save_safetensors_checkpoint(tmp_path, cfg, stored, torch.float32)
    text = json.loads((tmp_path / "config.json").read_text())
    text["model_type"] = "qwen3_vl_text"
    text["rope_scaling"] = {"rope_type": "default", "mrope_section": [2, 1, 1], "mrope_interleaved": True}
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "qwen3_vl", "text_config": text,
                                                      "vision_config": {"depth": 2}, "tie_word_embeddings": False}))
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    assert lm.config.model_type == "qwen3" and lm.config.qk_norm
    prompt = list(range(5, 22))
    assert torch.allclose(lm.prefill_logits(prompt), forward_logits(cfg, sd, prompt)[-1], atol=2e-4)
    from eredu_b200 import media as MM
    import numpy as np

    req = MM.MultimodalRequest().text("what is this").image(MM.RgbImage(np.zeros((4, 4, 3), np.uint8)))
    with pytest.raises(MM.MultimodalPreparationError):
        MM.prepare_for_text_model(req, lm.encode)
