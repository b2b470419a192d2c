"""Speculative decoding: greedy speculative output equals plain greedy output for any draft; a draft identical to the
target is always accepted; bookkeeping (bonus token, KV truncation, draft catch-up) survives many rounds."""
import dataclasses

import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.engine import Engine
from eredu_b200.runtime.speculative import SpeculativeDecoder


def _models(device, dtype, draft_seed):
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=512, hidden_size=256 if device == "cpu" else 512,
                              num_attention_heads=4 if device == "cpu" else 8, head_dim=64)
    sd = random_state(cfg, seed=0, std=0.08)
    target = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, device, dtype)
    dcfg = dataclasses.replace(cfg, num_hidden_layers=1)
    dsd = sd if draft_seed is None else random_state(dcfg, seed=draft_seed, std=0.08)
    draft = build_from_tensors(cfg if draft_seed is None else dcfg, dsd.__getitem__, dsd.__contains__, device, dtype)
    return cfg, target, draft


def _run(device, dtype, draft_seed, sp, k=4, n_new=30):
    cfg, target, draft = _models(device, dtype, draft_seed)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (11, 25)]
    plain = Engine(target, max_batch=2, max_seq_len=128).generate(prompts, sp, n_new)
    dec = SpeculativeDecoder(Engine(target, max_batch=2, max_seq_len=128, use_cuda_graph=False),
                             Engine(draft, max_batch=2, max_seq_len=128, use_cuda_graph=False), k=k)
    spec = dec.generate(prompts, sp, n_new)
    return plain, spec, dec.stats.summary()


@pytest.mark.parametrize("draft_seed", [None, 7])
def test_greedy_speculation_is_exact_cpu(draft_seed):
    plain, spec, stats = _run("cpu", torch.float32, draft_seed, SamplingParams(temperature=0.0))
    assert spec == plain
    if draft_seed is None:
        assert stats["acceptance_rate"] == 1.0 and stats["tokens_per_step"] == 5.0
    else:
        assert stats["acceptance_rate"] < 0.5


def test_stochastic_identical_draft_is_always_accepted_cpu():
    sp = SamplingParams(temperature=0.8, top_k=40, top_p=0.95, min_p=0.0, seed=11)
    plain, spec, stats = _run("cpu", torch.float32, None, sp, k=3, n_new=16)
    assert stats["acceptance_rate"] == 1.0
    # position-addressed randomness: accepted drafts and bonus tokens are the tokens plain sampling draws
    assert spec == plain


@pytest.mark.gpu
@pytest.mark.parametrize("draft_seed", [None, 7])
def test_greedy_speculation_is_exact_gpu(draft_seed):
    plain, spec, stats = _run("cuda", torch.bfloat16, draft_seed, SamplingParams(temperature=0.0), k=4, n_new=24)
    if draft_seed is None:
        assert stats["acceptance_rate"] == 1.0
    # bf16: the (k+1)-token verify pass and the 1-token decode pass round differently, so compare a prefix
    agree = sum(1 for a, b in zip(plain[0], spec[0]) if a == b)
    assert agree >= len(plain[0]) * 0.5 and len(spec[0]) == len(plain[0])


@pytest.mark.gpu
def test_stochastic_speculation_runs_gpu():
    sp = SamplingParams(temperature=0.8, top_k=40, top_p=0.95, min_p=0.0, seed=5)
    plain, spec, stats = _run("cuda", torch.bfloat16, 7, sp, k=4, n_new=24)
    assert all(len(o) == 24 for o in spec) and stats["rounds"] > 0


@pytest.mark.gpu
@pytest.mark.parametrize("draft_seed", [None, 7])
@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_graph_captured_round_matches_the_eager_decoder(draft_seed, temperature):
    """One CUDA graph per round (uniform two-token draft catch-up) emits exactly what the eager, ragged decoder emits:
    same kernels, same position-addressed uniforms, only the scheduling differs."""
    from eredu_b200.runtime.speculative import GraphSpeculativeDecoder

    sp = SamplingParams(temperature=temperature, top_k=40, top_p=0.95, min_p=0.0, seed=5)
    cfg, target, draft = _models("cuda", torch.bfloat16, draft_seed)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (11, 25)]
    eager = SpeculativeDecoder(Engine(target, max_batch=2, max_seq_len=128, use_cuda_graph=False),
                               Engine(draft, max_batch=2, max_seq_len=128, use_cuda_graph=False), k=4)
    want = eager.generate(prompts, sp, 24)
    graphed = GraphSpeculativeDecoder(Engine(target, max_batch=2, max_seq_len=128), Engine(draft, max_batch=2, max_seq_len=128), k=4)
    got = graphed.generate(prompts, sp, 24)
    assert [len(o) for o in got] == [24, 24]
    agree = sum(a == b for x, y in zip(want, got) for a, b in zip(x, y))
    # the draft's first step runs as a 2-query pass instead of a ragged prefill pass: bf16 rounding may flip a token,
    # after which a sampled (temperature > 0) continuation is a different, equally valid draw
    assert agree >= (24 if temperature == 0.0 else 4)
    s = graphed.stats.summary()
    assert s["rounds"] > 0 and s["emitted"] >= 48 - 2 * 5
    if draft_seed is None and temperature == 0.0:
        assert s["acceptance_rate"] > 0.6


def _hybrid(family, seed):
    from eredu_b200.models.moe import make_moe_factory

    if family == "lfm2":
        from test_lfm2 import lfm2_cfg

        cfg = lfm2_cfg()
        sd = random_state(cfg, seed=seed, std=0.08)
    elif family == "qwen3_next":
        from test_qwen_next import next_cfg, state_for

        cfg = next_cfg()
        sd = state_for(cfg, seed=seed) if "seed" in state_for.__code__.co_varnames else state_for(cfg)
    else:
        from test_nemotron_h import nh_cfg, state_for

        cfg = nh_cfg()
        sd = state_for(cfg, seed=seed)
    return cfg, build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())


@pytest.mark.parametrize("family", ["lfm2", "qwen3_next", "nemotron_h"])
@pytest.mark.parametrize("same_draft", [True, False])
def test_hybrid_models_roll_their_recurrent_state_back(family, same_draft):
    """Convolution histories and recurrent matrices leave the rejected proposals behind: greedy speculative output is
    the plain greedy output, with a draft that is always accepted and with one that almost never is."""
    cfg, target = _hybrid(family, 0)
    _, draft = (cfg, target) if same_draft else _hybrid(family, 5)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 21)]
    sp = SamplingParams(temperature=0.0)
    plain = Engine(target, max_batch=2, max_seq_len=96).generate(prompts, sp, 20)
    dec = SpeculativeDecoder(Engine(target, max_batch=2, max_seq_len=96, use_cuda_graph=False),
                             Engine(draft, max_batch=2, max_seq_len=96, use_cuda_graph=False), k=3)
    assert dec.t_hybrid and dec.d_hybrid
    assert dec.generate(prompts, sp, 20) == plain
    st = dec.stats.summary()
    assert st["acceptance_rate"] == 1.0 if same_draft else st["acceptance_rate"] < 0.6


def test_state_snapshot_round_trip():
    cfg, model = _hybrid("qwen3_next", 0)
    eng = Engine(model, max_batch=1, max_seq_len=64)
    seq = eng.new_sequence([5, 6, 7, 8, 9], max_new_tokens=8)
    eng.feed_logits(seq, [5, 6, 7, 8, 9])
    snap = eng.snapshot_state(seq)
    a = eng.step_logits(seq, 11)
    eng.restore_state(seq, snap)
    seq.kv_len -= 1
    assert torch.equal(eng.step_logits(seq, 11), a)
    eng.release(seq)
    dense = Engine(_models("cpu", torch.float32, None)[1], max_batch=1, max_seq_len=64)
    s2 = dense.new_sequence([1, 2, 3], max_new_tokens=4)
    assert dense.snapshot_state(s2) is None and not dense.kv.has_recurrent_state()
