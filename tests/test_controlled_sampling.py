"""Mirostat v2 state machine and grammar-constrained generation (llguidance masks) on CPU."""
import dataclasses
import json
import math

import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.ops import SamplingParams
from eredu_b200.ops.controlled import GrammarConstraint, MirostatV2, constrained_generate
from eredu_b200.runtime.engine import Engine
from test_text_streaming import make_bundle


def test_mirostat_truncation_update_and_fallback():
    m = MirostatV2(tau=3.0, eta=0.5, temperature=1.0, seed=1)
    assert m.mu == 6.0
    logits = torch.log(torch.tensor([0.5, 0.25, 0.125, 0.0625, 0.0625]))
    m.mu = 2.5   # surprises are 1, 2, 3, 4, 4 bits: the first two survive
    q = m.distribution(logits)
    assert torch.allclose(q, torch.tensor([2 / 3, 1 / 3, 0.0, 0.0, 0.0]), atol=1e-6)
    tok = m.sample(logits, position=5)
    assert tok in (0, 1)
    want = 2.5 - 0.5 * (-math.log2(float(q[tok])) - 3.0)   # probability AFTER truncation and renormalisation
    assert abs(m.mu - want) < 1e-6 and m.history == [tok]
    m.mu = 0.5   # below every surprise: only the argmax is kept
    q = m.distribution(logits)
    assert q.tolist() == [1.0, 0.0, 0.0, 0.0, 0.0]
    m.reset()
    assert m.mu == 6.0 and m.history == []
    with pytest.raises(ValueError):
        MirostatV2(tau=0.0)
    with pytest.raises(ValueError):
        m.accept(0, 0.0)
    # same seed / position -> same token; mu converges toward tau on a flat distribution
    a, b = MirostatV2(seed=7), MirostatV2(seed=7)
    flat = torch.zeros(64)
    assert [a.sample(flat, i) for i in range(20)] == [b.sample(flat, i) for i in range(20)]


def test_grammar_constraint_masks_rollback_and_generation(tmp_path):
    b = make_bundle(tmp_path)
    c = GrammarConstraint(b, "regex", r"(yes|no)!")
    mask = c.allow_mask(b.vocab_size())
    allowed = {b.decode([i], skip_special_tokens=False) for i in torch.nonzero(mask).flatten().tolist()}
    assert allowed and all(("yes".startswith(t) or "no".startswith(t) or t.startswith("yes") or t.startswith("no"))
                           for t in allowed if t)
    ids = b.encode("yes", add_special_tokens=False)
    fork = c.fork()
    for t in ids:
        c.commit(t)
    assert not c.is_complete()
    c.rollback(len(ids))                       # rejected speculation: back to the start
    assert torch.equal(c.allow_mask(b.vocab_size()), mask)
    with pytest.raises(ValueError):
        fork.commit(b.encode("maybe", add_special_tokens=False)[0])

    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=b.vocab_size(), eos_token_id=b.eos_ids[0])
    sd = random_state(cfg, seed=0, std=0.05)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32)
    eng = Engine(model, max_batch=1, max_seq_len=128)
    prompt = b.encode("answer:")
    out, reason = constrained_generate(eng, prompt, GrammarConstraint(b, "regex", r"(yes|no)!"),
                                       SamplingParams(temperature=0.0), max_new_tokens=16, eos_ids=b.eos_ids)
    assert b.decode(out) in ("yes!", "no!") and reason in ("grammar_complete", "eos")
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}}, "required": ["ok"], "additionalProperties": False}
    out, reason = constrained_generate(eng, prompt, GrammarConstraint(b, "json_schema", schema),
                                       SamplingParams(temperature=0.7, seed=3), max_new_tokens=48, eos_ids=b.eos_ids,
                                       mirostat=MirostatV2(temperature=0.7, seed=3))
    text = b.decode(out)
    if reason != "max_tokens":
        assert json.loads(text)["ok"] in (True, False)
    assert eng.kv.allocator.free_pages() == eng.kv.num_pages - 1


@pytest.mark.parametrize("same_draft", [True, False])
@pytest.mark.parametrize("spec", [("regex", r"(ab|ba){2,6}!"), ("json_schema", {"type": "object", "properties": {"ok": {"type": "boolean"}},
                                                                                   "required": ["ok"], "additionalProperties": False})])
def test_speculation_under_a_grammar_commits_what_plain_constrained_decoding_commits(tmp_path, same_draft, spec):
    """Proposals run the grammar ahead, the state is rolled back, target rows are masked along the proposed path: greedy
    output equals step-by-step constrained decoding whatever the draft proposes."""
    from eredu_b200.runtime.speculative import SpeculativeDecoder

    b = make_bundle(tmp_path)
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=b.vocab_size(), eos_token_id=b.eos_ids[0])
    sd = random_state(cfg, seed=0, std=0.05)
    target = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32)
    dcfg = dataclasses.replace(cfg, num_hidden_layers=1)
    dsd = random_state(dcfg, seed=9, std=0.05)
    draft = target if same_draft else build_from_tensors(dcfg, dsd.__getitem__, dsd.__contains__, "cpu", torch.float32)
    prompt = b.encode("answer:")
    sp = SamplingParams(temperature=0.0)
    want, want_reason = constrained_generate(Engine(target, max_batch=1, max_seq_len=128), prompt, GrammarConstraint(b, *spec), sp,
                                             max_new_tokens=24, eos_ids=b.eos_ids)
    dec = SpeculativeDecoder(Engine(target, max_batch=1, max_seq_len=128, use_cuda_graph=False),
                             Engine(draft, max_batch=1, max_seq_len=128, use_cuda_graph=False), k=3)
    seen = []
    got, reason = dec.generate_constrained(prompt, GrammarConstraint(b, *spec), sp, max_new_tokens=24, eos_ids=b.eos_ids,
                                           on_token=lambda t: seen.append(t))
    assert got == want and reason == want_reason and seen == got
    st = dec.stats.summary()
    if same_draft and st["proposed"]:
        assert st["acceptance_rate"] == 1.0
    assert dec.t.kv.allocator.free_pages() == dec.t.kv.num_pages - 1 and dec.d.kv.allocator.free_pages() == dec.d.kv.num_pages - 1
    # sampling keeps working (distribution-preserving, not draw-preserving): the grammar still holds
    got2, reason2 = dec.generate_constrained(prompt, GrammarConstraint(b, *spec), SamplingParams(temperature=0.9, seed=2),
                                             max_new_tokens=24, eos_ids=b.eos_ids)
    check = GrammarConstraint(b, *spec)
    for t in got2:
        check.commit(t)                                            # raises on a token the grammar does not allow
    assert reason2 in ("grammar_complete", "eos", "max_tokens")
