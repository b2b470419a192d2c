"""Continuous-batching server on CPU: scheduler-planned chunked prefill + slot-based decode reproduce the static
engine's tokens; late arrivals, cancellation, deadlines, request-local failures and consensus across gloo ranks."""
import dataclasses

import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.engine import Engine
from eredu_b200.runtime.server import ConsensusError, Server

from dist_util import run_ranks


def make_engine(max_batch=4):
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=512)
    sd = random_state(cfg, seed=0, std=0.05)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32)
    return Engine(model, max_batch=max_batch, max_seq_len=192)


def prompts(n, seed=3):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 512, (int(k),), generator=g).tolist() for k in torch.randint(5, 60, (n,), generator=g)]


def test_server_matches_static_engine_with_late_arrivals_and_chunked_prefill():
    ps = prompts(7)
    budgets = [6, 9, 4, 12, 7, 5, 8]
    sp = SamplingParams(temperature=0.0)
    ref_eng = make_engine()
    want = [ref_eng.generate([p], sp, n)[0] for p, n in zip(ps, budgets)]
    eng = make_engine(max_batch=3)   # fewer slots than requests: requests wait, join and leave
    srv = Server(eng, prefill_chunk=16, max_step_tokens=40)
    ids = [srv.submit(p, sp, n) for p, n in zip(ps[:4], budgets[:4])]
    for _ in range(5):
        srv.step()
    ids += [srv.submit(p, sp, n) for p, n in zip(ps[4:], budgets[4:])]   # arrive while others decode
    srv.run_until_idle(max_steps=500)
    for rid, w in zip(ids, want):
        r = srv.result(rid)
        assert r.tokens == w and r.finish_reason == "max_tokens"
    assert eng.kv.allocator.free_pages() == eng.kv.num_pages - 1   # every page came back
    assert srv.sched.report()["running"] == 0


def test_cancel_deadline_failure_and_streaming_stop():
    eng = make_engine()
    sp = SamplingParams(temperature=0.0)
    seen = []

    def stop_after_three(rid, tok):
        seen.append(tok)
        return "stop_sequence" if len(seen) == 3 else None

    fail_once = {"armed": True}

    def hook(kind, rid):
        if kind == "decode" and rid == ids[2] and fail_once["armed"]:
            fail_once["armed"] = False
            return True
        return False

    srv = Server(eng, prefill_chunk=32, fault_hook=hook)
    ps = prompts(4, seed=9)
    ids = [srv.submit(ps[0], sp, 50), srv.submit(ps[1], sp, 50, on_token=stop_after_three), srv.submit(ps[2], sp, 50),
           srv.submit(ps[3], sp, 9)]
    srv.step(now=0.0)
    srv.cancel(ids[0])      # work is in flight or not: either way the request ends as cancelled, never pre-empted
    srv.run_until_idle(max_steps=300)
    assert srv.result(ids[0]).finish_reason == "cancelled"
    assert srv.result(ids[1]).finish_reason == "stop_sequence" and len(srv.result(ids[1]).tokens) == 3
    assert srv.result(ids[2]).failed
    assert srv.result(ids[3]).finish_reason == "max_tokens" and len(srv.result(ids[3]).tokens) == 9
    assert eng.kv.allocator.free_pages() == eng.kv.num_pages - 1
    # a positive deadline in the past cancels at planning time
    rid = srv.submit(ps[3], sp, 5, deadline=1.0)
    srv.step(now=2.0)
    assert srv.result(rid).finish_reason == "deadline"


@pytest.mark.parametrize("world", [2])
def test_consensus_across_ranks(world, tmp_path):
    res = run_ranks("cpu_server", world, tmp_path)
    assert all(r["tokens"] == res[0]["tokens"] for r in res)
    # the request cancelled on the last rank ended as cancelled on every rank after the same number of tokens
    assert all(r["cancelled"] == res[0]["cancelled"] for r in res)
    assert res[0]["cancelled"][0] == "cancelled" and res[0]["cancelled"][1] < 40 and len(res[0]["cancelled"][2]) == 8
    assert all(r["diverged"] == "ConsensusError" for r in res)
    assert all(r["poisoned"] for r in res)
