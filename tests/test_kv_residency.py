"""KV host tier: park / resume keeps a sequence's continuation bit-identical; the server parks running requests
when the page pool runs out and brings them back."""
import dataclasses

import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.engine import Engine
from eredu_b200.runtime.kv_residency import KVHostTier, PagedCacheOptions
from eredu_b200.runtime.server import Server


def make_engine(device="cpu", dtype=torch.float32, max_batch=4, num_pages=None, big=False):
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=512)
    if big:
        cfg = dataclasses.replace(cfg, hidden_size=1024, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                                  intermediate_size=2048, vocab_size=4096, num_hidden_layers=3, tie_word_embeddings=False)
    sd = random_state(cfg, seed=0, std=0.05)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, device, dtype)
    return Engine(model, max_batch=max_batch, max_seq_len=128, num_pages=num_pages), cfg


def _park_resume(device, dtype, big):
    eng, cfg = make_engine(device, dtype, big=big)
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, cfg.vocab_size, (37,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0)
    want = eng.generate([prompt], sp, 10)[0]
    tier = KVHostTier(eng)
    seq = eng.new_sequence(prompt, sp, max_new_tokens=16)
    first = eng.prefill([seq])
    out = [int(first[0])]
    free_before = eng.kv.allocator.free_pages()
    assert tier.park(seq) and seq.pages == [] and eng.kv.allocator.free_pages() > free_before
    other = eng.new_sequence(prompt[::-1], sp, max_new_tokens=8)     # reuses (and overwrites) the freed pages
    eng.prefill([other])
    eng.release(other)
    assert tier.resume(seq) and len(seq.pages) > 0 and tier.report()["parked_now"] == 0
    seq.output.append(out[0])
    eng.start_decode([seq], first)
    for _ in range(9):
        toks = eng.decode_step()
        eng.commit(toks.tolist())
        out.append(int(toks[0]))
    eng._decode_state = None
    eng.release(seq)
    assert out == want
    assert tier.stats["bytes_to_host"] == tier.stats["bytes_to_device"] > 0


def test_park_resume_cpu():
    _park_resume("cpu", torch.float32, False)


@pytest.mark.gpu
def test_park_resume_gpu():
    _park_resume("cuda:0", torch.bfloat16, True)


def test_host_budget_and_victims():
    eng, cfg = make_engine()
    tier = KVHostTier(eng, PagedCacheOptions(host_budget_bytes=1, eviction="largest"))
    a = eng.new_sequence(list(range(20)), max_new_tokens=4)
    b = eng.new_sequence(list(range(50)), max_new_tokens=4)
    eng.prefill([a, b])
    assert tier.victim([a, b]) is b
    assert not tier.park(b) and b.pages and tier.report()["refused"] == 1      # over the host budget: nothing moves
    lru = KVHostTier(eng)
    lru.touch(b)
    lru.touch(a)
    assert lru.victim([a, b]) is b
    with pytest.raises(ValueError):
        KVHostTier(eng, PagedCacheOptions(block_size_tokens=32))


def test_server_parks_under_pressure_and_finishes_everything():
    sp = SamplingParams(temperature=0.0)
    ref, cfg = make_engine(max_batch=4)
    g = torch.Generator().manual_seed(8)
    ps = [torch.randint(0, cfg.vocab_size, (30,), generator=g).tolist() for _ in range(4)]
    want = [ref.generate([p], sp, 20)[0] for p in ps]
    # pool: room for two requests of (30 + 20) tokens = 4 pages each, plus the reserved page 0
    eng, _ = make_engine(max_batch=4, num_pages=2 * 4 + 1)
    tier = KVHostTier(eng)
    srv = Server(eng, prefill_chunk=64, kv_tier=tier)
    ids = [srv.submit(p, sp, 20) for p in ps[:2]]
    for _ in range(6):
        srv.step()
    ids += [srv.submit(p, sp, 20) for p in ps[2:]]        # no pages left: running requests are parked
    assert tier.report()["parked"] >= 1
    srv.run_until_idle(max_steps=2000)
    assert [srv.result(i).tokens for i in ids] == want
    assert tier.report()["parked_now"] == 0 and tier.report()["resumed"] == tier.report()["parked"]
    assert eng.kv.allocator.free_pages() == eng.kv.num_pages - 1


def test_disk_tier_behind_the_host_tier(tmp_path):
    """With a disk directory the host budget no longer refuses a park: the longest-parked sequence moves to a file and
    comes back bit-identically."""
    import os

    eng, cfg = make_engine()
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (33, 40, 21)]
    sp = SamplingParams(temperature=0.0)
    want = [eng.generate([p], sp, 6)[0] for p in prompts]
    probe = KVHostTier(eng)
    one = 3 * probe.page_bytes()                                   # 33..40 tokens = 3 pages each, 21 tokens = 2
    tier = KVHostTier(eng, PagedCacheOptions(host_budget_bytes=one, live_disk=str(tmp_path / "kv")))
    seqs, firsts = [], []
    for p in prompts:
        s = eng.new_sequence(p, sp, max_new_tokens=8)
        firsts.append(eng.prefill([s]))
        seqs.append(s)
    assert tier.park(seqs[0]) and tier.report()["on_disk_now"] == 0
    assert tier.park(seqs[1])                                      # the budget holds one: sequence 0 goes to disk
    r = tier.report()
    assert r["on_disk_now"] == 1 and r["spilled"] == 1 and r["host_bytes"] <= one and r["disk_bytes"] == one
    assert len(os.listdir(tmp_path / "kv")) == 1
    assert tier.park(seqs[2]) and tier.report()["on_disk_now"] == 2
    for i in (0, 2, 1):                                            # resume in another order; 0 comes back from its file
        assert tier.resume(seqs[i])
        out = [int(firsts[i][0])]
        seqs[i].output.append(out[0])
        eng.start_decode([seqs[i]], firsts[i])
        for _ in range(5):
            toks = eng.decode_step()
            eng.commit(toks.tolist())
            out.append(int(toks[0]))
        eng._decode_state = None
        eng.release(seqs[i])
        assert out == want[i]
    r = tier.report()
    assert r["parked_now"] == 0 and r["host_bytes"] == 0 and r["disk_bytes"] == 0 and os.listdir(tmp_path / "kv") == []
    assert r["bytes_from_disk"] == r["bytes_to_disk"] > 0
    # a disk budget that is too small refuses like a missing tier does; dropping a spilled sequence removes its file
    small = KVHostTier(eng, PagedCacheOptions(host_budget_bytes=one, live_disk=str(tmp_path / "kv2"), disk_budget_bytes=1))
    a = eng.new_sequence(prompts[0], sp, max_new_tokens=4)
    b = eng.new_sequence(prompts[1], sp, max_new_tokens=4)
    eng.prefill([a, b])
    assert small.park(a) and not small.park(b) and small.report()["refused"] == 1 and b.pages
    roomy = KVHostTier(eng, PagedCacheOptions(host_budget_bytes=one, live_disk=str(tmp_path / "kv3")))
    c = eng.new_sequence(prompts[2], sp, max_new_tokens=4)
    eng.prefill([c])
    assert roomy.park(b) and roomy.park(c) and len(os.listdir(tmp_path / "kv3")) == 1
    roomy.drop(b)
    assert os.listdir(tmp_path / "kv3") == [] and roomy.report()["disk_bytes"] == 0
