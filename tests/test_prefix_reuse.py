"""Prefix reuse over published KV pages: a request leases the longest sealed prefix of its prompt, prefills the rest, and
commits exactly the tokens of a cold run; pages are shared by reference count and evicted only when unreferenced."""
import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.engine import Engine
from eredu_b200.runtime.kv_cache import PAGE


def model(device="cpu", dtype=torch.float32):
    cfg = C.tiny_llama()
    sd = random_state(cfg, seed=0, std=0.08)
    return cfg, build_from_tensors(cfg, sd.__getitem__, sd.__contains__, device, dtype)


def prompts(cfg):
    g = torch.Generator().manual_seed(5)
    system = torch.randint(0, cfg.vocab_size, (50,), generator=g).tolist()
    return system, [system + torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (7, 20, 1)]


def test_hits_commit_the_tokens_of_a_cold_run():
    cfg, m = model()
    system, ps = prompts(cfg)
    sp = SamplingParams(temperature=0.0)
    cold = Engine(m, max_batch=2, max_seq_len=160)
    want = [cold.generate([p], sp, 12)[0] for p in ps]
    eng = Engine(m, max_batch=2, max_seq_len=160, prefix_cache=True)
    if not eng.prefix_cache:
        pytest.skip("host runtime module not built")
    total = eng.kv.allocator.free_pages()
    got = [eng.generate([p], sp, 12)[0] for p in ps]
    assert got == want
    st = eng.prefix_stats
    # the first request publishes the three full pages of the shared 50-token prefix, the later ones lease them
    assert st["lookups"] == 3 and st["hits"] == 2 and st["hit_tokens"] == 2 * 3 * PAGE
    assert eng.kv.allocator.free_pages() == total and eng.kv.allocator.cached_pages() > 0
    # a second turn extends a finished conversation: prompt + reply of the first request are reused page by page
    turn2 = ps[0] + want[0] + [3, 1, 4, 1, 5]
    before = st["hit_tokens"]
    assert eng.generate([turn2], sp, 8)[0] == cold.generate([turn2], sp, 8)[0]
    assert st["hit_tokens"] - before == (len(ps[0]) + 11) // PAGE * PAGE      # the reply's last token was never fed
    # identical prompts in one batch: the second is admitted after the first one's prefill published its pages
    a = eng.new_sequence(ps[1], sp, 4)
    eng.prefill([a])
    b = eng.new_sequence(ps[1], sp, 4)
    assert b.cached_tokens == (len(ps[1]) - 1) // PAGE * PAGE and b.pages[:3] == a.pages[:3]
    assert eng.kv.allocator.refcount(a.pages[0]) == 2
    eng.release(a)
    assert eng.kv.allocator.refcount(b.pages[0]) == 1
    eng.release(b)
    assert eng.kv.allocator.free_pages() == total


def test_a_prompt_of_whole_pages_still_prefills_its_last_token():
    cfg, m = model()
    g = torch.Generator().manual_seed(1)
    p = torch.randint(0, cfg.vocab_size, (2 * PAGE,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0)
    want = Engine(m, max_batch=1, max_seq_len=96).generate([p], sp, 6)[0]
    eng = Engine(m, max_batch=1, max_seq_len=96, prefix_cache=True)
    if not eng.prefix_cache:
        pytest.skip("host runtime module not built")
    assert eng.generate([p], sp, 6)[0] == want and eng.generate([p], sp, 6)[0] == want
    assert eng.prefix_stats["hit_tokens"] == PAGE            # one page leased, the second page re-prefilled for its logits


def test_published_pages_are_evicted_only_when_unreferenced():
    cfg, m = model()
    sp = SamplingParams(temperature=0.0)
    g = torch.Generator().manual_seed(2)
    eng = Engine(m, max_batch=1, max_seq_len=96, num_pages=7, prefix_cache=True)      # 6 usable pages
    if not eng.prefix_cache:
        pytest.skip("host runtime module not built")
    ps = [torch.randint(0, cfg.vocab_size, (40,), generator=g).tolist() for _ in range(3)]
    for p in ps:
        eng.generate([p], sp, 8)                 # 3 pages each, two of them published: the pool has to evict
    assert eng.kv.allocator.free_pages() == 6 and eng.kv.allocator.cached_pages() <= 6
    hold = eng.new_sequence(ps[2], sp, 8)
    assert hold.cached_tokens == 2 * PAGE
    with pytest.raises(RuntimeError):
        eng.new_sequence(ps[0] + ps[1], sp, 16)  # 6 pages wanted, 3 leased elsewhere: nothing referenced is taken
    assert eng.kv.allocator.refcount(hold.pages[0]) == 1
    eng.release(hold)
    assert eng.kv.allocator.free_pages() == 6


def test_models_with_recurrent_state_do_not_share_pages():
    from test_lfm2 import lfm2_cfg

    cfg = lfm2_cfg()
    sd = random_state(cfg, seed=3, std=0.08)
    m = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32)
    assert not Engine(m, max_batch=1, max_seq_len=64, prefix_cache=True).prefix_cache


@pytest.mark.gpu
def test_prefix_reuse_on_the_gpu_engine():
    cfg, m = model("cuda", torch.bfloat16)
    system, ps = prompts(cfg)
    sp = SamplingParams(temperature=0.0)
    eng = Engine(m, max_batch=2, max_seq_len=160, prefix_cache=True)
    assert eng.prefix_cache
    first = [eng.generate([p], sp, 12)[0] for p in ps]
    again = [eng.generate([p], sp, 12)[0] for p in ps]
    assert eng.prefix_stats["hit_tokens"] >= 5 * 3 * PAGE
    agree = sum(a == b for x, y in zip(first, again) for a, b in zip(x, y))
    assert agree >= 0.9 * 36          # the reused rows are bit-identical; the shorter prefill may round a near-tie differently
