"""Host and disk tiers under the published KV pages: evicted sealed pages are demoted (device -> host -> disk), a prompt
that continues through a demoted block gets it promoted into a fresh device page, and the tokens committed are those of
an engine that never evicted anything."""
import pytest
import torch

from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.engine import Engine
from eredu_b200.runtime.kv_cache import PAGE
from test_prefix_reuse import model


def small_pool_engine(m, tmp_path=None, host_blocks=64, disk_blocks=0, pages=11):
    probe = Engine(m, max_batch=1, max_seq_len=96, num_pages=pages, prefix_cache=True)
    if not probe.prefix_cache or not hasattr(probe.kv.allocator, "take_evicted"):
        pytest.skip("host runtime module not built")
    L, _, nkv, _, D = probe.kv.k.shape
    block = 2 * L * nkv * PAGE * D * probe.kv.k.element_size()
    return Engine(m, max_batch=1, max_seq_len=96, num_pages=pages, prefix_cache=True, kv_host_tier_bytes=host_blocks * block,
                  kv_disk_tier_dir=str(tmp_path / "kv") if tmp_path is not None else None, kv_disk_tier_bytes=disk_blocks * block)


def conversations(cfg, n=4, length=50):
    g = torch.Generator().manual_seed(11)
    return [torch.randint(0, cfg.vocab_size, (length,), generator=g).tolist() for _ in range(n)]


def test_evicted_prefixes_come_back_from_the_host_tier():
    cfg, m = model()
    sp = SamplingParams(temperature=0.0)
    convs = conversations(cfg)
    cold = Engine(m, max_batch=1, max_seq_len=96)
    want = {i: cold.generate([c + [7, 8, 9]], sp, 6)[0] for i, c in enumerate(convs)}
    eng = small_pool_engine(m)                     # 10 usable pages: one request of 50 + 3 + 6 tokens takes 4
    for c in convs:                                # four conversations: their published pages cannot all stay on the device
        eng.generate([c], sp, 4)
    st = eng.block_tiers.stats
    assert eng.kv.allocator.evictions > 0 and st["demoted"] == eng.kv.allocator.evictions and st["dropped"] == 0
    # follow-ups in order of age: the oldest conversations were evicted and are promoted from host memory
    for i, c in enumerate(convs):
        before = eng.prefix_stats["hit_tokens"]
        assert eng.generate([c + [7, 8, 9]], sp, 6)[0] == want[i], i
        assert eng.prefix_stats["hit_tokens"] - before == 3 * PAGE, i          # the whole 48-token prefix was reused every time
    assert st["promoted_host"] > 0 and st["promoted_disk"] == 0
    total = eng.kv.allocator.free_pages()
    assert total == eng.kv.allocator.num_pages - 1                             # nothing leaked: every page is free or cached


def test_host_overflow_spills_to_files_and_reads_back(tmp_path):
    cfg, m = model()
    sp = SamplingParams(temperature=0.0)
    convs = conversations(cfg, n=5)
    cold = Engine(m, max_batch=1, max_seq_len=96)
    eng = small_pool_engine(m, tmp_path, host_blocks=2, disk_blocks=32)
    for c in convs:
        eng.generate([c], sp, 4)
    st = eng.block_tiers.stats
    assert st["spilled"] > 0 and st["host_blocks"] <= 2
    files = list((tmp_path / "kv").glob("*.kvb"))
    assert len(files) == st["disk_blocks"] > 0 and all(f.stat().st_size == eng.block_tiers.block_bytes for f in files)
    assert eng.generate([convs[0] + [1, 2]], sp, 5)[0] == cold.generate([convs[0] + [1, 2]], sp, 5)[0]
    assert st["promoted_disk"] > 0
    eng.block_tiers.clear()
    assert not list((tmp_path / "kv").glob("*.kvb"))


def test_without_room_in_any_tier_blocks_are_dropped_and_recomputed(tmp_path):
    cfg, m = model()
    sp = SamplingParams(temperature=0.0)
    convs = conversations(cfg, n=4)
    cold = Engine(m, max_batch=1, max_seq_len=96)
    eng = small_pool_engine(m, tmp_path, host_blocks=1, disk_blocks=1)
    for c in convs:
        eng.generate([c], sp, 4)
    assert eng.block_tiers.stats["dropped"] > 0
    before = eng.prefix_stats["hit_tokens"]
    assert eng.generate([convs[0] + [5]], sp, 5)[0] == cold.generate([convs[0] + [5]], sp, 5)[0]
    assert eng.prefix_stats["hit_tokens"] - before < 3 * PAGE                   # a chain with a missing block ends there


def test_demotion_copies_the_page_before_its_new_owner_writes_it():
    """Direct check of the store: the K and V slabs of every layer survive the round trip bit for bit."""
    cfg, m = model()
    eng = small_pool_engine(m)
    kv, tiers = eng.kv, eng.block_tiers
    g = torch.Generator().manual_seed(3)
    kv.k.copy_(torch.randn(kv.k.shape, generator=g))
    kv.v.copy_(torch.randn(kv.v.shape, generator=g))
    want_k, want_v = kv.k[:, 5].clone(), kv.v[:, 5].clone()
    tiers.demote([(5, 1234), (6, 99)])
    assert tiers.where(1234) == "host" and tiers.where(99) == "host" and tiers.where(7) is None
    kv.k[:, 5].zero_()
    kv.v[:, 5].zero_()
    tiers.promote([(1234, 9)])
    assert torch.equal(kv.k[:, 9], want_k) and torch.equal(kv.v[:, 9], want_v)
    assert tiers.where(1234) is None and tiers.stats["promoted_host"] == 1
