"""Pinned transfer-buffer pool (per-purpose active / peak accounting, reuse by size class) and the Completion object."""
import pytest
import torch

from eredu_b200.ops.native import Completion
from eredu_b200.runtime.host_pool import HostTransferPool


def test_pool_accounts_by_kind_and_reuses_buffers():
    pool = HostTransferPool(cached_limit_bytes=3 << 20, pin=False)
    a = pool.acquire(5000, "kv")
    b = pool.acquire(1_500_000, "weights")
    assert a.numel() == 8192 and b.numel() == 2 << 20 and a.dtype == torch.uint8
    st = pool.stats()
    assert st["kv"]["active_bytes"] == 8192 and st["weights"]["active_bytes"] == 2 << 20 and st["active_bytes"] == 8192 + (2 << 20)
    v = pool.view(b, (3, 100), torch.float32)
    v.fill_(2.5)
    assert v.shape == (3, 100) and v.data_ptr() == b.data_ptr()
    pool.release(a)
    pool.release(b)
    with pytest.raises(ValueError):
        pool.release(b)                                    # double release
    st = pool.stats()
    assert st["active_bytes"] == 0 and st["cached_bytes"] == 8192 + (2 << 20) and st["kv"]["peak_bytes"] == 8192
    again = pool.acquire(6000, "experts")                  # same size class: the released buffer comes back
    assert again.data_ptr() == a.data_ptr() and pool.stats()["experts"]["reuses"] == 1
    big = pool.acquire(4 << 20, "weights")
    pool.release(big)                                      # beyond the cache limit: dropped, not kept pinned
    assert pool.stats()["cached_bytes"] == 2 << 20
    assert pool.trim() == 2 << 20 and pool.stats()["cached_bytes"] == 0
    with pytest.raises(ValueError):
        pool.acquire(16, "nonsense")


def test_kv_tier_stages_through_the_pool():
    from eredu_b200.models import config as C
    from eredu_b200.models.llama import build_from_tensors, random_state
    from eredu_b200.ops import SamplingParams
    from eredu_b200.runtime.engine import Engine
    from eredu_b200.runtime.kv_residency import KVHostTier

    cfg = C.tiny_llama()
    sd = random_state(cfg, seed=0, std=0.08)
    eng = Engine(build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32), max_batch=2, max_seq_len=64)
    tier = KVHostTier(eng)
    seq = eng.new_sequence(list(range(1, 20)), SamplingParams(temperature=0.0), 8)
    eng.prefill([seq])
    before = eng.kv.k[:, seq.pages[0]].clone()
    assert tier.park(seq) and tier.pool.stats()["kv"]["active_bytes"] > 0
    assert tier.resume(seq) and tier.pool.stats()["kv"]["active_bytes"] == 0 and tier.pool.stats()["cached_bytes"] > 0
    assert torch.equal(eng.kv.k[:, seq.pages[0]], before)
    assert tier.park(seq) and tier.pool.stats()["kv"]["reuses"] == 2      # K and V staging both came back from the cache
    tier.drop(seq)
    assert tier.pool.stats()["kv"]["active_bytes"] == 0


def test_completion_on_cpu_is_immediately_ready():
    c = Completion("cpu")
    assert c.is_ready()
    c.wait()


@pytest.mark.gpu
def test_completion_reports_at_the_recorded_point():
    from eredu_b200.ops import native

    dev = torch.device("cuda", 0)
    x = torch.randn(4096, 4096, device=dev)
    y = x @ x
    c = Completion(dev)
    c.wait(timeout_s=10.0)
    assert c.is_ready() and torch.isfinite(y).all()
    # a status recorded before the completion point surfaces at its wait and is cleared
    native.status_word(dev).fill_(4)
    c2 = Completion(dev)
    with pytest.raises(RuntimeError, match="peer flag"):
        c2.wait()
    native.check_status(dev)


def test_nvtx_ranges_fire_only_when_enabled():
    from eredu_b200.models import config as C
    from eredu_b200.models.llama import build_from_tensors, random_state
    from eredu_b200.ops import SamplingParams
    from eredu_b200.runtime.engine import Engine
    from eredu_b200.utils import nvtx

    cfg = C.tiny_llama()
    sd = random_state(cfg, seed=0, std=0.08)
    eng = Engine(build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32), max_batch=1, max_seq_len=64)
    before = nvtx.ranges_opened
    eng.generate([[1, 2, 3]], SamplingParams(temperature=0.0), 3)
    assert nvtx.ranges_opened == before and not nvtx.enabled()
    nvtx.enable(True)
    try:
        eng.generate([[1, 2, 3]], SamplingParams(temperature=0.0), 3)
        # one prefill range, two decode-step ranges, and a range per layer in each of the three passes
        assert nvtx.ranges_opened - before == 3 + 3 * cfg.num_hidden_layers
    finally:
        nvtx.enable(False)
