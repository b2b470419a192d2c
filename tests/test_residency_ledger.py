"""C++ residency ledger (tiers, budgets, reserve / publish / rollback, pins, eviction order, transfer generations) and
the process-wide cache byte pool."""
import pytest

from eredu_b200.lib import _eredu_host as H


def ledger(eviction="lru"):
    led = H.ResidencyLedger(device_budget_bytes=300, host_budget_bytes=-1, eviction=eviction)
    for i in range(5):
        led.add_unit(f"layer.{i}", 100, "cacheable", "host")
    led.add_unit("embed", 50, "pinned", "host")
    return led


def test_reserve_publish_evict_order():
    led = ledger()
    assert led.is_resident("layer.0", "host") and not led.is_resident("layer.0", "device")
    assert led.resident_bytes("host") == 550
    for i in range(3):
        assert led.reserve(f"layer.{i}", "device") == []
        led.publish(f"layer.{i}", "device")
    led.touch("layer.0", "device")                              # 1 is now the least recently used
    assert led.reserve("layer.3", "device") == ["layer.1"]
    led.publish("layer.3", "device")
    assert not led.is_resident("layer.1", "device") and led.resident_bytes("device") == 300
    # pins protect a copy; when nothing evictable is left the reservation is refused and nothing changes
    for u in ("layer.0", "layer.2", "layer.3"):
        led.pin(u, "device")
    with pytest.raises(RuntimeError, match="bytes short"):
        led.reserve("layer.4", "device")
    assert led.resident_bytes("device") == 300 and led.report()["device"]["refused"] == 1
    led.unpin("layer.2", "device")
    assert led.reserve("layer.4", "device") == ["layer.2"]
    led.rollback("layer.4", "device")                           # the transfer failed: bytes are returned
    assert led.resident_bytes("device") == 200 and not led.is_resident("layer.4", "device")
    with pytest.raises(RuntimeError):
        led.evict("layer.0", "device")                          # pinned
    with pytest.raises(RuntimeError):
        led.evict("layer.0", "host")                            # home copy
    with pytest.raises(RuntimeError):
        led.publish("layer.4", "device")                        # no reservation
    rep = led.report()
    assert rep["device"]["evictions"] == 2 and rep["device"]["evicted_bytes"] == 200 and rep["units"] == 6


def test_lfu_order_and_transfer_generations():
    led = ledger("lfu")
    for i in range(3):
        led.reserve(f"layer.{i}", "device")
        led.publish(f"layer.{i}", "device")
    led.touch("layer.0", "device"); led.touch("layer.0", "device"); led.touch("layer.1", "device")
    assert led.reserve("layer.3", "device") == ["layer.2"]      # never used again since it arrived
    g1 = led.begin_transfer("layer.3", "device")
    # the request is abandoned and issued again: the first completion is stale
    led.rollback("layer.3", "device")
    led.reserve("layer.3", "device")
    g2 = led.begin_transfer("layer.3", "device")
    assert g2 > g1 and not led.resolve_transfer("layer.3", "device", g1, "host", 0.001)
    assert not led.is_resident("layer.3", "device")
    assert led.resolve_transfer("layer.3", "device", g2, "host", 0.002)
    assert led.is_resident("layer.3", "device")
    led.record_prefetch("device", "hit"); led.record_prefetch("device", "late"); led.record_stall(0.5)
    rep = led.report()
    assert rep["transfers"]["host_to_device"] == {"count": 1, "bytes": 100, "seconds": 0.002}
    assert rep["stale_transfers"] == 1 and rep["device"]["prefetch"] == {"hit": 1, "late": 1, "miss": 0}
    assert rep["stalls"] == 1 and rep["stall_seconds"] == 0.5
    with pytest.raises(ValueError):
        led.record_prefetch("device", "maybe")
    with pytest.raises(IndexError):
        led.touch("nope", "device")
    with pytest.raises(ValueError):
        H.ResidencyLedger(eviction="fifo")


def test_cache_pool():
    pool = H.CachePool(device_bytes=1000, host_bytes=-1, transfer_bytes=256)
    a = pool.reserve("device", 600)
    assert a > 0 and pool.reserve("device", 500) == -1 and pool.used("device") == 600
    b = pool.reserve("device", 400)
    t = pool.reserve("transfer", 256)
    assert pool.reserve("transfer", 1) == -1
    pool.release(a)
    assert pool.used("device") == 400
    rep = pool.report()
    assert rep["device"]["peak_bytes"] == 1000 and rep["refused"] == 2 and rep["live_reservations"] == 2
    assert rep["host"]["budget_bytes"] is None
    with pytest.raises(IndexError):
        pool.release(a)
    pool.release(b); pool.release(t)
    assert pool.report()["live_reservations"] == 0
