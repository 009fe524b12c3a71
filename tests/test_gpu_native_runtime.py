"""Native device layer (C++ over the CUDA runtime): properties, streams, events, timer, pooled allocator."""
import pytest

pytestmark = pytest.mark.gpu


def test_device_stream_event_pool():
    from ghost_flow_b200.cuda import native

    assert native.device_count() >= 1
    p = native.device_properties(0)
    assert p["major"] == 10 and p["multiprocessors"] > 100 and p["total_memory"] > (100 << 30)
    free, total = native.memory_info(0)
    assert 0 < free <= total
    s = native.Stream(0)
    t = native.Timer()
    t.start(s)
    t.stop(s)
    assert t.elapsed_ms() >= 0.0
    ev = native.Event()
    ev.record(s)
    s.wait_event(ev)
    s.synchronize()
    assert s.query() and ev.query()
    pool = native.MemoryPool(0)
    a = pool.allocate(1000)
    b = pool.allocate(5000)
    st = pool.stats()
    assert st["current_usage"] == 1024 + 8192 and st["misses"] == 2 and st["live_blocks"] == 2
    pool.free(a)
    c = pool.allocate(900)                      # same size class: served from the cache
    assert c == a and pool.stats()["hits"] == 1
    pool.free(b)
    pool.free(c)
    assert pool.current_usage() == 0 and pool.peak_usage() == 1024 + 8192
    with pytest.raises(native.NativeCudaError):
        pool.free(12345)
    pool.close()
