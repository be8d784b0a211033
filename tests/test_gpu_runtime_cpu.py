"""Host-side checks of the device runtime: caching-allocator block logic (host-backed segments), memory guard policies with a fake memory query,
buffer pool rounding."""
import threading
import time

import pytest

from ferrotorch_b200 import gpu
from ferrotorch_b200.errors import FerrotorchError


def test_allocator_split_coalesce_reuse_and_budget():
    a = gpu.CudaAllocator(host_mode=True)
    p1 = a.malloc(1000)                       # rounds to 1024, carved out of a 2 MiB small segment
    p2 = a.malloc(3000)
    s = a.stats()
    assert s.allocated == 1024 + 3072 and s.reserved == 2 << 20 and s.num_segment_allocs == 1 and p2 == p1 + 1024
    a.free(p1)
    p3 = a.malloc(512)                        # fits in the freed 1024-byte block (split again)
    assert p3 == p1 and a.stats().num_cache_hits >= 1
    a.free(p2)
    a.free(p3)
    s = a.stats()
    assert s.allocated == 0 and s.live_blocks == 0 and s.reserved == 2 << 20
    p4 = a.malloc(1 << 20)                    # the segment coalesced back into one block: the largest small request fits at its start
    assert p4 == p1 and a.stats().num_segment_allocs == 1
    a.free(p4)
    big = a.malloc(5 << 20)                   # large pool: 20 MiB segment
    assert a.stats().reserved == (2 << 20) + (20 << 20)
    huge = a.malloc(33 << 20)                 # own segment, rounded to 2 MiB
    assert a.stats().reserved == (2 << 20) + (20 << 20) + (34 << 20)
    a.free(huge)
    assert a.empty_cache() == (2 << 20) + (34 << 20)        # whole free segments go back; the 20 MiB one is still in use
    a.set_budget(25 << 20)
    with pytest.raises(gpu.OutOfMemory):
        a.malloc(30 << 20)
    assert a.stats().num_ooms == 1 and a.stats().peak_allocated >= 38 << 20
    a.free(big)
    with pytest.raises(Exception):
        a.free(12345)
    # streams: a block freed on stream 1 is not handed to stream 2
    q1 = a.malloc(4096, stream=1)
    a.free(q1)
    q2 = a.malloc(4096, stream=2)
    assert q2 != q1
    q3 = a.malloc(4096, stream=1)
    assert q3 == q1
    a.close()


def test_memory_guard_policies_hooks_pressure_and_watchdog():
    state = {"used": 100}
    g = gpu.MemoryGuardBuilder().with_budget(1000).with_policy(gpu.OomPolicy.RETRY_AFTER_FREE).with_query(lambda: (state["used"], 2000)).build()
    order = []
    g.add_pre_oom_hook("late", lambda need: order.append("late") or 0, priority=10)

    def free_cache(need):
        order.append("cache")
        state["used"] -= 80
        return 80
    g.add_pre_oom_hook("cache", free_cache, priority=1)
    levels = []
    g.add_pressure_listener(lambda old, new: levels.append((old, new)))
    r1 = g.reserve(850)                                     # 100 + 850 = 950 <= 1000
    assert g.pressure() == gpu.PressureLevel.CRITICAL and levels[-1][1] == gpu.PressureLevel.CRITICAL
    r2 = g.reserve(100)                                     # over budget -> hooks run in priority order -> cache frees 80 -> fits
    assert order == ["cache"] and g.stats().oom_events == 1
    with pytest.raises(gpu.OutOfMemory):
        g.reserve(500)
    assert order[-1] == "late"
    r1.release()
    r2.release()
    assert g.stats().reserved_by_guard == 0 and g.pressure() == gpu.PressureLevel.NONE
    fail = gpu.MemoryGuard(100, gpu.OomPolicy.FAIL, query=lambda: (90, 200))
    with pytest.raises(gpu.OutOfMemory):
        fail.reserve(20)
    called = []
    ck = gpu.MemoryGuard(100, gpu.OomPolicy.CHECKPOINT_AND_FAIL, query=lambda: (90, 200))
    ck.on_oom = lambda n: called.append(n)
    with pytest.raises(gpu.OutOfMemory):
        ck.reserve(20)
    assert called == [20]
    # WAIT: another thread releases its reservation, the waiter proceeds
    w = gpu.MemoryGuard(100, gpu.OomPolicy.WAIT, query=lambda: (0, 200), wait_timeout_s=5)
    held = w.reserve(90)
    threading.Timer(0.1, held.release).start()
    t0 = time.monotonic()
    w.reserve(50).release()
    assert 0.05 < time.monotonic() - t0 < 4
    # watchdog pauses cooperative workers at CRITICAL and resumes them when pressure falls
    st = {"used": 99}
    wd = gpu.MemoryGuard(100, query=lambda: (st["used"], 200))
    wd.start_watchdog(0.01)
    time.sleep(0.1)
    assert wd.wait_if_paused(0.05) is False
    st["used"] = 10
    assert wd.wait_if_paused(2.0) is True
    wd.stop_watchdog()


def test_buffer_pool_rounding():
    assert gpu.BufferPool.round_len(1000) == 1024 and gpu.BufferPool.round_len(1 << 20) == 1 << 20 and gpu.BufferPool.round_len((1 << 20) + 1) == 2 << 20
    assert gpu.BufferPool.round_len(0) == 0


def test_allocator_canary_catches_a_write_past_the_end():
    import ctypes
    a = gpu.CudaAllocator(host_mode=True)
    a.set_canary(64)
    p = a.malloc(1000)
    ctypes.memset(p, 0x11, 1000)                 # exactly the requested bytes: fine
    a.free(p)
    assert a.canary_violations() == 0
    q = a.malloc(1000)
    ctypes.memset(q, 0x22, 1001)                 # one byte too far
    with pytest.raises(FerrotorchError, match="guard bytes"):
        a.free(q)
    assert a.canary_violations() == 1 and a.stats().allocated == 0     # the block went back to the pool all the same
    r = a.malloc(100)
    with pytest.raises(FerrotorchError):
        a.set_canary(0)                          # not while a block is live
    a.free(r)
    a.set_canary(0)
    a.close()
