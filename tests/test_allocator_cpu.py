"""Native caching allocator over a host backend: splitting, merging, caching, limits, the pressure path, tracing."""
import pytest

from mindspeed_b200.memory.allocator import HostCachingAllocator

MB = 1 << 20


def test_rounding_split_merge_and_cache():
    a = HostCachingAllocator()
    p1 = a.malloc(1000)
    assert a.block_size(p1) == 1024                         # rounded to 512 B
    p2 = a.malloc(3000)
    s = a.stats()
    assert s["num_segments"] == 1 and s["reserved_bytes"] == 2 * MB      # both live in one small segment
    assert s["allocated_bytes"] == 1024 + 3072
    a.free(p1)
    a.free(p2)
    s = a.stats()
    assert s["allocated_bytes"] == 0 and s["largest_free_block"] == 2 * MB   # neighbours merged back into one block
    p3 = a.malloc(1500 * 1024)                              # large pool: its own >= 20 MB segment
    assert a.stats()["reserved_bytes"] == 2 * MB + 20 * MB
    a.free(p3)
    p4 = a.malloc(5 * MB)
    assert p4 == p3 and a.stats()["num_segment_allocs"] == 2                 # served from the cached segment
    a.free(p4)
    assert a.empty_cache() == 22 * MB and a.stats()["reserved_bytes"] == 0 and a.backend_in_use() == 0
    a.close()


def test_streams_do_not_share_free_blocks():
    a = HostCachingAllocator()
    p = a.malloc(4096, stream=1)
    a.free(p)
    q = a.malloc(4096, stream=2)
    assert q != p and a.stats()["num_segments"] == 2
    r = a.malloc(4096, stream=1)
    assert r == p
    a.close()


def test_limit_and_pressure_callback_release_memory():
    a = HostCachingAllocator(backend_capacity_bytes=64 * MB)
    held = [a.malloc(20 * MB) for _ in range(3)]            # 60 MB of the fake 64 MB device
    assert all(held)
    assert a.malloc(20 * MB) is None                        # no callback: clean failure, not a crash
    calls = []

    def on_pressure(need, dev):
        calls.append(need)
        a.free(held.pop())                                  # "swap a tensor out"
        return 20 * MB

    a.set_pressure_callback(on_pressure)
    p = a.malloc(20 * MB)
    assert p and calls == [20 * MB] and a.stats()["num_pressure_events"] >= 2
    # a soft limit below the backend's capacity triggers the same path
    a.set_limit(40 * MB)
    a.free(p)
    a.free(held.pop())
    a.empty_cache()
    assert a.stats()["reserved_bytes"] == 20 * MB
    q = a.malloc(20 * MB)
    assert q and a.stats()["reserved_bytes"] == 40 * MB
    assert a.malloc(20 * MB) is not None                    # callback frees the last held block to make room
    a.close()


def test_trace_records_lifetimes_with_tags():
    a = HostCachingAllocator()
    a.enable_trace(100)
    a.set_tags(step=3, phase=0)
    p = a.malloc(10 * MB)
    a.set_tags(step=3, phase=1)
    a.free(p)
    ev = a.read_trace()
    assert [e["is_free"] for e in ev] == [False, True]
    assert ev[0]["addr"] == ev[1]["addr"] == p and ev[0]["size"] == 10 * MB
    assert (ev[0]["step"], ev[0]["phase"], ev[1]["phase"]) == (3, 0, 1)
    assert a.read_trace() == []
    a.close()
