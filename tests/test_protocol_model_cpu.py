"""The flag protocols of the fused compute+collective kernels, explored over every interleaving of the ranks' steps:
the protocols as implemented are free of deadlocks and stale reads; with one element removed the checker finds the race."""
import pytest

from mindspeed_b200.parallel import protocol_model as PM


@pytest.mark.parametrize("world", [2, 3])
def test_all_gather_gemm_protocol_is_race_free(world):
    v, states = PM.check(PM.all_gather_gemm_program(world, epochs=2, chunks=2 if world == 2 else 1))
    assert v is None, (v.kind, v.detail, v.trace[-6:])
    assert states > 100                                            # several interleavings were in fact explored


@pytest.mark.parametrize("world,all_reduce", [(2, False), (2, True), (3, False)])
def test_gemm_reduce_scatter_protocol_is_race_free(world, all_reduce):
    v, states = PM.check(PM.gemm_reduce_scatter_program(world, epochs=2, warps=2 if world == 2 else 1, all_reduce=all_reduce))
    assert v is None, (v.kind, v.detail, v.trace[-6:])
    assert states > 100


def test_removing_a_protocol_element_is_detected():
    # no entry handshake: a rank already in its next call overwrites rows a slower peer still reads, or bumps a counter the
    # peer's host has not zeroed yet
    v, _ = PM.check(PM.all_gather_gemm_program(2, epochs=2, chunks=1, entry_handshake=False))
    assert v is not None and v.kind in ("stale read", "deadlock")
    # consumer does not wait for the arrival counter: reads rows that have not arrived
    v, _ = PM.check(PM.all_gather_gemm_program(2, epochs=1, chunks=1, wait_ready=False))
    assert v is not None and v.kind == "stale read"
    # reduction does not wait for the owners' completion flags
    v, _ = PM.check(PM.gemm_reduce_scatter_program(2, epochs=1, warps=2, wait_done=False))
    assert v is not None and v.kind == "stale read"
    # no entry handshake in reduce-scatter: the next call's partial sums land in a staging area that is still being summed
    v, _ = PM.check(PM.gemm_reduce_scatter_program(2, epochs=2, warps=1, entry_handshake=False))
    assert v is not None and v.kind == "stale read" and v.trace


@pytest.mark.parametrize("world", [2, 3])
def test_moe_pull_protocol_needs_two_staging_slots_and_no_exit_flags(world):
    v, states = PM.check(PM.moe_pull_program(world, epochs=3, slots=2, readers=2 if world == 2 else 1))
    assert v is None and states > 50, v and (v.kind, v.detail)
    # one slot: the next call's staging copy overwrites rows a slower peer is still pulling
    v, _ = PM.check(PM.moe_pull_program(world, epochs=2, slots=1, readers=1))
    assert v is not None and v.kind == "stale read"
    # no handshake: a peer's rows are pulled before that peer has staged them
    v, _ = PM.check(PM.moe_pull_program(world, epochs=1, slots=2, readers=1, entry_handshake=False))
    assert v is not None and v.kind == "stale read"


def test_explorer_reports_deadlock_with_the_waiting_steps():
    progs = [[[[("wait_ge", "a", 1), ("store", 1, "b", 1)]]], [[[("wait_ge", "b", 1), ("store", 0, "a", 1)]]]]
    v, _ = PM.check(progs)
    assert v.kind == "deadlock" and "rank 0" in v.detail and "rank 1" in v.detail
    ok = [[[[("store", 1, "b", 1), ("wait_ge", "a", 1)]]], [[[("wait_ge", "b", 1), ("store", 0, "a", 1)]]]]
    assert PM.check(ok)[0] is None
    # fetch_add + conditional: exactly one of two threads sees itself as last
    last = [[[[("fetch_add", "c", 1), ("if_reg_ne", 1, 1), ("add", 0, "winners", 1)],
              [("fetch_add", "c", 1), ("if_reg_ne", 1, 1), ("add", 0, "winners", 1)]],
             [[("wait_ge", "winners", 1), ("write", 0, "x", 0, "ok"), ("read", "x", 0, "ok")]]]]
    assert PM.check(last)[0] is None


def test_heap_layout_guard_bytes_catch_a_write_past_a_buffer():
    import torch
    from mindspeed_b200.parallel.symm_mem import FLAG_BYTES, GUARD_BYTES, GUARD_PATTERN, HeapLayout
    plain, guarded = HeapLayout(1 << 16), HeapLayout(1 << 16, GUARD_BYTES)
    assert plain.alloc("a", 1500) == (FLAG_BYTES, True) and plain.alloc("b", 10) == (FLAG_BYTES + 2048, True)
    assert plain.alloc("a", 1000) == (FLAG_BYTES, False)              # named buffers are allocated once
    with pytest.raises(RuntimeError, match="too small"):
        plain.alloc("b", 5000)
    raw = torch.zeros(1 << 16, dtype=torch.uint8)
    offs = {}
    for name, n in (("a", 1500), ("b", 10), ("c", 4096)):
        offs[name], new = guarded.alloc(name, n)
        assert new
        guarded.fill_guard(raw, name)
    assert offs == {"a": FLAG_BYTES, "b": FLAG_BYTES + 2048 + GUARD_BYTES, "c": FLAG_BYTES + 3072 + 2 * GUARD_BYTES}
    assert guarded.check_guards(raw) == [] and plain.check_guards(raw) == []
    raw[offs["a"]:offs["a"] + 2048] = 7                                  # the whole (rounded) buffer is the kernel's to write
    assert guarded.check_guards(raw) == []
    raw[offs["b"] + 1024] = 0                                            # one byte past the end of b
    assert guarded.check_guards(raw) == ["b"]
    assert int(raw[offs["c"] + 4096]) == GUARD_PATTERN
    with pytest.raises(RuntimeError, match="exhausted"):
        guarded.alloc("huge", 1 << 16)
