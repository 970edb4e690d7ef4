"""Fault tolerance on the host only: heartbeats, disconnects, self-reports, dump planning, fault injection.
No GPU is involved and nothing is made to fault, trap or hang."""
import os
import time

import pytest


def _cluster(n, groups, dump_log, timeout_ms=300, interval_ms=50):
    from mindspeed_b200.ttp import TTPController, TTPProcessor
    ctl = TTPController(n, port=0, heartbeat_timeout_ms=timeout_ms, dump_timeout_s=5).start()
    procs = []
    for r in range(n):
        mine = [g for g in groups if r in g]
        procs.append(TTPProcessor(r, "127.0.0.1", ctl.port, mine, heartbeat_interval_ms=interval_ms,
                                  dump_fn=(lambda ranks, r=r: dump_log.append((r, tuple(ranks))))).start())
    return ctl, procs


def _shutdown(ctl, procs):
    for p in procs:
        p.close()
    ctl.stop()


def test_replica_groups_and_dump_selection():
    from mindspeed_b200.ttp import build_replica_groups, select_dump_ranks
    g = build_replica_groups(8, tp=2, pp=1)                       # dp=4 replicas for each tp rank
    assert sorted(map(sorted, g)) == [[0, 2, 4, 6], [1, 3, 5, 7]]
    plan = select_dump_ranks(g, {0, 1})
    assert plan["ok"] and plan["ranks"] == [2, 3]
    g2 = build_replica_groups(8, tp=2, use_distributed_optimizer=True, num_optimizer_instances=2)
    assert all(len(x) == 2 for x in g2) and len(g2) == 4
    assert not select_dump_ranks(g2, set(g2[0]))["ok"]          # a shard lost in both instances cannot be rebuilt


def test_heartbeat_timeout_triggers_pause_dump_exit():
    from mindspeed_b200.ttp import build_replica_groups
    groups = build_replica_groups(4, tp=2)
    log = []
    ctl, procs = _cluster(4, groups, log)
    try:
        time.sleep(0.2)
        assert ctl.state == "RUNNING"
        procs[2].stop_heartbeat()                                  # rank 2 "freezes"
        assert ctl.finished.wait(5.0)
        assert ctl.faulty == {2} and "heartbeat" in ctl.fault_reasons[2]
        assert ctl.plan["ok"] and ctl.plan["ranks"] == [0, 1]
        for r in (0, 1, 3):
            assert procs[r].paused.wait(2.0) and procs[r].exited.wait(2.0)
        assert sorted(x[0] for x in log) == [0, 1]
    finally:
        _shutdown(ctl, procs)


def test_disconnect_and_self_report():
    from mindspeed_b200.ttp import build_replica_groups
    groups = build_replica_groups(4, tp=1)
    log = []
    ctl, procs = _cluster(4, groups, log, timeout_ms=2000)
    try:
        procs[1].close()                                           # socket drops: detected without waiting for a time-out
        assert ctl.finished.wait(5.0)
        assert 1 in ctl.faulty and ctl.fault_reasons[1] == "disconnect"
        assert ctl.plan["ranks"] == [0]
    finally:
        _shutdown(ctl, procs)
    log2 = []
    ctl, procs = _cluster(2, [[0, 1]], log2, timeout_ms=2000)
    try:
        procs[0].report_fault("device: RuntimeError: CUDA error: an illegal memory access")
        assert ctl.finished.wait(5.0)
        assert ctl.plan["ranks"] == [1] and log2 and log2[0][0] == 1
    finally:
        _shutdown(ctl, procs)


def test_fault_injection_and_classification(monkeypatch):
    from mindspeed_b200.ttp import adaptor
    from mindspeed_b200.ttp import classify_exception, ttp_exception_handler, TTPPause
    adaptor._STATE.update(iteration=0, injected=False)
    monkeypatch.setenv("TTP_FAULT_INJECTION_ENABLED", "1")
    monkeypatch.setenv("TTP_FAULT_INJECTION_ITERATION", "3")
    monkeypatch.setenv("TTP_FAULT_INJECTION_RANK", "1")
    reports = []

    class FakeProc:
        def report_fault(self, reason):
            reports.append(reason)

    step = ttp_exception_handler(lambda: "ok", rank=1, processor=FakeProc())
    assert step() == "ok" and step() == "ok"
    with pytest.raises(RuntimeError, match="TTP_INJECTED_FAULT"):
        step()
    assert step() == "ok"                                         # injected once only
    assert reports and reports[0].startswith("device")
    assert classify_exception(RuntimeError("NCCL communicator was aborted")) == "device"
    assert classify_exception(ValueError("bad shape")) == "software"
    assert classify_exception(TTPPause()) == "pause"
