"""Glue between the training loop and the fault-tolerance control plane.

* ``install_ttp(args)``: rank 0 starts the controller, every rank starts a processor, the train step gets wrapped in
  ``ttp_exception_handler`` which classifies exceptions and reports them.
* fault injection for tests and drills: ``TTP_FAULT_INJECTION_ENABLED=1``, ``TTP_FAULT_INJECTION_ITERATION``,
  ``TTP_FAULT_INJECTION_RANK`` raise ``RuntimeError("TTP_INJECTED_FAULT ...")`` once on the chosen rank / iteration
  (reference: mindspeed/core/ttp/adaptor.py:25-61).  Injection happens on the host only; no device fault is ever provoked.
* the emergency dump writes a normal sharded checkpoint into ``--ttp-dump-dir`` from the selected healthy ranks
  (reference: mindspeed/core/ttp/recovery/dump_save.py:86-477); recovery is a relaunch that resumes from that directory.
"""
from __future__ import annotations

import functools
import os
from typing import Callable, Optional

from .controller import TTPController
from .processor import TTPPause, TTPProcessor
from .replica import build_replica_groups

_STATE = {"controller": None, "processor": None, "iteration": 0, "injected": False}

DEVICE_FAULT_MARKERS = ("CUDA error", "Xid", "uncorrectable", "ECC", "NCCL", "nccl", "timeout", "Timeout", "unspecified launch failure",
                        "device-side", "illegal memory", "bounded-wait", "TTP_INJECTED_FAULT")


def classify_exception(e: BaseException) -> str:
    """'device' for errors that mean this rank's GPU / communicator is unusable, 'pause' for controller pauses,
    'software' otherwise (reference string matching: recovery/exception_handler.py:118-131)."""
    if isinstance(e, TTPPause):
        return "pause"
    s = f"{type(e).__name__}: {e}"
    return "device" if any(m in s for m in DEVICE_FAULT_MARKERS) else "software"


def maybe_inject_fault(iteration: int, rank: int):
    if os.environ.get("TTP_FAULT_INJECTION_ENABLED", "0") != "1" or _STATE["injected"]:
        return
    if iteration == int(os.environ.get("TTP_FAULT_INJECTION_ITERATION", "-1")) and \
            rank == int(os.environ.get("TTP_FAULT_INJECTION_RANK", "-1")):
        _STATE["injected"] = True
        raise RuntimeError(f"TTP_INJECTED_FAULT at iteration {iteration} on rank {rank}")


def ttp_exception_handler(fn: Callable, rank: int, processor: Optional[TTPProcessor] = None):
    @functools.wraps(fn)
    def wrapped(*a, **k):
        _STATE["iteration"] += 1
        try:
            maybe_inject_fault(_STATE["iteration"], rank)
            return fn(*a, **k)
        except BaseException as e:  # noqa: BLE001 - everything is classified and re-raised
            kind = classify_exception(e)
            p = processor or _STATE["processor"]
            if p is not None and kind != "pause":
                p.report_fault(f"{kind}: {type(e).__name__}: {e}")
            raise
    return wrapped


def install_ttp(args, dump_fn=None):
    import torch.distributed as dist
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    groups = build_replica_groups(world, args.tensor_model_parallel_size, args.pipeline_model_parallel_size,
                                  args.context_parallel_size, args.use_distributed_optimizer,
                                  args.num_distributed_optimizer_instances)
    if rank == 0:
        _STATE["controller"] = TTPController(world, args.ttp_server_ip, args.ttp_server_port, args.ttp_heartbeat_timeout_ms,
                                             args.ttp_max_missed_count, args.ttp_dump_timeout_seconds).start()
    if dist.is_initialized():
        dist.barrier()
    mine = [g for g in groups if rank in g]
    _STATE["processor"] = TTPProcessor(rank, args.ttp_server_ip, args.ttp_server_port, mine, args.ttp_heartbeat_interval_ms,
                                       dump_fn=dump_fn, interrupt_main=True).start()
    return _STATE["processor"]
