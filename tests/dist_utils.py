"""Spawn ``world_size`` local CPU ranks over gloo and run a function on each.

The function must be importable (module-level).  Results (picklable) are returned in rank order.
A rank that raises makes the whole call raise with that rank's traceback; a hang is bounded by
``timeout`` seconds after which the children are terminated by exact pid.
"""
import os
import socket
import traceback

import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _plain(o):
    """Tensors travel back as numpy arrays (torch's shared-memory pickling needs the sender to stay alive)."""
    import torch
    if torch.is_tensor(o):
        return o.detach().cpu().numpy()
    if isinstance(o, (list, tuple)):
        return type(o)(_plain(x) for x in o)
    if isinstance(o, dict):
        return {k: _plain(v) for k, v in o.items()}
    return o


def _entry(rank, world, port, fn, args, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    try:
        import torch
        torch.set_num_threads(1)
        out = fn(rank, world, *args)
        q.put((rank, "ok", _plain(out)))
    except Exception:
        q.put((rank, "err", traceback.format_exc()))


def run_distributed(fn, world_size, *args, timeout=300):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world_size, port, fn, args, q)) for r in range(world_size)]
    for p in procs:
        p.start()
    results, errs = {}, []
    try:
        for _ in range(world_size):
            rank, status, payload = q.get(timeout=timeout)
            if status == "ok":
                results[rank] = payload
            else:
                errs.append((rank, payload))
                break
    finally:
        for p in procs:
            p.join(timeout=5 if errs else 30)
            if p.is_alive():
                p.terminate()
    if errs:
        raise RuntimeError(f"rank {errs[0][0]} failed:\n{errs[0][1]}")
    return [results[r] for r in range(world_size)]
