"""Checkpoint save / load in the ``torch_dist`` layout (and the legacy single-file ``torch`` layout).

Directory layout (Megatron compatible):
    <save>/latest_checkpointed_iteration.txt
    <save>/iter_0000010/.metadata, __<rank>_<n>.distcp      sharded tensors (model + optimizer)
    <save>/iter_0000010/common.pt                            everything that is not a sharded tensor
EMA weights are stored as extra ``ema.*`` optimizer-state keys (reference: mindspeed/checkpointing.py:43-153,322-410).
Device-to-host staging is synchronous (the reference forces the same: core/megatron_basic/megatron_basic.py:135-156);
``--async-save`` hands the file writing to a background thread after staging.
"""
from __future__ import annotations

import os
import threading
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..parallel import parallel_state as ps
from .sharded import ShardedTensor, model_sharded_state_dict, optimizer_sharded_state_dict

_ASYNC: List[threading.Thread] = []


def get_checkpoint_name(root, iteration):
    return os.path.join(root, f"iter_{iteration:07d}")


def _save_sharded(sts: Dict[str, ShardedTensor], path: str):
    """Write the chunks this rank owns (replica 0) and a merged ``.metadata``.

    File format: one ``__<rank>_0.distcp`` per rank holding {key: [(offset, tensor), ...]} and a ``.metadata`` index
    {key: {"shape", "dtype", "chunks": [(rank, offset, sizes)]}} merged on rank 0."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    mine, index = {}, {}
    for k, st in sts.items():
        if st.replica_id != 0:
            continue
        t = st.data.detach().cpu().contiguous()
        mine.setdefault(k, []).append((tuple(st.global_offset), t))
        index.setdefault(k, {"shape": tuple(st.global_shape), "dtype": str(t.dtype), "chunks": []})["chunks"].append(
            (rank, tuple(st.global_offset), tuple(t.shape)))
    os.makedirs(path, exist_ok=True)
    torch.save(mine, os.path.join(path, f"__{rank}_0.distcp"))
    gathered = [None] * world
    if world > 1:
        dist.all_gather_object(gathered, index)
    else:
        gathered = [index]
    if rank == 0:
        merged = {}
        for idx in gathered:
            for k, v in idx.items():
                m = merged.setdefault(k, {"shape": v["shape"], "dtype": v["dtype"], "chunks": []})
                if tuple(m["shape"]) != tuple(v["shape"]):
                    raise RuntimeError(f"checkpoint key {k} has inconsistent global shapes {m['shape']} vs {v['shape']}")
                m["chunks"].extend(v["chunks"])
        with open(os.path.join(path, ".metadata"), "wb") as f:
            torch.save(merged, f)


def _load_sharded(sts: Dict[str, ShardedTensor], path: str, strict: bool = True):
    """Fill every local shard from whichever saved chunks overlap it (works across layouts)."""
    with open(os.path.join(path, ".metadata"), "rb") as f:
        meta = torch.load(f, weights_only=False)
    cache = {}

    def rank_file(r):
        if r not in cache:
            cache[r] = torch.load(os.path.join(path, f"__{r}_0.distcp"), weights_only=False)
        return cache[r]

    missing = []
    for k, st in sts.items():
        if k not in meta:
            missing.append(k)
            continue
        m = meta[k]
        if tuple(m["shape"]) != tuple(st.global_shape):
            raise RuntimeError(f"{k}: checkpoint global shape {m['shape']} != expected {st.global_shape}")
        dst = st.data
        lo = st.global_offset
        hi = tuple(o + s for o, s in zip(lo, dst.shape))
        covered = 0
        for (r, off, sizes) in m["chunks"]:
            c_hi = tuple(o + s for o, s in zip(off, sizes))
            i_lo = tuple(max(a, b) for a, b in zip(lo, off))
            i_hi = tuple(min(a, b) for a, b in zip(hi, c_hi))
            if any(a >= b for a, b in zip(i_lo, i_hi)):
                continue
            src = None
            for (o2, t) in rank_file(r)[k]:
                if tuple(o2) == tuple(off):
                    src = t
            d_sl = tuple(slice(a - o, b - o) for a, b, o in zip(i_lo, i_hi, lo))
            s_sl = tuple(slice(a - o, b - o) for a, b, o in zip(i_lo, i_hi, off))
            with torch.no_grad():
                dst[d_sl].copy_(src[s_sl].to(dst.dtype))
            n = 1
            for a, b in zip(i_lo, i_hi):
                n *= (b - a)
            covered += n
        if covered < dst.numel() and strict:
            raise RuntimeError(f"{k}: checkpoint covers {covered} of {dst.numel()} elements of the local shard")
    if missing and strict:
        raise KeyError(f"keys missing from checkpoint: {missing[:5]} ...")
    return missing


def generate_state_dict(model, optimizer, opt_param_scheduler, iteration, args=None, rng=True):
    sharded: Dict[str, ShardedTensor] = {}
    for i, chunk in enumerate(model):
        pfx = "model." if len(model) == 1 else f"model{i}."
        sharded.update(model_sharded_state_dict(chunk, pfx))
    common = {"iteration": iteration, "checkpoint_version": 3.0}
    if args is not None:
        common["args"] = {k: v for k, v in vars(args).items() if isinstance(v, (int, float, str, bool, list, tuple, type(None)))}
    if optimizer is not None and hasattr(optimizer, "sharded_state_dict"):
        sharded.update(optimizer.sharded_state_dict())
        common["optimizer"] = {"step": optimizer.step_count, "param_groups": [dict(g) for g in optimizer.param_groups]}
    if opt_param_scheduler is not None:
        common["opt_param_scheduler"] = opt_param_scheduler.state_dict()
    if rng:
        from ..parallel.random import get_cuda_rng_tracker
        common["rng_state"] = {"torch": torch.get_rng_state(), "tracker": get_cuda_rng_tracker().get_states(),
                               "cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None}
    return sharded, common


def save_checkpoint(iteration, model, optimizer, opt_param_scheduler, args=None, save_dir=None, async_save=None):
    from ..training.global_vars import get_args
    if args is None:
        try:
            args = get_args()
        except RuntimeError:
            args = None
    save_dir = save_dir or args.save
    async_save = bool(getattr(args, "async_save", False)) if async_save is None else async_save
    path = get_checkpoint_name(save_dir, iteration)
    sharded, common = generate_state_dict(model, optimizer if not getattr(args, "no_save_optim", False) else None,
                                          opt_param_scheduler, iteration, args, rng=not getattr(args, "no_save_rng", False))
    rank = dist.get_rank() if dist.is_initialized() else 0
    os.makedirs(path, exist_ok=True)
    _save_sharded(sharded, path)                       # staging + write of this rank's file
    # rng state differs per rank: every rank keeps its own copy next to the shared common file
    torch.save({"rng_state": common.pop("rng_state", None)}, os.path.join(path, f"rng_{rank}.pt"))
    if rank == 0:
        torch.save(common, os.path.join(path, "common.pt"))
    if dist.is_initialized():
        dist.barrier()
    if rank == 0:
        with open(os.path.join(save_dir, "latest_checkpointed_iteration.txt"), "w") as f:
            f.write(str(iteration))
    if dist.is_initialized():
        dist.barrier()
    return path


def read_latest_iteration(load_dir) -> Optional[int]:
    p = os.path.join(load_dir, "latest_checkpointed_iteration.txt")
    if not os.path.exists(p):
        return None
    with open(p) as f:
        return int(f.read().strip())


def load_checkpoint(model, optimizer, opt_param_scheduler, load_dir=None, args=None, strict=True, iteration=None):
    from ..training.global_vars import get_args
    if args is None:
        try:
            args = get_args()
        except RuntimeError:
            args = None
    load_dir = load_dir or args.load
    it = iteration if iteration is not None else read_latest_iteration(load_dir)
    if it is None:
        return 0
    path = get_checkpoint_name(load_dir, it)
    load_optim = optimizer is not None and not getattr(args, "no_load_optim", False)
    sharded, _ = generate_state_dict(model, optimizer if load_optim else None, None, it, None, rng=False)
    _load_sharded(sharded, path, strict=strict)
    common = torch.load(os.path.join(path, "common.pt"), weights_only=False)
    if load_optim and "optimizer" in common:
        optimizer.step_count = common["optimizer"]["step"]
        for g, s in zip(optimizer.param_groups, common["optimizer"]["param_groups"]):
            g.update(s)
        # fp32 params update in place; bf16 models keep their master copy in the optimizer (already loaded)
        if hasattr(optimizer, "sharded") and optimizer.sharded:
            for chunk in model:
                if hasattr(chunk, "start_param_sync"):
                    chunk.start_param_sync(force_sync=True)
    elif optimizer is not None and hasattr(optimizer, "reload_model_params"):
        optimizer.reload_model_params()
    if opt_param_scheduler is not None and "opt_param_scheduler" in common:
        opt_param_scheduler.load_state_dict(common["opt_param_scheduler"])
    rank = dist.get_rank() if dist.is_initialized() else 0
    rp = os.path.join(path, f"rng_{rank}.pt")
    if os.path.exists(rp) and not getattr(args, "no_load_rng", False):
        rs = torch.load(rp, weights_only=False).get("rng_state")
        if rs is not None:
            from ..parallel.random import get_cuda_rng_tracker
            torch.set_rng_state(rs["torch"])
            get_cuda_rng_tracker().set_states(rs["tracker"])
            if rs.get("cuda") is not None and torch.cuda.is_available():
                torch.cuda.set_rng_state(rs["cuda"])
    return common.get("iteration", it)
