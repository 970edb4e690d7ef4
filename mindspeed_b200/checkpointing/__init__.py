"""Checkpoint save / load in the ``torch_dist`` format (and resume / reshard on load).

Directory layout (the one Megatron's ``torch_dist`` strategy writes):
    <save>/latest_checkpointed_iteration.txt
    <save>/iter_0000010/.metadata, __<rank>_<n>.distcp      torch.distributed.checkpoint files: sharded tensors
    <save>/iter_0000010/common.pt                            everything that is not a sharded tensor
    <save>/iter_0000010/rng_<rank>.pt                        per-rank RNG state
The ``.distcp`` / ``.metadata`` files are written and read through ``torch.distributed.checkpoint`` (FileSystemWriter /
FileSystemReader) with planners that take this package's chunk descriptions (key, global shape, offset of the local
chunk) directly, so any tool that reads DCP checkpoints can open them, and loading re-reads whichever saved chunks overlap
the new local shards under a different tensor / pipeline / data-parallel layout.  Model keys follow Megatron-core's
convention: no chunk prefix, and the per-layer tensors of ``decoder.layers`` stacked along a leading layer axis
(``decoder.layers.self_attention.linear_qkv.weight`` of shape [num_layers, ...]).  Optimizer state is keyed
``optimizer.state.{exp_avg,exp_avg_sq,fp32_param,...}.<param key>`` with this package's own chunking (one row per
tensor-parallel rank over the flattened local parameter), which Megatron's optimizer does not read.
EMA weights are stored as extra ``ema`` optimizer-state keys (reference: mindspeed/checkpointing.py:43-153,322-410).
Device-to-host staging is synchronous (the reference forces the same: core/megatron_basic/megatron_basic.py:135-156);
``--async-save`` then hands planning and file writing to a background thread that talks over its own gloo group, and the
training loop calls ``finalize_async_save`` before the next save and at exit.
"""
from __future__ import annotations

import os
import threading
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
from torch.distributed.checkpoint import FileSystemReader, FileSystemWriter
from torch.distributed.checkpoint.default_planner import DefaultLoadPlanner, DefaultSavePlanner
from torch.distributed.checkpoint.metadata import ChunkStorageMetadata, MetadataIndex, TensorProperties
from torch.distributed.checkpoint.planner import LoadPlan, SavePlan, TensorWriteData, WriteItem, WriteItemType
from torch.distributed.checkpoint.planner_helpers import create_read_items_for_chunk_list

from ..parallel import parallel_state as ps
from .sharded import ShardedTensor, model_sharded_state_dict, optimizer_sharded_state_dict

_ASYNC: List[threading.Thread] = []
_ASYNC_ERR: List[BaseException] = []
_CKPT_GROUP = {"group": None}


def get_checkpoint_name(root, iteration):
    return os.path.join(root, f"iter_{iteration:07d}")


class _ChunkSavePlanner(DefaultSavePlanner):
    """Plans one SHARD write item per local chunk whose ``replica_id`` is 0; the default global planning then merges all
    ranks' items into the checkpoint metadata (one tensor entry per key with the list of its chunks)."""

    def __init__(self, shards: Dict[str, ShardedTensor]):
        super().__init__(flatten_state_dict=False, flatten_sharded_tensors=False)
        # several local chunks may share a key (the layers of a stacked tensor): index by (key, offset)
        self.shards = {(st.key, tuple(st.global_offset)): st for st in shards.values() if st.replica_id == 0}

    def set_up_planner(self, state_dict, storage_meta=None, is_coordinator=False):
        super().set_up_planner({}, storage_meta, is_coordinator)

    def create_local_plan(self) -> SavePlan:
        items = []
        for (key, _), st in self.shards.items():
            t = st.data
            items.append(WriteItem(index=MetadataIndex(key, torch.Size(st.global_offset)), type=WriteItemType.SHARD,
                                   tensor_data=TensorWriteData(
                                       chunk=ChunkStorageMetadata(offsets=torch.Size(st.global_offset), sizes=t.size()),
                                       properties=TensorProperties.create_from_tensor(t), size=torch.Size(st.global_shape))))
        self.plan = SavePlan(items)
        return self.plan

    def lookup_object(self, index: MetadataIndex):
        return self.shards[(index.fqn, tuple(index.offset))].data


class _ChunkLoadPlanner(DefaultLoadPlanner):
    """Reads, for every local chunk, whichever saved chunks overlap it (any saved layout)."""

    def __init__(self, shards: Dict[str, ShardedTensor], strict: bool):
        super().__init__(flatten_state_dict=False, flatten_sharded_tensors=False, allow_partial_load=not strict)
        self.shards = {(st.key, tuple(st.global_offset)): st for st in shards.values()}
        self.strict, self.missing = strict, []

    def set_up_planner(self, state_dict, metadata=None, is_coordinator=False):
        super().set_up_planner({}, metadata, is_coordinator)

    def create_local_plan(self) -> LoadPlan:
        reqs = []
        for (key, _), st in self.shards.items():
            md = self.metadata.state_dict_metadata.get(key)
            if md is None:
                self.missing.append(key)
                continue
            if tuple(md.size) != tuple(st.global_shape):
                raise RuntimeError(f"{key}: checkpoint global shape {tuple(md.size)} != expected {tuple(st.global_shape)}")
            chunk = ChunkStorageMetadata(offsets=torch.Size(st.global_offset), sizes=st.data.size())
            items = create_read_items_for_chunk_list(key, md, [chunk])
            covered = 0
            for it in items:
                n = 1
                for l in it.lengths:
                    n *= int(l)
                covered += n
            if covered < st.data.numel() and self.strict:
                raise RuntimeError(f"{key}: checkpoint covers {covered} of {st.data.numel()} elements of the local shard")
            reqs += items
        if self.missing and self.strict:
            raise KeyError(f"keys missing from checkpoint: {self.missing[:5]} ...")
        return LoadPlan(reqs)

    def lookup_tensor(self, index: MetadataIndex) -> torch.Tensor:
        return self.shards[(index.fqn, tuple(index.offset))].data

    def commit_tensor(self, read_item, tensor) -> None:
        pass


def _use_dist() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def _ckpt_group():
    """A gloo group of all ranks used only by checkpoint threads, so their collectives never interleave with training's."""
    if _CKPT_GROUP["group"] is None:
        _CKPT_GROUP["group"] = dist.new_group(backend="gloo")
    return _CKPT_GROUP["group"]


def _stage(sts: Dict[str, ShardedTensor]) -> Dict[str, ShardedTensor]:
    """Host copies of the chunks this rank writes (replica 0): after this the training step may overwrite the originals."""
    out = {}
    for k, st in sts.items():
        if st.replica_id != 0:
            continue
        t = st.data.detach()
        t = t.cpu().clone() if not t.is_cuda else t.to("cpu", copy=True)
        out[k] = ShardedTensor(st.key, t.contiguous(), st.global_shape, st.global_offset, 0)
    return out


def _save_sharded(sts: Dict[str, ShardedTensor], path: str, group=None):
    os.makedirs(path, exist_ok=True)
    use = _use_dist()
    dcp.save({}, storage_writer=FileSystemWriter(path, single_file_per_rank=True), planner=_ChunkSavePlanner(sts),
             process_group=group if use else None, no_dist=not use)


def _load_sharded(sts: Dict[str, ShardedTensor], path: str, strict: bool = True):
    """Fill every local shard from whichever saved chunks overlap it (works across layouts).  Every rank reads on its own:
    no collective is involved, so ranks may ask for different keys."""
    planner = _ChunkLoadPlanner(sts, strict)
    dcp.load({}, storage_reader=FileSystemReader(path), planner=planner, no_dist=True)
    return planner.missing


def finalize_async_save(blocking: bool = True):
    """Wait for background checkpoint writes (all of them when ``blocking``, else only finished ones are reaped) and
    re-raise an error that happened in one."""
    for t in list(_ASYNC):
        if blocking or not t.is_alive():
            t.join()
            _ASYNC.remove(t)
    if _ASYNC_ERR:
        raise RuntimeError("asynchronous checkpoint save failed") from _ASYNC_ERR.pop(0)


def generate_state_dict(model, optimizer, opt_param_scheduler, iteration, args=None, rng=True):
    sharded: Dict[str, ShardedTensor] = {}
    from ..parallel.distributed.fsdp import FullyShardedDataParallel
    for chunk in model:      # keys carry global layer numbers, so chunks of one model never collide
        if isinstance(chunk, FullyShardedDataParallel):
            sharded.update(chunk.sharded_state_dict(""))       # flat per-parameter pieces of the rank's shard
        else:
            sharded.update(model_sharded_state_dict(chunk, ""))
    common = {"iteration": iteration, "checkpoint_version": 3.0}
    if args is not None:
        common["args"] = {k: v for k, v in vars(args).items() if isinstance(v, (int, float, str, bool, list, tuple, type(None)))}
    if optimizer is not None and hasattr(optimizer, "sharded_state_dict"):
        sharded.update(optimizer.sharded_state_dict())
        step = optimizer.step_count if hasattr(optimizer, "step_count") else optimizer.param_groups[0].get("step", 0)
        common["optimizer"] = {"step": step, "param_groups": [{k: v for k, v in g.items() if not torch.is_tensor(v)}
                                                              for g in optimizer.param_groups]}
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
    finalize_async_save(blocking=True)                 # at most one checkpoint in flight
    path = get_checkpoint_name(save_dir, iteration)
    sharded, common = generate_state_dict(model, optimizer if not getattr(args, "no_save_optim", False) else None,
                                          opt_param_scheduler, iteration, args, rng=not getattr(args, "no_save_rng", False))
    rank = dist.get_rank() if dist.is_initialized() else 0
    from ..parallel.distributed.fsdp import FullyShardedDataParallel as _FSDP
    if any(isinstance(c, _FSDP) for c in model):
        # the flat per-parameter tensors of a fully sharded model carry no shapes: keep them next to the checkpoint so that
        # checkpointing/convert_fsdp.py can rebuild the parameters without the model
        mine = {}
        for c in model:
            if isinstance(c, _FSDP):
                mine.update(c.layout(""))
        if _use_dist():
            parts = [None] * dist.get_world_size()
            dist.all_gather_object(parts, mine)
            mine = {k: v for part in parts for k, v in part.items()}
        common["fsdp_layout"] = mine
        inner = model[0].module
        common["num_layers"] = int(getattr(getattr(inner, "config", None), "num_layers", 0) or 0)
    os.makedirs(path, exist_ok=True)
    rng_state = {"rng_state": common.pop("rng_state", None)}

    def write(shards, group):
        _save_sharded(shards, path, group)
        # rng state differs per rank: every rank keeps its own copy next to the shared common file
        torch.save(rng_state, os.path.join(path, f"rng_{rank}.pt"))
        if rank == 0:
            torch.save(common, os.path.join(path, "common.pt"))
        if _use_dist():
            dist.barrier(group=group)
        if rank == 0:
            with open(os.path.join(save_dir, "latest_checkpointed_iteration.txt"), "w") as f:
                f.write(str(iteration))
        if _use_dist():
            dist.barrier(group=group)

    if not async_save:
        write(sharded, None)
        return path
    staged = _stage(sharded)                           # synchronous device-to-host copy; the step may now go on
    group = _ckpt_group() if _use_dist() else None

    def run():
        try:
            write(staged, group)
        except BaseException as e:   # surfaced by finalize_async_save
            _ASYNC_ERR.append(e)

    t = threading.Thread(target=run, name=f"ckpt-save-{iteration}", daemon=True)
    t.start()
    _ASYNC.append(t)
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
    for chunk in model:
        if hasattr(chunk, "post_load"):
            chunk.post_load()
    common = torch.load(os.path.join(path, "common.pt"), weights_only=False)
    if load_optim and "optimizer" in common:
        if hasattr(optimizer, "step_count"):
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
        # the schedule's shape (peak, warm-up, decay length) comes from this launch's flags; the checkpoint supplies the step
        # count, and with --use-checkpoint-opt_param-scheduler also the flags the schedule was saved with
        if getattr(args, "use_checkpoint_opt_param_scheduler", False) and "schedule" in common["opt_param_scheduler"]:
            for k, v in common["opt_param_scheduler"]["schedule"].items():
                setattr(opt_param_scheduler, k, v)
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


# ---------------------------------------------------------------------------------------------------------------------
# Fault dumps (TTP): collective-free, because some ranks are gone when a dump is requested.
# reference: mindspeed/core/training.py dump hooks of the TTP feature (mindspeed/features_manager/high_availability/*).
# ---------------------------------------------------------------------------------------------------------------------
def save_fault_dump(iteration, model, optimizer, dump_dir, save_optimizer=True, save_rng=True, keep=1):
    """Every calling rank writes ALL its local shards (replicas included) to ``<dump_dir>/iter_<n>/rank_<r>/`` as a
    self-contained torch.distributed.checkpoint directory planned without collectives, then prunes older dumps so that at
    most ``keep`` remain.  The ranks of one complete replica together hold the whole state."""
    import shutil
    rank = dist.get_rank() if dist.is_initialized() else 0
    sharded, common = generate_state_dict(model, optimizer if save_optimizer else None, None, iteration, None, rng=save_rng)
    everything = {k: ShardedTensor(st.key, st.data, st.global_shape, st.global_offset, 0) for k, st in sharded.items()}
    path = os.path.join(get_checkpoint_name(dump_dir, iteration), f"rank_{rank}")
    os.makedirs(path, exist_ok=True)
    dcp.save({}, storage_writer=FileSystemWriter(path, single_file_per_rank=True), planner=_ChunkSavePlanner(everything), no_dist=True)
    torch.save(common, os.path.join(path, "common.pt"))
    with open(os.path.join(path, "complete"), "w") as f:
        f.write(str(iteration))
    dumps = sorted(d for d in os.listdir(dump_dir) if d.startswith("iter_"))
    for old in dumps[:-max(1, int(keep))]:
        if old != os.path.basename(get_checkpoint_name(dump_dir, iteration)):
            shutil.rmtree(os.path.join(dump_dir, old, f"rank_{rank}"), ignore_errors=True)
    return path


def wait_for_fault_dump(dump_dir, ranks, timeout_s=60.0, poll_s=0.5):
    """Block until the newest dump under ``dump_dir`` holds a ``complete`` marker of every rank in ``ranks`` (they write
    independently); returns its iteration directory, or None when the time runs out."""
    import time as _time
    t0 = _time.time()
    while _time.time() - t0 <= timeout_s:
        dumps = sorted(d for d in os.listdir(dump_dir) if d.startswith("iter_")) if os.path.isdir(dump_dir) else []
        if dumps:
            p = os.path.join(dump_dir, dumps[-1])
            if all(os.path.exists(os.path.join(p, f"rank_{r}", "complete")) for r in ranks):
                return p
        _time.sleep(poll_s)
    return None


def load_fault_dump(model, optimizer, dump_path, rank=None, strict=True):
    """Reload this rank's own shards from a dump written by ``save_fault_dump`` under the same parallel layout."""
    rank = (dist.get_rank() if dist.is_initialized() else 0) if rank is None else rank
    path = os.path.join(dump_path, f"rank_{rank}")
    sharded, _ = generate_state_dict(model, optimizer, None, 0, None, rng=False)
    _load_sharded(sharded, path, strict=strict)
    common = torch.load(os.path.join(path, "common.pt"), weights_only=False)
    if optimizer is not None and "optimizer" in common:
        optimizer.step_count = common["optimizer"]["step"]
    return common.get("iteration", 0)
