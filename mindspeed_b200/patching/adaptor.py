"""Entry point for scripts written against ``megatron.*``: make those names resolve to this framework.

``patch_features()`` registers, for every public piece of the Megatron-core surface this framework provides, a patch
that installs it under the Megatron name (creating the ``megatron`` package tree as dummy modules when no checkout
is importable), plus harmless stand-ins for optional third-party modules (apex, transformer_engine, flash_attn,
amp_C).  ``repatch(args)`` re-evaluates the feature set after arguments changed (RL frameworks construct arguments
after import).  Nothing here is needed by the framework's own entry points.
reference: mindspeed/megatron_adaptor.py:23-63 (patch_features, repatch, delete_lock_file).
"""
from __future__ import annotations

import glob
import os
from typing import Optional

from .patch_utils import PatchesManager

_STATE = {"patched": False, "args": None}


def _surface():
    """(megatron dotted name, object) pairs."""
    from .. import checkpointing
    from ..models.gpt_model import GPTModel
    from ..optimizer import get_megatron_optimizer
    from ..parallel import cross_entropy, layers, mappings, parallel_state, random
    from ..parallel.distributed import ddp as _ddp
    from ..parallel.pipeline import schedules
    from ..training import training as _training
    out = [
        ("megatron.core.parallel_state", parallel_state),
        ("megatron.core.mpu", parallel_state),
        ("megatron.core.tensor_parallel.layers", layers),
        ("megatron.core.tensor_parallel.mappings", mappings),
        ("megatron.core.tensor_parallel.random", random),
        ("megatron.core.tensor_parallel.cross_entropy", cross_entropy),
        ("megatron.core.pipeline_parallel.schedules", schedules),
        ("megatron.core.models.gpt.GPTModel", GPTModel),
        ("megatron.core.optimizer.get_megatron_optimizer", get_megatron_optimizer),
        ("megatron.core.distributed.DistributedDataParallel", _ddp.DistributedDataParallel),
        ("megatron.training.pretrain", _training.pretrain),
        ("megatron.training.training.train_step", _training.train_step),
        ("megatron.training.checkpointing.save_checkpoint", checkpointing.save_checkpoint),
        ("megatron.training.checkpointing.load_checkpoint", checkpointing.load_checkpoint),
    ]
    return out


def _optional_dependency_stubs():
    from .compat import optional_dependency_stubs
    return optional_dependency_stubs()


def delete_lock_file(directory: Optional[str] = None):
    """Remove stale build lock files a crashed JIT build may have left (no-op when none exist)."""
    directory = directory or os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc", "build")
    removed = []
    for f in glob.glob(os.path.join(directory, "*.lock")):
        try:
            os.remove(f)
            removed.append(f)
        except OSError:
            pass
    return removed


def patch_features(args=None):
    if _STATE["patched"]:
        return
    delete_lock_file()
    for name, obj in _surface():
        PatchesManager.register_patch(name, obj, force_patch=True, create_dummy=True)
    for name, obj in _optional_dependency_stubs():
        try:
            __import__(name.split(".")[0])
        except ImportError:
            PatchesManager.register_patch(name, obj, create_dummy=True)
    PatchesManager.apply_patches()
    _STATE["patched"], _STATE["args"] = True, args


def repatch(args):
    """Arguments changed after import: drop every patch and apply the set again for the new arguments."""
    PatchesManager.remove_patches()
    _STATE["patched"] = False
    patch_features(args)
