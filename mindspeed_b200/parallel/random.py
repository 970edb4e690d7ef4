"""RNG state tracking and activation checkpointing for tensor parallelism.

* ``CudaRNGStatesTracker`` keeps named generator states so that dropout inside a
  tensor-parallel region uses a per-rank seed while everything else uses the
  data-parallel seed (Megatron-core ``tensor_parallel.random``).  Works on CPU
  (the default generator is forked) so the gloo tests cover it.
* ``checkpoint`` re-runs the forward in backward under the saved RNG states.
* ``CheckpointWithoutOutput`` is "recompute without keeping the output": the output's
  storage is released once its consumer has run and is re-materialised by a hook
  right before the consumer's backward (reference: mindspeed/core/tensor_parallel/random.py:94-193
  and mindspeed/core/memory/recompute/recompute_common.py:9-105).
"""
from __future__ import annotations

import contextlib
from typing import Dict

import torch

from . import parallel_state as ps

_MODEL_PARALLEL_RNG_TRACKER_NAME = "model-parallel-rng"
_EXPERT_PARALLEL_RNG_TRACKER_NAME = "expert-parallel-rng"
_DATA_PARALLEL_RNG_TRACKER_NAME = "data-parallel-rng"


def _get_state(cuda: bool):
    return torch.cuda.get_rng_state() if cuda else torch.get_rng_state()


def _set_state(state, cuda: bool):
    if cuda:
        torch.cuda.set_rng_state(state)
    else:
        torch.set_rng_state(state)


def _set_cuda_rng_state(new_state, device=-1, graph_safe=False):
    torch.cuda.set_rng_state(new_state) if torch.cuda.is_available() else torch.set_rng_state(new_state)


class CudaRNGStatesTracker:
    def __init__(self):
        self.reset()

    def is_initialized(self):
        return self._is_initialized

    def reset(self):
        self._is_initialized = False
        self.states_: Dict[str, torch.Tensor] = {}
        self.seeds_ = set()

    def get_states(self):
        return dict(self.states_)

    def set_states(self, states):
        self._is_initialized = True
        self.states_ = states

    def add(self, name, seed):
        self._is_initialized = True
        if seed in self.seeds_:
            raise RuntimeError(f"seed {seed} already exists")
        if name in self.states_:
            raise RuntimeError(f"rng state {name} already exists")
        self.seeds_.add(seed)
        cuda = torch.cuda.is_available()
        orig = _get_state(cuda)
        (torch.cuda.manual_seed if cuda else torch.manual_seed)(seed)
        self.states_[name] = _get_state(cuda)
        _set_state(orig, cuda)

    @contextlib.contextmanager
    def fork(self, name=_MODEL_PARALLEL_RNG_TRACKER_NAME):
        if name not in self.states_:
            raise RuntimeError(f"rng state {name} is not added")
        cuda = torch.cuda.is_available()
        orig = _get_state(cuda)
        _set_state(self.states_[name], cuda)
        try:
            yield
        finally:
            self.states_[name] = _get_state(cuda)
            _set_state(orig, cuda)


_TRACKER = CudaRNGStatesTracker()


def get_cuda_rng_tracker(use_te_rng_tracker=False, inference_rng_tracker=False):
    return _TRACKER


def get_expert_parallel_rng_tracker_name():
    return _EXPERT_PARALLEL_RNG_TRACKER_NAME


def get_data_parallel_rng_tracker_name():
    return _DATA_PARALLEL_RNG_TRACKER_NAME


def model_parallel_cuda_manual_seed(seed, te_rng_tracker=False, inference_rng_tracker=False):
    """default state: same across a tensor-parallel group; tracker state: differs per tp rank."""
    offset = seed + 2718
    tp_seed = offset + ps.get_tensor_model_parallel_rank()
    _TRACKER.reset()
    (torch.cuda.manual_seed if torch.cuda.is_available() else torch.manual_seed)(seed)
    _TRACKER.add(_DATA_PARALLEL_RNG_TRACKER_NAME, seed + 1)
    _TRACKER.add(_MODEL_PARALLEL_RNG_TRACKER_NAME, tp_seed)
    ep_seed = seed + 1024 + 100 * ps.get_expert_model_parallel_rank() + ps.get_expert_tensor_parallel_rank()
    _TRACKER.add(_EXPERT_PARALLEL_RNG_TRACKER_NAME, ep_seed)


class _CheckpointFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run_function, distribute_saved_activations, *args):
        ctx.run_function = run_function
        cuda = torch.cuda.is_available()
        ctx.cuda = cuda
        ctx.cpu_state = torch.get_rng_state()
        ctx.cuda_state = torch.cuda.get_rng_state() if cuda else None
        ctx.tracker_states = get_cuda_rng_tracker().get_states()
        with torch.no_grad():
            outputs = run_function(*args)
        ctx.tensor_idx = [i for i, a in enumerate(args) if torch.is_tensor(a)]
        ctx.others = [None if torch.is_tensor(a) else a for a in args]
        ctx.save_for_backward(*[args[i] for i in ctx.tensor_idx])
        return outputs

    @staticmethod
    def backward(ctx, *grads):
        args = list(ctx.others)
        for i, t in zip(ctx.tensor_idx, ctx.saved_tensors):
            args[i] = t
        bwd_cpu = torch.get_rng_state()
        bwd_cuda = torch.cuda.get_rng_state() if ctx.cuda else None
        bwd_tracker = get_cuda_rng_tracker().get_states()
        torch.set_rng_state(ctx.cpu_state)
        if ctx.cuda:
            torch.cuda.set_rng_state(ctx.cuda_state)
        get_cuda_rng_tracker().set_states(ctx.tracker_states)
        detached = [a.detach().requires_grad_(a.requires_grad) if torch.is_tensor(a) else a for a in args]
        with torch.enable_grad():
            outputs = ctx.run_function(*detached)
        torch.set_rng_state(bwd_cpu)
        if ctx.cuda:
            torch.cuda.set_rng_state(bwd_cuda)
        get_cuda_rng_tracker().set_states(bwd_tracker)
        if torch.is_tensor(outputs):
            outputs = (outputs,)
        pairs = [(o, g) for o, g in zip(outputs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([p[0] for p in pairs], [p[1] for p in pairs])
        in_grads = tuple(a.grad if torch.is_tensor(a) else None for a in detached)
        return (None, None) + in_grads


def checkpoint(function, distribute_saved_activations, *args):
    """Recompute ``function(*args)`` in backward instead of saving its intermediates."""
    return _CheckpointFn.apply(function, distribute_saved_activations, *args)


class CheckpointWithoutOutput:
    """Run ``fn`` without saving intermediates *and* drop its output after the consumer ran.

    usage:
        ckpt = CheckpointWithoutOutput()
        y = ckpt.checkpoint(fn, False, x)       # y is a normal tensor for the consumer
        z = consumer(y)
        ckpt.discard_output()                   # frees y's storage
        z.register_hook(ckpt.recompute)         # re-materialises y before consumer's backward
    """

    def __init__(self):
        self.run_function = None
        self.ctx = None
        self.outputs = None
        self.cuda = torch.cuda.is_available()

    def checkpoint(self, run_function, distribute_saved_activations, *args):
        self.run_function = run_function
        self.cpu_state = torch.get_rng_state()
        self.cuda_state = torch.cuda.get_rng_state() if self.cuda else None
        self.tracker_states = get_cuda_rng_tracker().get_states()
        out = _NoOutputFn.apply(self, *args)
        self.outputs = out if isinstance(out, tuple) else (out,)
        return out

    def discard_output(self):
        for o in self.outputs:
            o.untyped_storage().resize_(0)

    def recompute(self, _grad=None):
        if self.ctx is None:
            return
        args = self.ctx.saved_tensors
        cpu, cu, tr = torch.get_rng_state(), (torch.cuda.get_rng_state() if self.cuda else None), \
            get_cuda_rng_tracker().get_states()
        torch.set_rng_state(self.cpu_state)
        if self.cuda:
            torch.cuda.set_rng_state(self.cuda_state)
        get_cuda_rng_tracker().set_states(self.tracker_states)
        detached = [a.detach().requires_grad_(r) for a, r in zip(args, self.ctx.req)]
        with torch.enable_grad():
            outs = self.run_function(*detached)
        torch.set_rng_state(cpu)
        if self.cuda:
            torch.cuda.set_rng_state(cu)
        get_cuda_rng_tracker().set_states(tr)
        outs = outs if isinstance(outs, tuple) else (outs,)
        for old, new in zip(self.outputs, outs):
            n = new.untyped_storage().size()
            old.untyped_storage().resize_(n)
            with torch.no_grad():
                old.untyped_storage().copy_(new.untyped_storage())
        self.ctx.recomputed = (detached, outs)
        self.ctx = None
        self.outputs = None
        self.run_function = None


class _NoOutputFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, owner, *args):
        with torch.no_grad():
            out = owner.run_function(*args)
        ctx.save_for_backward(*[a.detach() if torch.is_tensor(a) else a for a in args])
        ctx.req = [a.requires_grad for a in args]
        ctx.recomputed = None
        owner.ctx = ctx
        return out

    @staticmethod
    def backward(ctx, *grads):
        if ctx.recomputed is None:
            raise RuntimeError("CheckpointWithoutOutput.recompute was not called before backward")
        detached, outs = ctx.recomputed
        for d, r in zip(detached, ctx.req):
            d.requires_grad_(r)
        pairs = [(o, g) for o, g in zip(outs, grads) if o.requires_grad and g is not None]
        torch.autograd.backward([p[0] for p in pairs], [p[1] for p in pairs])
        res = tuple(d.grad for d in detached)
        ctx.recomputed = None
        return (None,) + res
