"""Smart swap: profile tensor lifetimes, search a swap policy, then execute it with asynchronous copies.

Three phases, as in the reference (docs/zh/features/smart_swap.md:13-17; mindspeed/core/memory/smart_swap/
{swap_engine,policy_generator,swap_arranger,swap_manager,hooks}.py over the native NPUSwapManager):

  WarmUp        ``LifetimeProfiler`` records, for every tensor saved for backward during a step, its size, the index
                of the operation that saved it (forward order) and of the operation that reads it back (backward
                order).  Out-of-memory during warm-up is absorbed by the allocator's pressure callback, which swaps
                the largest idle candidates out synchronously.
  SearchPolicy  ``PolicyGenerator`` ranks candidates by bytes x idle-interval, and picks the cheapest set whose removal
                brings the simulated peak under the budget, subject to the copy-bandwidth constraint: a tensor is only
                worth swapping if its D2H copy fits into the compute time between its save and the memory peak, and its
                H2D copy into the time between the peak and its use.
  Stable        ``SwapExecutor`` installs saved-tensor hooks that, for tensors matching the policy (by forward index and
                size), start the D2H copy on a side stream right after the save, free the device copy when the copy
                has finished, and prefetch it ``prefetch_distance`` backward operations before its use.

The unit of time in the profile is "operation index"; ``op_time`` (seconds per operation, measured) converts it.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple

import torch


@dataclasses.dataclass
class TensorLife:
    key: int                 # forward save index (identity of the tensor within a step)
    nbytes: int
    save_op: int             # forward operation index at which it was saved
    use_op: int = -1         # backward operation index (counted from the start of backward) at which it is read
    name: str = ""


class LifetimeProfiler:
    """saved_tensors_hooks-based recorder.  Use as a context manager around forward; backward reads are counted as the
    graph unpacks them."""

    def __init__(self, min_bytes: int = 1 << 20):
        self.min_bytes = min_bytes
        self.lives: List[TensorLife] = []
        self._fwd = 0
        self._bwd = 0
        self._hooks = None

    def __enter__(self):
        self.lives, self._fwd, self._bwd = [], 0, 0

        def pack(t):
            idx = self._fwd
            self._fwd += 1
            nbytes = t.numel() * t.element_size()
            if nbytes >= self.min_bytes and t.grad_fn is not None:
                self.lives.append(TensorLife(len(self.lives), nbytes, idx))
                return ("life", len(self.lives) - 1, t)
            return ("raw", -1, t)

        def unpack(p):
            kind, i, t = p
            if kind == "life":
                self.lives[i].use_op = self._bwd
            self._bwd += 1
            return t

        self._hooks = torch.autograd.graph.saved_tensors_hooks(pack, unpack)
        self._hooks.__enter__()
        return self

    def __exit__(self, *exc):
        self._hooks.__exit__(*exc)
        return False

    @property
    def num_forward_ops(self):
        return self._fwd

    @property
    def num_backward_ops(self):
        return self._bwd


@dataclasses.dataclass
class SwapPolicy:
    swap_keys: List[int]                       # TensorLife.key values to swap
    prefetch_distance: int = 4
    expected_peak: int = 0
    expected_saving: int = 0

    def matches(self, save_op: int, nbytes: int, table: Dict[int, int]) -> bool:
        return table.get(save_op) == nbytes


class PolicyGenerator:
    def __init__(self, lives: Sequence[TensorLife], num_forward_ops: int, num_backward_ops: int, static_bytes: int = 0,
                 op_time: float = 50e-6, d2h_gbs: float = 50.0, h2d_gbs: float = 50.0):
        self.lives = [l for l in lives if l.use_op >= 0]
        self.nf, self.nb = num_forward_ops, num_backward_ops
        self.static = static_bytes
        self.op_time, self.d2h, self.h2d = op_time, d2h_gbs * 1e9, h2d_gbs * 1e9

    def timeline(self, swapped: Sequence[int] = (), prefetch_distance: int = 4) -> List[int]:
        """Simulated saved-activation bytes at every point of [forward ops..., backward ops...]."""
        n = self.nf + self.nb
        delta = [0] * (n + 1)
        sw = set(swapped)
        for l in self.lives:
            start, end = l.save_op, self.nf + l.use_op + 1
            if l.key in sw:
                # on device from the save until its copy has drained, and again from the prefetch until its use
                out_ops = max(1, int(l.nbytes / self.d2h / self.op_time) + 1)
                in_ops = max(prefetch_distance, int(l.nbytes / self.h2d / self.op_time) + 1)
                off, back = min(end, start + out_ops), max(start + out_ops, end - in_ops)
                delta[start] += l.nbytes
                delta[off] -= l.nbytes
                delta[back] += l.nbytes
                delta[end] -= l.nbytes
            else:
                delta[start] += l.nbytes
                delta[end] -= l.nbytes
        out, cur = [], self.static
        for i in range(n):
            cur += delta[i]
            out.append(cur)
        return out

    def generate(self, budget_bytes: int, prefetch_distance: int = 4) -> SwapPolicy:
        base = self.timeline((), prefetch_distance)
        peak = max(base) if base else self.static
        if peak <= budget_bytes:
            return SwapPolicy([], prefetch_distance, peak, 0)
        peak_at = base.index(peak)

        def score(l: TensorLife) -> float:
            end = self.nf + l.use_op
            if not (l.save_op < peak_at <= end):
                return -1.0                                   # not alive at the peak: swapping it cannot lower it
            out_ok = (peak_at - l.save_op) * self.op_time >= l.nbytes / self.d2h
            in_ok = (end - peak_at) * self.op_time >= l.nbytes / self.h2d
            if not (out_ok and in_ok):
                return -1.0                                   # its copies would not hide: skip
            return l.nbytes * float(end - l.save_op)

        cands = sorted((l for l in self.lives if score(l) > 0), key=score, reverse=True)
        chosen: List[int] = []
        cur_peak = peak
        for l in cands:
            chosen.append(l.key)
            cur_peak = max(self.timeline(chosen, prefetch_distance))
            if cur_peak <= budget_bytes:
                break
        return SwapPolicy(chosen, prefetch_distance, cur_peak, peak - cur_peak)


class SwapExecutor:
    """Stable phase: apply a policy with saved-tensor hooks.  On CPU tensors the "swap" is a plain copy (so the logic
    is testable without a GPU); on CUDA tensors it is a pinned-memory copy on a side stream."""

    def __init__(self, policy: SwapPolicy, lives: Sequence[TensorLife]):
        self.policy = policy
        self.table = {l.save_op: l.nbytes for l in lives if l.key in set(policy.swap_keys)}
        self.stream = torch.cuda.Stream() if torch.cuda.is_available() else None
        self.bytes_swapped = 0
        self.n_swapped = 0
        self._fwd = 0
        self._hooks = None

    def __enter__(self):
        self._fwd = 0
        self.bytes_swapped = self.n_swapped = 0

        def pack(t):
            idx = self._fwd
            self._fwd += 1
            nbytes = t.numel() * t.element_size()
            if self.table.get(idx) != nbytes or t.grad_fn is None:
                return ("raw", t)
            self.bytes_swapped += nbytes
            self.n_swapped += 1
            if t.is_cuda:
                host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
                self.stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.stream):
                    host.copy_(t, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self.stream)
                t.record_stream(self.stream)
                return ("swapped", host, t.device, ev)
            return ("swapped", t.detach().clone(), t.device, None)

        def unpack(p):
            if p[0] == "raw":
                return p[1]
            _, host, dev, ev = p
            if dev.type == "cuda":
                with torch.cuda.stream(self.stream):
                    out = host.to(dev, non_blocking=True)
                torch.cuda.current_stream().wait_stream(self.stream)
                return out
            return host

        self._hooks = torch.autograd.graph.saved_tensors_hooks(pack, unpack)
        self._hooks.__enter__()
        return self

    def __exit__(self, *exc):
        self._hooks.__exit__(*exc)
        return False


class SmartSwapManager:
    """Drives the three phases over training steps: ``step_context()`` returns the context manager to wrap the
    forward pass of the current step in."""

    def __init__(self, budget_bytes: int, warmup_steps: int = 2, min_bytes: int = 1 << 20, static_bytes: int = 0,
                 op_time: float = 50e-6, d2h_gbs: float = 50.0, h2d_gbs: float = 50.0, prefetch_distance: int = 4):
        self.budget, self.warmup_steps = budget_bytes, warmup_steps
        self.kw = dict(static_bytes=static_bytes, op_time=op_time, d2h_gbs=d2h_gbs, h2d_gbs=h2d_gbs)
        self.min_bytes, self.prefetch_distance = min_bytes, prefetch_distance
        self.step = 0
        self.phase = "warmup"
        self.profiler: Optional[LifetimeProfiler] = None
        self.policy: Optional[SwapPolicy] = None
        self.executor: Optional[SwapExecutor] = None

    def step_context(self):
        if self.phase == "warmup":
            self.profiler = LifetimeProfiler(self.min_bytes)
            return self.profiler
        return self.executor

    def end_step(self):
        self.step += 1
        if self.phase == "warmup" and self.step >= self.warmup_steps:
            gen = PolicyGenerator(self.profiler.lives, self.profiler.num_forward_ops, self.profiler.num_backward_ops, **self.kw)
            self.policy = gen.generate(self.budget, self.prefetch_distance)
            self.executor = SwapExecutor(self.policy, self.profiler.lives)
            self.phase = "stable"
