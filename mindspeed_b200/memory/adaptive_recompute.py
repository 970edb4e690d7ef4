"""Adaptive selective recompute: measure every candidate module, then recompute the cheapest set that fits the budget.

  profile    for the first ``profiling_steps`` steps each candidate module (by default every transformer layer and its
             attention / MLP children) is timed with events and the bytes it saves for backward are counted with
             saved-tensor hooks;
  solve      0/1 knapsack: choose the modules to recompute so that the saved-activation bytes drop below the budget
             at minimum extra forward time.  A parent and its children are alternatives (a recomputed parent already
             covers its children), handled by solving per top-level group over its "cut" options;
  apply      chosen modules run under activation checkpointing from then on.

Budget = ``--adaptive-recompute-device-size`` (MiB of device memory the job may use) minus the static footprint
(parameters, gradients, optimizer state) measured at the end of profiling.

``--adaptive-recompute-device-swap`` (``swap_while_profiling``): the profiling steps themselves must not run out of
memory, so while profiling every large activation saved for backward is parked in pinned host memory and fetched back
when backward needs it (``memory/host_offload.OffloadSaved``); the byte counts are unchanged by that.  Without an explicit
device size the budget is then ``auto_budget_fraction`` of the device's memory.  After the decision the swap stops and the
chosen modules recompute.  (The reference reaches the same end from the other side: its allocator swaps tensors out when
an allocation fails during profiling and the swapped volume tells the solver how much to free.)
reference: mindspeed/core/memory/adaptive_recomputing/adaptive_recompute.py (profiling + hooks),
adaptive_recompute_solver.py (knapsack over the module tree).
"""
from __future__ import annotations

import dataclasses
import time
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..parallel.random import checkpoint as _checkpoint


@dataclasses.dataclass
class ModuleProfile:
    name: str
    forward_time: float = 0.0        # seconds per call (mean)
    saved_bytes: int = 0             # bytes saved for backward inside the module (mean per call)
    input_bytes: int = 0             # what stays alive if the module is recomputed (its inputs)
    calls: int = 0
    parent: Optional[str] = None


def solve_recompute(profiles: Sequence[ModuleProfile], bytes_to_free: int, granularity: int = 1 << 20) -> List[str]:
    """Minimum-time set of modules to recompute that frees at least ``bytes_to_free``.

    Options per top-level group: recompute nothing, any subset of its children, or the whole group; across groups a
    knapsack (dynamic programme over freed bytes in units of ``granularity``)."""
    if bytes_to_free <= 0:
        return []
    by_parent: Dict[Optional[str], List[ModuleProfile]] = {}
    for p in profiles:
        by_parent.setdefault(p.parent, []).append(p)
    groups: List[List[Tuple[int, float, List[str]]]] = []     # per group: options (freed, cost, names)
    for top in by_parent.get(None, []):
        opts = [(0, 0.0, [])]
        gain = max(0, top.saved_bytes - top.input_bytes)
        opts.append((gain, top.forward_time, [top.name]))
        kids = by_parent.get(top.name, [])
        # subsets of children (children are few: attention, mlp, norms)
        for mask in range(1, 1 << min(len(kids), 6)):
            sel = [k for i, k in enumerate(kids[:6]) if mask >> i & 1]
            opts.append((sum(max(0, k.saved_bytes - k.input_bytes) for k in sel), sum(k.forward_time for k in sel),
                         [k.name for k in sel]))
        groups.append(opts)
    need = (bytes_to_free + granularity - 1) // granularity
    INF = float("inf")
    best = [INF] * (need + 1)
    best[0] = 0.0
    choice: List[List[Optional[int]]] = []
    for opts in groups:
        new = [INF] * (need + 1)
        pick: List[Optional[int]] = [None] * (need + 1)
        for have in range(need + 1):
            if best[have] == INF:
                continue
            for oi, (freed, cost, _) in enumerate(opts):
                tgt = min(need, have + freed // granularity)
                c = best[have] + cost
                if c < new[tgt]:
                    new[tgt] = c
                    pick[tgt] = (oi, have)
        choice.append(pick)
        best = new
    if best[need] == INF:
        # cannot free enough: recompute every top-level group (the most that can be done)
        return [o[1][2][0] for o in groups if len(o) > 1]
    names: List[str] = []
    at = need
    for gi in range(len(groups) - 1, -1, -1):
        oi, prev = choice[gi][at]
        names.extend(groups[gi][oi][2])
        at = prev
    return names


class _Ckpt(nn.Module):
    def __init__(self, inner):
        super().__init__()
        self.inner = inner
        self.enabled = True

    def forward(self, *args, **kw):
        if not self.enabled or not torch.is_grad_enabled() or kw or not any(isinstance(a, torch.Tensor) and a.requires_grad for a in args):
            return self.inner(*args, **kw)
        return _checkpoint(self.inner, False, *args)


class AdaptiveRecompute:
    def __init__(self, model: nn.Module, candidates: Optional[Sequence[str]] = None, profiling_steps: int = 2,
                 device_budget_bytes: Optional[int] = None, child_names: Sequence[str] = ("self_attention", "mlp"),
                 swap_while_profiling: bool = False, auto_budget_fraction: float = 0.9, swap_min_bytes: int = 1 << 20):
        self.model, self.profiling_steps, self.budget = model, profiling_steps, device_budget_bytes
        self.swap = None
        if swap_while_profiling:
            from .host_offload import OffloadSaved
            self.swap = OffloadSaved(min_bytes=swap_min_bytes)
            if self.budget is None and torch.cuda.is_available():
                total = torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory
                self.budget = int(auto_budget_fraction * total)
        self.swapped_bytes = 0                       # bytes parked on the host during profiling (all steps)
        self.step = 0
        self.profiles: Dict[str, ModuleProfile] = {}
        self.chosen: List[str] = []
        self._stack: List[Tuple[str, float, int]] = []
        self._saved_counter = 0
        self._handles = []
        names = list(candidates) if candidates is not None else self._default_candidates(model, child_names)
        mods = dict(model.named_modules())
        for n in names:
            parent = None
            for other in names:
                if other != n and n.startswith(other + "."):
                    parent = other if parent is None or len(other) > len(parent) else parent
            self.profiles[n] = ModuleProfile(n, parent=parent)
            self._handles.append(mods[n].register_forward_pre_hook(self._pre(n)))
            self._handles.append(mods[n].register_forward_hook(self._post(n)))
        self._hooks_ctx = None

    @staticmethod
    def _default_candidates(model, child_names):
        out = []
        for name, mod in model.named_modules():
            if type(mod).__name__ == "TransformerLayer":
                out.append(name)
                for c in child_names:
                    if hasattr(mod, c):
                        out.append(f"{name}.{c}")
        return out

    # -- profiling ------------------------------------------------------------------------------------------------
    def _pre(self, name):
        def hook(mod, args):
            if self.step >= self.profiling_steps or not torch.is_grad_enabled():
                return
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            inb = sum(a.numel() * a.element_size() for a in args if isinstance(a, torch.Tensor))
            self._stack.append((name, time.perf_counter(), self._saved_counter, inb))
        return hook

    def _post(self, name):
        def hook(mod, args, out):
            if self.step >= self.profiling_steps or not self._stack or self._stack[-1][0] != name:
                return
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            _, t0, saved0, inb = self._stack.pop()
            p = self.profiles[name]
            p.calls += 1
            k = p.calls
            p.forward_time += ((time.perf_counter() - t0) - p.forward_time) / k
            p.saved_bytes += int(((self._saved_counter - saved0) - p.saved_bytes) / k)
            p.input_bytes += int((inb - p.input_bytes) / k)
        return hook

    def step_context(self):
        """Wrap the forward pass of a step; counts saved bytes while profiling, no-op afterwards."""
        mgr = self

        class _Ctx:
            def __enter__(self_inner):
                if mgr.step < mgr.profiling_steps:
                    def pack(t):
                        mgr._saved_counter += t.numel() * t.element_size()
                        if mgr.swap is None:
                            return t
                        out = mgr.swap._pack(t)
                        if out is not t:
                            mgr.swapped_bytes += t.numel() * t.element_size()
                        return out
                    unpack = (lambda t: t) if mgr.swap is None else mgr.swap._unpack
                    mgr._hooks_ctx = torch.autograd.graph.saved_tensors_hooks(pack, unpack)
                    mgr._hooks_ctx.__enter__()
                return self_inner

            def __exit__(self_inner, *exc):
                if mgr._hooks_ctx is not None:
                    mgr._hooks_ctx.__exit__(*exc)
                    mgr._hooks_ctx = None
                return False
        return _Ctx()

    def end_step(self, static_bytes: Optional[int] = None):
        self.step += 1
        if self.step == self.profiling_steps:
            self._decide(static_bytes)

    def _decide(self, static_bytes):
        for h in self._handles:
            h.remove()
        self._handles = []
        total_saved = sum(p.saved_bytes for p in self.profiles.values() if p.parent is None)
        if self.budget is None:
            return
        if static_bytes is None:
            static_bytes = torch.cuda.memory_allocated() if torch.cuda.is_available() else 0
        to_free = static_bytes + total_saved - self.budget
        self.chosen = solve_recompute(list(self.profiles.values()), to_free)
        self.apply(self.chosen)

    def apply(self, names: Sequence[str]):
        for n in names:
            parent = self.model
            parts = n.split(".")
            for p in parts[:-1]:
                parent = getattr(parent, p)
            cur = getattr(parent, parts[-1])
            if not isinstance(cur, _Ckpt):
                setattr(parent, parts[-1], _Ckpt(cur))
