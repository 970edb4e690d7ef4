"""Adaptive memory optimisation: per module, keep its activations, recompute them, or park them in host memory.

Extends adaptive selective recompute (``memory/adaptive_recompute.py``) with a third action.  After the profiling steps
every candidate module has a forward time, the bytes it saves for backward and the bytes of its inputs; the host link is
timed once (pinned copies in both directions).  Then

  recompute   frees  (saved - inputs) * in_flight        costs  one more forward of the module
  swap        frees   saved * in_flight                  costs  what of the two transfers cannot hide behind the module's own
                                                                forward and backward:  2 * max(0, bytes / bandwidth - forward_time)
                                                                plus a fixed latency per transfer
  keep        frees   nothing                            costs  nothing

and a knapsack over the layers (a layer and its children are alternatives, as in the recompute solver) picks the cheapest
set of actions that brings the step under the device budget.  ``in_flight`` is the number of micro-batches whose
activations a pipeline stage holds at once (1 without pipeline parallelism).  Chosen modules are wrapped: recompute through
activation checkpointing, swap through ``memory.host_offload.OffloadSaved`` around their forward.
reference: mindspeed/core/memory/adaptive_memory/{adaptive_memory_profiling,adaptive_memory_solver,adaptive_memory_policy,
adaptive_memory_swap_manager,adaptive_memory_apply}.py (profile -> policy combinations -> knapsack -> hooks).
"""
from __future__ import annotations

import dataclasses
import time
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from .adaptive_recompute import AdaptiveRecompute, ModuleProfile, _Ckpt

KEEP, RECOMPUTE, SWAP = "keep", "recompute", "swap"


@dataclasses.dataclass
class HostLink:
    bytes_per_s: float = 50e9           # one direction; measured by ``measure_host_link`` on a GPU
    latency_s: float = 20e-6            # per transfer


def measure_host_link(nbytes: int = 256 << 20, repeats: int = 3) -> HostLink:
    """Time pinned host <-> device copies of ``nbytes`` with CUDA events; the default link on a machine without a GPU."""
    if not torch.cuda.is_available():
        return HostLink()
    dev = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    host = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    best = float("inf")
    for src, dst in ((dev, host), (host, dev)):
        for _ in range(repeats):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            dst.copy_(src, non_blocking=True)
            b.record()
            b.synchronize()
            best = min(best, nbytes / (a.elapsed_time(b) * 1e-3))
    small = torch.empty(1024, dtype=torch.uint8, device="cuda")
    hs = torch.empty(1024, dtype=torch.uint8, pin_memory=True)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(10):
        hs.copy_(small, non_blocking=True)
    b.record()
    b.synchronize()
    return HostLink(bytes_per_s=best, latency_s=a.elapsed_time(b) * 1e-4)


def module_options(p: ModuleProfile, link: HostLink, in_flight: int = 1, allow_swap: bool = True) -> List[Tuple[int, float, str]]:
    """[(bytes freed, seconds added, action)] for one module."""
    opts = [(0, 0.0, KEEP)]
    gain = max(0, p.saved_bytes - p.input_bytes) * in_flight
    if gain > 0:
        opts.append((gain, p.forward_time, RECOMPUTE))
    if allow_swap and p.saved_bytes > 0:
        exposed = max(0.0, p.saved_bytes / link.bytes_per_s - p.forward_time) + link.latency_s
        opts.append((p.saved_bytes * in_flight, 2.0 * exposed, SWAP))
    return opts


def solve_memory_policy(profiles: Sequence[ModuleProfile], bytes_to_free: int, link: HostLink, in_flight: int = 1,
                        allow_swap: bool = True, granularity: int = 1 << 20) -> Dict[str, str]:
    """{module name: "recompute" | "swap"} of minimum added time that frees at least ``bytes_to_free``."""
    if bytes_to_free <= 0:
        return {}
    by_parent: Dict[Optional[str], List[ModuleProfile]] = {}
    for p in profiles:
        by_parent.setdefault(p.parent, []).append(p)
    groups: List[List[Tuple[int, float, Dict[str, str]]]] = []
    for top in by_parent.get(None, []):
        opts: List[Tuple[int, float, Dict[str, str]]] = []
        for freed, cost, act in module_options(top, link, in_flight, allow_swap):
            opts.append((freed, cost, {} if act == KEEP else {top.name: act}))
        kids = by_parent.get(top.name, [])[:4]
        kid_opts = [module_options(k, link, in_flight, allow_swap) for k in kids]
        # every combination of child actions (3^4 at most) is an alternative to acting on the whole layer
        combos: List[Tuple[int, float, Dict[str, str]]] = [(0, 0.0, {})]
        for k, ko in zip(kids, kid_opts):
            combos = [(f + kf, c + kc, {**d, **({} if ka == KEEP else {k.name: ka})}) for f, c, d in combos for kf, kc, ka in ko]
        opts += [c for c in combos if c[2]]
        groups.append(opts)
    need = (bytes_to_free + granularity - 1) // granularity
    INF = float("inf")
    best = [INF] * (need + 1)
    best[0] = 0.0
    choice = []
    for opts in groups:
        new = [INF] * (need + 1)
        pick: List[Optional[Tuple[int, int]]] = [None] * (need + 1)
        for have in range(need + 1):
            if best[have] == INF:
                continue
            for oi, (freed, cost, _) in enumerate(opts):
                tgt = min(need, have + freed // granularity)
                c = best[have] + cost
                if c < new[tgt]:
                    new[tgt], pick[tgt] = c, (oi, have)
        choice.append(pick)
        best = new
    out: Dict[str, str] = {}
    if best[need] == INF:
        # not reachable: take, per layer, whatever frees the most
        for opts in groups:
            out.update(max(opts, key=lambda o: o[0])[2])
        return out
    at = need
    for gi in range(len(groups) - 1, -1, -1):
        oi, prev = choice[gi][at]
        out.update(groups[gi][oi][2])
        at = prev
    return out


class _Swap(nn.Module):
    """Forward of ``inner`` with everything autograd saves inside parked in pinned host memory."""

    def __init__(self, inner, min_bytes: int = 1 << 20, context=None):
        super().__init__()
        self.inner, self.min_bytes, self.context = inner, min_bytes, context

    def forward(self, *args, **kw):
        if not torch.is_grad_enabled():
            return self.inner(*args, **kw)
        if self.context is not None:
            ctx = self.context()
        else:
            from .host_offload import OffloadSaved
            ctx = OffloadSaved(min_bytes=self.min_bytes)
        with ctx:
            return self.inner(*args, **kw)


class AdaptiveMemory(AdaptiveRecompute):
    def __init__(self, model: nn.Module, candidates=None, profiling_steps: int = 2, device_budget_bytes: Optional[int] = None,
                 child_names: Sequence[str] = ("self_attention", "mlp"), link: Optional[HostLink] = None, in_flight: int = 1,
                 allow_swap: bool = True, swap_min_bytes: int = 1 << 20, swap_context=None, auto_budget_fraction: float = 0.9,
                 granularity: int = 1 << 20):
        super().__init__(model, candidates, profiling_steps, device_budget_bytes, child_names,
                         swap_while_profiling=allow_swap and torch.cuda.is_available(), auto_budget_fraction=auto_budget_fraction,
                         swap_min_bytes=swap_min_bytes)
        self.link, self.in_flight, self.allow_swap = link, max(1, in_flight), allow_swap
        self.swap_min_bytes, self.swap_context = swap_min_bytes, swap_context
        self.policy: Dict[str, str] = {}
        self.granularity = granularity              # unit of the knapsack over freed bytes

    def _decide(self, static_bytes):
        for h in self._handles:
            h.remove()
        self._handles = []
        if self.budget is None:
            return
        if self.link is None:
            self.link = measure_host_link()
        if static_bytes is None:
            static_bytes = torch.cuda.memory_allocated() if torch.cuda.is_available() else 0
        total_saved = sum(p.saved_bytes for p in self.profiles.values() if p.parent is None) * self.in_flight
        self.policy = solve_memory_policy(list(self.profiles.values()), static_bytes + total_saved - self.budget, self.link,
                                          self.in_flight, self.allow_swap, self.granularity)
        self.chosen = [n for n, a in self.policy.items() if a == RECOMPUTE]
        self.apply_policy(self.policy)

    def apply_policy(self, policy: Dict[str, str]):
        for name, act in policy.items():
            parent = self.model
            parts = name.split(".")
            for p in parts[:-1]:
                parent = getattr(parent, p)
            cur = getattr(parent, parts[-1])
            if isinstance(cur, (_Ckpt, _Swap)):
                continue
            setattr(parent, parts[-1], _Ckpt(cur) if act == RECOMPUTE else _Swap(cur, self.swap_min_bytes, self.swap_context))
