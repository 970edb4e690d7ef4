"""Tensor dump for run-to-run and cross-implementation comparison.

``install_data_dump(model, directory, steps, name_filter)`` registers forward and full-backward hooks on the selected
modules; during the chosen steps every hooked module's outputs and output gradients are written as
``<dir>/step<k>/rank<r>/<module>.<fwd|bwd>.<i>.pt`` together with a one-line summary (shape, dtype, mean, absmax, L2).
``compare_dumps(a, b)`` walks two dump directories and reports the first tensors that differ beyond a tolerance.
Together with ``utils.determinism`` this is the tool for bisecting a numerical difference between two runs.
reference: mindspeed/functional/npu_datadump (S5: determinism + data dump).
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn


def _summary(t: torch.Tensor) -> Dict:
    f = t.detach().float()
    return {"shape": list(t.shape), "dtype": str(t.dtype), "mean": float(f.mean()) if f.numel() else 0.0,
            "absmax": float(f.abs().max()) if f.numel() else 0.0, "l2": float(f.norm()) if f.numel() else 0.0}


class DataDump:
    def __init__(self, directory: str, steps: Iterable[int], rank: int = 0, save_tensors: bool = True):
        self.dir, self.steps, self.rank, self.save_tensors = directory, set(int(s) for s in steps), rank, save_tensors
        self.step = 0
        self.handles = []
        self.index: List[Dict] = []

    def active(self) -> bool:
        return self.step in self.steps

    def _write(self, name: str, kind: str, tensors):
        if not self.active():
            return
        d = os.path.join(self.dir, f"step{self.step}", f"rank{self.rank}")
        os.makedirs(d, exist_ok=True)
        ts = tensors if isinstance(tensors, (tuple, list)) else (tensors,)
        for i, t in enumerate(ts):
            if not isinstance(t, torch.Tensor):
                continue
            rec = {"module": name, "kind": kind, "index": i, **_summary(t)}
            self.index.append(rec)
            if self.save_tensors:
                torch.save(t.detach().cpu(), os.path.join(d, f"{name}.{kind}.{i}.pt"))
        with open(os.path.join(d, "index.jsonl"), "a") as f:
            for rec in self.index[-len(ts):]:
                f.write(json.dumps(rec) + "\n")

    def attach(self, model: nn.Module, name_filter: Optional[Callable[[str], bool]] = None):
        for name, mod in model.named_modules():
            if not name or (name_filter is not None and not name_filter(name)):
                continue
            self.handles.append(mod.register_forward_hook(lambda m, a, out, n=name: self._write(n, "fwd", out)))
            self.handles.append(mod.register_full_backward_hook(lambda m, gi, go, n=name: self._write(n, "bwd", go)))
        return self

    def end_step(self):
        self.step += 1

    def remove(self):
        for h in self.handles:
            h.remove()
        self.handles = []


def install_data_dump(model: nn.Module, directory: str, steps: Iterable[int] = (0,), name_filter=None, rank: int = 0) -> DataDump:
    return DataDump(directory, steps, rank).attach(model, name_filter)


def compare_dumps(dir_a: str, dir_b: str, rtol: float = 1e-3, atol: float = 1e-5) -> List[Tuple[str, float]]:
    """Relative paths of tensors present in both dumps whose max abs difference exceeds ``atol + rtol * absmax``."""
    bad = []
    for root, _, files in os.walk(dir_a):
        for fn in sorted(files):
            if not fn.endswith(".pt"):
                continue
            rel = os.path.relpath(os.path.join(root, fn), dir_a)
            other = os.path.join(dir_b, rel)
            if not os.path.exists(other):
                continue
            a, b = torch.load(os.path.join(root, fn)).float(), torch.load(other).float()
            if a.shape != b.shape:
                bad.append((rel, float("inf")))
                continue
            d = float((a - b).abs().max()) if a.numel() else 0.0
            if d > atol + rtol * float(a.abs().max() if a.numel() else 0.0):
                bad.append((rel, d))
    return bad
