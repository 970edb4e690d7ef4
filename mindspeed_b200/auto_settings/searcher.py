"""White-box, black-box and mixed search over the pruned configuration space; returns the top-k configurations
(reference: mindspeed/auto_settings/module/searcher.py:64-270)."""
from __future__ import annotations

from typing import Callable, List, Optional

from .cost_model import Estimate, estimate
from .hardware import Hardware
from .search_space import ModelDesc, SearchConfig, build_search_space


def white_search(model: ModelDesc, world: int, hw: Hardware, topk: int = 3) -> List[Estimate]:
    ests = [estimate(model, c, hw) for c in build_search_space(model, world, hw.gpus_per_node)]
    ok = [e for e in ests if e.fits]
    ok.sort(key=lambda e: e.step_ms)
    return ok[:topk]


def black_search(model: ModelDesc, world: int, hw: Hardware, run_config: Callable[[SearchConfig], Optional[float]], topk: int = 3,
                 budget: int = 16) -> List[Estimate]:
    """Measure real short runs.  ``run_config`` returns the measured step time in ms or None (failed / out of memory).
    Candidates are tried in white-box order so that the measuring budget goes to plausible configurations."""
    cands = white_search(model, world, hw, topk=budget)
    out = []
    for e in cands:
        ms = run_config(e.config)
        if ms is not None:
            out.append(Estimate(e.config, e.memory_gib, ms, True, {**e.detail, "measured": True, "predicted_ms": e.step_ms}))
    out.sort(key=lambda e: e.step_ms)
    return out[:topk]


def mixed_search(model, world, hw, run_config, topk=3, measure=4):
    """White-box ranking, then the best few are measured and re-ranked by the measurement."""
    return black_search(model, world, hw, run_config, topk=topk, budget=max(topk, measure))
