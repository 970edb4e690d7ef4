"""White-box, black-box and mixed search over the pruned configuration space; returns the top-k configurations
(reference: mindspeed/auto_settings/module/searcher.py:64-270)."""
from __future__ import annotations

from typing import Callable, List, Optional

from .cost_model import Estimate, estimate
from .hardware import Hardware
from .search_space import ModelDesc, SearchConfig, build_search_space


def white_search(model: ModelDesc, world: int, hw: Hardware, topk: int = 3, db=None, comm=None, prune: bool = True) -> List[Estimate]:
    """Rank the (pruned) space with the cost models; ``db`` / ``comm`` carry what earlier profiled runs taught them."""
    from .cost_model import memory_gib
    from .search_space import stage_1_prune
    space = build_search_space(model, world, hw.gpus_per_node)
    if prune:
        space = stage_1_prune(space, model, memory_gib, hw.hbm_gib)
    ests = [estimate(model, c, hw, db, comm) for c in space]
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


def mixed_search(model, world, hw, run_config, topk=3, measure=4, db=None, comm=None):
    """White-box ranking, the best few are measured, and - when the runs leave profiles (``run_config.last_trace``) - what the
    profiles say about operator efficiency and communication is fed back into the models before the space is ranked again;
    measured configurations keep their measured time in the final ranking."""
    measured = black_search(model, world, hw, run_config, topk=max(topk, measure), budget=max(topk, measure))
    if db is None or comm is None or not hasattr(run_config, "traces"):
        return measured[:topk]
    from .cost_model import learn_from_profile
    from .profiling_parse import parse_chrome_trace
    for cfg, path in run_config.traces:
        try:
            learn_from_profile(parse_chrome_trace(path), model, cfg, hw, db, comm)
        except (OSError, ValueError, KeyError):
            continue
    by_cfg = {e.config: e for e in measured}
    ranked = [by_cfg.get(e.config, e) for e in white_search(model, world, hw, topk=4 * topk, db=db, comm=comm)]
    ranked.sort(key=lambda e: e.step_ms)
    return ranked[:topk]
