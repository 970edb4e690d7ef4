"""Interleaved 1F1B (virtual pipeline): v chunks per rank, stage = chunk * pp + rank."""
from .. import parallel_state as ps
from .executor import run_plan
from .plan import build_plan

_CACHE = {}


def _plan(name, pp, n, vpp=None, split_w=True, pair_fb=None):
    """``pair_fb`` None: follow ``--moe-fb-overlap`` (F and B of different micro-batches share a slot and are interleaved)."""
    if pair_fb is None:
        try:
            from ...training.global_vars import get_args
            pair_fb = bool(getattr(get_args(), "moe_fb_overlap", False))
        except RuntimeError:
            pair_fb = False
    k = (name, pp, n, vpp, split_w, pair_fb)
    if k not in _CACHE:
        _CACHE[k] = build_plan(name, pp, n, vpp=vpp, split_w=split_w, pair_fb=pair_fb)
    return _CACHE[k]


def forward_backward_interleaved(*, forward_step_func, data_iterator, model, num_microbatches, seq_length, micro_batch_size,
                                 forward_only=False, collect_non_loss_data=False, **_):
    pp = ps.get_pipeline_model_parallel_world_size()
    vpp = len(model)
    nano, swap = False, False
    try:
        from ...training.global_vars import get_args
        nano, swap = bool(getattr(get_args(), "use_nanopipe", False)), bool(getattr(get_args(), "use_nanopipe_swap", False))
    except RuntimeError:
        pass
    # --use-nanopipe: weight gradients of the first backward steps of every rank move to the end of its schedule;
    # --use-nanopipe-swap parks what they need (layer inputs and output gradients) in pinned host memory meanwhile
    from ..weight_grad_store import WeightGradStore
    WeightGradStore.swap_to_host = nano and swap and not forward_only
    plan = _plan("nanopipe" if nano and not forward_only else "interleaved", pp, num_microbatches, vpp)
    return run_plan(plan, forward_step_func=forward_step_func, data_iterator=data_iterator, model=model,
                    num_microbatches=num_microbatches, seq_length=seq_length, micro_batch_size=micro_batch_size,
                    forward_only=forward_only, collect_non_loss_data=collect_non_loss_data)
