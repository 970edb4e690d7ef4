"""RiPipe: activation recompute placed by the pipeline scheduler instead of by the backward pass.

``--recompute-in-bubble``   the forward of a micro-batch runs without keeping activations; the schedule contains an
                            explicit recompute operation in front of the matching backward, which executes while the
                            stage waits for the downstream gradient (inside the pipeline bubble where one exists).
``--recompute-in-advance``  the recompute is additionally moved ahead of the operation before the backward, so the
                            rebuilt graph is ready when the gradient arrives.
Forwards that are followed directly by their own backward keep their activations (no recompute at all), which is what
removes the recompute of the last stage.  Works for 1F1B and interleaved placements.
reference: mindspeed/core/pipeline_parallel/ripipe_schedules.py:41-799, mindspeed/core/tensor_parallel/checkpoint_manager.py:4-62.
"""
from .. import parallel_state as ps
from .executor import run_plan
from .plan import build_plan

_CACHE = {}


def _plan(name, pp, n, vpp, mode):
    k = (name, pp, n, vpp, mode)
    if k not in _CACHE:
        _CACHE[k] = build_plan(name, pp, n, vpp=vpp, recompute=mode)
    return _CACHE[k]


def forward_backward_ripipe(*, forward_step_func, data_iterator, model, num_microbatches, seq_length, micro_batch_size,
                            forward_only=False, collect_non_loss_data=False, mode="bubble", **_):
    pp = ps.get_pipeline_model_parallel_world_size()
    models = model if isinstance(model, list) else [model]
    name = "interleaved" if len(models) > 1 else "1f1b"
    plan = _plan(name, pp, num_microbatches, len(models) if len(models) > 1 else None, mode)
    return run_plan(plan, forward_step_func=forward_step_func, data_iterator=data_iterator, model=model,
                    num_microbatches=num_microbatches, seq_length=seq_length, micro_batch_size=micro_batch_size,
                    forward_only=forward_only, collect_non_loss_data=collect_non_loss_data)


def forward_backward_recompute_in_bubble(**kw):
    return forward_backward_ripipe(mode="bubble", **kw)


def forward_backward_recompute_in_advance(**kw):
    return forward_backward_ripipe(mode="advance", **kw)
