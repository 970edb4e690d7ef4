"""DualPipeV: each rank holds two chunks in a V (stage r on the way down, stage 2pp-1-r on the way back), so the
embedding and the loss live on rank 0 and share the embedding weight; backward is split into input-gradient (B) and
weight-gradient (W) work and W fills the bubbles
(reference: mindspeed/core/pipeline_parallel/dualpipev/dualpipev_schedules.py:736-1606, dualpipev_chunks.py:43-53,561-570;
entry name kept: ``forward_backward_pipelining_with_cutinhalf``)."""
from .. import parallel_state as ps
from .executor import run_plan
from .interleaved import _plan


def forward_backward_pipelining_with_cutinhalf(*, forward_step_func, data_iterator, model, num_microbatches, seq_length,
                                               micro_batch_size, forward_only=False, collect_non_loss_data=False,
                                               dw_detach=True, order="greedy", **_):
    pp = ps.get_pipeline_model_parallel_world_size()
    try:
        from ...training.global_vars import get_args
        # --dualpipev-dw-detach: split every backward into input-gradient and weight-gradient work so that W fills bubbles
        dw_detach = bool(getattr(get_args(), "dualpipev_dw_detach", dw_detach))
    except RuntimeError:
        pass
    if len(model) != 2:
        raise RuntimeError("DualPipeV needs exactly two model chunks per rank")
    name = "dualpipev_greedy" if order == "greedy" else "dualpipev"
    plan = _plan(name, pp, num_microbatches, None, dw_detach)
    return run_plan(plan, forward_step_func=forward_step_func, data_iterator=data_iterator, model=model,
                    num_microbatches=num_microbatches, seq_length=seq_length, micro_batch_size=micro_batch_size,
                    forward_only=forward_only, collect_non_loss_data=collect_non_loss_data)
