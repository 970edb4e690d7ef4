"""DualPipe (bidirectional, non-V): two model replicas per rank fed from both ends of the pipeline; forward of one
direction overlaps backward of the other, W work fills the rest (DeepSeek-V3 technical report, section 3.2.1).
Not part of the reference tree; built from the paper on top of the same plan/executor machinery."""
from .. import parallel_state as ps
from .executor import run_plan
from .interleaved import _plan


def forward_backward_dualpipe(*, forward_step_func, data_iterator, model, num_microbatches, seq_length, micro_batch_size,
                              forward_only=False, collect_non_loss_data=False, **_):
    pp = ps.get_pipeline_model_parallel_world_size()
    plan = _plan("dualpipe", pp, num_microbatches, None, True)
    return run_plan(plan, forward_step_func=forward_step_func, data_iterator=data_iterator, model=model,
                    num_microbatches=num_microbatches, seq_length=seq_length, micro_batch_size=micro_batch_size,
                    forward_only=forward_only, collect_non_loss_data=collect_non_loss_data)
