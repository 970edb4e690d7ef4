"""Chimera: two 1F1B pipelines in opposite directions over the same ranks (Li & Hoefler, SC'21).  Rank r holds stage r
of the "down" replica (chunk 0) and stage pp-1-r of the "up" replica (chunk 1); half of the micro-batches enter each.
After the step the gradients of the two replicas of every stage are summed between the two ranks that hold them.
The reference tree has no Chimera; this is built from the paper."""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import parallel_state as ps
from .executor import run_plan
from .interleaved import _plan

_PAIR_GROUPS = {}


def _pair_group():
    """Group {r, pp-1-r} inside this pipeline group (created collectively, once)."""
    ranks = tuple(ps._ranks("pp"))
    if ranks in _PAIR_GROUPS:
        return _PAIR_GROUPS[ranks]
    pp = len(ranks)
    mine = None
    for all_ranks in ps.get_all_ranks("pp"):
        n = len(all_ranks)
        for i in range((n + 1) // 2):
            pair = sorted({all_ranks[i], all_ranks[n - 1 - i]})
            g = dist.new_group(pair) if len(pair) > 1 else None
            if dist.get_rank() in pair and tuple(all_ranks) == ranks:
                mine = (g, pair)
    _PAIR_GROUPS[ranks] = mine
    return mine


def _exchange(send0, send1, recv_like1, recv_like0, partner, group):
    """Send my chunk-0 list then my chunk-1 list; receive the partner's chunk-0 list (shaped like my chunk 1, which
    holds the same stage) then its chunk-1 list (shaped like my chunk 0)."""
    r1 = [torch.empty_like(t) for t in recv_like1]
    r0 = [torch.empty_like(t) for t in recv_like0]
    ops = [dist.P2POp(dist.isend, t.contiguous(), partner, group) for t in list(send0) + list(send1)]
    ops += [dist.P2POp(dist.irecv, t, partner, group) for t in r1 + r0]
    for r in dist.batch_isend_irecv(ops):
        r.wait()
    return r1, r0


def sync_replica_params(model):
    """Make the "up" replica (chunk 1 everywhere) equal to the "down" replica (chunk 0): the rank holding stage s of the
    down replica sends it to the rank holding stage s of the up replica.  Call once after construction."""
    g, pair = _pair_group()
    p0 = [p.data for p in model[0].parameters()]
    p1 = [p.data for p in model[1].parameters()]
    if g is None:
        for a, b in zip(p0, p1):
            b.copy_(a)
        return
    me = dist.get_rank()
    partner = pair[1] if me == pair[0] else pair[0]
    r1, _ = _exchange(p0, [], p1, [], partner, g)
    for dst, src in zip(p1, r1):
        dst.copy_(src)


def allreduce_replica_grads(model):
    """grad(stage s) = gradient from the down replica + gradient from the up replica, on both holders."""
    g, pair = _pair_group()

    def grads(chunk):
        out = []
        for p in chunk.parameters():
            gr = p.main_grad if hasattr(p, "main_grad") else p.grad
            if gr is None:
                gr = torch.zeros_like(p.data)
                p.grad = gr
            out.append(gr)
        return out

    g0, g1 = grads(model[0]), grads(model[1])
    if g is None:  # middle rank of an odd pipeline holds both replicas of its stage
        for a, b in zip(g0, g1):
            s = a + b
            a.copy_(s)
            b.copy_(s)
        return
    me = dist.get_rank()
    partner = pair[1] if me == pair[0] else pair[0]
    r1, r0 = _exchange(g0, g1, g1, g0, partner, g)
    for dst, src in zip(g1, r1):
        dst.add_(src)
    for dst, src in zip(g0, r0):
        dst.add_(src)


def forward_backward_chimera(*, forward_step_func, data_iterator, model, num_microbatches, seq_length, micro_batch_size,
                             forward_only=False, collect_non_loss_data=False, **_):
    pp = ps.get_pipeline_model_parallel_world_size()
    plan = _plan("chimera", pp, num_microbatches, None, False)
    return run_plan(plan, forward_step_func=forward_step_func, data_iterator=data_iterator, model=model,
                    num_microbatches=num_microbatches, seq_length=seq_length, micro_batch_size=micro_batch_size,
                    forward_only=forward_only, collect_non_loss_data=collect_non_loss_data)
