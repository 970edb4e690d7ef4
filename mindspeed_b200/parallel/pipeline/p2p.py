"""Pipeline point-to-point communication over NCCL (gloo on CPU).

send/recv pairs between adjacent stages.  Options mirrored from the reference
(mindspeed/core/pipeline_parallel/p2p_communication.py:23-105,460-542):
  * batched (``batch_isend_irecv``) or individual ops ordered even/odd by rank so that neighbours
    never both block in send;
  * optional second pipeline group so sends and receives of one step run on different communicators;
  * variable sequence lengths: the shape is exchanged first as an int64 triple.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .. import parallel_state as ps


def _dev():
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and \
        dist.get_backend(ps.get_pipeline_model_parallel_group()) != "gloo" else torch.device("cpu")


def warm_up_p2p(groups=None):
    """Create the point-to-point channels of every neighbour pair, in one fixed order on all ranks.

    NCCL builds the communicator of a rank pair inside the first send / receive between them, and that call blocks
    until the other side makes its matching call.  When ranks first touch two communicators in different orders (one
    posts a receive on the downward group while its neighbour posts one on the upward group), each blocks inside the
    creation of a different communicator and neither returns.  Walking the pairs (r, r+1) - and the wrap-around pair
    used by interleaved schedules - in rank order, group by group, rules that out; afterwards any posting order works.
    """
    pp = ps.get_pipeline_model_parallel_world_size()
    if pp <= 1:
        return
    if groups is None:
        groups = [ps.get_pipeline_model_parallel_group(), ps._group("pp_new_stream", check=False)]
    ranks = ps._ranks("pp")
    me = ps.get_pipeline_model_parallel_rank()
    dev = _dev()
    pairs = [(r, r + 1) for r in range(pp - 1)] + ([(pp - 1, 0)] if pp > 2 else [])
    for g in groups:
        if g is None:
            continue
        for a, b in pairs:
            for src, dst in ((a, b), (b, a)):
                if me == src:
                    dist.send(torch.zeros(1, device=dev), ranks[dst], group=g)
                elif me == dst:
                    dist.recv(torch.empty(1, device=dev), ranks[src], group=g)
    if dev.type == "cuda":
        torch.cuda.synchronize()


def _communicate_shapes(send_next, send_prev, recv_prev, recv_next, config):
    """Exchange 3-d shapes with the neighbours when sequence lengths vary."""
    group = ps.get_pipeline_model_parallel_group()
    ops, bufs = [], {}
    dev = _dev()

    def shape_t(t):
        return torch.tensor(list(t.shape), dtype=torch.int64, device=dev)

    if send_prev is not None:
        ops.append(dist.P2POp(dist.isend, shape_t(send_prev), ps.get_pipeline_model_parallel_prev_rank(), group))
    if recv_prev:
        bufs["prev"] = torch.empty(3, dtype=torch.int64, device=dev)
        ops.append(dist.P2POp(dist.irecv, bufs["prev"], ps.get_pipeline_model_parallel_prev_rank(), group))
    if send_next is not None:
        ops.append(dist.P2POp(dist.isend, shape_t(send_next), ps.get_pipeline_model_parallel_next_rank(), group))
    if recv_next:
        bufs["next"] = torch.empty(3, dtype=torch.int64, device=dev)
        ops.append(dist.P2POp(dist.irecv, bufs["next"], ps.get_pipeline_model_parallel_next_rank(), group))
    if ops:
        for r in dist.batch_isend_irecv(ops):
            r.wait()
    return (bufs["prev"].tolist() if "prev" in bufs else None), (bufs["next"].tolist() if "next" in bufs else None)


def _communicate(*, tensor_send_next, tensor_send_prev, recv_prev, recv_next, tensor_shape, config, wait_on_reqs=True):
    group = ps.get_pipeline_model_parallel_group()
    group2 = ps._group("pp_new_stream", check=False) if ps.model_parallel_is_initialized() else None
    dev = _dev()
    dtype = config.pipeline_dtype
    shape_prev = shape_next = tensor_shape
    if getattr(config, "variable_seq_lengths", False):
        shape_prev, shape_next = _communicate_shapes(tensor_send_next, tensor_send_prev, recv_prev, recv_next, config)
    t_prev = torch.empty(shape_prev, dtype=dtype, device=dev, requires_grad=True) if recv_prev else None
    t_next = torch.empty(shape_next, dtype=dtype, device=dev, requires_grad=True) if recv_next else None
    prev_r, next_r = ps.get_pipeline_model_parallel_prev_rank(), ps.get_pipeline_model_parallel_next_rank()
    reqs = []
    use_batch = getattr(config, "batch_p2p_comm", True) and group2 is None
    if use_batch:
        ops = []
        if tensor_send_prev is not None:
            ops.append(dist.P2POp(dist.isend, tensor_send_prev.contiguous(), prev_r, group))
        if t_prev is not None:
            ops.append(dist.P2POp(dist.irecv, t_prev, prev_r, group))
        if tensor_send_next is not None:
            ops.append(dist.P2POp(dist.isend, tensor_send_next.contiguous(), next_r, group))
        if t_next is not None:
            ops.append(dist.P2POp(dist.irecv, t_next, next_r, group))
        if ops:
            reqs = dist.batch_isend_irecv(ops)
    else:
        # even ranks send first, odd ranks receive first.  With a second group, traffic that moves up the ranks (send to
        # next / receive from previous) stays on the pipeline group and traffic that moves down uses the second one: a send
        # and its matching receive are always on the same communicator, and the two directions never queue behind each other
        down = group2 if group2 is not None else group
        even = ps.get_pipeline_model_parallel_rank() % 2 == 0
        seq = []
        s_next = (dist.isend, tensor_send_next, next_r, group)
        r_prev = (dist.irecv, t_prev, prev_r, group)
        s_prev = (dist.isend, tensor_send_prev, prev_r, down)
        r_next = (dist.irecv, t_next, next_r, down)
        seq = [s_next, r_prev, s_prev, r_next] if even else [r_prev, s_next, r_next, s_prev]
        for fn, t, peer, g in seq:
            if t is not None:
                reqs.append(fn(t.contiguous() if fn is dist.isend else t, peer, group=g))
    if wait_on_reqs:
        for r in reqs:
            r.wait()
        reqs = None
        if dev.type == "cuda" and getattr(config, "batch_p2p_sync", True):
            torch.cuda.synchronize()
    return t_prev, t_next, reqs


def _shape(shapes):
    return shapes[0] if isinstance(shapes, (list, tuple)) and isinstance(shapes[0], (list, tuple)) else shapes


def recv_forward(tensor_shapes, config):
    if ps.is_pipeline_first_stage():
        return None
    t, _, _ = _communicate(tensor_send_next=None, tensor_send_prev=None, recv_prev=True, recv_next=False,
                           tensor_shape=_shape(tensor_shapes), config=config)
    return t


def recv_backward(tensor_shapes, config):
    if ps.is_pipeline_last_stage():
        return None
    _, t, _ = _communicate(tensor_send_next=None, tensor_send_prev=None, recv_prev=False, recv_next=True,
                           tensor_shape=_shape(tensor_shapes), config=config)
    return t


def send_forward(output_tensor, config):
    if not ps.is_pipeline_last_stage():
        _communicate(tensor_send_next=output_tensor, tensor_send_prev=None, recv_prev=False, recv_next=False,
                     tensor_shape=None, config=config)


def send_backward(input_tensor_grad, config):
    if not ps.is_pipeline_first_stage():
        _communicate(tensor_send_next=None, tensor_send_prev=input_tensor_grad, recv_prev=False, recv_next=False,
                     tensor_shape=None, config=config)


def send_forward_recv_backward(output_tensor, tensor_shapes, config):
    if ps.is_pipeline_last_stage():
        return None
    _, t, _ = _communicate(tensor_send_next=output_tensor, tensor_send_prev=None, recv_prev=False, recv_next=True,
                           tensor_shape=_shape(tensor_shapes), config=config)
    return t


def send_backward_recv_forward(input_tensor_grad, tensor_shapes, config):
    if ps.is_pipeline_first_stage():
        return None
    t, _, _ = _communicate(tensor_send_next=None, tensor_send_prev=input_tensor_grad, recv_prev=True, recv_next=False,
                           tensor_shape=_shape(tensor_shapes), config=config)
    return t


def send_forward_recv_forward(output_tensor, recv_prev, tensor_shape, config, overlap_p2p_comm=False):
    t, _, reqs = _communicate(tensor_send_next=output_tensor, tensor_send_prev=None, recv_prev=recv_prev, recv_next=False,
                              tensor_shape=tensor_shape, config=config, wait_on_reqs=not overlap_p2p_comm)
    return (t, reqs) if overlap_p2p_comm else t


def send_backward_recv_backward(input_tensor_grad, recv_next, tensor_shape, config, overlap_p2p_comm=False):
    _, t, reqs = _communicate(tensor_send_next=None, tensor_send_prev=input_tensor_grad, recv_prev=False, recv_next=recv_next,
                              tensor_shape=tensor_shape, config=config, wait_on_reqs=not overlap_p2p_comm)
    return (t, reqs) if overlap_p2p_comm else t


def send_forward_backward_recv_forward_backward(output_tensor, input_tensor_grad, recv_prev, recv_next, tensor_shape, config):
    a, b, _ = _communicate(tensor_send_next=output_tensor, tensor_send_prev=input_tensor_grad, recv_prev=recv_prev,
                           recv_next=recv_next, tensor_shape=tensor_shape, config=config)
    return a, b
