"""Executes a pipeline ``Plan`` (plan.py) on this rank: lockstep slots of compute with point-to-point exchange between them.

Every tensor is sent in the slot after it was produced and received in that same slot; the order of the messages of a
slot is canonical (sorted by direction, chunk and micro-batch) on both ends.  Communication stays on NCCL point-to-point
(gloo on CPU).  Two modes:

  lock-step (default)   one ``batch_isend_irecv`` group per slot, waited for before the slot's compute.
  overlapped            (``--overlap-p2p-communication``) the receives of slot t+1 are posted BEFORE slot t's compute and the
                        sends of slot t+1 right after it, as individual isend / irecv calls; a receive is waited for only
                        when its slot starts, a send when its buffer is recycled.  So a slot's transfers fly while the slot
                        before it computes on the neighbour.  Messages that move up the ranks use the pipeline group, messages
                        that move down use the second pipeline group: inside one communicator the dependency between a
                        blocked receive and the send that feeds it then always points the same way along the ranks, so no
                        cycle of mutually waiting ranks can form (reference: the even / odd ordered async exchange and the
                        second group of mindspeed/core/pipeline_parallel/p2p_communication.py:460-542,
                        optimize_send_recv_comm/parallel_state.py:15-66).

B / W split: when the plan contains W operations for a chunk, its B runs with the weight-gradient store enabled
(linear layers queue their weight-gradient GEMMs, reference: mindspeed/core/weight_grad_store.py:63-240) and the W
operation pops that micro-batch's queue.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import parallel_state as ps
from ..weight_grad_store import WeightGradStore
from . import schedules as S
from .plan import Message, Op, Plan

_CURRENT = S._CURRENT
current_microbatch = S.current_microbatch


def _set_linear_deferral(module, flag: bool):
    for m in module.modules():
        if hasattr(m, "wgrad_deferral"):
            m.wgrad_deferral = flag


class _Replay:
    """Iterator wrapper that remembers what it handed out, so a scheduler-placed recompute sees the same batch."""

    def __init__(self, it):
        self.it, self.taken = it, []

    def __iter__(self):
        return self

    def __next__(self):
        b = next(self.it)
        self.taken.append(b)
        return b


def _rng_capture():
    st = {"cpu": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["cuda"] = torch.cuda.get_rng_state()
        from ..random import get_cuda_rng_tracker
        st["tracker"] = get_cuda_rng_tracker().get_states()
    return st


def _rng_restore(st):
    torch.set_rng_state(st["cpu"])
    if "cuda" in st:
        torch.cuda.set_rng_state(st["cuda"])
        from ..random import get_cuda_rng_tracker
        get_cuda_rng_tracker().set_states(st["tracker"])


def run_plan(plan: Plan, *, forward_step_func, data_iterator, model, num_microbatches, seq_length, micro_batch_size,
             forward_only=False, collect_non_loss_data=False):
    if not isinstance(model, list):
        model = [model]
    if not isinstance(data_iterator, list):
        data_iterator = [data_iterator] * len(model)
    config = S._cfg(model)
    pp_group = ps.get_pipeline_model_parallel_group()
    pp_ranks = ps._ranks("pp")
    rank = ps.get_pipeline_model_parallel_rank()
    pl = plan.placement
    Sn = pl.num_stages
    # what crosses a stage boundary: one [s, b, h] tensor, or the list given by ``config.pipeline_tensor_shapes``
    # (--use-multiparameter-pipeline-model-parallel).  Internally a payload is always a list; gradients exist for its
    # floating-point entries only.
    specs = S.get_tensor_specs(seq_length=seq_length, micro_batch_size=micro_batch_size, config=config)
    multi = S.is_multi_parameter(config)
    gspecs = [sp for sp in specs if sp[1].is_floating_point]
    # a chunk may hold no parameters at all (only no-op layers): take the device from any chunk that has some
    dev = next((p.device for m in model for p in m.parameters()),
               torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and dist.get_backend() != "gloo"
               else torch.device("cpu"))

    mb_sizes = getattr(config, "micro_batch_sizes", None)       # --optimized-mbs-list: the batch axis differs per micro-batch

    def specs_of(m):
        sp = specs if m.kind == "act" else gspecs
        if mb_sizes and not multi:
            b = mb_sizes[m.mb % len(mb_sizes)]
            sp = [((sh[0], b) + tuple(sh[2:]), dt) for sh, dt in sp]
        return sp

    def unwrap(payload):
        return payload if multi else payload[0]
    has_w = any(op.kind == "W" for ops in plan.table[rank] for op in ops)
    lazy = {(op.chunk, op.mb) for ops in plan.table[rank] for op in ops if op.kind == "R"}   # forwards that drop activations
    stash: Dict[Tuple[int, int], tuple] = {}
    inputs: Dict[Tuple[int, int], Optional[torch.Tensor]] = {}
    outputs: Dict[Tuple[int, int], torch.Tensor] = {}
    inbox: Dict[Tuple[str, int, int], torch.Tensor] = {}
    outbox: Dict[Tuple[str, int, int], torch.Tensor] = {}
    store: List = []
    total_tokens = torch.zeros([], dtype=torch.int)
    saved_vpp = (ps.get_virtual_pipeline_model_parallel_rank(), ps.get_virtual_pipeline_model_parallel_world_size())
    ctxs = []
    if not forward_only:
        for m in model:
            if hasattr(m, "no_sync"):
                c = m.no_sync()
                c.__enter__()
                ctxs.append(c)
    if has_w:
        for m in model:
            _set_linear_deferral(m, True)
    key = lambda m: (m.kind, m.src, m.dst, m.src_chunk, m.mb)
    group_down = ps._group("pp_new_stream", check=False)
    overlap = bool(getattr(config, "overlap_p2p_comm", False)) and group_down is not None

    def msgs(table, t):
        out = sorted(table.get((rank, t), []), key=key)
        return [m for m in out if m.kind == "act"] if forward_only else out

    def comm_of(m):
        return pp_group if m.dst > m.src else group_down

    pending_recv: Dict[int, list] = {}
    pending_send: List[tuple] = []
    grad_pool: List[torch.Tensor] = []

    def new_bufs(m):
        if m.kind == "grad" and grad_pool and not multi and not mb_sizes:
            return [grad_pool.pop()]
        return [torch.empty(sh, dtype=dt, device=dev) for sh, dt in specs_of(m)]

    def post_recvs(t):
        lst = []
        for m in msgs(plan.recvs, t):
            bufs = new_bufs(m)
            lst.append((m, bufs, [dist.irecv(b, pp_ranks[m.src], group=comm_of(m)) for b in bufs]))
        pending_recv[t] = lst

    def post_sends(t):
        for m in msgs(plan.sends, t):
            for ten in outbox.pop((m.kind, m.src_chunk, m.mb)):
                ten = ten.contiguous()
                pending_send.append((dist.isend(ten, pp_ranks[m.dst], group=comm_of(m)), ten))   # keep the tensor alive

    # ---- forward/backward overlap (--moe-fb-overlap): every chunk's layer stack keeps staged graphs; a slot that holds an F
    # and a B runs the B's layer backward interleaved with the F's layer forward on two streams ----
    fb_mode = bool(getattr(config, "moe_fb_overlap", False)) and not forward_only
    blocks = []
    if fb_mode:
        from ...models.transformer import TransformerBlock
        from ..moe.fb_overlap import StagedBlockState
        for chunk in model:
            blk = next(m for m in chunk.modules() if isinstance(m, TransformerBlock))
            blk.fb_state, blk.fb_partner = StagedBlockState(blk.layers), None
            blocks.append(blk)

    def enter(op):
        pipe, stage = pl.stage_of[(rank, op.chunk)]
        _CURRENT.update(chunk=op.chunk, mb=op.mb, pipe=pipe)
        ps.set_virtual_pipeline_model_parallel_world_size(None)
        ps.set_stage_override(stage == 0, stage == Sn - 1)
        return pipe, stage

    def fb_forward(op, partner=None):
        nonlocal total_tokens
        pipe, stage = enter(op)
        inp = None
        if stage > 0:
            inp = inbox.pop(("act", op.chunk, op.mb))
            for x in inp:
                if x.is_floating_point():
                    x.requires_grad_(True)
            inp = unwrap(inp)
        blocks[op.chunk].fb_partner = partner
        try:
            out, nt = S.forward_step(forward_step_func, data_iterator[op.chunk], model[op.chunk], num_microbatches, inp, store,
                                     config, collect_non_loss_data, current_microbatch=op.mb)
        finally:
            blocks[op.chunk].fb_partner = None
        total_tokens += nt.cpu() if torch.is_tensor(nt) else nt
        inputs[(op.chunk, op.mb)], outputs[(op.chunk, op.mb)] = inp, out
        if stage < Sn - 1:
            dr, dc = pl.holder(pipe, stage + 1)
            outs = list(out) if isinstance(out, (list, tuple)) else [out]
            if dr == rank:
                inbox[("act", dc, op.mb)] = [o.detach().clone() for o in outs]
            else:
                outbox[("act", op.chunk, op.mb)] = [o.detach() for o in outs]

    def fb_seed(op):
        """The part of a backward that lies after the layer stack (loss, output layer, final norm - or nothing): leaves the
        gradient of the stack's output in its detached leaf."""
        pipe, stage = enter(op)
        out = outputs.pop((op.chunk, op.mb))
        if stage == Sn - 1:
            loss = out
            if getattr(config, "grad_scale_func", None) is not None:
                loss = config.grad_scale_func(loss)
            loss.backward()
        else:
            og = inbox.pop(("grad", op.chunk, op.mb))
            torch.autograd.backward(out, unwrap(og))

    def fb_finish(op):
        pipe, stage = enter(op)
        inp = inputs.pop((op.chunk, op.mb))
        blocks[op.chunk].fb_state.backward((op.chunk, op.mb))
        if stage > 0:
            g = inp.grad if inp.grad is not None else torch.zeros_like(inp)
            dr, dc = pl.holder(pipe, stage - 1)
            if dr == rank:
                inbox[("grad", dc, op.mb)] = [g]
            else:
                outbox[("grad", op.chunk, op.mb)] = [g]

    def fb_slot(ops):
        fs = [o for o in ops if o.kind == "F"]
        bs = [o for o in ops if o.kind == "B"]
        if has_w and bs:
            WeightGradStore.enable(True)
        if len(fs) == 1 and len(bs) == 1:
            b = bs[0]
            fb_seed(b)
            fb_forward(fs[0], partner=(blocks[b.chunk].fb_state, (b.chunk, b.mb)))
            fb_finish(b)
        else:
            for o in ops:
                if o.kind == "F":
                    fb_forward(o)
                elif o.kind == "B":
                    fb_seed(o)
                    fb_finish(o)
        if has_w and bs:
            WeightGradStore.flush()
            WeightGradStore.enable(False)
        for o in ops:
            if o.kind == "W":
                WeightGradStore.pop()
            elif o.kind == "R":
                raise RuntimeError("scheduler-placed recompute is not combined with --moe-fb-overlap")

    try:
        if overlap:
            post_recvs(0)
        for t in range(plan.num_slots):
            if overlap:
                for m, bufs, reqs in pending_recv.pop(t):
                    for req in reqs:
                        req.wait()
                    inbox[(m.kind, m.dst_chunk, m.mb)] = bufs
                if t + 1 < plan.num_slots:
                    post_recvs(t + 1)            # flies while this slot computes here and the slot before it on the peer
                while pending_send and pending_send[0][0].is_completed():
                    pending_send.pop(0)
            else:
                sends, recvs = msgs(plan.sends, t), msgs(plan.recvs, t)
                ops, bufs = [], []
                allm = sorted(sends + recvs, key=key)
                for m in allm:
                    if m.src == rank and m in sends:
                        for ten in outbox.pop((m.kind, m.src_chunk, m.mb)):
                            ops.append(dist.P2POp(dist.isend, ten.contiguous(), pp_ranks[m.dst], pp_group))
                    else:
                        got = [torch.empty(sh, dtype=dt, device=dev) for sh, dt in specs_of(m)]
                        bufs.append((m, got))
                        for buf in got:
                            ops.append(dist.P2POp(dist.irecv, buf, pp_ranks[m.src], pp_group))
                if ops:
                    for r in dist.batch_isend_irecv(ops):
                        r.wait()
                for m, buf in bufs:
                    inbox[(m.kind, m.dst_chunk, m.mb)] = buf
            if fb_mode:
                fb_slot(plan.table[rank][t])
            for op in ([] if fb_mode else plan.table[rank][t]):
                if forward_only and op.kind != "F":
                    continue
                pipe, stage = pl.stage_of[(rank, op.chunk)]
                _CURRENT.update(chunk=op.chunk, mb=op.mb, pipe=pipe)
                ps.set_virtual_pipeline_model_parallel_world_size(None)
                ps.set_stage_override(stage == 0, stage == Sn - 1)
                chunk = model[op.chunk]
                if op.kind == "F":
                    inp = None
                    if stage > 0:
                        inp = inbox.pop(("act", op.chunk, op.mb))
                        for x in inp:
                            if x.is_floating_point():
                                x.requires_grad_(not forward_only)
                        inp = unwrap(inp)
                    drop = (op.chunk, op.mb) in lazy and not forward_only
                    if drop:
                        # RiPipe: run without building a graph, remember (input, batch, RNG) for the R op
                        rng = _rng_capture()
                        it = _Replay(data_iterator[op.chunk]) if data_iterator[op.chunk] is not None else None
                        with torch.no_grad():
                            out, nt = S.forward_step(forward_step_func, it, chunk, num_microbatches, inp, store, config,
                                                     collect_non_loss_data, current_microbatch=op.mb)
                        stash[(op.chunk, op.mb)] = (inp, it.taken if it is not None else None, rng)
                    else:
                        out, nt = S.forward_step(forward_step_func, data_iterator[op.chunk], chunk, num_microbatches, inp,
                                                 store, config, collect_non_loss_data, current_microbatch=op.mb)
                    total_tokens += nt.cpu() if torch.is_tensor(nt) else nt
                    if not forward_only and not drop:
                        inputs[(op.chunk, op.mb)] = inp
                        outputs[(op.chunk, op.mb)] = out
                    if stage < Sn - 1:
                        dr, dc = pl.holder(pipe, stage + 1)
                        outs = list(out) if isinstance(out, (list, tuple)) else [out]
                        if dr == rank:
                            inbox[("act", dc, op.mb)] = [o.detach().clone() for o in outs]
                        else:
                            outbox[("act", op.chunk, op.mb)] = [o.detach() for o in outs]
                elif op.kind == "R":
                    inp, batches, rng = stash.pop((op.chunk, op.mb))
                    now = _rng_capture()
                    _rng_restore(rng)
                    out, _ = S.forward_step(forward_step_func, iter(batches) if batches is not None else None, chunk,
                                            num_microbatches, inp, [], config, collect_non_loss_data, current_microbatch=op.mb)
                    _rng_restore(now)
                    inputs[(op.chunk, op.mb)] = inp
                    outputs[(op.chunk, op.mb)] = out
                elif op.kind == "B":
                    inp = inputs.pop((op.chunk, op.mb))
                    out = outputs.pop((op.chunk, op.mb))
                    og = None if stage == Sn - 1 else inbox.pop(("grad", op.chunk, op.mb))
                    if has_w:
                        WeightGradStore.enable(True)
                    g = S.backward_step(inp, out, None if og is None else unwrap(og), None, config)
                    if overlap and not multi and og is not None and og[0].is_leaf and not og[0].requires_grad:
                        grad_pool.append(og[0])  # the received output gradient has been consumed: reuse its storage
                    if has_w:
                        WeightGradStore.flush()
                        WeightGradStore.enable(False)
                    if stage > 0:
                        dr, dc = pl.holder(pipe, stage - 1)
                        gl = list(g) if isinstance(g, (list, tuple)) else [g]
                        if dr == rank:
                            inbox[("grad", dc, op.mb)] = gl
                        else:
                            outbox[("grad", op.chunk, op.mb)] = gl
                else:  # W
                    WeightGradStore.pop()
            if overlap and t + 1 < plan.num_slots:
                post_sends(t + 1)                # what this slot produced leaves now; nobody waits for it here
        for req, _ in pending_send:
            req.wait()
    finally:
        ps.set_stage_override(None, None)
        ps.set_virtual_pipeline_model_parallel_rank(saved_vpp[0])
        ps.set_virtual_pipeline_model_parallel_world_size(saved_vpp[1])
        for blk in blocks:
            blk.fb_state, blk.fb_partner = None, None
        if has_w:
            WeightGradStore.pop_all()
            WeightGradStore.enable(False)
            for m in model:
                _set_linear_deferral(m, False)
        for c in ctxs:
            c.__exit__(None, None, None)
    if not forward_only:
        if pl.replicas > 1:
            from .chimera import allreduce_replica_grads
            allreduce_replica_grads(model)
        fin = getattr(config, "finalize_model_grads_func", None)
        if fin is not None:
            fin(model, total_tokens if config.calculate_per_token_loss else None)
    return store
