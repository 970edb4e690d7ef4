"""Pipeline schedules (Megatron-core ``pipeline_parallel.schedules`` surface).

  get_forward_backward_func()  -> no pipelining | 1F1B | interleaved 1F1B | DualPipeV | DualPipe | Chimera
  every schedule has the signature
     f(forward_step_func, data_iterator, model, num_microbatches, seq_length, micro_batch_size,
       decoder_seq_length=None, forward_only=False, collect_non_loss_data=False, first_val_step=None)
  and returns the list of per-microbatch reduced-loss dicts on the last stage.

Selector reference: mindspeed/core/pipeline_parallel/schedules.py:34-59.
Point-to-point traffic stays on NCCL (``p2p.py``) and is overlapped with compute by issuing the
receive for the next step before running the current one.
"""
from __future__ import annotations

import contextlib
from typing import Callable, Iterator, List, Optional, Union

import torch

from .. import parallel_state as ps
from . import p2p

_SCHEDULE_OVERRIDE = {"name": None}
_CURRENT = {"chunk": 0, "mb": 0, "pipe": 0}   # the (chunk, micro-batch, pipeline) being executed


def current_microbatch():
    """Lets a forward_step_func or data iterator see which micro-batch the schedule is running."""
    return dict(_CURRENT)


def set_schedule(name: Optional[str]):
    """``--schedules-method``: None | 'dualpipev' | 'dualpipe' | 'chimera' | 'ripipe_bubble' | 'ripipe_advance'."""
    _SCHEDULE_OVERRIDE["name"] = name


def get_forward_backward_func():
    pp = ps.get_pipeline_model_parallel_world_size()
    name = _SCHEDULE_OVERRIDE["name"]
    if pp > 1:
        if name == "dualpipev":
            from .dualpipev import forward_backward_pipelining_with_cutinhalf
            return forward_backward_pipelining_with_cutinhalf
        if name == "dualpipe":
            from .dualpipe import forward_backward_dualpipe
            return forward_backward_dualpipe
        if name == "chimera":
            from .chimera import forward_backward_chimera
            return forward_backward_chimera
        if name == "ripipe_bubble":
            from .ripipe import forward_backward_recompute_in_bubble
            return forward_backward_recompute_in_bubble
        if name == "ripipe_advance":
            from .ripipe import forward_backward_recompute_in_advance
            return forward_backward_recompute_in_advance
        if ps.get_virtual_pipeline_model_parallel_world_size() is not None:
            return forward_backward_pipelining_with_interleaving
        return forward_backward_pipelining_without_interleaving
    return forward_backward_no_pipelining


def _cfg(model):
    m = model[0] if isinstance(model, list) else model
    while hasattr(m, "module") and not hasattr(m, "config"):
        m = m.module
    return m.config if hasattr(m, "config") else m.module.config


def _set_input(model, t):
    m = model
    while not hasattr(m, "set_input_tensor") and hasattr(m, "module"):
        m = m.module
    inner = m
    while hasattr(inner, "module") and not hasattr(inner, "set_input_tensor"):
        inner = inner.module
    inner.set_input_tensor(t)


def set_input_tensor(model, t):
    m = model
    while hasattr(m, "module"):
        m = m.module
    m.set_input_tensor(t)


def forward_step(forward_step_func, data_iterator, model, num_microbatches, input_tensor, forward_data_store, config,
                 collect_non_loss_data=False, checkpoint_activations_microbatch=None, is_first_microbatch=False,
                 current_microbatch=None):
    """One micro-batch forward.  ``forward_step_func(data_iterator, model) -> (output, loss_func)``;
    on the last stage ``loss_func(output) -> (loss, {name: value})`` or ``(loss, num_tokens, {...})``."""
    set_input_tensor(model, input_tensor)
    if current_microbatch is not None:
        _CURRENT["mb"] = current_microbatch
    ctx = torch.autocast("cuda", dtype=config.autocast_dtype) if getattr(config, "enable_autocast", False) else contextlib.nullcontext()
    with ctx:
        output_tensor, loss_func = forward_step_func(data_iterator, model)
    num_tokens = torch.tensor(0, dtype=torch.int)
    if ps.is_pipeline_last_stage():
        if not collect_non_loss_data:
            outputs = loss_func(output_tensor)
            # micro-batches of different sizes (--optimized-mbs-list) weigh in by their share of the step's samples
            sizes = getattr(config, "micro_batch_sizes", None)
            mb = _CURRENT.get("mb") if current_microbatch is None else current_microbatch
            share = (sizes[mb % len(sizes)] / sum(sizes)) if sizes and mb is not None else None
            if len(outputs) == 3:
                output_tensor, num_tokens, loss_reduced = outputs
                if not config.calculate_per_token_loss:
                    output_tensor = output_tensor / num_tokens.clamp(min=1)
                    output_tensor = output_tensor / num_microbatches if share is None else output_tensor * share
            else:
                output_tensor, loss_reduced = outputs
                output_tensor = output_tensor / num_microbatches if share is None else output_tensor * share
            forward_data_store.append(loss_reduced)
        else:
            forward_data_store.append(loss_func(output_tensor, non_loss_data=True))
    _set_aux_loss_scale(config, num_microbatches, output_tensor)
    return output_tensor, num_tokens


def _set_aux_loss_scale(config, num_microbatches, like):
    """Losses attached inside the model (MoE load balancing / z-loss, the sparse-attention indexer's KL loss) get the
    gradient scale of the main loss: the loss scaler's factor, divided by the micro-batch count when the main loss is
    averaged over micro-batches."""
    moe = getattr(config, "num_moe_experts", None) is not None
    dsa = getattr(config, "experimental_attention_variant", None) == "dsa"
    if not (moe or dsa):
        return
    dev = like.device if torch.is_tensor(like) else (like[0].device if like else "cpu")
    scale = torch.ones(1, device=dev)
    if getattr(config, "grad_scale_func", None) is not None:
        scale = config.grad_scale_func(scale)
    if not getattr(config, "calculate_per_token_loss", False):
        scale = scale / num_microbatches
    if moe:
        from ..moe.moe_utils import MoEAuxLossAutoScaler
        MoEAuxLossAutoScaler.set_loss_scale(scale)
    if dsa:
        from ...models.dsa import DSAIndexerLossScaler
        DSAIndexerLossScaler.set_loss_scale(scale)


_STORED_PLANS: dict = {}


def is_multi_parameter(config) -> bool:
    return bool(getattr(config, "use_multiparameter_pipeline_model_parallel", False)) and \
        bool(getattr(config, "pipeline_tensor_shapes", None))


def get_tensor_specs(*, seq_length, micro_batch_size, config):
    """[(shape, dtype)] of what one stage hands to the next: the [s, b, h] hidden state, or with
    ``--use-multiparameter-pipeline-model-parallel`` the entries of ``config.pipeline_tensor_shapes``
    ([{"shape": ..., "dtype": ...}], reference: mindspeed/features_manager/pipeline_parallel/multi_parameter.py:38-52)."""
    if is_multi_parameter(config):
        return [(tuple(d["shape"]), d["dtype"]) for d in config.pipeline_tensor_shapes]
    shape = get_tensor_shapes(seq_length=seq_length, micro_batch_size=micro_batch_size, config=config)[0]
    return [(shape, config.pipeline_dtype)]


def _backward_step_multi(inputs, outputs, output_grads, config):
    """Stage backward when the stage interface is a list of tensors: gradients flow through the floating-point entries
    (reference: mindspeed/core/pipeline_parallel/multiparameter_schedules.py:46-108)."""
    ins = [] if inputs is None else (list(inputs) if isinstance(inputs, (list, tuple)) else [inputs])
    outs = list(outputs) if isinstance(outputs, (list, tuple)) else [outputs]
    for x in ins:
        if x.is_floating_point() and x.requires_grad:
            x.retain_grad()
    if output_grads is None:
        loss = outs[0]
        if getattr(config, "grad_scale_func", None) is not None:
            loss = config.grad_scale_func(loss)
        loss.backward()
    else:
        grads = list(output_grads) if isinstance(output_grads, (list, tuple)) else [output_grads]
        fouts = [o for o in outs if o.is_floating_point()]
        pairs = [(o, g) for o, g in zip(fouts, grads) if o.requires_grad]
        torch.autograd.backward([p[0] for p in pairs], [p[1] for p in pairs])
    return [x.grad if x.grad is not None else torch.zeros_like(x) for x in ins if x.is_floating_point()]


def backward_step(input_tensor, output_tensor, output_tensor_grad, model_type, config):
    """Backward of one micro-batch; returns the gradient w.r.t. the stage input (None on the first stage)."""
    if isinstance(input_tensor, (list, tuple)) or isinstance(output_tensor, (list, tuple)):
        return _backward_step_multi(input_tensor, output_tensor, output_tensor_grad, config)
    if input_tensor is not None and input_tensor.requires_grad:
        input_tensor.retain_grad()
    if output_tensor_grad is None and getattr(config, "grad_scale_func", None) is not None:
        output_tensor = config.grad_scale_func(output_tensor)
    if output_tensor_grad is None:
        output_tensor.backward()
    else:
        torch.autograd.backward(output_tensor, grad_tensors=output_tensor_grad)
    g = None
    if input_tensor is not None:
        g = input_tensor.grad
    return g


def _no_sync(model, config):
    f = getattr(config, "no_sync_func", None)
    if f is not None:
        return f
    if isinstance(model, list):
        def multi():
            stack = contextlib.ExitStack()
            for m in model:
                if hasattr(m, "no_sync"):
                    stack.enter_context(m.no_sync())
            return stack
        return multi
    if hasattr(model, "no_sync"):
        return model.no_sync
    return contextlib.nullcontext


def forward_backward_no_pipelining(*, forward_step_func, data_iterator, model, num_microbatches, seq_length=None,
                                   micro_batch_size=None, decoder_seq_length=None, forward_only=False,
                                   collect_non_loss_data=False, first_val_step=None):
    if isinstance(model, list):
        model = model[0]
    if isinstance(data_iterator, list):
        data_iterator = data_iterator[0]
    config = _cfg(model)
    no_sync = _no_sync(model, config)
    store: List = []
    total_tokens = torch.zeros([], dtype=torch.int)
    if getattr(config, "moe_fb_overlap", False) and not forward_only and num_microbatches > 1:
        return _no_pipelining_fb_overlap(forward_step_func, data_iterator, model, num_microbatches, config, no_sync, store,
                                         total_tokens, collect_non_loss_data)
    with no_sync():
        for i in range(num_microbatches - 1):
            out, nt = forward_step(forward_step_func, data_iterator, model, num_microbatches, None, store, config,
                                   collect_non_loss_data, is_first_microbatch=(i == 0), current_microbatch=i)
            total_tokens += nt.cpu() if torch.is_tensor(nt) else nt
            if not forward_only:
                backward_step(None, out, None, None, config)
    out, nt = forward_step(forward_step_func, data_iterator, model, num_microbatches, None, store, config,
                           collect_non_loss_data, is_first_microbatch=(num_microbatches == 1),
                           current_microbatch=num_microbatches - 1)
    total_tokens += nt.cpu() if torch.is_tensor(nt) else nt
    if not forward_only:
        backward_step(None, out, None, None, config)
        fin = getattr(config, "finalize_model_grads_func", None)
        if fin is not None:
            fin([model], total_tokens.to(out.device) if config.calculate_per_token_loss else None)
    return store


def _no_pipelining_fb_overlap(forward_step_func, data_iterator, model, num_microbatches, config, no_sync, store, total_tokens,
                              collect_non_loss_data):
    """``--moe-fb-overlap`` without pipeline parallelism: the layer stack runs micro-batch i's forward interleaved, stage
    by stage, with micro-batch i-1's backward, so each all-to-all of one hides under the attention / expert compute of the
    other (reference: mindspeed/core/transformer/moe/moe_feature/fb_overlap/overlap_funcs/fwdbwd.py:37-380).

    The loss backward of a micro-batch only reaches the detached output of the layer stack; the stack's own backward is
    run by the next forward (or by ``finish``).  Every backward except the last micro-batch's runs under ``no_sync``."""
    from ...models.transformer import TransformerBlock
    from ..moe.fb_overlap import BlockOverlap
    block = next(m for m in model.modules() if isinstance(m, TransformerBlock))
    block.fb_overlap = BlockOverlap(block.layers)
    try:
        with no_sync():
            for i in range(num_microbatches):
                out, nt = forward_step(forward_step_func, data_iterator, model, num_microbatches, None, store, config,
                                       collect_non_loss_data, is_first_microbatch=(i == 0), current_microbatch=i)
                total_tokens += nt.cpu() if torch.is_tensor(nt) else nt
                if i < num_microbatches - 1:
                    backward_step(None, out, None, None, config)
        backward_step(None, out, None, None, config)
        block.fb_overlap.finish()
    finally:
        block.fb_overlap = None
    fin = getattr(config, "finalize_model_grads_func", None)
    if fin is not None:
        fin([model], total_tokens.to(out.device) if config.calculate_per_token_loss else None)
    return store


def get_tensor_shapes(*, seq_length, micro_batch_size, config, decoder_seq_length=None):
    s = seq_length // ps.get_context_parallel_world_size()
    if config.sequence_parallel:
        s //= ps.get_tensor_model_parallel_world_size()
    if getattr(config, "tp_2d", False):            # stages hand over the [s/x, b, h/y] tile
        return [(s // config.tp_x, micro_batch_size, config.hidden_size // config.tp_y)]
    return [(s, micro_batch_size, config.hidden_size)]


def forward_backward_pipelining_without_interleaving(*, forward_step_func, data_iterator, model, num_microbatches,
                                                     seq_length, micro_batch_size, decoder_seq_length=None,
                                                     forward_only=False, collect_non_loss_data=False, first_val_step=None):
    """Non-interleaved 1F1B: warm-up forwards, steady 1F1B, cool-down backwards."""
    stored = getattr(_cfg(model), "pp_schedule", None)
    if stored and not forward_only:
        # --pp-schedule-list: the order of forward and backward steps per rank is given; run it as a plan
        from .executor import run_plan
        from .plan import plan_from_stage_lists
        key = (ps.get_pipeline_model_parallel_world_size(), num_microbatches, id(stored))
        if key not in _STORED_PLANS:
            _STORED_PLANS[key] = plan_from_stage_lists(key[0], num_microbatches, stored)
        return run_plan(_STORED_PLANS[key], forward_step_func=forward_step_func, data_iterator=data_iterator, model=model,
                        num_microbatches=num_microbatches, seq_length=seq_length, micro_batch_size=micro_batch_size,
                        forward_only=forward_only, collect_non_loss_data=collect_non_loss_data)
    if is_multi_parameter(_cfg(model)) or (getattr(_cfg(model), "moe_fb_overlap", False) and not forward_only) \
            or getattr(_cfg(model), "micro_batch_sizes", None):
        # list-valued stage interfaces and forward/backward overlap are handled by the plan executor (same 1F1B order, as data)
        from .executor import run_plan
        from .interleaved import _plan
        plan = _plan("1f1b", ps.get_pipeline_model_parallel_world_size(), num_microbatches)
        return run_plan(plan, forward_step_func=forward_step_func, data_iterator=data_iterator, model=model,
                        num_microbatches=num_microbatches, seq_length=seq_length, micro_batch_size=micro_batch_size,
                        forward_only=forward_only, collect_non_loss_data=collect_non_loss_data)
    if isinstance(model, list):
        model = model[0]
    if isinstance(data_iterator, list):
        data_iterator = data_iterator[0]
    config = _cfg(model)
    no_sync = _no_sync(model, config)
    pp, rank = ps.get_pipeline_model_parallel_world_size(), ps.get_pipeline_model_parallel_rank()
    warm = min(pp - rank - 1, num_microbatches)
    remaining = num_microbatches - warm
    shapes = get_tensor_shapes(seq_length=seq_length, micro_batch_size=micro_batch_size, config=config)
    store: List = []
    inputs, outputs = [], []
    total_tokens = torch.zeros([], dtype=torch.int)
    sync_ctx = None

    def disable_sync():
        nonlocal sync_ctx
        if sync_ctx is None:
            sync_ctx = no_sync()
            sync_ctx.__enter__()

    def enable_sync():
        nonlocal sync_ctx
        if sync_ctx is not None:
            sync_ctx.__exit__(None, None, None)
            sync_ctx = None

    disable_sync()
    for i in range(warm):
        inp = p2p.recv_forward(shapes, config)
        out, nt = forward_step(forward_step_func, data_iterator, model, num_microbatches, inp, store, config,
                               collect_non_loss_data, is_first_microbatch=(i == 0), current_microbatch=i)
        p2p.send_forward(out, config)
        total_tokens += nt.cpu() if torch.is_tensor(nt) else nt
        if not forward_only:
            inputs.append(inp)
            outputs.append(out)
    if remaining > 0:
        inp = p2p.recv_forward(shapes, config)
    for i in range(remaining):
        last = i == remaining - 1
        out, nt = forward_step(forward_step_func, data_iterator, model, num_microbatches, inp, store, config,
                               collect_non_loss_data, is_first_microbatch=(i == 0 and warm == 0),
                               current_microbatch=i + warm)
        total_tokens += nt.cpu() if torch.is_tensor(nt) else nt
        if forward_only:
            p2p.send_forward(out, config)
            if not last:
                inp = p2p.recv_forward(shapes, config)
            continue
        out_grad = p2p.send_forward_recv_backward(out, shapes, config)
        inputs.append(inp)
        outputs.append(out)
        inp_b, out_b = inputs.pop(0), outputs.pop(0)
        if warm == 0 and last:
            enable_sync()
        g = backward_step(inp_b, out_b, out_grad, None, config)
        if last:
            inp = None
            p2p.send_backward(g, config)
        else:
            inp = p2p.send_backward_recv_forward(g, shapes, config)
    if not forward_only:
        for i in range(warm):
            if i == warm - 1:
                enable_sync()
            inp_b, out_b = inputs.pop(0), outputs.pop(0)
            out_grad = p2p.recv_backward(shapes, config)
            g = backward_step(inp_b, out_b, out_grad, None, config)
            p2p.send_backward(g, config)
        enable_sync()
        fin = getattr(config, "finalize_model_grads_func", None)
        if fin is not None:
            fin([model], total_tokens if config.calculate_per_token_loss else None)
    else:
        enable_sync()
    return store


def forward_backward_pipelining_with_interleaving(*, forward_step_func, data_iterator, model, num_microbatches,
                                                  seq_length, micro_batch_size, decoder_seq_length=None,
                                                  forward_only=False, collect_non_loss_data=False, first_val_step=None):
    from .interleaved import forward_backward_interleaved
    return forward_backward_interleaved(forward_step_func=forward_step_func, data_iterator=data_iterator, model=model,
                                        num_microbatches=num_microbatches, seq_length=seq_length,
                                        micro_batch_size=micro_batch_size, forward_only=forward_only,
                                        collect_non_loss_data=collect_non_loss_data)
