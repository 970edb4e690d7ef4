"""Several sub-models (e.g. a vision encoder and a language model) on disjoint rank ranges of one job, each with its
own tensor / pipeline / context parallel grid, exchanging activations and gradients across the model boundary.

  initialize_dist_train(cfg)   every rank builds the groups of every sub-model (group creation is collective) and keeps
                               the parallel state of the sub-model it belongs to, so ``parallel_state`` getters answer
                               for "my" sub-model afterwards.
  boundary exchange            last pipeline stage of model i  <->  first pipeline stage of model i+1.  When the two
                               sides have different numbers of boundary ranks n_src / n_dst:
                                 n_src <= n_dst   each source feeds n_dst / n_src destinations (same tensor); the
                                                  gradients coming back are summed
                                 n_src >  n_dst   each destination receives n_src / n_dst tensors and concatenates them
                                                  along ``concat_dim`` (batch); the gradient is split the same way
                               Every message is preceded by a fixed int64 header (dtype code, requires_grad, ndim,
                               shape) so the receiver can allocate without prior agreement on shapes.
  dist_forward_backward        non-pipelined schedule over micro-batches for the two roles (producer / consumer).

reference: mindspeed/core/multi_modal/dist_train/dist_parallel_state.py:137-1706 (per-model groups),
dist_communication.py:18-197 (header protocol, send/recv lists), dist_schedules.py:32-589 (schedules).
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import parallel_state as ps

HEADER_LEN = 12
_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int64, torch.int32, torch.int16, torch.int8,
           torch.uint8, torch.bool]
_DTYPE_CODE = {d: i for i, d in enumerate(_DTYPES)}


@dataclasses.dataclass
class SubModelConfig:
    name: str
    world_size: int
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    context_parallel_size: int = 1
    forward_only: bool = False
    main_dp: bool = False            # the sub-model whose data-parallel ranks load the data
    model_index: int = 0
    start_rank: int = 0


@dataclasses.dataclass
class DistTrainConfig:
    models: List[SubModelConfig]

    def validate(self, world: int) -> "DistTrainConfig":
        if not self.models:
            raise ValueError("dist-train needs at least one sub-model")
        start = 0
        for i, m in enumerate(self.models):
            m.model_index, m.start_rank = i, start
            mp = m.tensor_model_parallel_size * m.pipeline_model_parallel_size * m.context_parallel_size
            if m.world_size % mp != 0:
                raise ValueError(f"sub-model {m.name}: world_size {m.world_size} not divisible by tp*pp*cp = {mp}")
            start += m.world_size
        if start != world:
            raise ValueError(f"sub-model world sizes sum to {start}, the job has {world} ranks")
        if sum(1 for m in self.models if m.main_dp) > 1:
            raise ValueError("only one sub-model can be main_dp")
        names = [m.name for m in self.models]
        if len(set(names)) != len(names):
            raise ValueError("sub-model names must be unique")
        return self

    @staticmethod
    def from_list(items: Sequence[Dict]) -> "DistTrainConfig":
        return DistTrainConfig([SubModelConfig(**d) for d in items])


class _DistState:
    def __init__(self):
        self.cfg: Optional[DistTrainConfig] = None
        self.index: int = -1
        self.states: List[object] = []
        self.boundary: Dict[int, List[int]] = {}      # model index -> (first-stage ranks, last-stage ranks)
        self.first: Dict[int, List[int]] = {}
        self.last: Dict[int, List[int]] = {}


_D = _DistState()


def initialize_dist_train(cfg: DistTrainConfig, **extra_init_kwargs) -> None:
    world, rank = dist.get_world_size(), dist.get_rank()
    cfg.validate(world)
    _D.cfg, _D.states = cfg, []
    for m in cfg.models:
        ps.swap_state(None)
        ps.initialize_model_parallel(tensor_model_parallel_size=m.tensor_model_parallel_size,
                                     pipeline_model_parallel_size=m.pipeline_model_parallel_size,
                                     context_parallel_size=m.context_parallel_size, rank_offset=m.start_rank,
                                     sub_world_size=m.world_size, **extra_init_kwargs)
        st = ps.swap_state(None)
        _D.states.append(st)
        pp_groups = st.all_groups["pp"]
        _D.first[m.model_index] = sorted(g[0] for g in pp_groups)
        _D.last[m.model_index] = sorted(g[-1] for g in pp_groups)
        if m.start_rank <= rank < m.start_rank + m.world_size:
            _D.index = m.model_index
    ps.swap_state(_D.states[_D.index])


def destroy_dist_train():
    global _D
    for i, st in enumerate(_D.states):
        ps.swap_state(st)
        ps.destroy_model_parallel()
    _D = _DistState()


def get_dist_model_index(rank: Optional[int] = None) -> int:
    if rank is None:
        return _D.index
    for m in _D.cfg.models:
        if m.start_rank <= rank < m.start_rank + m.world_size:
            return m.model_index
    raise ValueError(f"rank {rank} belongs to no sub-model")


def get_dist_model_config(name: Optional[str] = None, index: Optional[int] = None) -> SubModelConfig:
    if name is not None:
        for m in _D.cfg.models:
            if m.name == name:
                return m
        raise KeyError(name)
    return _D.cfg.models[_D.index if index is None else index]


def is_in_model(name: str) -> bool:
    return get_dist_model_config(name).model_index == _D.index


# ---- boundary peers ------------------------------------------------------------------------------------------
def _peers(src_ranks: List[int], dst_ranks: List[int], me: int, i_am_src: bool) -> List[int]:
    ns, nd = len(src_ranks), len(dst_ranks)
    if ns <= nd:
        if nd % ns != 0:
            raise ValueError(f"boundary sizes {ns} -> {nd} must divide")
        f = nd // ns
        if i_am_src:
            k = src_ranks.index(me)
            return dst_ranks[k * f:(k + 1) * f]
        return [src_ranks[dst_ranks.index(me) // f]]
    if ns % nd != 0:
        raise ValueError(f"boundary sizes {ns} -> {nd} must divide")
    f = ns // nd
    if i_am_src:
        return [dst_ranks[src_ranks.index(me) // f]]
    k = dst_ranks.index(me)
    return src_ranks[k * f:(k + 1) * f]


def _on_boundary(kind: str) -> bool:
    r = dist.get_rank()
    return r in (_D.last if kind == "last" else _D.first)[_D.index]


# ---- header protocol -----------------------------------------------------------------------------------------
def encode_header(t: Optional[torch.Tensor]) -> torch.Tensor:
    h = [0] * HEADER_LEN
    if t is None:
        h[0] = -1
        return torch.tensor(h, dtype=torch.int64)
    if t.dim() > HEADER_LEN - 3:
        raise ValueError(f"tensors of more than {HEADER_LEN - 3} dimensions cannot cross a model boundary")
    h[0], h[1], h[2] = _DTYPE_CODE[t.dtype], int(t.requires_grad), t.dim()
    h[3:3 + t.dim()] = list(t.shape)
    return torch.tensor(h, dtype=torch.int64)


def decode_header(h: torch.Tensor):
    v = h.tolist()
    if v[0] == -1:
        return None
    return _DTYPES[v[0]], bool(v[1]), tuple(v[3:3 + v[2]])


def _device():
    return torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")


def _send(t: Optional[torch.Tensor], dst: int):
    dist.send(encode_header(t).to(_device()), dst)
    if t is not None:
        dist.send(t.detach().contiguous(), dst)


def _recv(src: int) -> Optional[torch.Tensor]:
    h = torch.empty(HEADER_LEN, dtype=torch.int64, device=_device())
    dist.recv(h, src)
    meta = decode_header(h.cpu())
    if meta is None:
        return None
    dtype, rg, shape = meta
    t = torch.empty(shape, dtype=dtype, device=_device())
    dist.recv(t, src)
    if rg and t.is_floating_point():
        t.requires_grad_(True)
    return t


# ---- public exchange -----------------------------------------------------------------------------------------
def send_to_next_model(t: torch.Tensor) -> None:
    """Called on the last pipeline stage of model i (no-op elsewhere or for the last model)."""
    i = _D.index
    if i + 1 >= len(_D.cfg.models) or not _on_boundary("last"):
        return
    for d in _peers(_D.last[i], _D.first[i + 1], dist.get_rank(), True):
        _send(t, d)


def recv_from_previous_model(concat_dim: int = 0) -> Optional[torch.Tensor]:
    """Called on the first pipeline stage of model i > 0; returns a leaf tensor (requires_grad as sent)."""
    i = _D.index
    if i == 0 or not _on_boundary("first"):
        return None
    parts = [_recv(s) for s in _peers(_D.last[i - 1], _D.first[i], dist.get_rank(), False)]
    if len(parts) == 1:
        return parts[0]
    rg = any(p.requires_grad for p in parts)
    out = torch.cat([p.detach() for p in parts], dim=concat_dim)
    return out.requires_grad_(rg) if rg else out


def send_grad_to_previous_model(grad: Optional[torch.Tensor], concat_dim: int = 0) -> None:
    i = _D.index
    if i == 0 or not _on_boundary("first"):
        return
    srcs = _peers(_D.last[i - 1], _D.first[i], dist.get_rank(), False)
    if len(srcs) == 1:
        _send(grad, srcs[0])
        return
    chunks = grad.chunk(len(srcs), dim=concat_dim) if grad is not None else [None] * len(srcs)
    for s, g in zip(srcs, chunks):
        _send(g, s)


def recv_grad_from_next_model() -> Optional[torch.Tensor]:
    i = _D.index
    if i + 1 >= len(_D.cfg.models) or not _on_boundary("last"):
        return None
    total = None
    for d in _peers(_D.last[i], _D.first[i + 1], dist.get_rank(), True):
        g = _recv(d)
        if g is not None:
            total = g if total is None else total + g
    return total


def dist_forward_backward(forward_step: Callable, data_iterator, model, num_microbatches: int, forward_only: bool = False,
                          concat_dim: int = 0) -> List[torch.Tensor]:
    """Non-pipelined schedule for one sub-model of a chain.

    ``forward_step(batch, model, boundary_input)`` returns the boundary output (intermediate models) or the loss
    (last model).  Producers send their output and later receive its gradient; consumers receive, run, and return
    the gradient of what they received.  Returns the list of losses (last model) or an empty list.
    """
    cfg = get_dist_model_config()
    last_model = _D.index == len(_D.cfg.models) - 1
    fwd_only = forward_only or cfg.forward_only
    losses, pending = [], []
    for _ in range(num_microbatches):
        batch = next(data_iterator) if data_iterator is not None else None
        x = recv_from_previous_model(concat_dim)
        ctx = torch.no_grad() if fwd_only else torch.enable_grad()
        with ctx:
            out = forward_step(batch, model, x)
        if last_model:
            losses.append(out.detach())
            if not fwd_only:
                (out / num_microbatches).backward()
            send_grad_to_previous_model(x.grad if (x is not None and x.requires_grad and not fwd_only) else None, concat_dim)
        else:
            send_to_next_model(out if not fwd_only else out.detach())
            pending.append((out, x))
            # one-in-flight: take the gradient back right away (the consumer is non-pipelined as well)
            g = recv_grad_from_next_model()
            o, xin = pending.pop()
            if not fwd_only and g is not None and o.requires_grad:
                o.backward(g)
            send_grad_to_previous_model(xin.grad if (xin is not None and xin.requires_grad and not fwd_only) else None, concat_dim)
    return losses
