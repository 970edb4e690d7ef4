"""Process-group topology for tensor / context / expert / data / pipeline parallelism.

One process drives one GPU (or one CPU rank under gloo).  The world is factored
as ``tp x cp x dp x pp`` for the dense part of the model and ``etp x ep x edp x pp``
for the expert part, following the Megatron-core ``order`` string convention
("tp-cp-ep-dp-pp": the left-most dimension varies fastest across ranks).  On top
of the Megatron-compatible getters this module creates, as first-class groups,
everything the reference bolts on afterwards through wrappers:

* a twin context-parallel group so that send and receive of a ring step travel
  on independent communicators   (reference: mindspeed/core/context_parallel/model_parallel_utils.py:22-56)
* hybrid Ulysses x ring sub-groups (reference: model_parallel_utils.py:59-118)
* double-ring window ranks         (reference: model_parallel_utils.py:121-212)
* 2-D tensor parallel tp-x / tp-y  (reference: mindspeed/core/tensor_parallel/tp_2d/parallel_state_2d.py:56-117)
* a second pipeline group for p2p on its own stream
                                   (reference: mindspeed/core/pipeline_parallel/optimize_send_recv_comm/parallel_state.py:15-66)
* optional removal of the gloo twins (reference: mindspeed/core/parallel_state.py:1077-1119)

Inside one NVSwitch domain every peer is one hop away, so none of the groups is
ordered for link locality; group membership is pure index arithmetic and can be
evaluated without any process group (``RankGenerator`` is usable on its own, which
is what the single-process tests and ``auto_settings`` do).
"""
from __future__ import annotations

import itertools
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

__all__ = [
    "RankGenerator",
    "initialize_model_parallel",
    "destroy_model_parallel",
    "model_parallel_is_initialized",
    "is_initialized",
]


# --------------------------------------------------------------------------------------
# Pure index arithmetic
# --------------------------------------------------------------------------------------
def _decompose(index: int, shape: Sequence[int]) -> List[int]:
    """Mixed-radix digits of ``index`` with shape[0] the fastest-varying digit."""
    out = []
    for s in shape:
        out.append(index % s)
        index //= s
    return out


def _compose(digits: Sequence[int], shape: Sequence[int]) -> int:
    idx, mul = 0, 1
    for d, s in zip(digits, shape):
        idx += d * mul
        mul *= s
    return idx


class RankGenerator:
    """Enumerates rank groups of a mixed-radix rank grid.

    ``order`` names the dimensions from fastest- to slowest-varying.  A token such
    as ``"tp-cp"`` asks for the groups obtained by letting tp and cp vary while all
    other coordinates are fixed.
    """

    def __init__(self, tp: int, ep: int, dp: int, pp: int, cp: int, order: str = "tp-cp-ep-dp-pp", rank_offset: int = 0):
        sizes = {"tp": tp, "ep": ep, "dp": dp, "pp": pp, "cp": cp}
        names = [n for n in order.split("-")]
        for n, s in sizes.items():
            if n not in names:
                if s != 1:
                    raise ValueError(f"dimension {n} has size {s} but is absent from order '{order}'")
                names.append(n)
        self.names = names
        self.sizes = [sizes[n] for n in names]
        self.world_size = 1
        for s in self.sizes:
            self.world_size *= s
        self.rank_offset = rank_offset
        self.tp, self.ep, self.dp, self.pp, self.cp = tp, ep, dp, pp, cp
        self.order = "-".join(names)

    def get_ranks(self, token: str) -> List[List[int]]:
        want = token.split("-")
        for w in want:
            if w not in self.names:
                raise ValueError(f"unknown dimension {w}")
        vary = [i for i, n in enumerate(self.names) if n in want]
        fixed = [i for i, n in enumerate(self.names) if n not in want]
        vary_shape = [self.sizes[i] for i in vary]
        fixed_shape = [self.sizes[i] for i in fixed]
        n_vary = 1
        for s in vary_shape:
            n_vary *= s
        n_fixed = self.world_size // n_vary
        groups = []
        for f in range(n_fixed):
            fd = _decompose(f, fixed_shape)
            ranks = []
            for v in range(n_vary):
                vd = _decompose(v, vary_shape)
                digits = [0] * len(self.names)
                for i, d in zip(fixed, fd):
                    digits[i] = d
                for i, d in zip(vary, vd):
                    digits[i] = d
                ranks.append(_compose(digits, self.sizes) + self.rank_offset)
            groups.append(ranks)
        return groups

    def coords(self, rank: int) -> Dict[str, int]:
        return dict(zip(self.names, _decompose(rank - self.rank_offset, self.sizes)))


# --------------------------------------------------------------------------------------
# Group registry
# --------------------------------------------------------------------------------------
@dataclass
class _Group:
    ranks: List[int]
    group: object = None  # torch ProcessGroup or None (single-process evaluation)

    @property
    def size(self) -> int:
        return len(self.ranks)


@dataclass
class _State:
    initialized: bool = False
    groups: Dict[str, _Group] = field(default_factory=dict)
    all_groups: Dict[str, List[List[int]]] = field(default_factory=dict)
    sizes: Dict[str, int] = field(default_factory=dict)
    vpp_rank: Optional[int] = None
    vpp_world: Optional[int] = None
    pp_split_rank: Optional[int] = None
    embedding_ranks: List[int] = field(default_factory=list)
    position_embedding_ranks: List[int] = field(default_factory=list)
    override_rank: Dict[str, Optional[int]] = field(default_factory=dict)
    override_world: Dict[str, Optional[int]] = field(default_factory=dict)
    rank: int = 0
    world: int = 1
    rank_offset: int = 0          # first global rank of this (sub-)world; generators work in sub-world-local ranks
    global_memory_buffer: object = None
    moe_tracker: dict = field(default_factory=dict)
    disable_gloo: bool = False
    dense_gen: Optional[RankGenerator] = None
    expert_gen: Optional[RankGenerator] = None


_S = _State()


def _world_info():
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def _new_group(ranks, backend=None, timeout=None, pg_options=None):
    """Collective across the whole world: every rank calls it for every group, in the same order."""
    if not (dist.is_available() and dist.is_initialized()):
        return None
    if backend == "gloo" and _S.disable_gloo:
        return None
    kwargs = {}
    if timeout is not None:
        kwargs["timeout"] = timeout
    if pg_options is not None:
        kwargs["pg_options"] = pg_options
    if backend is not None:
        kwargs["backend"] = backend
    return dist.new_group(ranks, **kwargs)


def _register(name: str, all_ranks: List[List[int]], backend=None, timeout=None, make_group=True, pg_options=None):
    """Create one process group per rank list; remember the one this rank is in."""
    if _S.rank_offset:
        all_ranks = [[r + _S.rank_offset for r in ranks] for ranks in all_ranks]
    _S.all_groups[name] = all_ranks
    mine = None
    for ranks in all_ranks:
        g = _new_group(ranks, backend=backend, timeout=timeout, pg_options=pg_options) if make_group else None
        if _S.rank in ranks:
            mine = _Group(list(ranks), g)
    if mine is not None:
        _S.groups[name] = mine
    return mine


def get_nccl_options(pg_name: str, nccl_comm_cfgs: dict):
    """Per-group NCCL options (cga cluster size, max/min CTAs) from a config dict.

    Mirrors Megatron-core's ``get_nccl_options``; the reference additionally
    threads a per-group buffer size through it (mindspeed/core/hccl_buffer/adaptor.py:16-57).
    On NVSwitch the interesting knobs are the CTA counts (how many SMs a
    collective may take away from an overlapped GEMM).
    """
    if pg_name in nccl_comm_cfgs and torch.cuda.is_available():
        opts = dist.ProcessGroupNCCL.Options()
        cfg = nccl_comm_cfgs[pg_name]
        opts.config.cga_cluster_size = cfg.get("cga_cluster_size", 4)
        opts.config.max_ctas = cfg.get("max_ctas", 32)
        opts.config.min_ctas = cfg.get("min_ctas", 1)
        return opts
    return None


def initialize_model_parallel(
    tensor_model_parallel_size: int = 1,
    pipeline_model_parallel_size: int = 1,
    virtual_pipeline_model_parallel_size: Optional[int] = None,
    pipeline_model_parallel_split_rank: Optional[int] = None,
    use_sharp: bool = False,
    context_parallel_size: int = 1,
    hierarchical_context_parallel_sizes: Optional[List[int]] = None,
    expert_model_parallel_size: int = 1,
    num_distributed_optimizer_instances: int = 1,
    expert_tensor_parallel_size: Optional[int] = None,
    nccl_communicator_config_path: Optional[str] = None,
    distributed_timeout_minutes: int = 30,
    order: str = "tp-cp-ep-dp-pp",
    encoder_tensor_model_parallel_size: int = 0,
    encoder_pipeline_model_parallel_size: int = 0,
    get_embedding_ranks=None,
    get_position_embedding_ranks=None,
    create_gloo_process_groups: bool = True,
    # ---- first-class extras (wrappers in the reference) ----
    use_cp_send_recv_overlap: bool = False,
    ulysses_degree_in_cp: Optional[int] = None,
    cp_window_size: int = 1,
    tp_2d: bool = False,
    tp_x: int = 1,
    tp_y: int = 1,
    optimize_send_recv_comm: bool = False,
    world_size: Optional[int] = None,
    rank: Optional[int] = None,
    rank_offset: int = 0,
    sub_world_size: Optional[int] = None,
) -> None:
    """Build every parallel group.  Signature follows Megatron-core 0.12 ``initialize_model_parallel``.

    ``world_size``/``rank`` may be passed explicitly to evaluate the topology in a
    single process without ``torch.distributed`` (no communicators are created then).
    ``rank_offset``/``sub_world_size`` lay the grid over the global ranks ``[offset, offset + size)`` only (one
    sub-model of a multi-model job); every rank of the job still has to make the call, because group creation is
    collective, and ranks outside the range simply end up without groups.
    """
    import datetime

    if _S.initialized:
        raise RuntimeError("model parallel groups are already initialized")
    r, w = _world_info()
    _S.rank = r if rank is None else rank
    _S.world = w if world_size is None else world_size
    if sub_world_size is not None:
        _S.world = sub_world_size
    _S.rank_offset = rank_offset
    make = dist.is_available() and dist.is_initialized() and world_size is None
    _S.disable_gloo = not create_gloo_process_groups
    timeout = datetime.timedelta(minutes=distributed_timeout_minutes) if make else None

    tp, pp, cp, ep = tensor_model_parallel_size, pipeline_model_parallel_size, context_parallel_size, expert_model_parallel_size
    etp = tp if expert_tensor_parallel_size is None else expert_tensor_parallel_size
    model_size = tp * pp * cp
    if _S.world % model_size != 0:
        raise RuntimeError(f"world_size ({_S.world}) is not divisible by tp*pp*cp ({model_size})")
    dp = _S.world // model_size
    expert_model_size = etp * ep * pp
    if _S.world % expert_model_size != 0:
        raise RuntimeError(f"world_size ({_S.world}) is not divisible by etp*ep*pp ({expert_model_size})")
    edp = _S.world // expert_model_size
    if virtual_pipeline_model_parallel_size is not None:
        if pp < 2:
            raise RuntimeError("interleaved schedule needs pipeline_model_parallel_size >= 2")
        _S.vpp_rank, _S.vpp_world = 0, virtual_pipeline_model_parallel_size
    _S.pp_split_rank = pipeline_model_parallel_split_rank

    dense = RankGenerator(tp=tp, ep=1, dp=dp, pp=pp, cp=cp, order=order)
    expert = RankGenerator(tp=etp, ep=ep, dp=edp, pp=pp, cp=1, order=order)
    _S.dense_gen, _S.expert_gen = dense, expert
    if dense.get_ranks("pp") != expert.get_ranks("pp"):
        raise RuntimeError("dense and expert rank grids disagree on pipeline groups")
    _S.sizes = dict(tp=tp, pp=pp, cp=cp, dp=dp, ep=ep, etp=etp, edp=edp)

    # Per-group NCCL settings: a YAML file ({group name: {max_ctas, min_ctas, cga_cluster_size}}) over these defaults.
    # The pipeline groups carry point-to-point transfers that are posted ahead of time and then wait for the peer while
    # this GPU computes; a waiting NCCL kernel holds its thread blocks, so those groups get few of them.
    nccl_cfgs = {"pp": {"max_ctas": 8, "cga_cluster_size": 2}, "pp_new_stream": {"max_ctas": 8, "cga_cluster_size": 2}}
    if nccl_communicator_config_path:
        import yaml
        with open(nccl_communicator_config_path) as f:
            nccl_cfgs.update(yaml.safe_load(f) or {})
    on_nccl = make and torch.cuda.is_available() and dist.get_backend() == "nccl"

    def reg(name, ranks, backend=None):
        opts = get_nccl_options(name, nccl_cfgs) if (on_nccl and backend is None) else None
        return _register(name, ranks, backend=backend, timeout=timeout, make_group=make, pg_options=opts)

    # data parallel (+ gloo twin, + with context parallel)
    reg("dp", dense.get_ranks("dp"))
    if create_gloo_process_groups:
        reg("dp_gloo", dense.get_ranks("dp"), backend="gloo")
    reg("dp_cp", dense.get_ranks("dp-cp"))
    if create_gloo_process_groups:
        reg("dp_cp_gloo", dense.get_ranks("dp-cp"), backend="gloo")

    # partial data parallel: several distributed-optimizer instances inside dp-cp
    dp_cp_groups = dense.get_ranks("dp-cp")
    n_inst = num_distributed_optimizer_instances
    if (dp * cp) % n_inst != 0:
        raise RuntimeError("dp*cp must be divisible by num_distributed_optimizer_instances")
    intra, inter = [], []
    per = dp * cp // n_inst
    for ranks in dp_cp_groups:
        for i in range(n_inst):
            intra.append(ranks[i * per:(i + 1) * per])
        for j in range(per):
            inter.append(ranks[j::per])
    reg("intra_partial_dp_cp", intra)
    if n_inst > 1:
        reg("inter_partial_dp_cp", inter)

    # context parallel
    reg("cp", dense.get_ranks("cp"))
    if use_cp_send_recv_overlap:
        reg("cp_overlap", dense.get_ranks("cp"))
    if hierarchical_context_parallel_sizes:
        prod = 1
        for s in hierarchical_context_parallel_sizes:
            prod *= s
        if prod != cp:
            raise RuntimeError("hierarchical_context_parallel_sizes must multiply to context_parallel_size")
        for lvl, ranks_lvl in enumerate(_hierarchical_groups(dense.get_ranks("cp"), hierarchical_context_parallel_sizes)):
            reg(f"hcp{lvl}", ranks_lvl)
        _S.sizes["hcp_levels"] = len(hierarchical_context_parallel_sizes)

    # hybrid context parallel: ulysses (contiguous) x ring (strided)
    if ulysses_degree_in_cp is not None and cp > 1:
        u = ulysses_degree_in_cp
        if cp % u != 0:
            raise RuntimeError("context_parallel_size must be divisible by ulysses_degree_in_cp")
        uly, ring = [], []
        for ranks in dense.get_ranks("cp"):
            for i in range(cp // u):
                uly.append(ranks[i * u:(i + 1) * u])
            for j in range(u):
                ring.append(ranks[j::u])
        reg("cp_ulysses", uly)
        reg("cp_ring", ring)
        if use_cp_send_recv_overlap:
            reg("cp_ring_overlap", ring)
        _S.sizes["cp_ulysses"], _S.sizes["cp_ring"] = u, cp // u

    # double ring windows
    ring_size = _S.sizes.get("cp_ring", cp)
    if cp_window_size > 1:
        if ring_size % cp_window_size != 0 or not (1 <= cp_window_size < ring_size):
            raise RuntimeError("cp_window_size must divide the ring size and be smaller than it")
    _S.sizes["cp_window"] = cp_window_size

    # model parallel, tensor parallel, pipeline parallel
    reg("mp", dense.get_ranks("tp-pp"))
    reg("tp", dense.get_ranks("tp"))
    reg("pp", dense.get_ranks("pp"))
    if optimize_send_recv_comm and pp > 1:
        reg("pp_new_stream", dense.get_ranks("pp"))

    # embedding groups (first & last pipeline stage, plus split rank)
    emb_all, pos_all = [], []
    for ranks in dense.get_ranks("pp"):
        if get_embedding_ranks is not None:
            e = get_embedding_ranks(ranks, pipeline_model_parallel_split_rank)
        else:
            e = _default_embedding_ranks(ranks, pipeline_model_parallel_split_rank)
        if get_position_embedding_ranks is not None:
            p = get_position_embedding_ranks(ranks, pipeline_model_parallel_split_rank)
        else:
            p = _default_position_embedding_ranks(ranks, pipeline_model_parallel_split_rank)
        emb_all.append(e)
        pos_all.append(p)
        if _S.rank - _S.rank_offset in ranks:
            _S.embedding_ranks = [x + _S.rank_offset for x in e]
            _S.position_embedding_ranks = [x + _S.rank_offset for x in p]
    reg("embd", emb_all)
    reg("pos_embd", pos_all)

    reg("tp_dp_cp", dense.get_ranks("tp-dp-cp"))
    reg("tp_dp", dense.get_ranks("tp-dp"))
    reg("tp_cp", dense.get_ranks("tp-cp"))
    # amax reduction group for fp8 delayed scaling = tp x cp
    _S.all_groups["amax"] = _S.all_groups["tp_cp"]
    if "tp_cp" in _S.groups:
        _S.groups["amax"] = _S.groups["tp_cp"]

    # expert groups
    reg("ep", expert.get_ranks("ep"))
    reg("etp", expert.get_ranks("tp"))
    reg("etp_ep", expert.get_ranks("tp-ep"))
    reg("etp_ep_pp", expert.get_ranks("tp-ep-pp"))
    reg("edp", expert.get_ranks("dp"))
    if create_gloo_process_groups:
        reg("edp_gloo", expert.get_ranks("dp"), backend="gloo")

    # 2-D tensor parallel: tp = tp_x * tp_y, x fastest
    if tp_2d:
        if tp_x * tp_y != tp:
            raise RuntimeError("tp_x * tp_y must equal tensor_model_parallel_size")
        xs, ys = [], []
        for ranks in dense.get_ranks("tp"):
            for j in range(tp_y):
                xs.append(ranks[j * tp_x:(j + 1) * tp_x])
            for i in range(tp_x):
                ys.append(ranks[i::tp_x])
        reg("tp_x", xs)
        reg("tp_y", ys)
        reg("tp_x_overlap", xs)
        reg("tp_y_overlap", ys)
        # union of tp-y and cp for attention under 2-D TP
        # (reference: mindspeed/core/tensor_parallel_y_union_cp.py:26-99)
        uni = []
        for ranks in dense.get_ranks("tp-cp"):
            # ranks enumerates tp fastest then cp
            for i in range(tp_x):
                uni.append([ranks[c * tp + j * tp_x + i] for c in range(cp) for j in range(tp_y)])
        reg("tp_y_cp", uni)
        _S.sizes["tp_x"], _S.sizes["tp_y"] = tp_x, tp_y

    _S.initialized = True


def _hierarchical_groups(cp_groups, sizes):
    """For each level, the rank lists obtained by varying that level's digit only."""
    out = []
    for lvl in range(len(sizes)):
        lvl_groups = []
        for ranks in cp_groups:
            n = len(ranks)
            other = [s for i, s in enumerate(sizes) if i != lvl]
            n_other = n // sizes[lvl]
            for o in range(n_other):
                od = _decompose(o, other)
                g = []
                for v in range(sizes[lvl]):
                    digits = od[:lvl] + [v] + od[lvl:]
                    g.append(ranks[_compose(digits, sizes)])
                lvl_groups.append(g)
        out.append(lvl_groups)
    return out


def _default_embedding_ranks(pp_ranks, split_rank=None):
    if len(pp_ranks) == 1:
        return [pp_ranks[0]]
    if split_rank is not None and pp_ranks[split_rank] not in (pp_ranks[0], pp_ranks[-1]):
        return [pp_ranks[0], pp_ranks[split_rank], pp_ranks[-1]]
    return [pp_ranks[0], pp_ranks[-1]]


def _default_position_embedding_ranks(pp_ranks, split_rank=None):
    if split_rank is not None and len(pp_ranks) > 1 and pp_ranks[split_rank] != pp_ranks[0]:
        return [pp_ranks[0], pp_ranks[split_rank]]
    return [pp_ranks[0]]


def swap_state(new_state=None):
    """Install ``new_state`` (a fresh empty one when None) as the module's parallel state and return the previous
    one.  Multi-model jobs build one state per sub-model and keep the one of the sub-model this rank belongs to."""
    global _S
    old = _S
    _S = new_state if new_state is not None else _State()
    return old


def destroy_model_parallel() -> None:
    global _S
    if dist.is_available() and dist.is_initialized():
        seen = set()
        for g in _S.groups.values():
            if g.group is not None and id(g.group) not in seen:
                seen.add(id(g.group))
                try:
                    dist.destroy_process_group(g.group)
                except Exception:  # group may be shared or already gone
                    pass
    _S = _State()


def model_parallel_is_initialized() -> bool:
    return _S.initialized


is_initialized = model_parallel_is_initialized


def is_unitialized() -> bool:  # historical spelling kept by Megatron
    return not _S.initialized


# --------------------------------------------------------------------------------------
# Getters
# --------------------------------------------------------------------------------------
def _g(name: str, check: bool = True) -> Optional[_Group]:
    g = _S.groups.get(name)
    if g is None and check:
        raise RuntimeError(f"parallel group '{name}' is not initialized")
    return g


def _group(name, check=True):
    g = _g(name, check)
    return None if g is None else g.group


def _ranks(name):
    return _g(name).ranks


def _size(name, key=None):
    ov = _S.override_world.get(name)
    if ov is not None:
        return ov
    g = _S.groups.get(name)
    if g is None:
        return _S.sizes.get(key or name, 1) if not _S.initialized else 1
    return g.size


def _rank_in(name):
    ov = _S.override_rank.get(name)
    if ov is not None:
        return ov
    g = _S.groups.get(name)
    if g is None:
        return 0
    return g.ranks.index(_S.rank)


def get_all_ranks(name: str) -> List[List[int]]:
    """Every rank list of a named group kind (available without communicators)."""
    return _S.all_groups[name]


# tensor parallel
def get_tensor_model_parallel_group(check_initialized=True):
    return _group("tp", check_initialized)


def get_tensor_model_parallel_world_size():
    return _size("tp")


def get_tensor_model_parallel_rank():
    return _rank_in("tp")


def get_tensor_model_parallel_src_rank():
    return _ranks("tp")[0]


def get_tensor_model_parallel_ranks():
    return _ranks("tp")


def set_tensor_model_parallel_world_size(v):
    _S.override_world["tp"] = v


def set_tensor_model_parallel_rank(v):
    _S.override_rank["tp"] = v


def get_model_parallel_group():
    return _group("mp")


# pipeline parallel
def get_pipeline_model_parallel_group():
    return _group("pp")


def get_pipeline_model_parallel_group_for_new_stream():
    return _group("pp_new_stream")


def get_pipeline_model_parallel_world_size():
    return _size("pp")


def get_pipeline_model_parallel_rank():
    return _rank_in("pp")


def set_pipeline_model_parallel_world_size(v):
    _S.override_world["pp"] = v


def set_pipeline_model_parallel_rank(v):
    _S.override_rank["pp"] = v


def get_pipeline_model_parallel_split_rank():
    return _S.pp_split_rank


def set_pipeline_model_parallel_split_rank(v):
    _S.pp_split_rank = v


def get_pipeline_model_parallel_first_rank():
    return _ranks("pp")[0]


def get_pipeline_model_parallel_last_rank():
    return _ranks("pp")[-1]


def get_pipeline_model_parallel_next_rank():
    r = _ranks("pp")
    return r[(get_pipeline_model_parallel_rank() + 1) % len(r)]


def get_pipeline_model_parallel_prev_rank():
    r = _ranks("pp")
    return r[(get_pipeline_model_parallel_rank() - 1) % len(r)]


def get_virtual_pipeline_model_parallel_rank():
    return _S.vpp_rank


def set_virtual_pipeline_model_parallel_rank(v):
    _S.vpp_rank = v


def get_virtual_pipeline_model_parallel_world_size():
    return _S.vpp_world


def set_virtual_pipeline_model_parallel_world_size(v):
    _S.vpp_world = v


_STAGE_OVERRIDE = {"first": None, "last": None}


def set_stage_override(first, last):
    """Schedules whose chunk placement is not ``chunk*pp + rank`` (V-shaped, bidirectional) tell the model code
    explicitly whether the chunk being run is the first / last model stage."""
    _STAGE_OVERRIDE["first"], _STAGE_OVERRIDE["last"] = first, last


def is_pipeline_first_stage(ignore_virtual=False):
    if not ignore_virtual and _STAGE_OVERRIDE["first"] is not None:
        return _STAGE_OVERRIDE["first"]
    if not ignore_virtual and _S.vpp_world is not None and _S.vpp_rank != 0:
        return False
    return get_pipeline_model_parallel_rank() == 0


def is_pipeline_last_stage(ignore_virtual=False):
    if not ignore_virtual and _STAGE_OVERRIDE["last"] is not None:
        return _STAGE_OVERRIDE["last"]
    if not ignore_virtual and _S.vpp_world is not None and _S.vpp_rank != _S.vpp_world - 1:
        return False
    return get_pipeline_model_parallel_rank() == get_pipeline_model_parallel_world_size() - 1


def is_rank_in_embedding_group(ignore_virtual=False):
    if _S.rank not in _S.embedding_ranks:
        return False
    if ignore_virtual:
        return True
    if _S.rank == _S.embedding_ranks[0]:
        return is_pipeline_first_stage(ignore_virtual=False)
    if _S.rank == _S.embedding_ranks[-1]:
        return is_pipeline_last_stage(ignore_virtual=False)
    return True


def is_rank_in_position_embedding_group():
    return _S.rank in _S.position_embedding_ranks


def get_embedding_group():
    return _group("embd", check=False)


def get_position_embedding_group():
    return _group("pos_embd", check=False)


def is_pipeline_stage_before_split(rank=None):
    if get_pipeline_model_parallel_world_size() == 1 or _S.pp_split_rank is None:
        return True
    rank = get_pipeline_model_parallel_rank() if rank is None else rank
    return rank < _S.pp_split_rank


def is_pipeline_stage_after_split(rank=None):
    if get_pipeline_model_parallel_world_size() == 1 or _S.pp_split_rank is None:
        return True
    rank = get_pipeline_model_parallel_rank() if rank is None else rank
    return rank >= _S.pp_split_rank


def is_pipeline_stage_at_split():
    r = get_pipeline_model_parallel_rank()
    return is_pipeline_stage_before_split(r) and is_pipeline_stage_after_split(r + 1)


# data parallel
def get_data_parallel_group(with_context_parallel=False, partial_data_parallel=False):
    if partial_data_parallel:
        return _group("intra_partial_dp_cp")
    return _group("dp_cp" if with_context_parallel else "dp")


def get_data_parallel_group_gloo(with_context_parallel=False, partial_data_parallel=False):
    """Gloo twin, or the device group itself when gloo groups are disabled
    (reference: mindspeed/core/parallel_state.py:1077-1108)."""
    if _S.disable_gloo:
        return get_data_parallel_group(with_context_parallel, partial_data_parallel)
    return _group("dp_cp_gloo" if with_context_parallel else "dp_gloo")


def get_inter_partial_data_parallel_group():
    return _group("inter_partial_dp_cp", check=False)


def get_data_parallel_world_size(with_context_parallel=False, partial_data_parallel=False):
    if partial_data_parallel:
        return _size("intra_partial_dp_cp")
    return _size("dp_cp" if with_context_parallel else "dp")


def get_data_parallel_rank(with_context_parallel=False, partial_data_parallel=False):
    if partial_data_parallel:
        return _rank_in("intra_partial_dp_cp")
    return _rank_in("dp_cp" if with_context_parallel else "dp")


def get_data_parallel_src_rank(with_context_parallel=False):
    return _ranks("dp_cp" if with_context_parallel else "dp")[0]


def get_data_parallel_ranks(with_context_parallel=False):
    return _ranks("dp_cp" if with_context_parallel else "dp")


# context parallel
def get_context_parallel_group(check_initialized=True):
    return _group("cp", check_initialized)


def get_context_parallel_group_for_send_recv_overlap(check_initialized=True):
    return _group("cp_overlap", check=False)


def get_context_parallel_global_ranks(check_initialized=True):
    return _ranks("cp")


def get_context_parallel_world_size():
    return _size("cp")


def get_context_parallel_rank():
    return _rank_in("cp")


def get_hierarchical_context_parallel_groups(check_initialized=True):
    n = _S.sizes.get("hcp_levels", 0)
    return [_group(f"hcp{i}") for i in range(n)]


def get_context_parallel_group_for_hybrid_ulysses():
    return _group("cp_ulysses")


def get_context_parallel_for_hybrid_ulysses_world_size():
    return _size("cp_ulysses")


def get_context_parallel_for_hybrid_ulysses_rank():
    return _rank_in("cp_ulysses")


def get_context_parallel_group_for_hybrid_ring():
    return _group("cp_ring")


def get_context_parallel_for_hybrid_ring_world_size():
    return _size("cp_ring")


def get_context_parallel_for_hybrid_ring_rank():
    return _rank_in("cp_ring")


def get_context_parallel_for_hybrid_ring_global_ranks():
    return _ranks("cp_ring")


def get_context_parallel_group_for_hybrid_ring_overlap():
    return _group("cp_ring_overlap", check=False)


def get_cp_window_size():
    return _S.sizes.get("cp_window", 1)


def get_ring_ranks_for_intra_window(ring_ranks=None, rank=None):
    """Ranks of this rank's window (inner ring) under ``--cp-window-size``
    (reference: model_parallel_utils.py:121-160)."""
    ring_ranks = ring_ranks if ring_ranks is not None else (_ranks("cp_ring") if "cp_ring" in _S.groups else _ranks("cp"))
    rank = _S.rank if rank is None else rank
    w = get_cp_window_size()
    i = ring_ranks.index(rank)
    start = (i // w) * w
    return ring_ranks[start:start + w]


def get_ring_ranks_for_inter_window_kv(ring_ranks=None, rank=None):
    """Outer-ring ranks used to prefetch the next window's KV: same offset in every window."""
    ring_ranks = ring_ranks if ring_ranks is not None else (_ranks("cp_ring") if "cp_ring" in _S.groups else _ranks("cp"))
    rank = _S.rank if rank is None else rank
    w = get_cp_window_size()
    i = ring_ranks.index(rank)
    return ring_ranks[i % w::w]


def get_ring_ranks_for_inter_window_dkv(ring_ranks=None, rank=None):
    """Outer-ring ranks for the dKV return path.  The gradient of the block received
    from window k-1 has to land on the rank that owns it after the inner ring has
    rotated a full turn, which shifts the inner offset by one per window hop
    (reference: model_parallel_utils.py:186-201)."""
    ring_ranks = ring_ranks if ring_ranks is not None else (_ranks("cp_ring") if "cp_ring" in _S.groups else _ranks("cp"))
    rank = _S.rank if rank is None else rank
    w = get_cp_window_size()
    n = len(ring_ranks)
    i = ring_ranks.index(rank)
    n_win = n // w
    win, off = i // w, i % w
    out = []
    for k in range(n_win):
        out.append(ring_ranks[((win + k) % n_win) * w + (off + k) % w])
    # rotate so that the list starts at window 0 for a canonical order
    return out


# combined groups
def get_tensor_and_data_parallel_group(with_context_parallel=False):
    return _group("tp_dp_cp" if with_context_parallel else "tp_dp")


def get_tensor_and_data_parallel_world_size(with_context_parallel=False):
    return _size("tp_dp_cp" if with_context_parallel else "tp_dp")


def get_tensor_and_context_parallel_group():
    return _group("tp_cp")


def get_tensor_and_context_parallel_world_size():
    return _size("tp_cp")


def get_tensor_and_context_parallel_rank():
    return _rank_in("tp_cp")


def get_amax_reduction_group(with_context_parallel=True, tp_only_amax_red=False):
    if tp_only_amax_red or not with_context_parallel:
        return _group("tp")
    return _group("amax")


# expert parallel
def get_expert_model_parallel_group(check_initialized=True):
    return _group("ep", check_initialized)


def get_expert_model_parallel_world_size():
    return _size("ep")


def get_expert_model_parallel_rank():
    return _rank_in("ep")


def set_expert_model_parallel_world_size(v):
    _S.override_world["ep"] = v


def set_expert_model_parallel_rank(v):
    _S.override_rank["ep"] = v


def get_expert_tensor_parallel_group(check_initialized=True):
    return _group("etp", check_initialized)


def get_expert_tensor_parallel_world_size():
    return _size("etp")


def get_expert_tensor_parallel_rank():
    return _rank_in("etp")


def set_expert_tensor_parallel_world_size(v):
    _S.override_world["etp"] = v


def set_expert_tensor_parallel_rank(v):
    _S.override_rank["etp"] = v


def get_expert_tensor_and_model_parallel_group(check_initialized=True):
    return _group("etp_ep", check_initialized)


def get_expert_tensor_and_model_parallel_world_size():
    return _size("etp_ep")


def get_expert_tensor_and_model_parallel_rank():
    return _rank_in("etp_ep")


def get_expert_tensor_model_pipeline_parallel_group():
    return _group("etp_ep_pp")


def get_expert_data_parallel_group(check_initialized=True):
    return _group("edp", check_initialized)


def get_expert_data_parallel_group_gloo():
    if _S.disable_gloo:
        return _group("edp")
    return _group("edp_gloo")


def get_expert_data_parallel_rank():
    return _rank_in("edp")


def get_expert_data_parallel_world_size():
    return _size("edp")


# legacy alias kept by Megatron for dp-modulo-ep
get_data_modulo_expert_parallel_group = get_expert_data_parallel_group
get_data_modulo_expert_parallel_rank = get_expert_data_parallel_rank
get_data_modulo_expert_parallel_group_gloo = get_expert_data_parallel_group_gloo


# 2-D tensor parallel
def get_tensor_model_parallel_group_for_nd1_dim1(check_initialized=True):
    return _group("tp_x", check_initialized)


def get_tensor_model_parallel_group_for_nd1_dim2(check_initialized=True):
    return _group("tp_y", check_initialized)


def get_tp_x_group():
    return _group("tp_x")


def get_tp_y_group():
    return _group("tp_y")


def get_tp_x_overlap_group():
    return _group("tp_x_overlap")


def get_tp_y_overlap_group():
    return _group("tp_y_overlap")


def get_tp_x_world_size():
    return _size("tp_x")


def get_tp_y_world_size():
    return _size("tp_y")


def get_tp_x_rank():
    return _rank_in("tp_x")


def get_tp_y_rank():
    return _rank_in("tp_y")


def get_tp_x_ranks():
    return _ranks("tp_x")


def get_tp_y_ranks():
    return _ranks("tp_y")


def get_tp_y_cp_group():
    return _group("tp_y_cp")


def get_tp_y_cp_world_size():
    return _size("tp_y_cp")


def get_tp_y_cp_rank():
    return _rank_in("tp_y_cp")


# misc
class GlobalMemoryBuffer:
    """Named scratch tensors reused across calls (all-gather outputs and the like)."""

    def __init__(self):
        self.buffer = {}

    def get_tensor(self, tensor_shape, dtype, name, device=None):
        import math

        numel = math.prod(tensor_shape)
        key = (name, dtype)
        buf = self.buffer.get(key)
        if buf is None or buf.numel() < numel:
            if device is None:
                device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
            buf = torch.empty(numel, dtype=dtype, device=device, requires_grad=False)
            self.buffer[key] = buf
        return buf[:numel].view(*tensor_shape)


def get_global_memory_buffer():
    if _S.global_memory_buffer is None:
        _S.global_memory_buffer = GlobalMemoryBuffer()
    return _S.global_memory_buffer


def destroy_global_memory_buffer():
    _S.global_memory_buffer = None


def get_moe_layer_wise_logging_tracker():
    return _S.moe_tracker


def get_rank():
    return _S.rank


def get_world_size():
    return _S.world


def get_sizes() -> Dict[str, int]:
    return dict(_S.sizes)
