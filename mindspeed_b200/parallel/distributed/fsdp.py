"""Fully sharded data parallel (ZeRO-3), hybrid sharding and LayerZeRO (ZeRO-3 inside a sub-group + ZeRO-1 across it).

One ``ShardedUnit`` per wrapped sub-module (normally a transformer layer):

  storage     every parameter of the unit lives in one flat buffer, padded to the shard-group size; each rank keeps
              1/S of it (``flat_shard``).  With ``zero1_over_replicas`` the optimizer additionally owns only 1/R of that
              shard (``opt_param``), i.e. optimizer state is split over all S*R data-parallel ranks while parameters
              are only split over the S ranks of the (NVLink-local) shard group - the LayerZeRO layout.
  forward     pre-hook: all-gather the flat buffer over the shard group (the next unit's gather is issued right away
              on a side stream when prefetching is on), parameters become views into it; post-hook: free it
              (``reshard_after_forward``).
  backward    pre-hook: all-gather again; when the last parameter gradient of the unit has been accumulated: flatten
              the gradients, reduce-scatter over the shard group, then all-reduce (HSDP) or reduce-scatter (LayerZeRO)
              over the replica group, and free the full buffer.
  step        ``FullyShardedDataParallel.optimizer_params()`` are ordinary leaf tensors, so any optimizer works;
              ``post_step()`` re-assembles ``flat_shard`` from the owned slices in the LayerZeRO layout.

A YAML / dict plan chooses which sub-modules become units, the mixed-precision dtypes and the two group sizes.
Runs on NCCL and (for tests) gloo.
reference: mindspeed/core/distributed/torch_fully_sharded_data_parallel/* (fully_shard adaptor with YAML plan) and
mindspeed/core/distributed/layerzero/* (ZeRO-1 over DP + ZeRO-3 over a sub-group).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Iterable, List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import mappings as M
from ...utils.patterns import match as _match


@dataclasses.dataclass
class FSDPPlan:
    """Which modules to shard and how.  ``wrap`` holds class names or glob patterns over qualified module names."""
    wrap: Sequence[str] = ("TransformerLayer",)
    ignore: Sequence[str] = ()                # modules (class names / patterns) whose parameters stay whole on every rank:
    #                                           not sharded, gradients averaged over the data-parallel ranks after backward
    shard_size: Optional[int] = None          # ranks per shard group (None: the whole data-parallel group)
    zero1_over_replicas: bool = False         # LayerZeRO: optimizer state also split over the replica group
    reshard_after_forward: bool = True
    param_dtype: Optional[str] = None         # dtype parameters are gathered in (e.g. "bfloat16"); None keeps theirs
    reduce_dtype: Optional[str] = "float32"   # dtype of the gradient reduction
    prefetch: bool = True

    @staticmethod
    def from_yaml(path: str) -> "FSDPPlan":
        import yaml
        with open(path) as f:
            d = yaml.safe_load(f) or {}
        return FSDPPlan.from_dict(d)

    @staticmethod
    def from_dict(d: Dict) -> "FSDPPlan":
        d = dict(d.get("fsdp", d))
        known = {f.name for f in dataclasses.fields(FSDPPlan)}
        bad = set(d) - known
        if bad:
            raise ValueError(f"unknown FSDP plan keys: {sorted(bad)}")
        if "wrap" in d and isinstance(d["wrap"], str):
            d["wrap"] = [d["wrap"]]
        return FSDPPlan(**d)


def _dtype(name):
    return None if name is None else getattr(torch, name)


def build_groups(dp_ranks: List[int], shard_size: Optional[int], all_dp_rank_lists: Optional[List[List[int]]] = None):
    """(shard_group, replica_group) of the calling rank.  Shard groups are contiguous runs of ``shard_size`` ranks
    (contiguous ranks share an NVSwitch domain), replica groups are strided across them.  Group creation is a
    collective over the whole job: when several data-parallel groups exist (one per tensor-parallel index) pass all
    of them in ``all_dp_rank_lists`` so that every rank creates every group in the same order."""
    me = dist.get_rank()
    shard_g = rep_g = None
    for ranks_all in (all_dp_rank_lists or [dp_ranks]):
        world = len(ranks_all)
        s = shard_size or world
        if world % s != 0:
            raise ValueError(f"shard size {s} must divide the data-parallel size {world}")
        for i in range(0, world, s):
            ranks = ranks_all[i:i + s]
            g = dist.new_group(ranks)
            if me in ranks:
                shard_g = g
        for j in range(s):
            ranks = ranks_all[j::s]
            g = dist.new_group(ranks) if len(ranks) > 1 else None
            if me in ranks:
                rep_g = g
    return shard_g, rep_g


class ShardedUnit:
    def __init__(self, module: nn.Module, shard_group, replica_group, plan: FSDPPlan, name: str = "", grad_scale: float = 1.0):
        self.module, self.shard_group, self.replica_group, self.plan, self.name = module, shard_group, replica_group, plan, name
        self.grad_scale = grad_scale
        self.S = M._ws(shard_group)
        self.R = M._ws(replica_group)
        self.s_rank = M._rk(shard_group)
        self.r_rank = M._rk(replica_group)
        self.params: List[nn.Parameter] = [p for p in module.parameters(recurse=True) if not getattr(p, "_fsdp_owned", False)]
        for p in self.params:
            p._fsdp_owned = True
        ids = {id(p): n for n, p in module.named_parameters(recurse=True)}
        self.param_names = [ids.get(id(p), f"param{i}") for i, p in enumerate(self.params)]
        # tensor-parallel bookkeeping: a parameter split over the tensor-parallel ranks holds different values on each of
        # them; the rest is duplicated there (its gradient norm counts once), and the duplicated ones that see only a
        # sequence slice per rank (norm weights under sequence parallelism) need their gradients summed over those ranks
        self.tp_sharded = [bool(getattr(p, "tensor_model_parallel", False)) or not getattr(p, "allreduce", True) for p in self.params]
        self.seq_replicated = [bool(getattr(p, "sequence_parallel", False)) for p in self.params]
        self.shapes = [p.shape for p in self.params]
        self.numels = [p.numel() for p in self.params]
        # where a tensor-parallel parameter is split (axis, and 2 for the gated FC1 whose rows are [gate; up] per rank)
        self.tp_dims = [int(getattr(p, "partition_dim", -1)) if getattr(p, "tensor_model_parallel", False) else None for p in self.params]
        self.tp_strides = [int(getattr(p, "partition_stride", 1)) for p in self.params]
        total = sum(self.numels)
        div = self.S * (self.R if plan.zero1_over_replicas else 1)
        self.padded = ((total + div - 1) // div) * div
        self.total = total
        dev = self.params[0].device if self.params else torch.device("cpu")
        self.master_dtype = self.params[0].dtype if self.params else torch.float32
        self.gather_dtype = _dtype(plan.param_dtype) or self.master_dtype
        self.reduce_dtype = _dtype(plan.reduce_dtype) or self.master_dtype
        flat = torch.zeros(self.padded, dtype=self.master_dtype, device=dev)
        off = 0
        for p, n in zip(self.params, self.numels):
            flat[off:off + n].copy_(p.detach().reshape(-1))
            off += n
        per = self.padded // self.S
        self.per = per
        self.flat_shard = flat[self.s_rank * per:(self.s_rank + 1) * per].clone()
        self.flat_shard_grad: Optional[torch.Tensor] = None
        if plan.zero1_over_replicas and self.R > 1:
            own = per // self.R
            self.own = own
            self.opt_param = nn.Parameter(self.flat_shard[self.r_rank * own:(self.r_rank + 1) * own].clone())
        else:
            self.own = per
            self.opt_param = nn.Parameter(self.flat_shard)   # shares storage: the optimizer updates the shard in place
            self.flat_shard = self.opt_param.data
        self.full: Optional[torch.Tensor] = None
        self._pending_grads = 0
        self._reduced = False
        self._gather_work = None
        self._free_params()
        self._install_hooks()

    # -- (un)sharding ------------------------------------------------------------------------------------------
    def _free_params(self):
        for p in self.params:
            p.data = torch.empty(0, dtype=self.gather_dtype, device=self.flat_shard.device)
        self.full = None

    def start_unshard(self):
        """Issue the all-gather (asynchronously where the backend allows); ``finish_unshard`` makes it visible."""
        if self.full is not None or self._gather_work is not None:
            return
        shard = self.flat_shard.to(self.gather_dtype)
        if self.S == 1:
            self._gather_work = (shard.clone(), None)
            return
        out = torch.empty(self.padded, dtype=self.gather_dtype, device=shard.device)
        work = dist.all_gather_into_tensor(out, shard.contiguous(), group=self.shard_group, async_op=True)
        self._gather_work = (out, work)

    def finish_unshard(self):
        if self.full is not None:
            return
        if self._gather_work is None:
            self.start_unshard()
        out, work = self._gather_work
        self._gather_work = None
        if work is not None:
            work.wait()
        self.full = out
        off = 0
        for p, n, shp in zip(self.params, self.numels, self.shapes):
            p.data = out[off:off + n].view(shp)
            off += n

    def reshard(self):
        self._free_params()

    # -- hooks -------------------------------------------------------------------------------------------------
    def _install_hooks(self):
        self.module.register_forward_pre_hook(self._pre_forward)
        self.module.register_forward_hook(self._post_forward)
        self.module.register_full_backward_pre_hook(self._pre_backward)
        for p in self.params:
            if p.requires_grad:
                p.register_post_accumulate_grad_hook(self._grad_ready)
        self.next_unit: Optional["ShardedUnit"] = None
        self.prev_unit: Optional["ShardedUnit"] = None

    def _pre_forward(self, mod, args):
        self.finish_unshard()
        if self.plan.prefetch and self.next_unit is not None:
            self.next_unit.start_unshard()

    def _post_forward(self, mod, args, out):
        if self.plan.reshard_after_forward:
            self.reshard()

    def _pre_backward(self, mod, grad_out):
        self.finish_unshard()
        self._pending_grads = sum(1 for p in self.params if p.requires_grad)
        self._reduced = False
        # the unit after this one (in forward order) has finished its backward entirely once ours starts: only now is
        # it safe to drop its gathered weights (autograd re-reads a parameter's current storage when it unpacks it)
        if self.next_unit is not None and self.next_unit._reduced:
            self.next_unit.reshard()
        if self.plan.prefetch and self.prev_unit is not None:
            self.prev_unit.start_unshard()

    def _grad_ready(self, p):
        self._pending_grads -= 1
        if self._pending_grads == 0:
            self.reduce_grads()

    def reduce_grads(self):
        """Flatten, reduce-scatter over the shard group, reduce over the replica group; accumulates into .grad of
        the optimizer's parameter (several micro-batches add up)."""
        if self._reduced:
            return
        self._reduced = True
        dev = self.flat_shard.device
        self._sum_sequence_parallel_grads()
        flat = torch.zeros(self.padded, dtype=self.reduce_dtype, device=dev)
        off = 0
        for p, n in zip(self.params, self.numels):
            if p.grad is not None:
                flat[off:off + n].copy_(p.grad.reshape(-1))
                p.grad = None
            off += n
        world = self.S * self.R
        flat.mul_(self.grad_scale / world)
        g = M.reduce_scatter_first_dim(flat, self.shard_group) if self.S > 1 else flat
        if self.R > 1:
            if self.plan.zero1_over_replicas:
                g = M.reduce_scatter_first_dim(g, self.replica_group)
            else:
                dist.all_reduce(g, group=self.replica_group)
        g = g.to(self.opt_param.dtype)
        if self.opt_param.grad is None:
            self.opt_param.grad = g
        else:
            self.opt_param.grad.add_(g)

    def _sum_sequence_parallel_grads(self):
        """Parameters that every tensor-parallel rank holds in full but applies to its own slice of the sequence (norm
        weights under sequence parallelism): their gradient is the sum over the tensor-parallel ranks."""
        from .. import parallel_state as ps
        if not ps.model_parallel_is_initialized() or ps.get_tensor_model_parallel_world_size() == 1:
            return
        grads = [p.grad for p, sr in zip(self.params, self.seq_replicated) if sr and p.grad is not None]
        if not grads:
            return
        flat = torch.cat([g.reshape(-1).float() for g in grads])
        dist.all_reduce(flat, group=ps.get_tensor_model_parallel_group())
        off = 0
        for g in grads:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()

    def local_range(self):
        """[lo, hi) of the flat (padded) parameter space that this rank's optimizer parameter covers."""
        lo = self.s_rank * self.per
        if self.plan.zero1_over_replicas and self.R > 1:
            lo += self.r_rank * self.own
        return lo, lo + self.own

    def param_slices(self, lo: int, hi: int):
        """(index, name, start inside the parameter, start inside [lo, hi), length) for every parameter that overlaps the
        flat range [lo, hi)."""
        out, off = [], 0
        for i, (name, n) in enumerate(zip(self.param_names, self.numels)):
            a, b = max(lo, off), min(hi, off + n)
            if b > a:
                out.append((i, name, a - off, a - lo, b - a))
            off += n
        return out

    def norm_weight_mask(self):
        """1 where an element of the local optimizer parameter counts towards the global gradient norm on this rank:
        parameters duplicated over the tensor-parallel ranks count on tensor-parallel rank 0 only; padding never."""
        from .. import parallel_state as ps
        lo, hi = self.local_range()
        mask = torch.zeros(hi - lo, dtype=torch.float32, device=self.flat_shard.device)
        tp_rank = ps.get_tensor_model_parallel_rank() if ps.model_parallel_is_initialized() else 0
        for i, _, _, at, n in self.param_slices(lo, hi):
            if self.tp_sharded[i] or tp_rank == 0:
                mask[at:at + n] = 1.0
        return mask

    def post_step(self):
        """LayerZeRO: rebuild the parameter shard from the slices the replicas own."""
        if self.plan.zero1_over_replicas and self.R > 1:
            out = M.all_gather_first_dim(self.opt_param.data, self.replica_group)
            self.flat_shard.copy_(out)

    # -- state -------------------------------------------------------------------------------------------------
    def full_parameters(self) -> List[torch.Tensor]:
        """Unsharded master-precision copies (collective over the shard group)."""
        full = M.all_gather_first_dim(self.flat_shard, self.shard_group) if self.S > 1 else self.flat_shard
        out, off = [], 0
        for n, shp in zip(self.numels, self.shapes):
            out.append(full[off:off + n].view(shp).clone())
            off += n
        return out


class FullyShardedDataParallel(nn.Module):
    """Wraps ``module``; every sub-module matched by the plan becomes a ShardedUnit, the remaining parameters form one
    root unit.  ``dp_group_ranks`` lists the global ranks of the data-parallel group in order."""

    def __init__(self, module: nn.Module, plan: Optional[FSDPPlan] = None, dp_group_ranks: Optional[List[int]] = None,
                 shard_group=None, replica_group=None, grad_scale: float = 1.0, root_unit: bool = True,
                 all_dp_rank_lists: Optional[List[List[int]]] = None):
        """``grad_scale`` multiplies the averaged gradients (expert parameters under expert parallelism need 1/ep:
        their owner already holds the sum over the expert-parallel ranks' tokens).  ``root_unit=False`` leaves the
        parameters outside the matched sub-modules alone (another wrapper owns them)."""
        super().__init__()
        self.module = module
        self.plan = plan or FSDPPlan()
        if shard_group == "local":          # explicit single-rank sharding (no communication at all)
            shard_group = replica_group = None
        elif shard_group is None and dist.is_initialized():
            ranks = dp_group_ranks or list(range(dist.get_world_size()))
            shard_group, replica_group = build_groups(ranks, self.plan.shard_size, all_dp_rank_lists)
        self.shard_group, self.replica_group = shard_group, replica_group
        self.units: List[ShardedUnit] = []
        self.ignored: List[nn.Parameter] = []
        self._dp_ranks = dp_group_ranks
        for name, sub in module.named_modules():
            if name and any(sub.__class__.__name__ == pat or _match(name, pat) for pat in self.plan.ignore):
                for p in sub.parameters():
                    if not getattr(p, "_fsdp_owned", False):
                        p._fsdp_owned = True               # keeps every unit from taking it
                        self.ignored.append(p)
        for name, sub in module.named_modules():
            if sub is module:
                continue
            if self._matches(name, sub) and any(not getattr(p, "_fsdp_owned", False) for p in sub.parameters()):
                self.units.append(ShardedUnit(sub, shard_group, replica_group, self.plan, name, grad_scale))
        if root_unit and any(not getattr(p, "_fsdp_owned", False) for p in module.parameters()):
            self.units.insert(0, ShardedUnit(module, shard_group, replica_group, self.plan, "<root>", grad_scale))
        # forward order == registration order for sequential stacks; used for prefetching only
        body = [u for u in self.units if u.name != "<root>"]
        for a, b in zip(body[:-1], body[1:]):
            a.next_unit, b.prev_unit = b, a

    def _matches(self, name: str, sub: nn.Module) -> bool:
        cls = type(sub).__name__
        return any(pat == cls or _match(name, pat) for pat in self.plan.wrap)

    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    # ---- surface the training loop expects from a data-parallel wrapper ----
    @property
    def config(self):
        return self.module.config

    def zero_grad_buffer(self):
        self.zero_grad()

    def no_sync(self):
        import contextlib
        return contextlib.nullcontext()       # gradients of several micro-batches accumulate in the sharded .grad

    def start_param_sync(self, *a, **kw):
        return None                           # parameters are gathered on demand by the forward / backward hooks

    def set_input_tensor(self, t):
        return self.module.set_input_tensor(t)

    def optimizer_params(self) -> List[nn.Parameter]:
        return [u.opt_param for u in self.units] + [p for p in self.ignored if p.requires_grad]

    def _sync_ignored(self):
        """Average the gradients of the unsharded (``plan.ignore``) parameters over shard and replica group."""
        for group in (self.shard_group, self.replica_group):
            n = M._ws(group)
            if n > 1:
                for p in self.ignored:
                    if p.grad is not None:
                        dist.all_reduce(p.grad, group=group)
                        p.grad /= n

    def finish_grad_sync(self):
        """Reduce units whose backward never fired completely (unused parameters)."""
        if self.ignored:
            self._sync_ignored()
        for u in self.units:
            if not u._reduced and (u._pending_grads > 0 or any(p.grad is not None for p in u.params)):
                u.reduce_grads()
        for u in self.units:
            u._reduced = False
            u._pending_grads = 0
            u.reshard()

    def zero_grad(self, set_to_none: bool = True):
        for u in self.units:
            u.opt_param.grad = None
        for p in self.ignored:
            p.grad = None

    def post_step(self):
        for u in self.units:
            u.post_step()

    def full_state_dict(self) -> Dict[str, torch.Tensor]:
        """Unsharded parameters by their original names (collective)."""
        out = {}
        names = {id(p): n for n, p in self.module.named_parameters()}
        for u in self.units:
            for p, t in zip(u.params, u.full_parameters()):
                if id(p) in names:
                    out[names[id(p)]] = t
        for p in self.ignored:                         # whole on every rank already
            if id(p) in names:
                out[names[id(p)]] = p.detach().clone()
        return out

    def post_load(self):
        """After a checkpoint has been read into the parameter shards: the optimizer's own slice (a separate tensor in the
        LayerZeRO layout) follows."""
        for u in self.units:
            if u.plan.zero1_over_replicas and u.R > 1:
                u.opt_param.data.copy_(u.flat_shard[u.r_rank * u.own:(u.r_rank + 1) * u.own])

    def sharded_state_dict(self, prefix: str = ""):
        """Every parameter as a flat 1-D global tensor of which this rank holds one contiguous piece: written with
        ``torch.distributed.checkpoint`` and readable under any other shard-group / replica-group size.  Parameters that are
        split over tensor-parallel ranks (and everything of another pipeline stage) get the rank in their key: resharding
        across those dimensions is left to the DDP checkpoint path."""
        from ...checkpointing.sharded import ShardedTensor
        from .. import parallel_state as ps
        mp = ps.model_parallel_is_initialized()
        tp, tpr = (ps.get_tensor_model_parallel_world_size(), ps.get_tensor_model_parallel_rank()) if mp else (1, 0)
        ppr = ps.get_pipeline_model_parallel_rank() if mp and ps.get_pipeline_model_parallel_world_size() > 1 else None
        out = {}
        for u in self.units:
            lo, hi = u.s_rank * u.per, (u.s_rank + 1) * u.per            # the parameter shard (complete on every replica)
            for i, name, start, at, n in u.param_slices(lo, hi):
                qual = name if u.name == "<root>" else f"{u.name}.{name}"
                key = f"{prefix}fsdp.{qual}"
                if tp > 1 and u.tp_sharded[i]:
                    key += f".tp{tpr}of{tp}"
                if ppr is not None:
                    key += f".pp{ppr}"
                replica = u.r_rank + (0 if (u.tp_sharded[i] or tp == 1) else tpr * 1000)
                out[key] = ShardedTensor(key, u.flat_shard[at:at + n], (u.numels[i],), (start,), replica_id=replica)
        return out

    def layout(self, prefix: str = "") -> Dict[str, dict]:
        """What a reader of ``sharded_state_dict`` needs to turn the flat tensors back into parameters, per checkpoint key:
        the qualified parameter name, the local shape, the tensor-parallel split (rank, size, axis, stride) or None, and the
        global number of the layer the parameter belongs to (pipeline stages number their layers locally)."""
        from .. import parallel_state as ps
        mp = ps.model_parallel_is_initialized()
        tp, tpr = (ps.get_tensor_model_parallel_world_size(), ps.get_tensor_model_parallel_rank()) if mp else (1, 0)
        ppr = ps.get_pipeline_model_parallel_rank() if mp and ps.get_pipeline_model_parallel_world_size() > 1 else None
        inner = self.module
        numbers = {}
        if hasattr(inner, "decoder"):
            numbers = {i: l.layer_number - 1 for i, l in enumerate(inner.decoder.layers) if hasattr(l, "layer_number")}
        out = {}
        for u in self.units:
            for i, name in enumerate(u.param_names):
                qual = name if u.name == "<root>" else f"{u.name}.{name}"
                key = f"{prefix}fsdp.{qual}"
                split = None
                if tp > 1 and u.tp_sharded[i]:
                    key += f".tp{tpr}of{tp}"
                    split = (tpr, tp, u.tp_dims[i], u.tp_strides[i])
                if ppr is not None:
                    key += f".pp{ppr}"
                parts = qual.split(".")
                layer = None
                if "layers" in parts:
                    j = parts.index("layers")
                    if j + 1 < len(parts) and parts[j + 1].isdigit():
                        layer = numbers.get(int(parts[j + 1]))
                        parts = parts[:j + 1] + parts[j + 2:]
                out[key] = {"name": ".".join(parts), "shape": tuple(u.shapes[i]), "tp": split, "layer": layer,
                            "expert": not getattr(u.params[i], "allreduce", True)}
        return out

    def memory_summary(self) -> Dict[str, int]:
        shard = sum(u.flat_shard.numel() * u.flat_shard.element_size() for u in self.units)
        opt = sum(u.opt_param.numel() * u.opt_param.element_size() for u in self.units)
        full = sum(u.padded * torch.empty((), dtype=u.gather_dtype).element_size() for u in self.units)
        return {"param_shard_bytes": shard, "optimizer_param_bytes": opt, "unsharded_bytes": full}


def fully_shard(module: nn.Module, plan=None, **kw) -> FullyShardedDataParallel:
    """Entry point matching the torch ``fully_shard`` call shape; ``plan`` may be an FSDPPlan, a dict or a YAML path."""
    if isinstance(plan, str):
        plan = FSDPPlan.from_yaml(plan)
    elif isinstance(plan, dict):
        plan = FSDPPlan.from_dict(plan)
    return FullyShardedDataParallel(module, plan, **kw)


class ShardedAdamW:
    """AdamW over the flat shards of one or more ``FullyShardedDataParallel`` wrappers, with the optimizer surface of the
    training loop (``step() -> (ok, grad_norm, num_zeros)``, ``zero_grad``, ``param_groups``).  Weight decay skips
    one-dimensional parameters (norm weights, biases) through a per-element mask laid out like the flat shard; the
    gradient norm for clipping is reduced over the ranks that hold different shards."""

    def __init__(self, wrappers: Sequence[FullyShardedDataParallel], lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 clip_grad: float = 0.0):
        self.wrappers = list(wrappers)
        if any(w.ignored for w in self.wrappers):
            raise NotImplementedError("FSDP plan 'ignore' keeps parameters outside the flat shards this optimizer updates; use it "
                                      "with an optimizer built over optimizer_params() (the engine), not with the training loop")
        self.param_groups = [dict(lr=lr, weight_decay=weight_decay, betas=betas, eps=eps, step=0)]
        self.clip_grad = clip_grad
        self.state = []
        for w in self.wrappers:
            for u in w.units:
                mask = torch.zeros(u.padded, dtype=torch.float32, device=u.flat_shard.device)
                off = 0
                for n, shp in zip(u.numels, u.shapes):
                    if len(shp) > 1:
                        mask[off:off + n] = 1.0
                    off += n
                lo = u.s_rank * u.per
                m = mask[lo:lo + u.per]
                if u.plan.zero1_over_replicas and u.R > 1:
                    m = m[u.r_rank * u.own:(u.r_rank + 1) * u.own]
                self.state.append(dict(unit=u, wd_mask=m.clone(), m=torch.zeros_like(u.opt_param, dtype=torch.float32),
                                       v=torch.zeros_like(u.opt_param, dtype=torch.float32), norm_mask=u.norm_weight_mask()))

    def zero_grad(self, set_to_none=True):
        for w in self.wrappers:
            w.zero_grad()

    def get_loss_scale(self):
        return torch.ones(1)

    def reload_model_params(self):
        return None

    @torch.no_grad()
    def step(self):
        g = self.param_groups[0]
        g["step"] += 1
        t, lr, wd, (b1, b2), eps = g["step"], g["lr"], g["weight_decay"], g["betas"], g["eps"]
        grad_norm = None
        coef = 1.0
        if self.clip_grad and self.clip_grad > 0:
            sq = torch.zeros((), dtype=torch.float32, device=self.state[0]["m"].device)
            for st in self.state:
                gr = st["unit"].opt_param.grad
                if gr is not None:
                    sq += (gr.float().pow(2) * st["norm_mask"]).sum()
            u0 = self.state[0]["unit"]
            if u0.S > 1:
                dist.all_reduce(sq, group=u0.shard_group)
            if u0.plan.zero1_over_replicas and u0.R > 1:
                dist.all_reduce(sq, group=u0.replica_group)
            from .. import parallel_state as ps
            if ps.model_parallel_is_initialized():
                mpg = ps.get_model_parallel_group()
                if mpg is not None and dist.get_world_size(mpg) > 1:
                    dist.all_reduce(sq, group=mpg)       # tensor- and pipeline-parallel ranks hold other parameters
            grad_norm = float(sq.sqrt())
            coef = min(1.0, self.clip_grad / (grad_norm + 1e-6))
        bc1, bc2 = 1.0 - b1 ** t, 1.0 - b2 ** t
        for st in self.state:
            p = st["unit"].opt_param
            if p.grad is None:
                continue
            gr = p.grad.float() * coef
            st["m"].mul_(b1).add_(gr, alpha=1 - b1)
            st["v"].mul_(b2).addcmul_(gr, gr, value=1 - b2)
            upd = (st["m"] / bc1) / ((st["v"] / bc2).sqrt() + eps)
            p.data.mul_(1.0 - lr * wd * st["wd_mask"].to(p.dtype))
            p.data.add_(upd.to(p.dtype), alpha=-lr)
        for w in self.wrappers:
            w.post_step()
        return True, grad_norm, None

    def sharded_state_dict(self, prefix: str = "optimizer."):
        """Adam moments laid out like ``FullyShardedDataParallel.sharded_state_dict``: flat per-parameter pieces."""
        from ...checkpointing.sharded import ShardedTensor
        from .. import parallel_state as ps
        mp = ps.model_parallel_is_initialized()
        tp, tpr = (ps.get_tensor_model_parallel_world_size(), ps.get_tensor_model_parallel_rank()) if mp else (1, 0)
        ppr = ps.get_pipeline_model_parallel_rank() if mp and ps.get_pipeline_model_parallel_world_size() > 1 else None
        out = {}
        for st in self.state:
            u = st["unit"]
            lo, hi = u.local_range()
            split = u.plan.zero1_over_replicas and u.R > 1
            for i, name, start, at, n in u.param_slices(lo, hi):
                qual = name if u.name == "<root>" else f"{u.name}.{name}"
                suffix = (f".tp{tpr}of{tp}" if tp > 1 and u.tp_sharded[i] else "") + (f".pp{ppr}" if ppr is not None else "")
                replica = (0 if split else u.r_rank) + (0 if (u.tp_sharded[i] or tp == 1) else tpr * 1000)
                for kind, buf in (("exp_avg", st["m"]), ("exp_avg_sq", st["v"])):
                    key = f"{prefix}fsdp.{kind}.{qual}{suffix}"
                    out[key] = ShardedTensor(key, buf[at:at + n], (u.numels[i],), (start,), replica_id=replica)
        return out

    def state_dict(self):
        return {"step": self.param_groups[0]["step"], "m": [s["m"] for s in self.state], "v": [s["v"] for s in self.state]}

    def load_state_dict(self, sd):
        self.param_groups[0]["step"] = sd["step"]
        for s, m, v in zip(self.state, sd["m"], sd["v"]):
            s["m"].copy_(m)
            s["v"].copy_(v)

