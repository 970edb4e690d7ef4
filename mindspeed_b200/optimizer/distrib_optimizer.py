"""Mixed-precision optimizer over the data-parallel flat buffers, optionally sharded (ZeRO-1).

State lives per bucket as flat fp32 tensors covering this rank's shard (``use_distributed_optimizer``)
or the whole bucket.  One step:

  finish grad sync -> (unscale) -> sum of squared grads on device -> all-reduce -> clip coefficient on
  device (no host sync) -> fused AdamW per hyper-parameter segment: reads fp32 grad, updates fp32
  master/m/v and writes the bf16 model parameter shard in the same pass -> parameter all-gather.

Parameters with equal (weight-decay, lr multiplier) that are adjacent in the buffer form one segment,
so a 32-layer model is a few hundred launches of a bandwidth-bound kernel.

reference: Megatron ``DistributedOptimizer`` as patched by mindspeed/optimizer/distrib_optimizer.py and
mindspeed/core/optimizer/fix_duplicate_allgather.py:10-109; AdamW semantics mindspeed/core/optimizer/adamw.py:23-62;
EMA variant mindspeed/core/optimizer/fused_ema_adamw/fused_ema_adamw.py:8-211.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import adam as adam_ops
from ..parallel import parallel_state as ps
from ..parallel.layers import param_is_not_tensor_parallel_duplicate
from .config import OptimizerConfig


@dataclass
class _Segment:
    start: int          # offsets relative to the state tensors of the bucket
    end: int
    wd_mult: float
    lr_mult: float
    in_norm: bool


class _BucketState:
    def __init__(self, buf, bucket, sharded, use_master, ema, reuse=False):
        self.buf, self.bucket = buf, bucket
        if sharded:
            self.lo, self.hi = buf.shard_range(bucket)
        else:
            self.lo, self.hi = bucket.start, bucket.end
        n = self.hi - self.lo
        dev = buf.grad_data.device
        self.grad = buf.grad_data[self.lo:self.hi]
        self.param16 = buf.param_data[self.lo:self.hi] if buf.param_data is not None else None
        self.residual = None
        if use_master and reuse and self.param16.dtype == torch.bfloat16:
            # master = (bf16 parameter, 16-bit residual): the parameter already is the rounded master, residual starts at 0x8000-offset zero
            # a bf16 value widened to fp32 has zero low bits, so its stored form is (same bf16, 0x8000): no temporaries needed
            self.residual = torch.full((n,), -32768, dtype=torch.int16, device=dev)
            self.master = None
        elif use_master:
            self.master = self.param16.float()
        else:
            self.master = self.param16  # fp32 params: update in place
            self.param16 = None
        self.m = torch.zeros(n, dtype=torch.float32, device=dev)
        self.v = torch.zeros(n, dtype=torch.float32, device=dev)
        self.ema = self.master.clone() if (ema and self.master is not None) else None
        self.segments: List[_Segment] = []

    def param_view(self, sl):
        """fp32 models: the parameter buffer itself is the master."""
        return self.buf.param_data[self.lo:self.hi][sl]

    master_fp32 = param_view


def _default_wd_mult(name, p):
    no_wd = name.endswith(".bias") or p.dim() == 1
    return 0.0 if no_wd else 1.0


def build_segments(bucket, names, lo, hi, cond) -> List[_Segment]:
    """Hyper-parameter segments of the slice [lo, hi) of a bucket (offsets relative to ``lo``).  Parameters are walked in
    buffer order (``bucket.params`` is reverse layer order, ascending offset); neighbours with equal
    (weight-decay multiplier, lr multiplier, counted-in-norm) closer than the 64-element alignment padding merge.
    Segment ends are rounded up to a multiple of 4 inside that padding (never past ``hi``) because the vectorised
    kernels work on groups of four; the padding holds zeros with zero gradients, which AdamW leaves at zero.
    ``cond(name, param) -> (wd_mult, lr_mult, in_norm)``."""
    out: List[_Segment] = []
    cur = None
    for p in bucket.params:
        ps_, pe_ = bucket.param_ranges[id(p)]
        s, e = max(ps_, lo), min(pe_, hi)
        if s >= e:
            continue
        e = min(hi, (e + 3) // 4 * 4)
        wdm, lrm, in_norm = cond(names.get(id(p), ""), p)
        seg = _Segment(s - lo, e - lo, wdm, lrm, in_norm)
        if cur is not None and (cur.wd_mult, cur.lr_mult, cur.in_norm) == (wdm, lrm, in_norm) and seg.start - cur.end < 64:
            cur.end = max(cur.end, seg.end)
        else:
            if cur is not None and seg.start < cur.end:     # rounding of the previous end reached into this parameter's padding
                seg.start = cur.end
            if seg.start < seg.end:
                out.append(seg)
                cur = seg
    return out


class DistributedOptimizer:
    """Works for both sharded (ZeRO-1) and replicated state; exposes the Megatron optimizer surface
    (``step``, ``zero_grad``, ``state_dict``, ``get_loss_scale``, ``param_groups``)."""

    def __init__(self, config: OptimizerConfig, model_chunks, no_weight_decay_cond: Optional[Callable] = None,
                 scale_lr_cond: Optional[Callable] = None, lr_mult: float = 1.0):
        self.config = config
        self.model_chunks = model_chunks
        self.sharded = config.use_distributed_optimizer
        self.step_count = 0
        self.param_groups = [dict(lr=config.lr, weight_decay=config.weight_decay, betas=(config.adam_beta1, config.adam_beta2),
                                  eps=config.adam_eps, step=0, is_expert_parallel=False)]
        self.states: List[_BucketState] = []
        self.expert_states: List[_BucketState] = []
        self._dev = None
        for chunk in model_chunks:
            names = {id(p): n for n, p in chunk.module.named_parameters()}
            for is_expert, bufs, out in ((False, chunk.buffers, self.states), (True, chunk.expert_buffers, self.expert_states)):
                for buf in bufs:
                    self._dev = buf.grad_data.device
                    use_master = buf.param_dtype != torch.float32
                    for b in buf.buckets:
                        st = _BucketState(buf, b, self.sharded and buf.dp_size > 1, use_master, config.use_ema,
                                          reuse=config.reuse_fp32_param)
                        def cond(name, p):
                            if no_weight_decay_cond is not None:
                                wdm = 0.0 if no_weight_decay_cond(name, p) else 1.0
                            else:
                                wdm = _default_wd_mult(name, p)
                            lrm = lr_mult if (scale_lr_cond is not None and scale_lr_cond(name, p)) else 1.0
                            in_norm = param_is_not_tensor_parallel_duplicate(p) and not getattr(p, "shared", False)
                            return wdm, lrm, in_norm
                        st.segments = build_segments(b, names, st.lo, st.hi, cond)
                        # launches of the fused peer-memory step handshake with every peer, so each rank must issue the
                        # same number per bucket: the layout is deterministic, every rank can count every rank's segments
                        st.max_segments = len(st.segments)
                        if self.sharded and buf.dp_size > 1:
                            per = b.numel // buf.dp_size
                            st.max_segments = max(len(build_segments(b, names, b.start + r * per, b.start + (r + 1) * per, cond))
                                                  for r in range(buf.dp_size))
                        out.append(st)
        dev = self._dev or torch.device("cpu")
        self._norm_sq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._coef = torch.ones(1, dtype=torch.float32, device=dev)
        self._found_inf = torch.zeros(1, dtype=torch.float32, device=dev)
        self._norm = torch.zeros(1, dtype=torch.float32, device=dev)

    # ---- Megatron surface ----
    def zero_grad(self, set_to_none=True):
        for chunk in self.model_chunks:
            for p in chunk.module.parameters():
                p.grad = None

    def get_loss_scale(self):
        return torch.ones(1, device=self._dev)

    def scale_loss(self, loss):
        return loss

    def reload_model_params(self):
        for st in self.states + self.expert_states:
            if st.residual is not None:
                st.residual.fill_(-32768)
            elif st.param16 is not None:
                st.master.copy_(st.param16)

    def _all_states(self):
        return self.states + self.expert_states

    def _grad_norm_sq(self):
        self._norm_sq.zero_()
        for st in self._all_states():
            for sg in st.segments:
                if sg.in_norm:
                    adam_ops.l2norm_sq(st.grad[sg.start:sg.end], out=self._norm_sq, accumulate=True)
        if dist.is_available() and dist.is_initialized() and ps.model_parallel_is_initialized():
            if self.sharded and ps.get_data_parallel_world_size(with_context_parallel=True) > 1:
                dist.all_reduce(self._norm_sq, group=ps.get_data_parallel_group(with_context_parallel=True))
            mp = ps.get_model_parallel_group()
            if mp is not None and dist.get_world_size(mp) > 1:
                dist.all_reduce(self._norm_sq, group=mp)
        return self._norm_sq

    @torch.no_grad()
    def step(self):
        cfg = self.config
        self.step_count += 1
        self.param_groups[0]["step"] = self.step_count
        lr = self.param_groups[0]["lr"]
        wd = self.param_groups[0]["weight_decay"]
        on_gpu = self._dev is not None and self._dev.type == "cuda"
        grad_norm = None
        coef_dev, coef_host = None, 1.0
        if any(getattr(st.buf, "fused", False) for st in self._all_states()):
            return self._step_fused(lr, wd)      # computes the norm itself, on the reduced gradients
        if cfg.clip_grad > 0.0 or cfg.log_num_zeros_in_grad:
            nsq = self._grad_norm_sq()
            if on_gpu:
                adam_ops.clip_coef(nsq, cfg.clip_grad, self._coef, self._found_inf, self._norm)
                coef_dev = self._coef
                grad_norm = self._norm
            else:
                nrm = math.sqrt(float(nsq.item()))
                grad_norm = nrm
                if not math.isfinite(nrm):
                    return False, grad_norm, None
                coef_host = min(1.0, cfg.clip_grad / (nrm + 1e-6)) if cfg.clip_grad > 0 else 1.0
        for st in self._all_states():
            for sg in st.segments:
                sl = slice(sg.start, sg.end)
                if st.residual is not None:
                    from ..memory.reuse_param import adam_flat_reuse
                    adam_flat_reuse(st.param16[sl], st.residual[sl], st.grad[sl], st.m[sl], st.v[sl], lr * sg.lr_mult,
                                    cfg.adam_beta1, cfg.adam_beta2, cfg.adam_eps, wd * sg.wd_mult, self.step_count, coef_host,
                                    True, found_inf=self._found_inf if (on_gpu and coef_dev is not None) else None,
                                    grad_scale_dev=coef_dev)
                    continue
                adam_ops.adam_flat(st.master[sl], st.grad[sl], st.m[sl], st.v[sl],
                                   None if st.param16 is None else st.param16[sl], lr * sg.lr_mult, cfg.adam_beta1,
                                   cfg.adam_beta2, cfg.adam_eps, wd * sg.wd_mult, self.step_count, coef_host, True,
                                   ema=None if st.ema is None else st.ema[sl], ema_decay=cfg.ema_decay,
                                   found_inf=self._found_inf if (on_gpu and coef_dev is not None) else None,
                                   grad_scale_dev=coef_dev)
        if self.sharded:
            for chunk in self.model_chunks:
                chunk.start_param_sync(force_sync=not chunk.ddp_config.overlap_param_gather)
        return True, grad_norm, None

    def _step_fused(self, lr, wd):
        """Every (bucket, segment) as peer-memory kernel launches: pull-reduce gradients from the data-parallel peers,
        AdamW on the owned shard, push the new bf16 weights to every peer.  With clipping the reduction (and the
        squared norm) is a first pass, the update a second one that reads the clip coefficient on the device."""
        import ctypes
        from ..ops import gemm as G
        from ..ops import loader
        from ..ops.fused_dist_opt import _Args
        cfg = self.config
        L = loader.require_lib()
        clip = cfg.clip_grad > 0.0
        st_word = G.status_word(self._dev)

        def launch(st, sg, pull, do_adam, push, use_clip):
            buf = st.buf
            h = buf.heap
            a = _Args()
            gsz = buf.grad_data.element_size()
            for r in range(h.world):
                a.peer_grad[r] = h.ptr(r, buf.grad_off)
                a.peer_param[r] = h.ptr(r, buf.param_off)
                a.flag_peer[r] = h.ptr(r, 0)
            sl = slice(sg.start, sg.end)
            a.reduced = st.reduced[sl].data_ptr()
            a.master, a.m, a.v = st.master[sl].data_ptr(), st.m[sl].data_ptr(), st.v[sl].data_ptr()
            a.sumsq = self._norm_sq.data_ptr() if (pull and sg.in_norm and clip) else None
            a.clip_coef = self._coef.data_ptr() if use_clip else None
            a.found_inf = self._found_inf.data_ptr() if use_clip else None
            a.n, a.shard_offset = sg.end - sg.start, st.lo + sg.start
            a.grad_scale = float(buf.gradient_scaling_factor) * (1.0 / h.world if buf.ddp_config.average_in_collective else 1.0)
            a.lr, a.beta1, a.beta2, a.eps, a.wd = lr * sg.lr_mult, cfg.adam_beta1, cfg.adam_beta2, cfg.adam_eps, wd * sg.wd_mult
            a.step, a.world, a.rank = self.step_count, h.world, h.rank
            a.grad_is_bf16 = int(buf.grad_data.dtype == torch.bfloat16)
            a.pull, a.do_adam, a.push = int(pull), int(do_adam), int(push)
            a.epoch = h.next_epoch()
            a.flag_local = h.ptr(h.rank, 0)
            a.status = st_word.data_ptr()
            loader.check(L.msb_dist_opt_fused(ctypes.byref(a), ctypes.c_void_p(loader.stream_ptr())), "dist_opt_fused")
            st.last_epoch = a.epoch

        def padded(st):
            """This rank's segments followed by empty ones up to the group-wide maximum for the bucket: an empty launch
            still performs the entry handshake and the exit flag, so every rank's epoch sequence is the same."""
            empty = _Segment(0, 0, 0.0, 1.0, False)
            return list(st.segments) + [empty] * (getattr(st, "max_segments", len(st.segments)) - len(st.segments))

        states = [st for st in self._all_states()]
        for st in states:
            if not getattr(st.buf, "fused", False) or st.residual is not None or st.master is None:
                raise RuntimeError("--use-fused-dist-opt needs bf16 parameters with fp32 masters in every buffer "
                                   "(not --reuse-fp32-param) and a data-parallel group of 2..8 GPUs")
            if not hasattr(st, "reduced"):
                st.reduced = torch.zeros_like(st.m)
        grad_norm = None
        if clip:
            self._norm_sq.zero_()
            for st in states:
                for sg in padded(st):
                    launch(st, sg, True, False, False, False)
            dist.all_reduce(self._norm_sq, group=ps.get_data_parallel_group(with_context_parallel=True))
            mp = ps.get_model_parallel_group()
            if mp is not None and dist.get_world_size(mp) > 1:
                dist.all_reduce(self._norm_sq, group=mp)
            adam_ops.clip_coef(self._norm_sq, cfg.clip_grad, self._coef, self._found_inf, self._norm)
            grad_norm = self._norm
            for st in states:
                for sg in padded(st):
                    launch(st, sg, False, True, True, True)
        else:
            for st in states:
                for sg in padded(st):
                    launch(st, sg, True, True, True, False)
        for st in states:                    # the next forward reads the parameter buffer: wait (bounded) for every peer's pushes
            h = st.buf.heap
            loader.check(L.msb_dist_opt_wait_params(ctypes.c_void_p(h.ptr(h.rank, 0)), ctypes.c_uint(st.last_epoch), h.world,
                                                    ctypes.c_void_p(st_word.data_ptr()), 0, ctypes.c_void_p(loader.stream_ptr())),
                         "dist_opt_wait_params")
        return True, grad_norm, None

    # ---- EMA helpers (reference: fused_ema_adamw store/restore/copy_to) ----
    def ema_swap_in(self):
        """Put EMA weights into the model (for evaluation); returns a token to restore."""
        saved = []
        for st in self._all_states():
            tgt = st.param16 if st.param16 is not None else st.master
            saved.append(tgt.clone())
            tgt.copy_(st.ema)
        if self.sharded:
            for chunk in self.model_chunks:
                chunk.start_param_sync(force_sync=True)
        return saved

    def ema_swap_out(self, saved):
        for st, s in zip(self._all_states(), saved):
            tgt = st.param16 if st.param16 is not None else st.master
            tgt.copy_(s)
        if self.sharded:
            for chunk in self.model_chunks:
                chunk.start_param_sync(force_sync=True)

    # ---- state dict ----
    def state_dict(self):
        out = {"step": self.step_count, "param_groups": [{k: v for k, v in g.items()} for g in self.param_groups], "buckets": []}
        for st in self._all_states():
            d = {"lo": st.lo, "hi": st.hi, "exp_avg": st.m, "exp_avg_sq": st.v}
            if st.residual is not None:
                d["residual"] = st.residual
            elif st.param16 is not None:
                d["master"] = st.master
            if st.ema is not None:
                d["ema"] = st.ema
            out["buckets"].append(d)
        return out

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        for g, s in zip(self.param_groups, sd["param_groups"]):
            g.update(s)
        for st, d in zip(self._all_states(), sd["buckets"]):
            st.m.copy_(d["exp_avg"])
            st.v.copy_(d["exp_avg_sq"])
            if "residual" in d and st.residual is not None:
                st.residual.copy_(d["residual"])
            if "master" in d and st.param16 is not None and st.master is not None:
                st.master.copy_(d["master"])
            if "ema" in d and st.ema is not None:
                st.ema.copy_(d["ema"])

    def sharded_state_dict(self, model_sharded_state_dict=None, is_loading=False, sharding_type="fully_sharded_bucket_space"):
        from ..checkpointing.sharded import optimizer_sharded_state_dict
        return optimizer_sharded_state_dict(self, sharding_type)


def get_megatron_optimizer(config: OptimizerConfig, model_chunks, no_weight_decay_cond=None, scale_lr_cond=None, lr_mult=1.0):
    """Factory with the reference's ``--optimizer-selection`` / ``--optimizer`` switches."""
    if config.optimizer == "muon":
        from .muon import build_muon_optimizer
        return build_muon_optimizer(config, model_chunks)
    try:
        from ..training.global_vars import get_args
        virt = getattr(get_args(), "virtual_optimizer", None)
    except RuntimeError:
        virt = None
    if virt:
        from .virtual_adam import VirtualDistributedOptimizer
        return VirtualDistributedOptimizer(config, model_chunks, virt, no_weight_decay_cond, scale_lr_cond, lr_mult)
    if config.swap_optimizer:
        from .swap_optimizer import SwapDistributedOptimizer
        return SwapDistributedOptimizer(config, model_chunks, no_weight_decay_cond, scale_lr_cond, lr_mult)
    if getattr(config, "compress_optimizer", False):
        from .compressed_states import CompressedStateDistributedOptimizer
        return CompressedStateDistributedOptimizer(config, model_chunks, no_weight_decay_cond, scale_lr_cond, lr_mult)
    if config.quant_states:
        from .low_precision import QuantStateDistributedOptimizer
        return QuantStateDistributedOptimizer(config, model_chunks, no_weight_decay_cond, scale_lr_cond, lr_mult)
    if config.optimizer_selection == "fused_ema_adamw":
        config.use_ema = True
    return DistributedOptimizer(config, model_chunks, no_weight_decay_cond, scale_lr_cond, lr_mult)
