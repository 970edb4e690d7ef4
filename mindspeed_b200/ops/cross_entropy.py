"""Fused vocabulary-parallel cross entropy (csrc/kernels/cross_entropy.cu).

Forward: one kernel pass over the local logits for (max, sum-exp, target logit), three [tokens]
all-reduces over the tensor-parallel group, one tiny kernel for the loss.  Backward: the gradient
is written in place over the logits buffer (saved by reference, not copied), in the logits' own
dtype.  The logits tensor must therefore not be used by the caller after the loss is computed,
which holds for the language-model head.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import loader
from ._dtypes import code


def available() -> bool:
    return loader.lib() is not None


class _FusedCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, group, ignore_index):
        L = loader.require_lib()
        world = 1 if group is None else dist.get_world_size(group)
        rank = 0 if group is None else dist.get_rank(group)
        lg = logits if logits.is_contiguous() else logits.contiguous()
        vloc = lg.shape[-1]
        rows = lg.numel() // vloc
        tgt = target.reshape(-1).contiguous().long()
        dev = lg.device
        stats = torch.empty(4, rows, dtype=torch.float32, device=dev)
        lmax, lsum, picked, loss = stats[0], stats[1], stats[2], stats[3]
        st = ctypes.c_void_p(loader.stream_ptr())
        ll = ctypes.c_longlong
        loader.check(L.msb_ce_stats(loader.p(lg), loader.p(tgt), loader.p(lmax), loader.p(lsum), loader.p(picked),
                                    ll(rows), vloc, ll(rank * vloc), ll(ignore_index), code(lg.dtype), st), "ce_stats")
        if world > 1:
            gmax = lmax.clone()
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
            loader.check(L.msb_ce_rescale(loader.p(lsum), loader.p(lmax), loader.p(gmax), ll(rows), st), "ce_rescale")
            both = stats[1:3]
            dist.all_reduce(both, group=group)
        else:
            gmax = lmax
        loader.check(L.msb_ce_loss(loader.p(gmax), loader.p(lsum), loader.p(picked), loader.p(tgt), loader.p(loss),
                                   ll(rows), ll(ignore_index), st), "ce_loss")
        ctx.save_for_backward(lg, tgt, gmax, lsum)
        ctx.rank, ctx.vloc, ctx.ignore = rank, vloc, ignore_index
        return loss.clone().reshape(target.shape)

    @staticmethod
    def backward(ctx, g):
        L = loader.require_lib()
        lg, tgt, gmax, gsum = ctx.saved_tensors
        rows = lg.numel() // ctx.vloc
        gout = g.reshape(-1).float().contiguous()
        ll = ctypes.c_longlong
        loader.check(L.msb_ce_grad(loader.p(lg), loader.p(tgt), loader.p(gmax), loader.p(gsum), loader.p(gout), ll(rows),
                                   ctx.vloc, ll(ctx.rank * ctx.vloc), ll(ctx.ignore), code(lg.dtype),
                                   ctypes.c_void_p(loader.stream_ptr())), "ce_grad")
        return lg, None, None, None


def fused_vocab_parallel_cross_entropy(logits, target, group=None, ignore_index=-100):
    return _FusedCE.apply(logits, target, group, ignore_index)
