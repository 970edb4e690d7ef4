"""3-D convolution with the depth (frame) dimension split over a process group.

Each rank holds a contiguous slab of frames.  A kernel of depth k with stride 1 needs k-1 extra frames across slab
boundaries ("halo"): before the convolution every rank receives the missing frames from its depth neighbours, and
in backward the gradient of the halo is sent back and added to the neighbour's slab gradient.  The weights are
replicated; their gradients are all-reduced over the group.

Padding along depth is applied only at the two outer ends of the full volume, so the concatenated outputs of all
ranks equal the unsplit convolution.  Requirements: depth stride 1, dilation 1, slab depth >= halo.
reference: mindspeed/multi_modal/conv3d/conv3d_depth_parallel.py:8-205.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .. import mappings as M


class _HaloExchange(torch.autograd.Function):
    """x [N, C, D_local, H, W] -> [N, C, left + D_local + right, H, W] with neighbour frames attached."""

    @staticmethod
    def forward(ctx, x, group, left, right):
        n, r = M._ws(group), M._rk(group)
        ctx.group, ctx.left, ctx.right, ctx.n, ctx.r = group, left, right, n, r
        parts = []
        reqs = []
        recv_l = recv_r = None
        if left > 0 and r > 0:
            recv_l = torch.empty_like(x[:, :, :left])
            reqs.append(dist.irecv(recv_l, dist.get_global_rank(group, r - 1), group=group))
        if right > 0 and r < n - 1:
            recv_r = torch.empty_like(x[:, :, :right])
            reqs.append(dist.irecv(recv_r, dist.get_global_rank(group, r + 1), group=group))
        if left > 0 and r < n - 1:      # my last frames are my right neighbour's left halo
            reqs.append(dist.isend(x[:, :, -left:].contiguous(), dist.get_global_rank(group, r + 1), group=group))
        if right > 0 and r > 0:
            reqs.append(dist.isend(x[:, :, :right].contiguous(), dist.get_global_rank(group, r - 1), group=group))
        for q in reqs:
            q.wait()
        if recv_l is not None:
            parts.append(recv_l)
        parts.append(x)
        if recv_r is not None:
            parts.append(recv_r)
        return torch.cat(parts, dim=2) if len(parts) > 1 else x.clone()

    @staticmethod
    def backward(ctx, g):
        group, left, right, n, r = ctx.group, ctx.left, ctx.right, ctx.n, ctx.r
        has_l, has_r = left > 0 and r > 0, right > 0 and r < n - 1
        lo = left if has_l else 0
        hi = g.shape[2] - (right if has_r else 0)
        gx = g[:, :, lo:hi].clone()
        reqs = []
        add_r = add_l = None
        if left > 0 and r < n - 1:      # gradient of the frames I sent to the right comes back from the right
            add_r = torch.empty_like(gx[:, :, :left])
            reqs.append(dist.irecv(add_r, dist.get_global_rank(group, r + 1), group=group))
        if right > 0 and r > 0:
            add_l = torch.empty_like(gx[:, :, :right])
            reqs.append(dist.irecv(add_l, dist.get_global_rank(group, r - 1), group=group))
        if has_l:
            reqs.append(dist.isend(g[:, :, :left].contiguous(), dist.get_global_rank(group, r - 1), group=group))
        if has_r:
            reqs.append(dist.isend(g[:, :, hi:].contiguous(), dist.get_global_rank(group, r + 1), group=group))
        for q in reqs:
            q.wait()
        if add_r is not None:
            gx[:, :, -left:] += add_r
        if add_l is not None:
            gx[:, :, :right] += add_l
        return gx, None, None, None


class Conv3dDepthParallel(nn.Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, bias=True, group=None,
                 conv: Optional[nn.Conv3d] = None):
        super().__init__()
        self.conv = conv if conv is not None else nn.Conv3d(in_channels, out_channels, kernel_size, stride, padding, bias=bias)
        c = self.conv
        if c.stride[0] != 1 or c.dilation[0] != 1:
            raise ValueError("depth-parallel convolution needs depth stride 1 and dilation 1")
        if isinstance(c.padding, str):
            raise ValueError("string padding modes are not supported")
        self.group = group
        self.kd, self.pd = c.kernel_size[0], c.padding[0]
        for p in self.conv.parameters():
            p.depth_parallel_replicated = True

    def forward(self, x):
        """x: this rank's slab [N, C, D_local, H, W]; returns this rank's slab of the output."""
        n, r = M._ws(self.group), M._rk(self.group)
        c = self.conv
        if n == 1:
            return c(x)
        total_halo = self.kd - 1
        left = self.pd                      # frames needed before the slab (same as the padding at the outer end)
        right = total_halo - self.pd
        if left < 0 or right < 0:
            raise ValueError("depth padding larger than kernel depth - 1 is not supported")
        if x.shape[2] < max(left, right):
            raise ValueError("slab depth smaller than the halo")
        y = _HaloExchange.apply(x, self.group, left, right)
        pad_front = self.pd if r == 0 else 0
        pad_back = self.pd if r == n - 1 else 0
        # with stride 1 each rank must produce exactly D_local frames except at the ends when padding < (k-1)/2
        if right > 0 and r == n - 1 and pad_back < right:
            pass    # the last rank simply has fewer valid output frames, as the unsplit convolution does
        if pad_front or pad_back:
            y = F.pad(y, (0, 0, 0, 0, pad_front, pad_back))
        return F.conv3d(y, c.weight, c.bias, stride=c.stride, padding=(0, c.padding[1], c.padding[2]), dilation=c.dilation,
                        groups=c.groups)

    def allreduce_weight_grads(self):
        """Sum the replicated weights' gradients over the depth group (call after backward)."""
        if M._ws(self.group) == 1:
            return
        for p in self.conv.parameters():
            if p.grad is not None:
                dist.all_reduce(p.grad, group=self.group)
