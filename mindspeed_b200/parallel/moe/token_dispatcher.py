"""MoE token dispatchers: all-gather and all-to-all (+ overlapped variant).

All-to-all contract (reference: mindspeed/core/transformer/moe/moe_feature/overlap/token_dispatcher.py:519-975):
  preprocess     tokens per expert -> input_splits / output_splits (one host sync for the split sizes)
  permute-1      local sort by global expert id
  all-to-all-v   tokens (and their probabilities as a second tensor) over the expert-parallel group
  permute-2      regroup the received [source rank][local expert] chunks to [local expert][source rank]
  experts        grouped GEMM on expert-sorted rows
  combine        exact reverse, probabilities applied in the final un-permute
With ``overlap=True`` the probability all-to-all and the shared expert run on side streams while the token
all-to-all is in flight.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .. import mappings as M
from .. import parallel_state as ps
from .moe_utils import permute, sort_chunks_by_idxs, unpermute


class MoETokenDispatcher:
    def __init__(self, config):
        self.config = config
        self.ep_group = ps.get_expert_model_parallel_group(check_initialized=False)
        self.ep_size = ps.get_expert_model_parallel_world_size()
        self.ep_rank = ps.get_expert_model_parallel_rank()
        self.tp_size = ps.get_expert_tensor_parallel_world_size()
        self.shared_experts = None

    def set_shared_experts(self, se):
        self.shared_experts = se


class _GatherRowsAsync(torch.autograd.Function):
    """All-gather along dim 0 that returns before the collective has finished: the caller keeps the work handle and
    waits on it right before the first use.  Backward is the matching reduce-scatter."""

    @staticmethod
    def forward(ctx, x, group, holder):
        ctx.group = group
        world = dist.get_world_size(group)
        out = torch.empty((x.shape[0] * world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        holder.append(dist.all_gather_into_tensor(out, x.contiguous(), group=group, async_op=True))
        return out

    @staticmethod
    def backward(ctx, dout):
        world = dist.get_world_size(ctx.group)
        dx = torch.empty((dout.shape[0] // world,) + tuple(dout.shape[1:]), dtype=dout.dtype, device=dout.device)
        dist.reduce_scatter_tensor(dx, dout.contiguous(), group=ctx.group)
        return dx, None, None


class MoEAllGatherTokenDispatcher(MoETokenDispatcher):
    """Every EP rank gathers all tokens, computes its local experts on the ones routed to them, and the results are
    reduce-scattered back (reference: moe_layer_overlap_allgather.py; docs megatron-moe-allgather-dispatcher.md).

    ``overlap`` (``--moe-allgather-overlap-comm``): the layer calls ``pre_gather`` before the router, so the all-gather of
    the hidden states - the large transfer, which does not depend on the routing - is in flight while the router (and the
    shared expert) compute; only the small gathers of probabilities and routing map follow the router."""

    def __init__(self, num_local_experts, local_expert_indices, config, overlap: bool = False):
        super().__init__(config)
        self.num_local_experts, self.local_expert_indices = num_local_experts, local_expert_indices
        self.group = ps.get_expert_tensor_and_model_parallel_group(check_initialized=False)
        self.gsize = ps.get_expert_tensor_and_model_parallel_world_size()
        self.overlap = overlap
        self._pre = None

    def pre_gather(self, hidden):
        """Start the all-gather of the hidden states; ``token_permutation`` picks the result up."""
        if not self.overlap or self.gsize <= 1:
            return
        holder = []
        h = hidden.reshape(-1, hidden.shape[-1])
        self._pre = (_GatherRowsAsync.apply(h, self.group, holder), holder)

    def token_permutation(self, hidden, probs, routing_map):
        self.hidden_shape = hidden.shape
        h = hidden.reshape(-1, hidden.shape[-1])
        pre, self._pre = self._pre, None
        if self.gsize > 1:
            if pre is not None:
                h, holder = pre
                for w in holder:
                    w.wait()
            else:
                h = M.gather_from_sequence_parallel_region(h, group=self.group)
            probs = M.gather_from_sequence_parallel_region(probs, group=self.group)
            with torch.no_grad():
                routing_map = M.all_gather_first_dim(routing_map.to(torch.uint8), self.group).bool()
        lo, hi = self.local_expert_indices[0], self.local_expert_indices[-1] + 1
        self.local_map = routing_map[:, lo:hi].contiguous()
        self.local_probs = probs[:, lo:hi].contiguous()
        tokens_per_expert = self.local_map.sum(0).cpu()
        self.restore_shape = h.shape
        permuted, self.sorted_indices = permute(h, self.local_map)
        pprobs = self.local_probs.t().contiguous().masked_select(self.local_map.t().contiguous())
        return permuted, tokens_per_expert, pprobs

    def token_unpermutation(self, expert_out, bias=None):
        out = unpermute(expert_out, self.sorted_indices, self.restore_shape)
        if self.gsize > 1:
            out = M.reduce_scatter_to_sequence_parallel_region(out, group=self.group)
        return out.view(self.hidden_shape), None


class MoEAlltoAllTokenDispatcher(MoETokenDispatcher):
    def __init__(self, num_local_experts, local_expert_indices, config, overlap: bool = False):
        super().__init__(config)
        self.num_local_experts, self.local_expert_indices = num_local_experts, local_expert_indices
        self.num_experts = config.num_moe_experts
        if self.tp_size > 1:
            raise NotImplementedError("the all-to-all dispatcher runs with expert tensor parallel size 1 "
                                      "(use --moe-tp-extend-ep to turn tensor-parallel ranks into expert-parallel ones)")
        self.overlap = overlap
        self.fused_permute = config.optimization_level >= 1 or getattr(config, "use_fused_moe_token_permute_and_unpermute", False)
        # chunk order after the all-to-all is [src rank][local expert]; experts want [local expert][src rank]
        idx = torch.arange(self.ep_size * num_local_experts).reshape(self.ep_size, num_local_experts)
        self.sort_fwd = idx.t().reshape(-1).tolist()
        self.sort_bwd = torch.arange(self.ep_size * num_local_experts).reshape(num_local_experts, self.ep_size).t().reshape(-1).tolist()
        self._side = None

    def preprocess(self, routing_map):
        E_loc, ep = self.num_local_experts, self.ep_size
        local_counts = routing_map.sum(dim=0).to(torch.int64)  # [E]
        if ep > 1:
            allc = torch.empty(ep, self.num_experts, dtype=torch.int64, device=local_counts.device)
            dist.all_gather_into_tensor(allc, local_counts.contiguous(), group=self.ep_group) if dist.get_backend(self.ep_group) != "gloo" \
                else dist.all_gather(list(allc.unbind(0)), local_counts.contiguous(), group=self.ep_group)
            mine = allc[:, self.local_expert_indices[0]:self.local_expert_indices[-1] + 1]  # [ep, E_loc]
            host = torch.cat([local_counts.reshape(ep, E_loc).sum(1), mine.reshape(-1)]).cpu()  # single D2H sync
            self.input_splits = host[:ep].tolist()
            per_src_expert = host[ep:].reshape(ep, E_loc)
            self.output_splits = per_src_expert.sum(1).tolist()
            self.chunk_sizes = per_src_expert.reshape(-1).tolist()
            tokens_per_expert = per_src_expert.sum(0)
        else:
            host = local_counts.cpu()
            self.input_splits = self.output_splits = None
            self.chunk_sizes = host.tolist()
            tokens_per_expert = host
        return tokens_per_expert

    def token_permutation(self, hidden, probs, routing_map):
        self.hidden_shape = hidden.shape
        h = hidden.reshape(-1, hidden.shape[-1])
        self.routing_map, self.probs = routing_map, probs
        tokens_per_expert = self.preprocess(routing_map)
        self.restore_shape = h.shape
        permuted, self.sorted_indices = permute(h, routing_map, fused=self.fused_permute)
        pprobs = probs.t().contiguous().masked_select(routing_map.t().contiguous())
        if self.ep_size > 1:
            if self.overlap and permuted.is_cuda:
                if self._side is None:
                    self._side = torch.cuda.Stream()
                self._side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self._side):
                    gprobs = M.all_to_all(self.ep_group, pprobs.unsqueeze(-1), self.output_splits, self.input_splits).squeeze(-1)
                gtokens = M.all_to_all(self.ep_group, permuted, self.output_splits, self.input_splits)
                torch.cuda.current_stream().wait_stream(self._side)
            else:
                gtokens = M.all_to_all(self.ep_group, permuted, self.output_splits, self.input_splits)
                gprobs = M.all_to_all(self.ep_group, pprobs.unsqueeze(-1), self.output_splits, self.input_splits).squeeze(-1)
        else:
            gtokens, gprobs = permuted, pprobs
        if self.num_local_experts > 1 and self.ep_size > 1:
            gtokens, gprobs = sort_chunks_by_idxs(gtokens, self.chunk_sizes, self.sort_fwd, gprobs)
        return gtokens, tokens_per_expert, gprobs

    def token_unpermutation(self, expert_out, bias=None):
        """``expert_out`` rows are already weighted by the router probabilities (applied in the expert activation)."""
        if self.num_local_experts > 1 and self.ep_size > 1:
            sizes = [self.chunk_sizes[i] for i in self.sort_fwd]
            expert_out = sort_chunks_by_idxs(expert_out, sizes, self.sort_bwd)
        if self.ep_size > 1:
            expert_out = M.all_to_all(self.ep_group, expert_out, self.input_splits, self.output_splits)
        out = unpermute(expert_out, self.sorted_indices, self.restore_shape, fused=self.fused_permute)
        return out.view(self.hidden_shape), None
