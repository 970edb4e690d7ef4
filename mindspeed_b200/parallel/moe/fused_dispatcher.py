"""All-to-all token dispatcher whose transfers are peer-memory kernels instead of NCCL all-to-all-v.

Selected by ``--moe-alltoall-mc2`` at optimisation level 2.  Contract and return values are those of
``MoEAlltoAllTokenDispatcher``; what changes is how rows move:

  library path   permute (sort by expert) -> all-to-all-v tokens -> all-to-all-v probabilities -> regroup chunks
  this path      one kernel: every expert owner gathers its rows (and their probabilities) from the peers'
                 unpermuted hidden states directly into [local expert][source rank] order
  way back       one kernel: every token owner pulls and sums its k expert outputs (un-permute + all-to-all fused)

The only host synchronisation is the one the library path also has (split sizes / tokens per expert).  When some
rank would receive more rows than the staging slot holds (capacity = ``MSB200_MOE_STAGE_FACTOR`` x tokens x top-k,
default 2.0) every rank takes the library path for that call - all ranks see the same count matrix, so the choice
is consistent without further communication.
reference: mindspeed/core/transformer/moe/moe_feature/overlap/token_dispatcher.py:519-975 and the --moe-alltoall-mc2
feature (mindspeed/features_manager/moe/fused_mc2.py) that swaps in fused dispatch / combine vendor ops.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ...ops import moe_comm as MC
from .token_dispatcher import MoEAlltoAllTokenDispatcher


class FusedAlltoAllTokenDispatcher(MoEAlltoAllTokenDispatcher):
    def __init__(self, num_local_experts, local_expert_indices, config):
        super().__init__(num_local_experts, local_expert_indices, config, overlap=False)
        self._comm = None
        self._fused_now = False
        self.fused_calls = 0
        self.fallback_calls = 0

    # -- helpers ------------------------------------------------------------------------------------------------
    def _capacity_rows(self, T: int) -> int:
        topk = int(getattr(self.config, "moe_router_topk", 1) or 1)
        return max(128, int(MC.stage_factor() * T * topk))

    def _eligible(self, h: torch.Tensor) -> bool:
        return (h.is_cuda and h.dtype == torch.bfloat16 and 2 <= self.ep_size <= MC.MAX_RANKS
                and (h.shape[1] * h.element_size()) % 16 == 0 and self.num_experts == self.num_local_experts * self.ep_size
                and getattr(self.config, "moe_expert_capacity_factor", None) is None)   # token dropping: library path

    def _counts(self, routing_map, T):
        """[ep, E + 1] on the device: per-expert counts of every source rank, last column = its token count."""
        local = torch.cat([routing_map.sum(dim=0).to(torch.int64), torch.tensor([T], dtype=torch.int64, device=routing_map.device)])
        allc = torch.empty(self.ep_size, self.num_experts + 1, dtype=torch.int64, device=local.device)
        dist.all_gather_into_tensor(allc, local.contiguous(), group=self.ep_group)
        return allc

    # -- dispatcher contract ------------------------------------------------------------------------------------
    def token_permutation(self, hidden, probs, routing_map):
        h = hidden.reshape(-1, hidden.shape[-1])
        if not self._eligible(h):
            self._fused_now = False
            self.fallback_calls += 1
            return super().token_permutation(hidden, probs, routing_map)
        self.hidden_shape = hidden.shape
        T, H = h.shape
        E, E_loc, ep = self.num_experts, self.num_local_experts, self.ep_size
        allc = self._counts(routing_map, T)
        topk = int(getattr(self.config, "moe_router_topk", 1) or 1)
        cap_rows = self._capacity_rows(T)
        if self._comm is None:
            self._comm = MC.context(self.ep_group, MC.slot_bytes_needed(T, H, E, cap_rows, h.element_size()))
        # index tables and staging copies are queued BEFORE the host read of the counts, so the GPU works through them
        # while the host waits; only the output allocation and the kernel launch depend on host-side numbers
        plan = MC.build_plan_fused(routing_map, probs.reshape(T, E), allc, self.ep_rank, ep, T * topk)
        staged = MC.prestage_dispatch(self._comm, plan, h, probs.reshape(T, E))
        host = allc.cpu()                                              # the one host synchronisation of the layer
        if not bool((host[:, E] == T).all()):
            raise NotImplementedError("the fused MoE dispatcher needs the same number of tokens on every expert-parallel rank")
        counts_h = host[:, :E]
        if int(counts_h[self.ep_rank].sum()) != T * topk:
            raise NotImplementedError("the fused MoE dispatcher needs exactly top-k routed experts per token")
        recv_per_rank = counts_h.reshape(ep, ep, E_loc).sum(dim=(0, 2))   # rows every owner receives
        lo = self.ep_rank * E_loc
        tokens_per_expert = counts_h[:, lo:lo + E_loc].sum(0)
        if int(recv_per_rank.max()) > cap_rows:
            # same decision on every rank (all see the same count matrix); the staged slot is simply not used
            self._fused_now = False
            self.fallback_calls += 1
            return super().token_permutation(hidden, probs, routing_map)
        plan.R = int(recv_per_rank[self.ep_rank])
        self._plan, self._cap_rows, self._fused_now = plan, cap_rows, True
        self.fused_calls += 1
        rows, row_probs = MC.dispatch(h, probs.reshape(T, E), self._comm, plan, cap_rows, staged)
        return rows, tokens_per_expert, row_probs

    def token_unpermutation(self, expert_out, bias=None):
        if not self._fused_now:
            return super().token_unpermutation(expert_out, bias)
        out = MC.combine(expert_out, self._comm, self._plan, self._cap_rows)
        return out.view(self.hidden_shape), None
