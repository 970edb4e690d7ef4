"""Search space of parallel configurations and its first-stage pruning
(reference rules: mindspeed/auto_settings/module/search/stage_1_prune.py:33-102)."""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import List, Optional


@dataclass(frozen=True)
class ModelDesc:
    num_layers: int
    hidden_size: int
    ffn_hidden_size: int
    num_attention_heads: int
    num_query_groups: int
    vocab_size: int
    seq_length: int
    global_batch_size: int
    num_experts: Optional[int] = None
    moe_topk: int = 2
    moe_ffn_hidden_size: Optional[int] = None
    gated: bool = True
    kv_channels: int = 128

    @staticmethod
    def from_args(a):
        return ModelDesc(a.num_layers, a.hidden_size, a.ffn_hidden_size, a.num_attention_heads, a.num_query_groups or a.num_attention_heads,
                         a.padded_vocab_size or a.vocab_size, a.seq_length, a.global_batch_size, a.num_experts, a.moe_router_topk,
                         a.moe_ffn_hidden_size, bool(a.swiglu), a.kv_channels or a.hidden_size // a.num_attention_heads)

    def dense_params_per_layer(self):
        d = self.kv_channels
        attn = self.hidden_size * (self.num_attention_heads * d + 2 * self.num_query_groups * d) + self.num_attention_heads * d * self.hidden_size
        mlp = self.hidden_size * self.ffn_hidden_size * (3 if self.gated else 2)
        return attn, mlp

    def expert_params_per_layer(self):
        if not self.num_experts:
            return 0
        f = self.moe_ffn_hidden_size or self.ffn_hidden_size
        return self.num_experts * self.hidden_size * f * (3 if self.gated else 2)


@dataclass(frozen=True)
class SearchConfig:
    tp: int = 1
    cp: int = 1
    pp: int = 1
    vpp: int = 1
    dp: int = 1
    ep: int = 1
    mbs: int = 1
    recompute_layers: int = 0          # full recompute of this many layers per stage
    sequence_parallel: bool = True
    use_distributed_optimizer: bool = True
    fused_tp_comm: bool = True         # the fused all-gather/GEMM/reduce-scatter kernels

    def to_flags(self) -> List[str]:
        f = ["--tensor-model-parallel-size", str(self.tp), "--context-parallel-size", str(self.cp),
             "--pipeline-model-parallel-size", str(self.pp), "--micro-batch-size", str(self.mbs)]
        if self.ep > 1:
            f += ["--expert-model-parallel-size", str(self.ep)]
        if self.tp > 1 and self.sequence_parallel:
            f += ["--sequence-parallel"]
            if self.fused_tp_comm:
                f += ["--use-fused-tp-comm"]
        if self.use_distributed_optimizer:
            f += ["--use-distributed-optimizer"]
        if self.recompute_layers > 0:
            f += ["--recompute-granularity", "full", "--recompute-method", "block", "--recompute-num-layers", str(self.recompute_layers)]
        return f

    def as_dict(self):
        return asdict(self)


def _pow2_upto(n):
    out, v = [], 1
    while v <= n:
        out.append(v)
        v *= 2
    return out


def build_search_space(model: ModelDesc, world: int, gpus_per_node: int = 8, min_seq_per_cp: int = 4096, max_mbs: int = 2) -> List[SearchConfig]:
    out = []
    for tp in _pow2_upto(min(world, gpus_per_node)):
        if model.num_attention_heads % tp or model.num_query_groups % tp:
            continue
        for cp in _pow2_upto(world // tp):
            if model.seq_length % (2 * cp) or (cp > 1 and model.seq_length // cp < min_seq_per_cp):
                continue
            for pp in _pow2_upto(world // (tp * cp)):
                if model.num_layers % pp:
                    continue
                dp = world // (tp * cp * pp)
                if tp * cp * pp * dp != world:
                    continue
                eps = [1]
                if model.num_experts:
                    eps = [e for e in _pow2_upto(cp * dp) if model.num_experts % e == 0 and (cp * dp) % e == 0]
                for ep in eps:
                    for mbs in range(1, max_mbs + 1):
                        if model.global_batch_size % (dp * mbs):
                            continue
                        n_mb = model.global_batch_size // (dp * mbs)
                        if pp > 1 and n_mb < pp:
                            continue
                        per_stage = model.num_layers // pp
                        for rl in sorted({0, per_stage // 2, per_stage}):
                            out.append(SearchConfig(tp=tp, cp=cp, pp=pp, dp=dp, ep=ep, mbs=mbs, recompute_layers=rl))
    return out


def stage_1_prune(configs: List[SearchConfig], model: ModelDesc, memory_fn, budget_gib: float) -> List[SearchConfig]:
    """First-stage pruning before anything is timed (reference rules: mindspeed/auto_settings/module/search/
    stage_1_prune.py:33-102):
      * drop what cannot fit: configurations whose modelled memory exceeds the budget even with every layer recomputed;
      * among configurations that differ only in the number of recomputed layers keep the smallest count that fits
        (more recompute is never faster);
      * drop pipeline splits with fewer micro-batches than 2 x stages (bubble above one third) when a configuration with the
        same tensor / context sizes and a shallower pipeline fits;
      * drop context parallelism when the same configuration without it fits (it only adds ring traffic)."""
    by_key = {}
    for c in configs:
        mem = memory_fn(model, c)["total"]
        if mem > budget_gib:
            continue
        k = (c.tp, c.cp, c.pp, c.vpp, c.dp, c.ep, c.mbs, c.sequence_parallel, c.use_distributed_optimizer, c.fused_tp_comm)
        if k not in by_key or c.recompute_layers < by_key[k].recompute_layers:
            by_key[k] = c
    kept = list(by_key.values())
    fits = {(c.tp, c.cp, c.pp, c.ep, c.mbs) for c in kept}
    out = []
    for c in kept:
        n_mb = model.global_batch_size // (c.dp * c.mbs)
        shallower = any((c.tp, c.cp, p, c.ep, c.mbs) in fits for p in range(1, c.pp))
        if c.pp > 1 and n_mb < 2 * c.pp and shallower:
            continue
        if c.cp > 1 and any((c.tp, q, c.pp, e, c.mbs) in fits for q in range(1, c.cp) for e in (c.ep, max(1, c.ep // 2))):
            continue
        out.append(c)
    return out
