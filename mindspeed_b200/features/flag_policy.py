"""What happens to a registered flag that no code path reads.

Every command-line flag of the reference is accepted by the parser so that existing launch scripts keep working
(reference flag surface: mindspeed/arguments.py:27-929 and the ``register_args`` of mindspeed/features_manager/*).
A flag must then do one of three things, and ``tests/test_flag_policy_cpu.py`` fails when a flag does none:

  * be read by the framework (the normal case);
  * appear in ``NO_EFFECT`` with the reason why it changes nothing here (a knob of the reference's hardware or software
    stack without a counterpart on this one, a launcher-only value, or a behaviour this framework always has);
    setting it prints one notice at start-up instead of silently doing nothing;
  * appear in ``UNSUPPORTED`` with a message; setting it to a non-default value stops the run in ``validate_args``.
"""
from __future__ import annotations

from typing import Dict

NO_EFFECT: Dict[str, str] = {
    # --- knobs of the reference's device / communication stack ---
    "aiqos": "per-communicator QoS classes exist only on the reference's interconnect",
    "aiqos-enable-roce": "per-communicator QoS classes exist only on the reference's interconnect",
    "aiqos-mode": "per-communicator QoS classes exist only on the reference's interconnect",
    "aiqos-schedule": "per-communicator QoS classes exist only on the reference's interconnect",
    "hccl-ep-group-buffer-adaptive-factor": "communicator buffer sizing of the reference's collective library; NCCL sizes are set with --nccl-group-buffer",
    "hccl-op-mode": "execution mode of the reference's collective library",
    "jit-compile": "operator JIT switch of the reference's device runtime; kernels here are built ahead of time",
    "use-fusion-attn-v2": "selects between two vendor attention ops; there is one attention kernel family here",
    "megatron-cp-in-bnsd": "layout hint for the vendor attention op; the tcgen05 kernels read strided [s, b, n, d] directly",
    "attention-mask-on-cpu": "the causal mask is generated inside the attention kernels, no mask tensor is built",
    "square-alibi-mask": "shape of the ALiBi bias tensor on the unfused path; the bias here is evaluated from the head slopes block by block, no bias tensor of either shape exists",
    "fill-neg-inf": "mask fill value of the unfused softmax path; masked scores are -inf in every kernel here",
    "te-gmm-mode": "grouped-GEMM backend choice of the reference's TE shim; one grouped kernel here",
    "no-use-gmm-fp8": "grouped-GEMM backend choice of the reference's TE shim; fp8 experts follow --fp8-format",
    "fp8-reuse-quantized-weight": "quantised weights are always cached across micro-batches (models/te_compat.py)",
    "transformer-impl": "one implementation (this package's modules with the TE-compatible surface)",
    "use-mcore-models": "the core model classes are the only ones",
    # --- always-on behaviours ---
    "use-fused-lightning-indexer": "the indexer, the sparse attention and the KL loss of --experimental-attention-variant dsa are one implementation (ops/lightning_indexer.py, ops/sparse_attention.py); there is no separate unfused path to switch from",
    "use-fused-sparse-flash-attention": "the indexer, the sparse attention and the KL loss of --experimental-attention-variant dsa are one implementation (ops/lightning_indexer.py, ops/sparse_attention.py); there is no separate unfused path to switch from",
    "use-fused-lightning-indexer-kl-loss": "the indexer, the sparse attention and the KL loss of --experimental-attention-variant dsa are one implementation (ops/lightning_indexer.py, ops/sparse_attention.py); there is no separate unfused path to switch from",
    "shape-order": "layout hint for the vendor attention op; the kernels here read strided [s, b, n, d] directly",
    "enable-token-rearrange-opt": "the DeepSpeed-style MoE here always dispatches through index arithmetic on the one-hot routing; there is no slower einsum path to switch from",
    "skip-bias-add": "every parallel linear here returns its bias separately when the caller fuses the add; there is no switch",
    "use-fused-ring-attention-update": "ring attention carries log-sum-exp values and merges partial results inside its own autograd function; the max / sum form of the update is the stand-alone op ops/misc.ring_attention_update",
    "use-legacy-models": "the core model classes are the only ones",
    "spec": "layer specifications are chosen from the model flags (MLA, MoE, TE-compatible modules); there is no module-spec import",
    "timing-log-level": "step time and throughput are always logged; there are no nested timers to select",
    "timing-log-option": "step time and throughput are always logged; there are no nested timers to select",
    "no-barrier-with-level-1-timing": "step time and throughput are always logged; there are no nested timers to select",
    "no-bias-gelu-fusion": "bias + GeLU run unfused unless the optimisation level enables the fused activation kernels",
    "no-rope-fusion": "the rotary kernel follows --optimization-level / --use-fused-rotary-pos-emb",
    "auto-detect-ckpt-format": "one checkpoint format (torch.distributed.checkpoint) is read and written",
    "dist-ckpt-format": "one checkpoint format (torch.distributed.checkpoint) is read and written",
    "no-shared-storage": "every rank writes its own shard files and reads what it needs; no rank relies on another's local disk",
    "short-seq-prob": "option of the BERT-style sample builder; GPT samples are packed to the full sequence length",
    "img-h": "read by vision-language model definitions built on this package (parallel/multimodal), not by the GPT entry point",
    "img-w": "read by vision-language model definitions built on this package (parallel/multimodal), not by the GPT entry point",
    "patch-dim": "read by vision-language model definitions built on this package (parallel/multimodal), not by the GPT entry point",
    "mbs-idx": "index used by the reference's profiling launcher while it tries the entries of a micro-batch size list; the list itself is --optimized-mbs-list",
    "ampipe-tp-sp-comm-overlap": "the tensor-parallel communication of the attention output projection is already fused with its GEMM (--use-ascend-mc2 / level 2); --ampipe-degree pipelines what follows it",
    "moe-hierarchical-alltoallv": "two-level all-to-all for fabrics where the ranks inside a node are closer than the ones across; inside one NVSwitch domain every peer is one hop away and the exchange is flat (peer-memory dispatch at level 2)",
    "no-create-attention-mask-in-dataloader": "the data path never builds attention masks; the kernels generate the causal mask",
    "overlap-param-gather-with-optimizer-step": "parameter all-gathers start bucket by bucket right after the update (--overlap-param-gather); there is no separate staging to overlap",
    "mla-mm-split": "whether the latent up-projection runs as one GEMM or as separate no-position / rotary and key / value GEMMs; here it is one GEMM per projection whose output is split by views",
    "mla-up-proj-tp-overlap": "tensor-parallel communication of the projections is fused with their GEMMs at level 2 (--use-ascend-mc2)",
    "mtp-mem-efficient-logits": "the multi-token-prediction heads compute their loss with the vocabulary-parallel cross-entropy kernels on the 16-bit logits; no fp32 copy of the logits is kept",
    "adaptive-cp-only-reschedule": "adaptive CP here always keeps the sequence order and only schedules the exchanges",
    "adaptive-cp-without-coarse": "the mask is coarsened to context-parallel rank granularity for scheduling only; nothing else uses the coarse form",
    "gemm-gradient-accumulation-fusion": "weight gradients always accumulate into main_grad inside the GEMM epilogue",
    "no-bias-swiglu-fusion": "SwiGLU is fused whenever the optimisation level allows; level 0 gives the unfused path",
    "coc-mode": "sub-mode of the chunk-pipelining path; --use-ascend-coc / --coc-fused-kernel select the back end",
    "enable-overlap-ag-with-matmul": "the fused all-gather -> GEMM kernel always overlaps",
    "enable-overlap-matmul-with-rs": "the fused GEMM -> reduce-scatter kernel always overlaps",
    "enable-backward-overlap-ag-with-matmul": "backward uses the same fused kernels as forward",
    "moe-permutation-async-comm": "the dispatcher's collectives are already asynchronous with respect to the permute kernels",
    "moe-dynamic-padding": "the grouped GEMM takes ragged expert row ranges, no padding is needed",
    "ckpt-fully-parallel-save": "every rank always writes its own shard file",
    "dist-ckpt-optim-sharding-type": "one optimizer-state chunking is implemented (see checkpointing/sharded.py)",
    "mock-data": "synthetic data is used whenever no --data-path is given",
    # --- launcher-only values (consumed by auto_settings / torchrun, not by a rank) ---
    "master-addr": "launcher value", "node-rank": "launcher value", "nproc-per-node": "launcher value",
    "target-nnodes": "search target of --auto-settings only",
    "auto-settings-log-level": "verbosity of --auto-settings only",
    "num-workers": "the synthetic and indexed datasets are read in-process",
    "tokenizer-not-use-fast": "passed to the HF tokenizer only by the data tools",
}

UNSUPPORTED: Dict[str, str] = {
}


def check_flags(args, parser) -> None:
    """Called at the end of ``validate_args``: stop on unsupported flags, print one notice per no-effect flag that was set."""
    from ..utils.logging import print_rank_0
    dests = {}
    for a in parser._actions:
        for o in a.option_strings:
            if o.startswith("--"):
                dests[o[2:]] = (a.dest, a.default)
    bad = []
    for flag, why in UNSUPPORTED.items():
        if flag in dests:
            dest, default = dests[flag]
            if getattr(args, dest, default) != default:
                bad.append(f"--{flag}: {why}")
    if bad:
        raise NotImplementedError("flags without an implementation were set:\n  " + "\n  ".join(bad))
    for flag, why in NO_EFFECT.items():
        if flag in dests:
            dest, default = dests[flag]
            if getattr(args, dest, default) != default:
                print_rank_0(f"note: --{flag} has no effect here ({why})")
