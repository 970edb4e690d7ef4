"""Argument presets for the benchmark configurations (shapes only; parallel layout is added by the caller)."""
from __future__ import annotations

from typing import List


def _common(seq, gbs, vocab, std=0.02) -> List[str]:
    return ["--seq-length", str(seq), "--max-position-embeddings", str(seq), "--micro-batch-size", "1",
            "--global-batch-size", str(gbs), "--vocab-size", str(vocab), "--make-vocab-size-divisible-by", "1",
            "--init-method-std", str(std), "--hidden-dropout", "0", "--attention-dropout", "0", "--bf16",
            "--lr", "1e-4", "--lr-decay-style", "constant", "--weight-decay", "0.1", "--clip-grad", "1.0",
            "--adam-beta2", "0.95", "--untie-embeddings-and-output-weights", "--disable-bias-linear",
            "--normalization", "RMSNorm", "--norm-epsilon", "1e-5", "--swiglu", "--position-embedding-type", "rope",
            "--use-flash-attn", "--mock-data", "--seed", "1234"]


def llama3_8b(seq=8192, gbs=64) -> List[str]:
    """32 layers, hidden 4096, 32 heads / 8 KV heads, SwiGLU 14336, RMSNorm 1e-5, RoPE theta 5e5, vocab 128256."""
    return ["--num-layers", "32", "--hidden-size", "4096", "--num-attention-heads", "32", "--group-query-attention",
            "--num-query-groups", "8", "--ffn-hidden-size", "14336", "--rotary-base", "500000"] + _common(seq, gbs, 128256)


def llama2_13b(seq=32768, gbs=8) -> List[str]:
    """40 layers, hidden 5120, 40 heads MHA, SwiGLU 13824, vocab 32000."""
    return ["--num-layers", "40", "--hidden-size", "5120", "--num-attention-heads", "40", "--ffn-hidden-size", "13824",
            "--rotary-base", "10000"] + _common(seq, gbs, 32000)


def mixtral_8x7b(seq=4096, gbs=64) -> List[str]:
    """32 layers, hidden 4096, 32/8 heads, 8 experts top-2 softmax, expert FFN 14336, aux loss 0.01, vocab 32000."""
    return ["--num-layers", "32", "--hidden-size", "4096", "--num-attention-heads", "32", "--group-query-attention",
            "--num-query-groups", "8", "--ffn-hidden-size", "14336", "--rotary-base", "1000000", "--num-experts", "8",
            "--moe-router-topk", "2", "--moe-aux-loss-coeff", "0.01", "--moe-token-dispatcher-type", "alltoall",
            "--moe-grouped-gemm", "--moe-router-load-balancing-type", "aux_loss"] + _common(seq, gbs, 32000)


def deepseek_v3_reduced(seq=4096, gbs=16) -> List[str]:
    """16 layers (first 2 dense, FFN 12288), hidden 4096, MLA 32 heads, 64 routed experts top-6 sigmoid + 1 shared,
    expert FFN 1536, vocab 129280, N(0, 0.006) init."""
    return ["--num-layers", "16", "--hidden-size", "4096", "--num-attention-heads", "32", "--ffn-hidden-size", "12288",
            "--multi-latent-attention", "--q-lora-rank", "1536", "--kv-lora-rank", "512", "--qk-nope-head-dim", "128",
            "--qk-rope-head-dim", "64", "--v-head-dim", "128", "--num-experts", "64", "--moe-router-topk", "6",
            "--moe-router-score-function", "sigmoid", "--moe-router-enable-expert-bias", "--moe-ffn-hidden-size", "1536",
            "--moe-shared-expert-intermediate-size", "1536", "--first-k-dense-replace", "2",
            "--moe-token-dispatcher-type", "alltoall", "--moe-grouped-gemm", "--moe-router-load-balancing-type", "seq_aux_loss",
            "--moe-aux-loss-coeff", "0.0001", "--rotary-base", "10000"] + _common(seq, gbs, 129280, std=0.006)


def tiny_gpt() -> List[str]:
    return ["--num-layers", "2", "--hidden-size", "256", "--num-attention-heads", "4", "--ffn-hidden-size", "1024",
            "--seq-length", "128", "--max-position-embeddings", "128", "--micro-batch-size", "2", "--global-batch-size", "4",
            "--vocab-size", "1024", "--make-vocab-size-divisible-by", "1", "--lr", "1e-4", "--lr-decay-style", "constant",
            "--hidden-dropout", "0", "--attention-dropout", "0", "--seed", "1234", "--init-method-std", "0.02",
            "--weight-decay", "0.0", "--untie-embeddings-and-output-weights"]


PRESETS = {"llama3-8b": llama3_8b, "llama2-13b": llama2_13b, "mixtral-8x7b": mixtral_8x7b,
           "deepseek-v3-reduced": deepseek_v3_reduced, "tiny-gpt": tiny_gpt}
