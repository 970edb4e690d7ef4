"""Tokenizers behind ``--tokenizer-type``: HuggingFace wrapper, byte-level fallback and the null tokenizer."""
from .tokenizer import ByteLevelTokenizer, NullTokenizer, PretrainedFromHF, build_tokenizer

__all__ = ["build_tokenizer", "PretrainedFromHF", "NullTokenizer", "ByteLevelTokenizer"]
