"""Tokenizer wrappers with the Megatron tokenizer interface (``tokenize``, ``detokenize``, ``vocab_size``, ``eod``, ...).

  PretrainedFromHF   transformers.AutoTokenizer loaded from a local directory (``--tokenizer-name-or-path``); a pad token
                     is added when the model has none; the padded vocabulary size follows --make-vocab-size-divisible-by
  NullTokenizer      integer ids in, integer ids out (synthetic data, benchmarks); eod = vocab_size - 1
  ByteLevelTokenizer UTF-8 bytes + specials, no files needed (smoke tests, data tools without a model directory)
reference: mindspeed/tokenizer/tokenizer.py:24-63 (PretrainedFromHF), mindspeed/features_manager/tokenizer/build_tokenizer.py:16-23.
"""
from __future__ import annotations

from typing import Dict, List, Optional


def _pad_vocab(n: int, divisible_by: int, tp: int) -> int:
    m = divisible_by * tp
    return ((n + m - 1) // m) * m


class _Base:
    name = "base"

    def tokenize(self, text: str) -> List[int]:
        raise NotImplementedError

    def detokenize(self, ids) -> str:
        raise NotImplementedError

    @property
    def vocab_size(self) -> int:
        raise NotImplementedError

    @property
    def eod(self) -> int:
        raise NotImplementedError

    @property
    def pad(self) -> int:
        return self.eod

    @property
    def eos(self) -> int:
        return self.eod


class NullTokenizer(_Base):
    name = "NullTokenizer"

    def __init__(self, vocab_size: int):
        self._n = int(vocab_size) + 1
        self._eod = int(vocab_size)

    def tokenize(self, text):
        return [int(x) for x in str(text).split()]

    def detokenize(self, ids):
        return " ".join(str(int(i)) for i in ids)

    @property
    def vocab_size(self):
        return self._n

    @property
    def eod(self):
        return self._eod


class ByteLevelTokenizer(_Base):
    name = "ByteLevelTokenizer"
    BOS, EOS, PAD = 256, 257, 258

    def tokenize(self, text):
        return list(text.encode("utf-8"))

    def detokenize(self, ids):
        return bytes(int(i) for i in ids if int(i) < 256).decode("utf-8", errors="replace")

    @property
    def vocab_size(self):
        return 259

    @property
    def eod(self):
        return self.EOS

    @property
    def pad(self):
        return self.PAD

    @property
    def bos(self):
        return self.BOS


class PretrainedFromHF(_Base):
    name = "PretrainedFromHF"

    def __init__(self, name_or_path: str, vocab_extra_ids: int = 0, model_max_length: Optional[int] = None, use_fast: bool = True,
                 trust_remote_code: bool = False):
        import transformers
        kw = {}
        if model_max_length:
            kw["model_max_length"] = model_max_length
        self.tokenizer = transformers.AutoTokenizer.from_pretrained(name_or_path, use_fast=use_fast, local_files_only=True,
                                                                    trust_remote_code=trust_remote_code, **kw)
        if vocab_extra_ids:
            self.tokenizer.add_special_tokens({"additional_special_tokens": [f"<extra_id_{i}>" for i in range(vocab_extra_ids)]})
        if self.tokenizer.pad_token_id is None:
            if self.tokenizer.eos_token is not None:
                self.tokenizer.pad_token = self.tokenizer.eos_token
            else:
                self.tokenizer.add_special_tokens({"pad_token": "<pad>"})
        self.encoder = self.tokenizer.get_vocab()
        self.decoder = {v: k for k, v in self.encoder.items()}

    def tokenize(self, text):
        return self.tokenizer.encode(text, add_special_tokens=False)

    def detokenize(self, ids):
        return self.tokenizer.decode(list(ids))

    def apply_chat_template(self, messages, **kw):
        return self.tokenizer.apply_chat_template(messages, **kw)

    @property
    def vocab(self):
        return self.encoder

    @property
    def inv_vocab(self):
        return self.decoder

    @property
    def vocab_size(self):
        return len(self.tokenizer)

    @property
    def eod(self):
        t = self.tokenizer
        return t.eos_token_id if t.eos_token_id is not None else t.pad_token_id

    @property
    def pad(self):
        return self.tokenizer.pad_token_id

    @property
    def bos(self):
        return self.tokenizer.bos_token_id

    @property
    def eos(self):
        return self.tokenizer.eos_token_id


class GPT2BPETokenizer(_Base):
    """Byte-level BPE from a ``vocab.json`` (token -> id) and a ``merges.txt`` (one merge per line, highest priority first), the
    file pair GPT-2 style models ship (``--tokenizer-type GPT2BPETokenizer --vocab-file ... --merge-file ...``).  Text is cut
    into words by the GPT-2 pattern, every word's UTF-8 bytes are mapped to printable code points, and adjacent symbols are
    merged in priority order.  The end-of-document token is ``<|endoftext|>``."""
    name = "GPT2BPETokenizer"
    PATTERN = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""

    def __init__(self, vocab_file: str, merge_file: str):
        import json
        import regex
        with open(vocab_file, encoding="utf-8") as f:
            self.encoder = json.load(f)
        self.decoder = {v: k for k, v in self.encoder.items()}
        with open(merge_file, encoding="utf-8") as f:
            lines = [l.rstrip("\n") for l in f if l.strip() and not l.startswith("#version")]
        self.ranks = {tuple(l.split()): i for i, l in enumerate(lines)}
        bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
        cs, n = bs[:], 0
        for b in range(256):                       # bytes without a printable form get code points above 255
            if b not in bs:
                bs.append(b)
                cs.append(256 + n)
                n += 1
        self.byte_enc = {b: chr(c) for b, c in zip(bs, cs)}
        self.byte_dec = {c: b for b, c in self.byte_enc.items()}
        self.pat = regex.compile(self.PATTERN)
        self.cache: Dict[str, List[str]] = {}
        if "<|endoftext|>" not in self.encoder:
            raise ValueError("vocab file has no <|endoftext|> token")

    def _bpe(self, word: str) -> List[str]:
        if word in self.cache:
            return self.cache[word]
        sym = list(word)
        while len(sym) > 1:
            best = min(zip(sym, sym[1:]), key=lambda pr: self.ranks.get(pr, float("inf")))
            if best not in self.ranks:
                break
            out, i = [], 0                         # merge every occurrence of the best-ranked pair, left to right
            while i < len(sym):
                if i + 1 < len(sym) and (sym[i], sym[i + 1]) == best:
                    out.append(sym[i] + sym[i + 1])
                    i += 2
                else:
                    out.append(sym[i])
                    i += 1
            sym = out
        self.cache[word] = sym
        return sym

    def tokenize(self, text):
        ids = []
        for w in self.pat.findall(text):
            mapped = "".join(self.byte_enc[b] for b in w.encode("utf-8"))
            ids.extend(self.encoder[t] for t in self._bpe(mapped))
        return ids

    def detokenize(self, ids):
        text = "".join(self.decoder[int(i)] for i in ids)
        return bytearray(self.byte_dec[c] for c in text).decode("utf-8", errors="replace")

    @property
    def vocab_size(self):
        return len(self.encoder)

    @property
    def eod(self):
        return self.encoder["<|endoftext|>"]


def build_tokenizer(args):
    """Build from ``--tokenizer-type`` and set ``args.padded_vocab_size`` when it is not fixed yet."""
    kind = getattr(args, "tokenizer_type", "NullTokenizer")
    if kind == "PretrainedFromHF":
        path = getattr(args, "tokenizer_name_or_path", None) or getattr(args, "tokenizer_model", None)
        if not path:
            raise ValueError("--tokenizer-name-or-path is required for PretrainedFromHF")
        tok = PretrainedFromHF(path, getattr(args, "vocab_extra_ids", 0), getattr(args, "seq_length", None),
                               not getattr(args, "tokenizer_not_use_fast", False))
    elif kind == "GPT2BPETokenizer":
        if not getattr(args, "vocab_file", None) or not getattr(args, "merge_file", None):
            raise ValueError("GPT2BPETokenizer needs --vocab-file and --merge-file")
        tok = GPT2BPETokenizer(args.vocab_file, args.merge_file)
    elif kind == "ByteLevelTokenizer":
        tok = ByteLevelTokenizer()
    elif kind == "NullTokenizer":
        tok = NullTokenizer(getattr(args, "vocab_size", None) or 32000)
    else:
        raise ValueError(f"unknown tokenizer type {kind}")
    if getattr(args, "padded_vocab_size", None) in (None, 0):
        args.padded_vocab_size = _pad_vocab(tok.vocab_size, getattr(args, "make_vocab_size_divisible_by", 128),
                                            getattr(args, "tensor_model_parallel_size", 1))
    return tok
