"""Dataset handlers: turn raw records into token sequences and write them as indexed datasets.

  GeneralPretrainHandler   {"text": ...}                               -> input_ids (+ eod per document)
  AlpacaHandler            {"instruction", "input", "output"}          -> prompt / response with loss only on the response
  SharegptHandler          {"conversations": [{"from", "value"}, ...]} -> multi-turn, loss on assistant turns
Each instruction handler writes three aligned datasets: ``input_ids``, ``attention_mask``, ``labels`` (-100 on prompt).
reference: mindspeed/tools/data_handler.py:70-505 (handler family), mindspeed/tools/preprocess_data.py:172 (driver).
"""
from __future__ import annotations

import json
from typing import Dict, Iterable, Iterator, List, Optional

import numpy as np

from .indexed_dataset import IndexedDatasetBuilder, best_dtype

IGNORE = -100


class BaseHandler:
    keys = ("input_ids",)

    def __init__(self, tokenizer, seq_length: Optional[int] = None, append_eod: bool = True):
        self.tok, self.seq_length, self.append_eod = tokenizer, seq_length, append_eod

    def encode(self, record: Dict) -> Optional[Dict[str, List[int]]]:
        raise NotImplementedError

    def records(self, path: str) -> Iterator[Dict]:
        with open(path) as f:
            head = f.read(1)
            f.seek(0)
            if head == "[":
                yield from json.load(f)
            else:
                for line in f:
                    line = line.strip()
                    if line:
                        yield json.loads(line)

    def serialize_to_disk(self, records: Iterable[Dict], output_prefix: str) -> Dict[str, int]:
        builders = {}
        for k in self.keys:
            dt = np.int32 if k == "labels" else best_dtype(self.tok.vocab_size)
            builders[k] = IndexedDatasetBuilder(f"{output_prefix}_{k}_document", dt)
        n_docs = n_tok = skipped = 0
        for rec in records:
            enc = self.encode(rec)
            if enc is None or not enc["input_ids"]:
                skipped += 1
                continue
            for k in self.keys:
                builders[k].add_item(enc[k])
                builders[k].end_document()
            n_docs += 1
            n_tok += len(enc["input_ids"])
        for b in builders.values():
            b.finalize()
        return {"documents": n_docs, "tokens": n_tok, "skipped": skipped}

    def _clip(self, enc):
        if self.seq_length:
            return {k: v[:self.seq_length] for k, v in enc.items()}
        return enc


class GeneralPretrainHandler(BaseHandler):
    def __init__(self, tokenizer, text_key: str = "text", **kw):
        super().__init__(tokenizer, **kw)
        self.text_key = text_key

    def encode(self, record):
        text = record.get(self.text_key)
        if not text:
            return None
        ids = list(self.tok.tokenize(text))
        if self.append_eod:
            ids.append(self.tok.eod)
        return {"input_ids": ids}


class _InstructionHandler(BaseHandler):
    keys = ("input_ids", "attention_mask", "labels")

    def _build(self, turns):
        """turns: list of (text, is_response)."""
        ids, labels = [], []
        for text, is_resp in turns:
            t = list(self.tok.tokenize(text))
            if is_resp and self.append_eod:
                t.append(self.tok.eod)
            ids += t
            labels += t if is_resp else [IGNORE] * len(t)
        return self._clip({"input_ids": ids, "attention_mask": [1] * len(ids), "labels": labels})


class AlpacaHandler(_InstructionHandler):
    PROMPT_INPUT = ("Below is an instruction that describes a task, paired with an input that provides further context. "
                    "Write a response that appropriately completes the request.\n\n### Instruction:\n{instruction}\n\n### Input:\n{input}\n\n### Response:\n")
    PROMPT_NO_INPUT = ("Below is an instruction that describes a task. Write a response that appropriately completes the request.\n\n"
                       "### Instruction:\n{instruction}\n\n### Response:\n")

    def encode(self, record):
        if "instruction" not in record or "output" not in record:
            return None
        tpl = self.PROMPT_INPUT if record.get("input") else self.PROMPT_NO_INPUT
        return self._build([(tpl.format(instruction=record["instruction"], input=record.get("input", "")), False),
                            (record["output"], True)])


class SharegptHandler(_InstructionHandler):
    ROLES = {"human": "USER", "user": "USER", "gpt": "ASSISTANT", "assistant": "ASSISTANT", "system": "SYSTEM"}

    def encode(self, record):
        conv = record.get("conversations") or record.get("messages")
        if not conv:
            return None
        turns = []
        for m in conv:
            role = self.ROLES.get((m.get("from") or m.get("role") or "").lower())
            text = m.get("value") if "value" in m else m.get("content", "")
            if role is None:
                continue
            if role == "ASSISTANT":
                turns.append((f"{role}: ", False))
                turns.append((text, True))
                turns.append(("\n", False))
            else:
                turns.append((f"{role}: {text}\n", False))
        if not any(r for _, r in turns):
            return None
        return self._build(turns)


HANDLERS = {"GeneralPretrainHandler": GeneralPretrainHandler, "AlpacaHandler": AlpacaHandler, "AlpacaStyleInstructionHandler": AlpacaHandler,
            "SharegptHandler": SharegptHandler, "SharegptStyleInstructionHandler": SharegptHandler, "MOSSInstructionHandler": SharegptHandler}


def get_handler(name: str, tokenizer, **kw) -> BaseHandler:
    if name not in HANDLERS:
        raise ValueError(f"unknown handler {name}; choose from {sorted(HANDLERS)}")
    return HANDLERS[name](tokenizer, **kw)
