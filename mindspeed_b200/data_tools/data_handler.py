"""Dataset handlers: turn raw records into token sequences and write them as indexed datasets.

  GeneralPretrainHandler               {"text": ...} (any keys)                  -> input_ids (+ eod per document); optional sentence
                                                                                 splitting and padding to a multiple
  AlpacaPretrainHandler                {"instruction", "input", "output"}        -> one chat-formatted text, trained on every token
  StackOverflowPythonPretrainHandler   {"title", "question_body", "answer_body"} -> question / response text
  AlpacaHandler                        {"instruction", "input", "output"}        -> prompt / response, loss on the response only
  GeneralInstructionHandler            configurable keys; with human / assistant prefixes the instruction field is split into turns
  BelleMultiTurnInstructionHandler     "Human:" / "Assistant:" turns inside the instruction field
  LeetcodePythonInstructionHandler     problem statement -> code + explanation
  SharegptHandler                      {"conversations": [{"from", "value"}, ...]} -> multi-turn, loss on assistant turns
  MOSSInstructionHandler               {"chat": {"turn_1": {"Human", "MOSS"}, ...}} -> one sample PER TURN (history as prompt)
  MOSSMultiTurnHandler                 the same records -> one sample per dialogue, role marker ids between turns
Each instruction handler writes three aligned datasets: ``input_ids``, ``attention_mask``, ``labels`` (-100 on prompt).
Records are read from JSON, JSON-lines, CSV, plain text (one document per line) or Parquet files, or a directory of them.
reference: mindspeed/tools/data_handler.py:70-554 (handler family and file formats), mindspeed/tools/preprocess_data.py:172 (driver).
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
        yield from read_records(path)

    def serialize_to_disk(self, records: Iterable[Dict], output_prefix: str) -> Dict[str, int]:
        builders = {}
        for k in self.keys:
            dt = np.int32 if k == "labels" else best_dtype(self.tok.vocab_size)
            builders[k] = IndexedDatasetBuilder(f"{output_prefix}_{k}_document", dt)
        n_docs = n_tok = skipped = 0
        for rec in records:
            enc = self.encode(rec)
            encs = enc if isinstance(enc, list) else [enc]           # some handlers give several samples per record
            encs = [e for e in encs if e is not None and e["input_ids"]]
            if not encs:
                skipped += 1
                continue
            for e in encs:
                parts = e.get("sentences")                            # sentence-split documents: one item per sentence
                if parts:
                    for part in parts:
                        builders["input_ids"].add_item(part)
                    builders["input_ids"].end_document()
                else:
                    for k in self.keys:
                        builders[k].add_item(e[k])
                        builders[k].end_document()
                n_docs += 1
                n_tok += len(e["input_ids"])
        for b in builders.values():
            b.finalize()
        return {"documents": n_docs, "tokens": n_tok, "skipped": skipped}

    def _clip(self, enc):
        if self.seq_length:
            return {k: v[:self.seq_length] for k, v in enc.items()}
        return enc


class GeneralPretrainHandler(BaseHandler):
    """``text_key`` may name several fields (comma separated); they are joined by a newline.  ``split_sentences`` stores one
    item per sentence (a document is then a run of items); ``pad_to_multiple_of`` pads each document with the id
    ``vocab_size`` (one past the vocabulary, dropped from the loss by the training data path) so that its length, end-of-
    document token included, is a multiple - the layout context parallelism wants for packed documents."""

    def __init__(self, tokenizer, text_key: str = "text", split_sentences: bool = False, pad_to_multiple_of: int = 1,
                 keep_newlines: bool = False, **kw):
        super().__init__(tokenizer, **kw)
        self.text_keys = [k for k in str(text_key).split(",") if k]
        self.split_sentences, self.pad, self.keep_newlines = split_sentences, max(1, int(pad_to_multiple_of)), keep_newlines

    def text(self, record) -> Optional[str]:
        parts = [record.get(k) for k in self.text_keys]
        parts = [p for p in parts if p]
        return "\n".join(parts) if parts else None

    def encode(self, record):
        text = self.text(record)
        if not text:
            return None
        sentences = split_sentences(text, self.keep_newlines) if self.split_sentences else [text]
        parts = [list(self.tok.tokenize(s)) for s in sentences if s]
        parts = [p for p in parts if p]
        if not parts:
            return None
        if self.pad > 1:
            n = sum(len(p) for p in parts) + (1 if self.append_eod else 0)
            parts[-1] += [self.tok.vocab_size] * (-n % self.pad)
        if self.append_eod:
            parts[-1].append(self.tok.eod)
        ids = [t for p in parts for t in p]
        out = {"input_ids": ids}
        if self.split_sentences:
            out["sentences"] = parts
        return out


class AlpacaPretrainHandler(GeneralPretrainHandler):
    """Instruction records flattened into one chat-style text each; every token is trained on."""
    FORMAT = ("A chat between a curious user and an artificial intelligence assistant. The assistant gives helpful, detailed, and "
              "polite answers to the user's questions. USER: Below is an instruction that describes a task. Write a response that "
              "appropriately completes the request.\n\n### Instruction:\n{instruction}\n\n{inputs}### Response: ASSISTANT: {response}")

    def text(self, record):
        if not record.get("instruction") or record.get("output") is None:
            return None
        inputs = f"### Input:\n{record['input']}\n\n" if record.get("input") else ""
        return self.FORMAT.format(instruction=record["instruction"], inputs=inputs, response=record["output"])


class StackOverflowPythonPretrainHandler(GeneralPretrainHandler):
    def text(self, record):
        if not record.get("title") or not record.get("answer_body"):
            return None
        return (f"In python, {record['title']}\n### Question:\n{record.get('question_body', '')}\n"
                f"### Response:\n{record['answer_body']}\n")


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


class GeneralInstructionHandler(_InstructionHandler):
    """Instruction / input / output records under configurable field names.  With ``human_prefix`` and ``assistant_prefix`` the
    instruction field holds earlier turns ("Human: .. Assistant: .. Human: ..") which become prompt turns; the output field is
    the final response.  ``train_on_inputs`` puts the loss on the prompt tokens too."""
    instruction_key, input_key, output_key = "instruction", "input", "output"
    human_prefix: Optional[str] = None
    assistant_prefix: Optional[str] = None
    USER, ASSISTANT = "USER: ", "ASSISTANT: "

    def __init__(self, tokenizer, train_on_inputs: bool = False, instruction_key=None, input_key=None, output_key=None, **kw):
        super().__init__(tokenizer, **kw)
        self.train_on_inputs = train_on_inputs
        self.instruction_key = instruction_key or self.instruction_key
        self.input_key, self.output_key = input_key or self.input_key, output_key or self.output_key

    def messages(self, record) -> Optional[List[tuple]]:
        """[(role, text)] with role "user" / "assistant"; the last one is the response that is trained on."""
        ins, out = record.get(self.instruction_key), record.get(self.output_key)
        if not ins or out is None:
            return None
        if not (self.human_prefix and self.assistant_prefix):
            extra = record.get(self.input_key)
            return [("user", ins + ("\n" + extra if extra else "")), ("assistant", out)]
        msgs = []
        for chunk in ins.split(self.human_prefix):
            if not chunk.strip():
                continue
            parts = chunk.split(self.assistant_prefix)
            msgs.append(("user", parts[0].strip()))
            if len(parts) > 1 and parts[1].strip():
                msgs.append(("assistant", parts[1].strip()))
        if msgs and msgs[-1][0] == "assistant":       # the field ends with an open "Assistant:" - the answer is the output field
            msgs.pop()
        msgs.append(("assistant", out.strip()))
        return msgs

    def encode(self, record):
        msgs = self.messages(record)
        if not msgs:
            return None
        turns = []
        for i, (role, text) in enumerate(msgs):
            last = i == len(msgs) - 1
            if role == "user":
                turns.append((self.USER + text + "\n", self.train_on_inputs))
            else:
                turns.append((self.ASSISTANT, self.train_on_inputs))
                turns.append((text, last or self.train_on_inputs))
                if not last:
                    turns.append(("\n", self.train_on_inputs))
        return self._build(turns)


class BelleMultiTurnInstructionHandler(GeneralInstructionHandler):
    human_prefix, assistant_prefix = "Human:", "Assistant:"


class LeetcodePythonInstructionHandler(GeneralInstructionHandler):
    instruction_key, input_key, output_key = "code_with_problem", "code_only", "explanation_only"

    def messages(self, record):
        prob, code, expl = (record.get(k) for k in (self.instruction_key, self.input_key, self.output_key))
        if not prob or code is None or expl is None:
            return None
        return [("user", prob.split("```", 1)[0].strip()), ("assistant", code + "\n" + expl)]


def _moss_turns(record):
    chat = record.get("chat")
    if not isinstance(chat, dict):
        return []
    out = []
    for turn in chat.values():
        if not turn:
            continue
        user = turn.get("Human", "").replace("<eoh>", "").replace("<|Human|>: ", "").strip()
        bot = turn.get("MOSS", "").replace("<|MOSS|>:", "").replace("<eom>", "").strip()
        out.append((user, bot))
    return out


class MOSSInstructionHandler(GeneralInstructionHandler):
    """One training sample per dialogue turn: the history up to the turn is the prompt, the turn's reply the response."""

    def encode(self, record):
        samples, history = [], []
        for user, bot in _moss_turns(record):
            history.append(("user", user))
            history.append(("assistant", bot))
            turns = []
            for i, (role, text) in enumerate(history):
                last = i == len(history) - 1
                if role == "user":
                    turns.append((self.USER + text + "\n", self.train_on_inputs))
                else:
                    turns.append((self.ASSISTANT, self.train_on_inputs))
                    turns.append((text, last or self.train_on_inputs))
                    if not last:
                        turns.append(("\n", self.train_on_inputs))
            samples.append(self._build(turns))
        return samples or None


class MOSSMultiTurnHandler(_InstructionHandler):
    """One sample per dialogue: ``user_token`` ids, the user's text, ``assistant_token`` ids, the reply - for every turn - and a
    closing end-of-document id.  The loss covers the replies (and the closing id) only.  The marker ids default to the two
    reserved role ids of the Baichuan vocabulary and are parameters for any other."""

    def __init__(self, tokenizer, user_token=(195,), assistant_token=(196,), **kw):
        super().__init__(tokenizer, **kw)
        self.user_token, self.assistant_token = list(user_token), list(assistant_token)

    def encode(self, record):
        ids, labels = [], []
        for user, bot in _moss_turns(record):
            u, a = list(self.tok.tokenize(user)), list(self.tok.tokenize(bot))
            ids += self.user_token + u + self.assistant_token + a
            labels += [IGNORE] * (len(self.user_token) + len(u) + len(self.assistant_token)) + a
        if not ids:
            return None
        ids.append(self.tok.eod)
        labels.append(self.tok.eod)
        return self._clip({"input_ids": ids, "attention_mask": [1] * len(ids), "labels": labels})


# ---------------------------------------------------------------------------------------------------------------------
# input files
# ---------------------------------------------------------------------------------------------------------------------
_FORMATS = {".json": "json", ".jsonl": "json", ".csv": "csv", ".txt": "text", ".parquet": "parquet"}


def data_files(path: str) -> List[str]:
    """``path`` itself, or - for a directory - its files of the format that occurs most often (by extension)."""
    import os
    if not os.path.isdir(path):
        return [path]
    by_fmt: Dict[str, List[str]] = {}
    for root, _, files in os.walk(path):
        for f in sorted(files):
            fmt = _FORMATS.get(os.path.splitext(f)[1].lower())
            if fmt:
                by_fmt.setdefault(fmt, []).append(os.path.join(root, f))
    if not by_fmt:
        raise ValueError(f"no .json / .jsonl / .csv / .txt / .parquet files under {path}")
    return sorted(max(by_fmt.values(), key=len))


def read_records(path: str) -> Iterator[Dict]:
    import os
    for f in data_files(path):
        fmt = _FORMATS.get(os.path.splitext(f)[1].lower(), "json")
        if fmt == "json":
            with open(f) as fh:
                head = fh.read(1)
                fh.seek(0)
                if head == "[":
                    yield from json.load(fh)
                else:
                    for line in fh:
                        line = line.strip()
                        if line:
                            yield json.loads(line)
        elif fmt == "text":
            with open(f) as fh:
                for line in fh:
                    if line.strip():
                        yield {"text": line.rstrip("\n")}
        elif fmt == "csv":
            import csv
            with open(f, newline="") as fh:
                yield from csv.DictReader(fh)
        else:
            import pyarrow.parquet as pq
            for batch in pq.ParquetFile(f).iter_batches():
                yield from batch.to_pylist()


def split_sentences(text: str, keep_newlines: bool = False) -> List[str]:
    """Sentence boundaries after ``.``, ``!``, ``?`` (and their CJK forms) followed by white space, and at newlines."""
    import re
    out = []
    for line in (text.splitlines(keepends=keep_newlines) if not keep_newlines else [text]):
        for s in re.split(r"(?<=[.!?\u3002\uff01\uff1f])\s+", line):
            if s.strip():
                out.append(s if keep_newlines else s.strip())
    return out


HANDLERS = {"GeneralPretrainHandler": GeneralPretrainHandler, "AlpacaPretrainHandler": AlpacaPretrainHandler,
            "StackOverflowPythonPretrainHandler": StackOverflowPythonPretrainHandler,
            "AlpacaHandler": AlpacaHandler, "AlpacaStyleInstructionHandler": AlpacaHandler,
            "GeneralInstructionHandler": GeneralInstructionHandler,
            "BelleMultiTurnInstructionHandler": BelleMultiTurnInstructionHandler,
            "LeetcodePythonInstructionHandler": LeetcodePythonInstructionHandler,
            "SharegptHandler": SharegptHandler, "SharegptStyleInstructionHandler": SharegptHandler,
            "MOSSInstructionHandler": MOSSInstructionHandler, "MOSSMultiTurnHandler": MOSSMultiTurnHandler}


def get_handler(name: str, tokenizer, **kw) -> BaseHandler:
    if name not in HANDLERS:
        raise ValueError(f"unknown handler {name}; choose from {sorted(HANDLERS)}")
    return HANDLERS[name](tokenizer, **kw)
