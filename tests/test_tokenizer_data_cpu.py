"""Tokenizers, indexed datasets, data handlers, preprocessing CLI and mask / position utilities."""
import json
import math
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch


def _hf_dir(tmp_path):
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    vocab = {w: i for i, w in enumerate(["<unk>", "<s>", "</s>", "hello", "world", "the", "cat", "sat", "###", "Instruction", ":", "."])}
    t = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    t.pre_tokenizer = pre_tokenizers.Whitespace()
    fast = PreTrainedTokenizerFast(tokenizer_object=t, unk_token="<unk>", bos_token="<s>", eos_token="</s>")
    d = tmp_path / "tok"
    fast.save_pretrained(str(d))
    return str(d)


def test_tokenizers(tmp_path):
    from mindspeed_b200.tokenizer import build_tokenizer
    a = SimpleNamespace(tokenizer_type="PretrainedFromHF", tokenizer_name_or_path=_hf_dir(tmp_path), padded_vocab_size=None,
                        make_vocab_size_divisible_by=8, tensor_model_parallel_size=2, vocab_extra_ids=0, seq_length=64)
    tok = build_tokenizer(a)
    ids = tok.tokenize("hello world the cat")
    assert ids == [3, 4, 5, 6] and tok.detokenize(ids) == "hello world the cat"
    assert tok.eod == 2 and tok.pad == 2 and a.padded_vocab_size % 16 == 0 and a.padded_vocab_size >= tok.vocab_size
    b = SimpleNamespace(tokenizer_type="NullTokenizer", vocab_size=100, padded_vocab_size=None, make_vocab_size_divisible_by=128,
                        tensor_model_parallel_size=1)
    nt = build_tokenizer(b)
    assert nt.tokenize("1 2 3") == [1, 2, 3] and nt.eod == 100 and b.padded_vocab_size == 128
    bt = build_tokenizer(SimpleNamespace(tokenizer_type="ByteLevelTokenizer", padded_vocab_size=1))
    assert bt.detokenize(bt.tokenize("héllo")) == "héllo"
    with pytest.raises(ValueError):
        build_tokenizer(SimpleNamespace(tokenizer_type="Nope"))


def test_indexed_dataset_roundtrip_and_merge(tmp_path):
    from mindspeed_b200.data_tools import IndexedDatasetBuilder, MMapIndexedDataset
    p1, p2 = str(tmp_path / "a"), str(tmp_path / "b")
    b = IndexedDatasetBuilder(p1, np.uint16)
    b.add_item([1, 2, 3]); b.end_document()
    b.add_item([4, 5]); b.add_item([6]); b.end_document()
    b.finalize()
    c = IndexedDatasetBuilder(p2, np.uint16)
    c.add_item([7, 8, 9, 10]); c.end_document()
    c.merge_file(p1)
    c.finalize()
    ds = MMapIndexedDataset(p2)
    assert len(ds) == 4 and [x.tolist() for x in ds[:]] == [[7, 8, 9, 10], [1, 2, 3], [4, 5], [6]]
    assert ds.doc_idx.tolist() == [0, 1, 2, 4] and ds.num_tokens == 10 and ds.get(0, 1, 2).tolist() == [8, 9]


def test_handlers_and_cli(tmp_path):
    from mindspeed_b200.data_tools import MMapIndexedDataset, get_handler
    from mindspeed_b200.data_tools import preprocess_data
    from mindspeed_b200.tokenizer import ByteLevelTokenizer
    tok = ByteLevelTokenizer()
    h = get_handler("AlpacaHandler", tok)
    enc = h.encode({"instruction": "Say hi", "input": "", "output": "hi"})
    n_resp = len("hi") + 1
    assert enc["labels"][-n_resp:] == enc["input_ids"][-n_resp:] and set(enc["labels"][:-n_resp]) == {-100}
    s = get_handler("SharegptHandler", tok).encode({"conversations": [{"from": "human", "value": "q"}, {"from": "gpt", "value": "a"}]})
    assert sum(1 for x in s["labels"] if x != -100) == 2 and len(s["labels"]) == len(s["input_ids"])
    src = tmp_path / "d.jsonl"
    src.write_text("\n".join(json.dumps({"text": t}) for t in ["abc", "", "hello"]))
    assert preprocess_data.main(["--input", str(src), "--output-prefix", str(tmp_path / "out")]) == 0
    ds = MMapIndexedDataset(str(tmp_path / "out_input_ids_document"))
    assert len(ds) == 2 and ds[0].tolist() == list(b"abc") + [tok.eod]


def test_handler_family(tmp_path):
    from mindspeed_b200.data_tools import MMapIndexedDataset, get_handler, preprocess_data
    from mindspeed_b200.data_tools.data_handler import data_files, read_records, split_sentences
    from mindspeed_b200.tokenizer import ByteLevelTokenizer
    tok = ByteLevelTokenizer()
    dec = lambda ids: bytes(i for i in ids if 0 <= i < 256).decode()
    trained = lambda e: dec([t for t, l in zip(e["input_ids"], e["labels"]) if l != -100])

    # pretrain-style handlers: text built from the record, every token trained
    e = get_handler("AlpacaPretrainHandler", tok).encode({"instruction": "Add", "input": "1 2", "output": "3"})
    t = dec(e["input_ids"])
    assert "### Instruction:\nAdd" in t and "### Input:\n1 2" in t and t.endswith("ASSISTANT: 3") and e["input_ids"][-1] == tok.eod
    assert "### Input" not in dec(get_handler("AlpacaPretrainHandler", tok).encode({"instruction": "Hi", "output": "x"})["input_ids"])
    e = get_handler("StackOverflowPythonPretrainHandler", tok).encode({"title": "sort a list", "question_body": "how?", "answer_body": "sorted(x)"})
    assert dec(e["input_ids"]) == "In python, sort a list\n### Question:\nhow?\n### Response:\nsorted(x)\n"
    # several text fields, sentence splitting, padding to a multiple with the id one past the vocabulary
    h = get_handler("GeneralPretrainHandler", tok, text_key="title,body", split_sentences=True, pad_to_multiple_of=8)
    e = h.encode({"title": "One. Two!", "body": "Three? Four"})
    assert [dec(p) for p in e["sentences"]] == ["One.", "Two!", "Three?", "Four"]
    assert len(e["input_ids"]) % 8 == 0 and e["input_ids"][-1] == tok.eod and e["input_ids"][-2] == tok.vocab_size
    assert split_sentences("a b. c d\ne") == ["a b.", "c d", "e"]

    # instruction handlers: loss on the final response only
    g = get_handler("GeneralInstructionHandler", tok)
    e = g.encode({"instruction": "Translate", "input": "chat", "output": "cat"})
    assert dec(e["input_ids"]) == "USER: Translate\nchat\nASSISTANT: cat" and trained(e) == "cat"
    assert trained(get_handler("GeneralInstructionHandler", tok, train_on_inputs=True).encode(
        {"instruction": "a", "output": "b"})) == "USER: a\nASSISTANT: b"
    b = get_handler("BelleMultiTurnInstructionHandler", tok).encode(
        {"instruction": "Human: hi\nAssistant: hello\nHuman: bye\nAssistant:", "output": "see you"})
    assert dec(b["input_ids"]) == "USER: hi\nASSISTANT: hello\nUSER: bye\nASSISTANT: see you" and trained(b) == "see you"
    l = get_handler("LeetcodePythonInstructionHandler", tok).encode(
        {"code_with_problem": "Two sum.\n```python\nx```", "code_only": "def f(): pass", "explanation_only": "hash map"})
    assert dec(l["input_ids"]) == "USER: Two sum.\nASSISTANT: def f(): pass\nhash map" and trained(l) == "def f(): pass\nhash map"

    # MOSS dialogues: one sample per turn with the history as prompt / one sample per dialogue with role marker ids
    rec = {"chat": {"turn_1": {"Human": "<|Human|>: q1<eoh>", "MOSS": "<|MOSS|>: a1<eom>"},
                    "turn_2": {"Human": "<|Human|>: q2<eoh>", "MOSS": "<|MOSS|>: a2<eom>"}}}
    per_turn = get_handler("MOSSInstructionHandler", tok).encode(rec)
    assert [trained(x) for x in per_turn] == ["a1", "a2"]
    assert dec(per_turn[1]["input_ids"]) == "USER: q1\nASSISTANT: a1\nUSER: q2\nASSISTANT: a2"
    m = get_handler("MOSSMultiTurnHandler", tok, user_token=(300,), assistant_token=(301,)).encode(rec)
    assert m["input_ids"] == [300] + list(b"q1") + [301] + list(b"a1") + [300] + list(b"q2") + [301] + list(b"a2") + [tok.eod]
    assert [x for x in m["labels"] if x != -100] == list(b"a1") + list(b"a2") + [tok.eod]

    # input formats: a directory of text files (majority format wins), csv, parquet; the CLI writes one dataset per turn
    d = tmp_path / "corpus"
    d.mkdir()
    (d / "a.txt").write_text("first doc\nsecond doc\n")
    (d / "b.txt").write_text("third doc\n")
    (d / "c.json").write_text(json.dumps([{"text": "ignored"}]))
    assert [os.path.basename(f) for f in data_files(str(d))] == ["a.txt", "b.txt"]
    assert [r["text"] for r in read_records(str(d))] == ["first doc", "second doc", "third doc"]
    (tmp_path / "x.csv").write_text("instruction,output\nsay a,a\nsay b,b\n")
    assert [r["output"] for r in read_records(str(tmp_path / "x.csv"))] == ["a", "b"]
    import pyarrow as pa
    import pyarrow.parquet as pq
    pq.write_table(pa.table({"text": ["p1", "p2"]}), str(tmp_path / "y.parquet"))
    assert [r["text"] for r in read_records(str(tmp_path / "y.parquet"))] == ["p1", "p2"]
    src = tmp_path / "moss.jsonl"
    src.write_text(json.dumps(rec))
    assert preprocess_data.main(["--input", str(src), "--output-prefix", str(tmp_path / "moss"), "--handler-name",
                                 "MOSSInstructionHandler"]) == 0
    ids, lab = MMapIndexedDataset(str(tmp_path / "moss_input_ids_document")), MMapIndexedDataset(str(tmp_path / "moss_labels_document"))
    assert len(ids) == 2 and len(lab) == 2 and len(ids[1]) == len(lab[1]) > len(ids[0])
    assert preprocess_data.main(["--input", str(d), "--output-prefix", str(tmp_path / "sent"), "--split-sentences"]) == 0
    sd = MMapIndexedDataset(str(tmp_path / "sent_input_ids_document"))
    assert len(sd) == 3 and sd.doc_idx.tolist() == [0, 1, 2, 3]


def test_alibi_masks_and_eod_reset():
    from mindspeed_b200.models import attention_masks as AM
    s8 = AM.alibi_slopes(8)
    assert torch.allclose(s8, torch.tensor([2.0 ** -(i + 1) for i in range(8)]))
    assert AM.alibi_slopes(12).shape == (12,)
    b = AM.alibi_bias(8, 4, 4, tp_rank=1, tp_size=2)
    assert b.shape == (4, 4, 4) and b[0, 3, 0] == -3 * s8[4] and b[0, 0, 3] == 0
    m = AM.compressed_causal_mask()
    assert m.shape == (2048, 2048) and not m[5, 5] and m[5, 6] and AM.compressed_causal_mask() is m
    toks = torch.tensor([[5, 6, 0, 7, 8, 9, 0, 4]])
    r = AM.eod_reset(toks, eod_token=0, build_dense_mask=True)
    assert r["position_ids"].tolist() == [[0, 1, 2, 0, 1, 2, 3, 0]]
    assert r["cu_seqlens"].tolist() == [0, 3, 7, 8] and r["max_seqlen"] == 4
    assert r["loss_mask"].tolist() == [[1, 1, 0, 1, 1, 1, 0, 1]]
    dm = r["attention_mask"][0, 0]
    assert not dm[4, 3] and dm[4, 2] and dm[3, 4]          # attends within its document only, causally
