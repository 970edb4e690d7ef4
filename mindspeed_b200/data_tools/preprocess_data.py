"""``python -m mindspeed_b200.data_tools.preprocess_data --input data.jsonl --output-prefix out/corpus
       --tokenizer-type PretrainedFromHF --tokenizer-name-or-path DIR --handler-name AlpacaHandler``
Tokenises a JSON / JSON-lines / CSV / text / Parquet file (or a directory of them) with the chosen handler and writes indexed datasets next to ``--output-prefix``.
reference: mindspeed/tools/preprocess_data.py:172."""
from __future__ import annotations

import argparse
import json
import sys

from ..tokenizer import build_tokenizer
from .data_handler import get_handler


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", required=True)
    ap.add_argument("--output-prefix", required=True)
    ap.add_argument("--handler-name", default="GeneralPretrainHandler")
    ap.add_argument("--tokenizer-type", default="ByteLevelTokenizer")
    ap.add_argument("--tokenizer-name-or-path", default=None)
    ap.add_argument("--vocab-size", type=int, default=None)
    ap.add_argument("--seq-length", type=int, default=None)
    ap.add_argument("--no-append-eod", action="store_true")
    ap.add_argument("--json-key", "--json-keys", dest="json_key", default="text", help="text field(s), comma separated")
    ap.add_argument("--split-sentences", action="store_true", help="pretrain handlers: one stored item per sentence")
    ap.add_argument("--pad-to-multiple-of", type=int, default=1,
                    help="pretrain handlers: pad every document to a multiple of this many tokens")
    ap.add_argument("--train-on-inputs", action="store_true", help="instruction handlers: loss on the prompt tokens too")
    ap.add_argument("--append-eod", action="store_true", help="accepted for script compatibility: the end-of-document token is "
                    "appended unless --no-append-eod is given")
    ap.add_argument("--keep-newlines", action="store_true", help="--split-sentences: sentences keep their line breaks")
    ap.add_argument("--vocab-file", default=None, help="GPT2BPETokenizer: vocab.json")
    ap.add_argument("--merge-file", default=None, help="GPT2BPETokenizer: merges.txt")
    ap.add_argument("--tokenizer-not-use-fast", action="store_true")
    ap.add_argument("--make-vocab-size-divisible-by", type=int, default=128)
    ap.add_argument("--pad-vocab-size-to", type=int, default=None)
    ap.add_argument("--workers", type=int, default=1, help="accepted; records are tokenised in this process")
    ap.add_argument("--log-interval", type=int, default=100)
    ap.add_argument("--dataset-impl", default="mmap", choices=["mmap", "lazy", "cached"], help="accepted; the files are memory-mapped")
    a = ap.parse_args(argv)
    a.padded_vocab_size = 1          # not needed here; stops build_tokenizer from touching parallel sizes
    tok = build_tokenizer(a)
    kw = dict(seq_length=a.seq_length, append_eod=not a.no_append_eod)
    from .data_handler import HANDLERS, GeneralInstructionHandler, GeneralPretrainHandler
    cls = HANDLERS.get(a.handler_name)
    if cls is not None and issubclass(cls, GeneralPretrainHandler):
        kw.update(split_sentences=a.split_sentences, pad_to_multiple_of=a.pad_to_multiple_of, keep_newlines=a.keep_newlines)
        if cls is GeneralPretrainHandler:
            kw["text_key"] = a.json_key
    if cls is not None and issubclass(cls, GeneralInstructionHandler):
        kw["train_on_inputs"] = a.train_on_inputs
    h = get_handler(a.handler_name, tok, **kw)
    stats = h.serialize_to_disk(h.records(a.input), a.output_prefix)
    print(json.dumps(stats))
    return 0


if __name__ == "__main__":
    sys.exit(main())
