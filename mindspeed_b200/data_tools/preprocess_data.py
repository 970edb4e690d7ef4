"""``python -m mindspeed_b200.data_tools.preprocess_data --input data.jsonl --output-prefix out/corpus
       --tokenizer-type PretrainedFromHF --tokenizer-name-or-path DIR --handler-name AlpacaHandler``
Tokenises a JSON / JSON-lines file with the chosen handler and writes indexed datasets next to ``--output-prefix``.
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
    ap.add_argument("--json-key", default="text")
    a = ap.parse_args(argv)
    a.padded_vocab_size = 1          # not needed here; stops build_tokenizer from touching parallel sizes
    tok = build_tokenizer(a)
    kw = dict(seq_length=a.seq_length, append_eod=not a.no_append_eod)
    if a.handler_name == "GeneralPretrainHandler":
        kw["text_key"] = a.json_key
    h = get_handler(a.handler_name, tok, **kw)
    stats = h.serialize_to_disk(h.records(a.input), a.output_prefix)
    print(json.dumps(stats))
    return 0


if __name__ == "__main__":
    sys.exit(main())
