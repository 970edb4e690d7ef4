"""GPT pre-training samples from indexed token datasets (``--data-path``).

An indexed dataset is a ``.bin`` of token ids plus an ``.idx`` of sequence lengths / offsets / document boundaries
(``data_tools/indexed_dataset.py`` reads this package's own format and Megatron's ``MMIDIDX`` format).  A sample is
``seq_length + 1`` consecutive tokens of the stream obtained by concatenating the split's documents in a per-epoch shuffled
order, so no token is padded and documents are packed across sample boundaries; samples of an epoch are visited in a second
shuffled order.  Everything is a pure function of (seed, epoch, index): any rank can build any sample without shared index
files, and resuming at a consumed-sample count needs no state.

``--split a,b,c`` divides the documents (in file order) into train / validation / test ranges.  Several datasets are
blended by weight (``--data-path w1 prefix1 w2 prefix2 ...``): global sample i goes to the dataset whose achieved share
lags its weight the most, so every prefix of the sample sequence respects the weights.
``--reset-position-ids`` / ``--reset-attention-mask`` / ``--eod-mask-loss`` act on the end-of-document token as in
Megatron's ``_get_ltor_masks_and_position_ids`` (reference data path: mindspeed/tools/preprocess_data.py:172 builds the files;
Megatron's GPTDataset consumes them).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..data_tools.indexed_dataset import MMapIndexedDataset


def parse_split(split: str) -> Tuple[float, float, float]:
    parts = [float(x) for x in str(split).replace("/", ",").split(",") if x != ""]
    parts = (parts + [0.0, 0.0, 0.0])[:3]
    tot = sum(parts)
    if tot <= 0:
        raise ValueError(f"--split {split!r} has no positive entry")
    return tuple(p / tot for p in parts)


def split_documents(n_docs: int, split: str) -> List[Tuple[int, int]]:
    """[(first, last+1)] document ranges of train / validation / test."""
    fr = parse_split(split)
    bounds = [0]
    for f in fr:
        bounds.append(bounds[-1] + int(round(f * n_docs)))
    bounds[-1] = n_docs
    for i in range(1, 4):
        bounds[i] = min(max(bounds[i], bounds[i - 1]), n_docs)
    return [(bounds[i], bounds[i + 1]) for i in range(3)]


class GPTDataset(torch.utils.data.Dataset):
    def __init__(self, indexed: MMapIndexedDataset, doc_range: Tuple[int, int], seq_length: int, seed: int = 1234,
                 eod_token: Optional[int] = None, reset_position_ids: bool = False, reset_attention_mask: bool = False,
                 eod_mask_loss: bool = False, num_samples: Optional[int] = None):
        self.ix, self.seq, self.seed = indexed, int(seq_length), int(seed)
        self.eod, self.reset_pos, self.reset_mask, self.eod_mask_loss = eod_token, reset_position_ids, reset_attention_mask, eod_mask_loss
        d0, d1 = doc_range
        # a document = the sequences [doc_idx[d], doc_idx[d+1]); token count per document
        di = np.asarray(indexed.doc_idx, dtype=np.int64)
        lens = np.asarray(indexed.lengths, dtype=np.int64)
        csum = np.concatenate([[0], np.cumsum(lens)])
        self.doc_first_seq = di[d0:d1]
        self.doc_tokens = csum[di[d0 + 1:d1 + 1]] - csum[di[d0:d1]]
        self.doc_token_start = csum[di[d0:d1]]                    # position of the document's first token in the .bin stream
        self.tokens_per_epoch = int(self.doc_tokens.sum())
        if self.tokens_per_epoch <= self.seq:
            raise ValueError(f"split holds {self.tokens_per_epoch} tokens, fewer than one sample of {self.seq + 1}")
        self.samples_per_epoch = (self.tokens_per_epoch - 1) // self.seq
        self.num_samples = int(num_samples) if num_samples is not None else self.samples_per_epoch
        self._epoch_cache: Dict[int, Tuple[np.ndarray, np.ndarray, np.ndarray]] = {}
        self._flat = np.frombuffer(indexed._bin, dtype=indexed.dtype)

    def __len__(self):
        return self.num_samples

    def _epoch(self, e: int):
        c = self._epoch_cache.get(e)
        if c is None:
            rs = np.random.RandomState((self.seed + 7919 * e) % (2 ** 31))
            order = rs.permutation(len(self.doc_tokens))
            cum = np.concatenate([[0], np.cumsum(self.doc_tokens[order])])
            shuffle = np.random.RandomState((self.seed + 104729 * (e + 1)) % (2 ** 31)).permutation(self.samples_per_epoch)
            if len(self._epoch_cache) > 2:
                self._epoch_cache.pop(next(iter(self._epoch_cache)))
            c = self._epoch_cache[e] = (order, cum, shuffle)
        return c

    def tokens_of(self, idx: int) -> np.ndarray:
        e, i = divmod(int(idx), self.samples_per_epoch)
        order, cum, shuffle = self._epoch(e)
        start = int(shuffle[i]) * self.seq
        need = self.seq + 1
        out = np.empty(need, dtype=np.int64)
        d = int(np.searchsorted(cum, start, side="right")) - 1
        got = 0
        while got < need:
            doc = int(order[d])
            off = start + got - int(cum[d])
            take = min(need - got, int(self.doc_tokens[doc]) - off)
            s = int(self.doc_token_start[doc]) + off
            out[got:got + take] = self._flat[s:s + take]
            got += take
            d += 1
        return out

    def __getitem__(self, idx):
        text = torch.from_numpy(self.tokens_of(idx))
        tokens, labels = text[:-1].contiguous(), text[1:].contiguous()
        loss_mask = torch.ones(self.seq)
        position_ids = torch.arange(self.seq)
        item = {"tokens": tokens, "labels": labels, "loss_mask": loss_mask, "position_ids": position_ids}
        if self.eod is not None:
            is_eod = tokens == self.eod
            if self.eod_mask_loss:
                loss_mask[is_eod] = 0.0
            if self.reset_pos or self.reset_mask:
                # a new document starts after every end-of-document token
                doc_id = torch.cumsum(is_eod.long(), 0) - is_eod.long()
                if self.reset_pos:
                    first = torch.zeros(self.seq, dtype=torch.long)
                    starts = torch.nonzero(is_eod).flatten() + 1
                    starts = starts[starts < self.seq]
                    first[starts] = starts
                    first = torch.cummax(first, 0).values
                    item["position_ids"] = position_ids - first
                if self.reset_mask:
                    item["document_ids"] = doc_id
        return item


class BlendedDataset(torch.utils.data.Dataset):
    """Weighted mixture: sample i is drawn from the dataset whose count lags ``weight * (i + 1)`` the most."""

    def __init__(self, datasets: Sequence[GPTDataset], weights: Sequence[float], num_samples: int):
        w = np.asarray(weights, dtype=np.float64)
        self.datasets, self.weights, self.num_samples = list(datasets), w / w.sum(), int(num_samples)
        which = np.empty(self.num_samples, dtype=np.int16)
        local = np.empty(self.num_samples, dtype=np.int64)
        counts = np.zeros(len(w), dtype=np.int64)
        for i in range(self.num_samples):
            k = int(np.argmax(self.weights * (i + 1) - counts))
            which[i], local[i] = k, counts[k]
            counts[k] += 1
        self.which, self.local = which, local

    def __len__(self):
        return self.num_samples

    def __getitem__(self, idx):
        idx = int(idx) % self.num_samples
        return self.datasets[int(self.which[idx])][int(self.local[idx])]


def parse_data_path(data_path: Sequence[str]) -> Tuple[List[float], List[str]]:
    """["prefix"] or ["w1", "prefix1", "w2", "prefix2", ...] -> (weights, prefixes)."""
    items = list(data_path)
    if len(items) == 1:
        return [1.0], items
    if len(items) % 2 != 0:
        raise ValueError("--data-path takes one prefix, or weight / prefix pairs")
    return [float(x) for x in items[0::2]], items[1::2]


def build_train_valid_test_datasets(data_path: Sequence[str], split: str, seq_length: int, seed: int,
                                    train_valid_test_num_samples: Sequence[Optional[int]] = (None, None, None), eod_token=None,
                                    reset_position_ids=False, reset_attention_mask=False, eod_mask_loss=False):
    weights, prefixes = parse_data_path(data_path)
    per_split: List[List[Optional[GPTDataset]]] = [[], [], []]
    for prefix in prefixes:
        ix = MMapIndexedDataset(prefix)
        n_docs = len(ix.doc_idx) - 1
        for s, (a, b) in enumerate(split_documents(n_docs, split)):
            if b <= a:
                per_split[s].append(None)
                continue
            try:
                per_split[s].append(GPTDataset(ix, (a, b), seq_length, seed + s, eod_token, reset_position_ids,
                                               reset_attention_mask, eod_mask_loss))
            except ValueError:
                per_split[s].append(None)
    out = []
    for s in range(3):
        ds = [(d, w) for d, w in zip(per_split[s], weights) if d is not None]
        n = train_valid_test_num_samples[s]
        if not ds:
            out.append(None)
        elif len(ds) == 1:
            if n is not None:
                ds[0][0].num_samples = int(n)
            out.append(ds[0][0])
        else:
            total = int(n) if n is not None else sum(d.samples_per_epoch for d, _ in ds)
            for d, _ in ds:
                d.num_samples = 1 << 62             # a member is indexed by the blend, epochs wrap inside it
            out.append(BlendedDataset([d for d, _ in ds], [w for _, w in ds], total))
    return tuple(out)
