"""Synthetic and indexed token datasets.

``SyntheticGPTDataset`` draws token ids i.i.d. uniform from a seeded generator; labels are the ids
shifted by one (the layout the benchmark configs prescribe).  ``get_batch`` slices the batch for this
context-parallel rank.
"""
from __future__ import annotations

import torch

from ..parallel import parallel_state as ps
from ..parallel.context_parallel.batch_utils import get_batch_on_this_cp_rank


class SyntheticGPTDataset(torch.utils.data.Dataset):
    def __init__(self, vocab_size, seq_length, num_samples, seed=1234):
        self.vocab_size, self.seq_length, self.num_samples, self.seed = vocab_size, seq_length, num_samples, seed

    def __len__(self):
        return self.num_samples

    def __getitem__(self, idx):
        g = torch.Generator().manual_seed(self.seed * 1000003 + idx)
        text = torch.randint(0, self.vocab_size, (self.seq_length + 1,), generator=g, dtype=torch.int64)
        return {"tokens": text[:-1], "labels": text[1:], "loss_mask": torch.ones(self.seq_length),
                "position_ids": torch.arange(self.seq_length)}


class BatchIterator:
    """Yields micro-batches for this data-parallel rank in global-sample order."""

    def __init__(self, dataset, micro_batch_size, dp_rank, dp_size, start=0, pin=False, device=None, micro_batch_sizes=None):
        self.ds, self.mbs, self.r, self.n = dataset, micro_batch_size, dp_rank, dp_size
        self.cursor, self.pin, self.device = start, pin, device
        # --optimized-mbs-list: the micro-batches of a step have these sizes, in this order, step after step
        self.sizes, self._k = (list(micro_batch_sizes) if micro_batch_sizes else None), 0

    def __iter__(self):
        return self

    def __next__(self):
        items = []
        mbs = self.mbs
        if self.sizes:
            mbs = self.sizes[self._k % len(self.sizes)]
            self._k += 1
        for i in range(mbs):
            idx = (self.cursor + self.r * mbs + i) % len(self.ds)
            items.append(self.ds[idx])
        self.cursor += mbs * self.n
        batch = {k: torch.stack([it[k] for it in items]) for k in items[0]}
        if self.pin and torch.cuda.is_available():
            batch = {k: v.pin_memory() for k, v in batch.items()}
        return batch


def fixed_sub_seq_boundaries(seq_length: int, sub_seq_length: int):
    """[0, L, 2L, ..., seq_length]: sub-sequences of L tokens, the last one taking what is left
    (reference: mindspeed/core/transformer/flash_attention/reset_attention_mask/utils.py:206-211)."""
    return list(range(0, seq_length, sub_seq_length)) + [seq_length]


def _fixed_sub_seq_boundaries(seq_length):
    """Boundaries set by ``--reset-attention-mask --fix-sub-seq-length L`` (0 < L <= seq_length), else None."""
    try:
        from .global_vars import get_args
        args = get_args()
    except RuntimeError:
        return None
    L = getattr(args, "fix_sub_seq_length", None)
    if not getattr(args, "reset_attention_mask", False) or L is None or not (0 < L <= seq_length):
        return None
    return fixed_sub_seq_boundaries(seq_length, L)


def get_batch(data_iterator, device=None, return_packed=False):
    """tokens, labels, loss_mask, attention_mask(None: causal), position_ids for this cp rank; with ``return_packed`` a sixth
    value: None, or for batches that carry ``document_ids`` (packed documents, --reset-attention-mask) a dict with the
    documents' boundaries ``cu_seqlens`` (host integers) and, when the positions restart per document, ``position_ids``."""
    batch = next(data_iterator)
    packed = None
    doc = batch.pop("document_ids", None) if isinstance(batch, dict) else None
    fixed = _fixed_sub_seq_boundaries(batch["tokens"].shape[1]) if return_packed else None
    if fixed is not None:
        packed = {"cu_seqlens": fixed}                 # the same for every row of the batch
    elif doc is not None:
        if doc.shape[0] != 1:
            raise ValueError("packed documents (--reset-attention-mask) take micro-batch size 1")
        d = doc[0].cpu()
        starts = torch.nonzero(d[1:] != d[:-1]).flatten() + 1
        packed = {"cu_seqlens": [0] + starts.tolist() + [int(d.numel())]}
    if device is not None:
        batch = {k: v.to(device, non_blocking=True) for k, v in batch.items()}
    batch = get_batch_on_this_cp_rank(batch)
    if fixed is not None:
        # positions restart in every sub-sequence (the rotary embedding of a packed layout follows the boundaries)
        pos = torch.arange(fixed[-1], device=batch["position_ids"].device)
        start = torch.zeros_like(pos)
        for a in fixed[1:-1]:
            start[a:] = a
        batch["position_ids"] = (pos - start).unsqueeze(0).expand_as(batch["position_ids"]).contiguous()
        packed["position_ids"] = batch["position_ids"][:1]            # one row: the same for the whole batch
    elif packed is not None and bool((batch["position_ids"][0, 1:] < batch["position_ids"][0, :-1]).any()):
        packed["position_ids"] = batch["position_ids"]
    out = (batch["tokens"], batch["labels"], batch["loss_mask"], None, batch["position_ids"])
    return out + (packed,) if return_packed else out
