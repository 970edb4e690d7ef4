"""Memory-mapped indexed dataset: one ``.bin`` of concatenated token ids and one ``.idx`` with per-sequence lengths,
byte offsets and document boundaries.

.idx layout (little endian):  magic b"MSB200IDX\\0" | u64 version | u8 dtype code | u64 n_sequences | u64 n_documents
                              | i32 lengths[n_sequences] | i64 offsets[n_sequences] | i64 doc_index[n_documents]
Reading maps both files, so a multi-hundred-GB corpus costs no resident memory and every data-parallel rank can open it.
reference: the indexed-dataset builder used by mindspeed/tools/preprocess_data.py:172 (Megatron's MMapIndexedDataset).
"""
from __future__ import annotations

import os
import struct
from typing import List, Sequence

import numpy as np

MAGIC = b"MSB200IDX\x00"
DTYPES = {1: np.uint8, 2: np.uint16, 3: np.int32, 4: np.int64}
CODES = {np.dtype(v): k for k, v in DTYPES.items()}


def best_dtype(vocab_size: int):
    return np.uint16 if vocab_size < 65500 else np.int32


class IndexedDatasetBuilder:
    def __init__(self, prefix: str, dtype=np.int32):
        self.prefix, self.dtype = prefix, np.dtype(dtype)
        os.makedirs(os.path.dirname(os.path.abspath(prefix)) or ".", exist_ok=True)
        self._bin = open(prefix + ".bin", "wb")
        self.lengths: List[int] = []
        self.doc_idx: List[int] = [0]

    def add_item(self, ids: Sequence[int]):
        a = np.asarray(ids, dtype=self.dtype)
        self._bin.write(a.tobytes(order="C"))
        self.lengths.append(int(a.size))

    def end_document(self):
        self.doc_idx.append(len(self.lengths))

    def merge_file(self, other_prefix: str):
        other = MMapIndexedDataset(other_prefix)
        if other.dtype != self.dtype:
            raise ValueError("cannot merge datasets of different dtypes")
        base = len(self.lengths)
        self.lengths.extend(int(x) for x in other.lengths)
        self.doc_idx.extend(base + int(d) for d in other.doc_idx[1:])
        with open(other_prefix + ".bin", "rb") as f:
            while True:
                buf = f.read(1 << 24)
                if not buf:
                    break
                self._bin.write(buf)

    def finalize(self):
        self._bin.close()
        lengths = np.asarray(self.lengths, dtype=np.int32)
        offsets = np.zeros(len(lengths), dtype=np.int64)
        if len(lengths) > 1:
            np.cumsum(lengths[:-1].astype(np.int64) * self.dtype.itemsize, out=offsets[1:])
        with open(self.prefix + ".idx", "wb") as f:
            f.write(MAGIC)
            f.write(struct.pack("<QBQQ", 1, CODES[self.dtype], len(lengths), len(self.doc_idx)))
            f.write(lengths.tobytes())
            f.write(offsets.tobytes())
            f.write(np.asarray(self.doc_idx, dtype=np.int64).tobytes())


# Megatron's index files ("MMIDIDX", version 1) have the same sections in the same order with their own dtype codes; corpora
# tokenised for the reference (mindspeed/tools/preprocess_data.py writes this format) are read as they are.
MEGATRON_MAGIC = b"MMIDIDX\x00\x00"
MEGATRON_DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float64, 7: np.float32, 8: np.uint16}


class MMapIndexedDataset:
    def __init__(self, prefix: str):
        with open(prefix + ".idx", "rb") as f:
            head = f.read(len(MAGIC))
            if head == MAGIC:
                table = DTYPES
            elif head[:len(MEGATRON_MAGIC)] == MEGATRON_MAGIC:
                table = MEGATRON_DTYPES
                f.seek(len(MEGATRON_MAGIC))
            else:
                raise ValueError(f"{prefix}.idx is neither this package's nor Megatron's indexed-dataset format")
            _, code, n, nd = struct.unpack("<QBQQ", f.read(25))
            header = f.tell()
        self.dtype = np.dtype(table[code])
        idx = np.memmap(prefix + ".idx", mode="r", dtype=np.uint8)
        o = header
        self.lengths = np.frombuffer(idx, dtype=np.int32, count=n, offset=o); o += 4 * n
        self.offsets = np.frombuffer(idx, dtype=np.int64, count=n, offset=o); o += 8 * n
        self.doc_idx = np.frombuffer(idx, dtype=np.int64, count=nd, offset=o)
        self._bin = np.memmap(prefix + ".bin", mode="r", dtype=np.uint8) if os.path.getsize(prefix + ".bin") else np.zeros(0, np.uint8)

    def __len__(self):
        return len(self.lengths)

    def __getitem__(self, i):
        if isinstance(i, slice):
            return [self[j] for j in range(*i.indices(len(self)))]
        if i < 0:
            i += len(self)
        return np.frombuffer(self._bin, dtype=self.dtype, count=int(self.lengths[i]), offset=int(self.offsets[i]))

    def get(self, i, offset=0, length=None):
        a = self[i]
        return a[offset:offset + length if length is not None else None]

    @property
    def num_tokens(self):
        return int(self.lengths.astype(np.int64).sum())
