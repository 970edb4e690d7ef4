"""Measured operator times, keyed by operator and shape, persisted between searches.

A black-box or mixed search profiles a handful of configurations; what it learns about individual operators (this GEMM
shape takes 0.21 ms, attention at s = 8192 with 4 heads takes 0.14 ms) is worth keeping, because the white-box model can
then price other configurations that contain the same shapes without running them.  Entries live in a SQLite file
(one table: operator, shape signature, dtype, FLOPs, bytes, time, sample count); ``lookup`` returns the exact shape when it
has been seen and otherwise scales the nearest entry of the same operator by the ratio of FLOPs (bytes for bandwidth-bound
operators), which is exact for a fixed efficiency and a good first guess elsewhere.
reference: mindspeed/auto_settings/module/operator/operator_database.py and operator_profile_get.py (profiled operator
shapes in a database that later searches query).
"""
from __future__ import annotations

import sqlite3
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple


@dataclass
class OpRecord:
    op: str
    shape: Tuple[int, ...]
    dtype: str
    flops: float
    bytes: float
    ms: float
    samples: int = 1


class OperatorDB:
    def __init__(self, path: str = ":memory:"):
        self.conn = sqlite3.connect(path)
        self.conn.execute("CREATE TABLE IF NOT EXISTS ops (op TEXT, shape TEXT, dtype TEXT, flops REAL, bytes REAL, ms REAL, "
                          "samples INTEGER, PRIMARY KEY (op, shape, dtype))")
        self.conn.commit()

    @staticmethod
    def _sig(shape: Sequence[int]) -> str:
        return "x".join(str(int(s)) for s in shape)

    def record(self, op: str, shape: Sequence[int], ms: float, flops: float = 0.0, nbytes: float = 0.0, dtype: str = "bf16"):
        """Running mean over repeated measurements of the same (operator, shape, dtype)."""
        sig = self._sig(shape)
        row = self.conn.execute("SELECT ms, samples FROM ops WHERE op=? AND shape=? AND dtype=?", (op, sig, dtype)).fetchone()
        if row:
            n = row[1] + 1
            self.conn.execute("UPDATE ops SET ms=?, samples=? WHERE op=? AND shape=? AND dtype=?",
                              (row[0] + (ms - row[0]) / n, n, op, sig, dtype))
        else:
            self.conn.execute("INSERT INTO ops VALUES (?,?,?,?,?,?,1)", (op, sig, dtype, flops, nbytes, ms))
        self.conn.commit()

    def exact(self, op: str, shape: Sequence[int], dtype: str = "bf16") -> Optional[OpRecord]:
        row = self.conn.execute("SELECT flops, bytes, ms, samples FROM ops WHERE op=? AND shape=? AND dtype=?",
                                (op, self._sig(shape), dtype)).fetchone()
        return OpRecord(op, tuple(shape), dtype, row[0], row[1], row[2], row[3]) if row else None

    def lookup(self, op: str, shape: Sequence[int], flops: float = 0.0, nbytes: float = 0.0, dtype: str = "bf16") -> Optional[float]:
        """Time in ms: the exact entry, else the nearest entry of this operator scaled by work; None when the operator has
        never been measured."""
        hit = self.exact(op, shape, dtype)
        if hit:
            return hit.ms
        key, want = ("flops", flops) if flops > 0 else ("bytes", nbytes)
        if want <= 0:
            return None
        rows = self.conn.execute(f"SELECT {key}, ms FROM ops WHERE op=? AND dtype=? AND {key}>0", (op, dtype)).fetchall()
        if not rows:
            return None
        work, ms = min(rows, key=lambda r: abs(r[0] - want) / want)
        return ms * want / work

    def efficiency(self, op: str, peak_flops: float, dtype: str = "bf16") -> Optional[float]:
        """FLOP-weighted achieved fraction of ``peak_flops`` over every measured shape of the operator."""
        rows = self.conn.execute("SELECT flops, ms FROM ops WHERE op=? AND dtype=? AND flops>0", (op, dtype)).fetchall()
        if not rows:
            return None
        return sum(r[0] for r in rows) / (sum(r[1] for r in rows) * 1e-3) / peak_flops

    def __len__(self):
        return self.conn.execute("SELECT COUNT(*) FROM ops").fetchone()[0]
