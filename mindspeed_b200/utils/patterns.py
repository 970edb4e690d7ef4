"""Module-name patterns used by the parallel plans: ``*`` matches within one dotted segment, ``**`` across segments."""
from __future__ import annotations

import functools
import re


@functools.lru_cache(maxsize=512)
def _compile(pattern: str):
    out, i = [], 0
    while i < len(pattern):
        if pattern.startswith("**", i):
            out.append(".*")
            i += 2
        elif pattern[i] == "*":
            out.append("[^.]*")
            i += 1
        elif pattern[i] == "?":
            out.append("[^.]")
            i += 1
        else:
            out.append(re.escape(pattern[i]))
            i += 1
    return re.compile("".join(out) + r"\Z")


def match(name: str, pattern: str) -> bool:
    return _compile(pattern).match(name) is not None
