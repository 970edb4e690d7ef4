"""Lossless compression of the activations a transformer layer saves for backward (``--compress-activation``).

For the selected layers every tensor that autograd saves during the layer's forward goes through
``torch.autograd.graph.saved_tensors_hooks``: floating-point tensors above a size threshold are replaced by their
compressed form (exponent / mantissa split with block-wise bit packing, ``ops/compress.py``: bit-exact, ~30 % smaller for
bf16) and restored when backward asks for them; parameters, small tensors and integer tensors pass through untouched.
On a GPU the encode runs on a side stream, ordered after the producer, so it overlaps the rest of the layer's forward; the
decode is waited for where backward needs the tensor.

Layer selection follows the reference's flag grammar: ``"0"`` = every layer, otherwise a comma list of 1-based layer
numbers and ``a-b`` ranges (reference: mindspeed/features_manager/compress/compress.py:13-34; hook placement
mindspeed/core/memory/compress/adaptor.py:22-52, compress_activation.py CompressHook).
``--compress-dense level0|level1`` applies the same hooks to the dense MLP only (level0: its input, level1: everything it
saves; reference: mindspeed/features_manager/compress_dense/compress_dense.py:18-28).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..ops import compress as C

MIN_NUMEL = 1 << 16          # smaller tensors are not worth a kernel sequence


def parse_layers(spec, num_layers: int) -> List[int]:
    """"0" -> all layers; "1,3-5" -> [1, 3, 4, 5]; lists pass through."""
    if spec in (None, "", False):
        return []
    if isinstance(spec, (list, tuple)):
        return [int(x) for x in spec]
    if spec is True or str(spec) == "0":
        return list(range(1, num_layers + 1))
    out: List[int] = []
    for elem in str(spec).split(","):
        elem = elem.strip()
        if not elem:
            continue
        if "-" in elem:
            a, b = (int(x) for x in elem.split("-"))
            out.extend(range(a, b + 1))
        else:
            out.append(int(elem))
    bad = [x for x in out if not (1 <= x <= num_layers)]
    if bad:
        raise ValueError(f"--compress-activation names layers {bad} outside 1..{num_layers}")
    return sorted(set(out))


class _Packed:
    __slots__ = ("data", "event", "requires_grad")

    def __init__(self, data, event):
        self.data, self.event = data, event


class CompressSavedActivations:
    """Context manager: saved tensors of the enclosed forward are stored compressed.  ``stats`` accumulates raw and stored
    bytes so the saving can be reported."""

    stats = {"raw": 0, "stored": 0, "tensors": 0}
    _side = {}

    def __init__(self, min_numel: Optional[int] = None, only: Optional[Sequence[int]] = None):
        self.min_numel = MIN_NUMEL if min_numel is None else min_numel
        self.only = set(only) if only is not None else None      # data pointers that may be compressed (None: all)
        self._hooks = None

    @classmethod
    def _stream(cls, device):
        if device.type != "cuda":
            return None
        s = cls._side.get(device)
        if s is None:
            s = cls._side[device] = torch.cuda.Stream(device=device)
        return s

    def _pack(self, t: torch.Tensor):
        if (not t.is_floating_point() or t.dtype not in C._LAYOUT or t.numel() < self.min_numel or isinstance(t, torch.nn.Parameter)
                or not t.is_contiguous() or (self.only is not None and t.data_ptr() not in self.only)):
            return t
        side = self._stream(t.device)
        if side is None:
            comp, ev = C.compress(t), None
        else:
            side.wait_stream(torch.cuda.current_stream())
            t.record_stream(side)
            with torch.cuda.stream(side):
                comp = C.compress(t)
                ev = side.record_event()
        st = CompressSavedActivations.stats
        st["raw"] += t.numel() * t.element_size()
        st["stored"] += comp.nbytes
        st["tensors"] += 1
        return _Packed(comp, ev)

    @staticmethod
    def _unpack(obj):
        if not isinstance(obj, _Packed):
            return obj
        if obj.event is not None:
            torch.cuda.current_stream().wait_event(obj.event)
        return C.decompress(obj.data)

    def __enter__(self):
        self._hooks = torch.autograd.graph.saved_tensors_hooks(self._pack, self._unpack)
        self._hooks.__enter__()
        return self

    def __exit__(self, *exc):
        return self._hooks.__exit__(*exc)


def reset_stats():
    CompressSavedActivations.stats.update(raw=0, stored=0, tensors=0)
