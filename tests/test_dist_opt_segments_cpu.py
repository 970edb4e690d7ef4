"""Segments of the distributed optimizer: every data-parallel rank must be able to compute every rank's segment list, so
the fused peer-memory step can issue the same number of (handshaking) launches per bucket on all ranks."""
import types

import torch

from mindspeed_b200.optimizer.distrib_optimizer import build_segments


def _bucket(shapes, dp):
    params, ranges, off = [], {}, 0
    for shp in shapes:
        p = torch.nn.Parameter(torch.zeros(shp))
        start = (off + 63) // 64 * 64
        ranges[id(p)] = (start, start + p.numel())
        off = start + p.numel()
        params.append(p)
    numel = (off + dp * 64 - 1) // (dp * 64) * (dp * 64)
    return types.SimpleNamespace(params=params, param_ranges=ranges, start=0, end=numel, numel=numel)


def _cond(name, p):
    return (0.0 if p.dim() == 1 else 1.0), 1.0, True


def test_segment_counts_differ_per_rank_and_padding_equalises_them():
    # a transformer-ish bucket: matrices (weight decay) interleaved with norm vectors / biases (none), odd sizes included
    shapes = [(96, 64), (64,), (64, 96), (37,), (3, 5), (128, 64), (64,), (64,), (200, 3), (7,)] * 3
    for dp in (2, 4, 8):
        b = _bucket(shapes, dp)
        per = b.numel // dp
        lists = [build_segments(b, {}, r * per, (r + 1) * per, _cond) for r in range(dp)]
        counts = [len(l) for l in lists]
        assert len(set(counts)) > 1 or dp == 2            # the raw counts are rank dependent ...
        target = max(counts)                              # ... every rank can compute the maximum and pad to it
        for r, segs in enumerate(lists):
            assert len(segs) + (target - len(segs)) == target
            prev_end = 0
            for sg in segs:
                assert sg.start % 4 == 0 and sg.end % 4 == 0 and 0 <= sg.start < sg.end <= per
                assert sg.start >= prev_end               # disjoint, ascending
                prev_end = sg.end
        # every parameter element is covered by exactly one segment of exactly one rank, with its own hyper-parameters
        for p in b.params:
            s, e = b.param_ranges[id(p)]
            wd = 0.0 if p.dim() == 1 else 1.0
            for pos in (s, (s + e) // 2, e - 1):
                r = pos // per
                hit = [sg for sg in lists[r] if sg.start <= pos - r * per < sg.end]
                assert len(hit) == 1 and hit[0].wd_mult == wd


def test_merges_neighbours_with_equal_hyper_parameters():
    b = _bucket([(64, 64), (64, 64), (64,), (64,), (64, 64)], 1)
    segs = build_segments(b, {}, 0, b.numel, _cond)
    assert [(s.wd_mult) for s in segs] == [1.0, 0.0, 1.0]
