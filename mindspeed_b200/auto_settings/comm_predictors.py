"""Per-dimension communication time models: a line ``t = w * x + b`` over ``x = traffic / bandwidth``.

For every parallel dimension (tp, cp, dp, ep, pp and the fused tp kernels, "mc2" in the reference) the time of one
collective is modelled as a fixed cost ``b`` plus ``w`` times the ideal transfer time.  Without measurements the line is the
hardware description itself (w = 1, b = latency).  When profiled samples exist (``profiling_parse`` gives communication
time per class for a known configuration, hence known traffic) the line is fitted to them by least squares, separately for
total and for exposed (non-overlapped) time, so the model learns both the achieved bandwidth fraction and how much of the
communication a schedule hides.
reference: mindspeed/auto_settings/module/communication/{tp,cp,dp,ep,pp,mc2}_comm_perf_predictor.py (linear model per
dimension fitted on parsed profiles, tp_comm_perf_predictor.py:43-57) and communication_profile.py.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Tuple

from .hardware import Hardware

DIMS = ("tp", "mc2", "cp", "ep", "pp", "dp")


@dataclass
class LinearModel:
    w: float = 1.0
    b: float = 0.0
    samples: List[Tuple[float, float]] = field(default_factory=list)

    def add(self, x: float, t: float):
        self.samples.append((float(x), float(t)))

    def fit(self):
        n = len(self.samples)
        if n == 0:
            return self
        if n == 1:
            x, t = self.samples[0]
            self.w = max((t - self.b) / x, 0.0) if x > 0 else self.w      # one point: keep the latency, learn the slope
            return self
        sx = sum(x for x, _ in self.samples); st = sum(t for _, t in self.samples)
        sxx = sum(x * x for x, _ in self.samples); sxt = sum(x * t for x, t in self.samples)
        den = n * sxx - sx * sx
        if abs(den) < 1e-30:
            self.w = st / sx if sx > 0 else self.w
            return self
        self.w = (n * sxt - sx * st) / den
        self.b = (st - self.w * sx) / n
        if self.b < 0:                           # a negative fixed cost is noise: refit through the origin
            self.b, self.w = 0.0, sxt / sxx
        return self

    def predict(self, x: float) -> float:
        return max(0.0, self.w * x + self.b)


class CommPredictors:
    """One (total, exposed) pair of lines per dimension; ``x`` is seconds of ideal transfer, results are seconds."""

    def __init__(self, hw: Hardware):
        self.hw = hw
        lat = {"tp": hw.collective_latency_us, "mc2": hw.collective_latency_us, "cp": hw.p2p_latency_us, "ep": hw.collective_latency_us,
               "pp": hw.p2p_latency_us, "dp": hw.collective_latency_us}
        self.total: Dict[str, LinearModel] = {d: LinearModel(1.0, lat[d] * 1e-6) for d in DIMS}
        # default exposure: pipeline and tensor-parallel collectives sit on the critical path, the fused kernels hide all but
        # fill / drain, ring steps and the data-parallel reduction are mostly overlapped
        expo = {"tp": 1.0, "mc2": 0.15, "cp": 0.2, "ep": 1.0, "pp": 1.0, "dp": 0.3}
        self.exposed: Dict[str, LinearModel] = {d: LinearModel(expo[d], lat[d] * 1e-6 * expo[d]) for d in DIMS}

    def bandwidth(self, dim: str, span: int) -> float:
        """Bytes per second available to one GPU for a collective of ``dim`` spanning ``span`` ranks."""
        hw = self.hw
        if span > hw.gpus_per_node:
            return hw.internode_gbs * 1e9
        return (hw.allreduce_bus_gbs if dim == "dp" else hw.nvlink_gbs) * 1e9

    def x(self, dim: str, nbytes: float, span: int) -> float:
        return nbytes / self.bandwidth(dim, span)

    def add_sample(self, dim: str, nbytes: float, span: int, total_s: float, exposed_s: float = None):
        x = self.x(dim, nbytes, span)
        self.total[dim].add(x, total_s)
        if exposed_s is not None:
            self.exposed[dim].add(x, exposed_s)

    def fit(self):
        for d in DIMS:
            self.total[d].fit()
            self.exposed[d].fit()
        return self

    def time(self, dim: str, nbytes: float, span: int, exposed: bool = False) -> float:
        if nbytes <= 0 or span <= 1:
            return 0.0
        m = (self.exposed if exposed else self.total)[dim]
        return m.predict(self.x(dim, nbytes, span))
