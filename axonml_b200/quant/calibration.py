"""Calibration statistics (crates/axonml-quant/src/calibration.rs:19-230): running min / max /
mean / std and a histogram, ``CalibrationMethod`` {MinMax, Percentile(x10), Entropy, MeanStd(x10)}."""
from __future__ import annotations

import dataclasses
import enum

import torch

from .types import QuantType


class CalibrationMethod(enum.Enum):
    MinMax = "minmax"
    Percentile = "percentile"
    Entropy = "entropy"
    MeanStd = "meanstd"

    def with_arg(self, arg: int):
        """Percentile and MeanStd carry an integer argument scaled by 10 (999 = 99.9 %, 30 = 3 sigma)."""
        return (self, arg)


@dataclasses.dataclass
class CalibrationData:
    min: float
    max: float
    mean: float
    std: float
    histogram: torch.Tensor
    num_bins: int
    count: int

    @classmethod
    def new(cls, tensor: torch.Tensor, num_bins: int = 2048) -> "CalibrationData":
        t = tensor.detach().float().flatten()
        lo, hi = float(t.min()), float(t.max())
        hist = torch.histc(t, bins=num_bins, min=lo, max=hi if hi > lo else lo + 1e-8)
        return cls(lo, hi, float(t.mean()), float(t.std(unbiased=False)), hist, num_bins, t.numel())

    def update(self, tensor: torch.Tensor) -> None:
        t = tensor.detach().float().flatten()
        n2 = t.numel()
        lo, hi = min(self.min, float(t.min())), max(self.max, float(t.max()))
        if lo != self.min or hi != self.max:   # re-bin the old histogram onto the new range
            centers = torch.linspace(self.min, self.max, self.num_bins)
            self.histogram = torch.histc(centers, bins=self.num_bins, min=lo, max=hi) * 0 + \
                torch.zeros(self.num_bins).index_add(0, ((centers - lo) / max(hi - lo, 1e-12) * (self.num_bins - 1)).long(), self.histogram)
        self.histogram = self.histogram + torch.histc(t, bins=self.num_bins, min=lo, max=hi if hi > lo else lo + 1e-8)
        mean = (self.mean * self.count + float(t.sum())) / (self.count + n2)
        var = (self.count * (self.std ** 2 + (self.mean - mean) ** 2) + float(((t - mean) ** 2).sum())) / (self.count + n2)
        self.min, self.max, self.mean, self.std, self.count = lo, hi, mean, var ** 0.5, self.count + n2

    def dynamic_range(self) -> float: return self.max - self.min

    def symmetric_scale(self, quant_type: QuantType) -> float:
        qmax = {8: 127.0, 5: 15.0, 4: 7.0}.get(quant_type.nominal_bits(), 127.0)
        return max(abs(self.min), abs(self.max)) / qmax

    def asymmetric_scale(self, quant_type: QuantType):
        levels = float(2 ** quant_type.nominal_bits() - 1)
        scale = (self.max - self.min) / levels if self.max > self.min else 1.0
        return scale, self.min

    def percentile(self, p: float) -> float:
        c = self.histogram.cumsum(0)
        target = p / 100.0 * float(c[-1])
        idx = int(torch.searchsorted(c, torch.tensor(target)).clamp(max=self.num_bins - 1))
        return self.min + (idx + 0.5) * (self.max - self.min) / self.num_bins


def calibrate(tensor: torch.Tensor, method=CalibrationMethod.MinMax) -> CalibrationData:
    arg = None
    if isinstance(method, tuple):
        method, arg = method
    d = CalibrationData.new(tensor)
    if method is CalibrationMethod.Percentile:
        p = (arg if arg is not None else 999) / 10.0
        hi, lo = d.percentile(p), d.percentile(100.0 - p)
        d.min, d.max = lo, hi
    elif method is CalibrationMethod.MeanStd:
        k = (arg if arg is not None else 30) / 10.0
        d.min, d.max = d.mean - k * d.std, d.mean + k * d.std
    elif method is CalibrationMethod.Entropy:
        # keep the clipping threshold that minimises KL(P || quantised P) over candidate ranges
        t = tensor.detach().float().abs().flatten()
        best, best_kl = float(t.max()), float("inf")
        ref = torch.histc(t, bins=2048, min=0, max=float(t.max()) + 1e-12) + 1e-6
        ref = ref / ref.sum()
        for frac in (1.0, 0.99, 0.97, 0.95, 0.9, 0.8, 0.7):
            thr = float(t.max()) * frac
            q = torch.histc(t.clamp(max=thr), bins=2048, min=0, max=float(t.max()) + 1e-12) + 1e-6
            q = q / q.sum()
            kl = float((ref * (ref / q).log()).sum()) + (1 - frac) * 0.01
            if kl < best_kl:
                best, best_kl = thr, kl
        d.min, d.max = -best, best
    return d


def calibrate_batch(tensors, method=CalibrationMethod.MinMax) -> CalibrationData:
    tensors = list(tensors)
    d = CalibrationData.new(tensors[0])
    for t in tensors[1:]:
        d.update(t)
    if method is not CalibrationMethod.MinMax:
        return calibrate(torch.cat([t.flatten() for t in tensors]), method)
    return d
