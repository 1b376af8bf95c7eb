"""Audio transforms (crates/axonml-audio/src/transforms.rs:18-517): Resample, MelSpectrogram
(STFT via torch.fft instead of the reference's own DFT loop), MFCC, TimeStretch, PitchShift,
AddNoise, NormalizeAudio, TrimSilence."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..data.transforms import Transform


class Resample(Transform):
    def __init__(self, orig_freq: int, new_freq: int): self.orig, self.new = orig_freq, new_freq
    @classmethod
    def new(cls, orig_freq, new_freq): return cls(orig_freq, new_freq)
    def apply(self, x):
        if self.orig == self.new:
            return x
        n = int(round(x.shape[-1] * self.new / self.orig))
        return F.interpolate(x.reshape(1, 1, -1).float(), size=n, mode="linear", align_corners=False).reshape(*x.shape[:-1], n)


def _hz_to_mel(f): return 2595.0 * math.log10(1.0 + f / 700.0)
def _mel_to_hz(m): return 700.0 * (10 ** (m / 2595.0) - 1.0)


def mel_filterbank(n_mels: int, n_fft: int, sample_rate: int, f_min: float = 0.0, f_max: float | None = None):
    f_max = f_max or sample_rate / 2
    pts = torch.linspace(_hz_to_mel(f_min), _hz_to_mel(f_max), n_mels + 2)
    hz = torch.tensor([_mel_to_hz(float(m)) for m in pts])
    bins = torch.floor((n_fft + 1) * hz / sample_rate).long()
    fb = torch.zeros(n_mels, n_fft // 2 + 1)
    for m in range(1, n_mels + 1):
        l, c, r = int(bins[m - 1]), int(bins[m]), int(bins[m + 1])
        for k in range(l, c):
            fb[m - 1, k] = (k - l) / max(c - l, 1)
        for k in range(c, r):
            fb[m - 1, k] = (r - k) / max(r - c, 1)
    return fb


class MelSpectrogram(Transform):
    def __init__(self, sample_rate: int = 16000, n_fft: int = 400, hop_length: int = 160, n_mels: int = 40):
        self.sr, self.n_fft, self.hop, self.n_mels = sample_rate, n_fft, hop_length, n_mels
        self.fb = mel_filterbank(n_mels, n_fft, sample_rate)

    @classmethod
    def new(cls, sample_rate=16000): return cls(sample_rate)
    @classmethod
    def with_params(cls, sample_rate, n_fft, hop_length, n_mels): return cls(sample_rate, n_fft, hop_length, n_mels)

    def apply(self, x):
        x = x.float()
        spec = torch.stft(x, self.n_fft, self.hop, window=torch.hann_window(self.n_fft, device=x.device),
                          return_complex=True, center=True).abs() ** 2
        return self.fb.to(x.device) @ spec


class MFCC(Transform):
    def __init__(self, sample_rate: int = 16000, n_mfcc: int = 13, n_mels: int = 40):
        self.mel, self.n_mfcc = MelSpectrogram(sample_rate, n_mels=n_mels), n_mfcc
        n = n_mels
        k = torch.arange(n_mfcc).unsqueeze(1)
        i = torch.arange(n).unsqueeze(0)
        self.dct = torch.cos(math.pi / n * (i + 0.5) * k) * math.sqrt(2.0 / n)

    @classmethod
    def new(cls, sample_rate=16000, n_mfcc=13): return cls(sample_rate, n_mfcc)
    def apply(self, x): return self.dct.to(x.device) @ torch.log(self.mel(x) + 1e-6)


class TimeStretch(Transform):
    def __init__(self, rate: float): self.rate = rate
    def apply(self, x):
        n = max(1, int(round(x.shape[-1] / self.rate)))
        return F.interpolate(x.reshape(1, 1, -1).float(), size=n, mode="linear", align_corners=False).reshape(*x.shape[:-1], n)


def _phase_vocoder(x: torch.Tensor, stretch: float, n_fft: int) -> torch.Tensor:
    """``x`` made ``stretch`` times longer at the same pitch: short-time spectra re-spaced in time,
    magnitudes interpolated between neighbouring frames, phases advanced by each bin's measured
    instantaneous frequency."""
    hop = n_fft // 4
    win = torch.hann_window(n_fft, dtype=torch.float32)
    spec = torch.stft(x.float(), n_fft, hop, window=win, return_complex=True, pad_mode="constant")           # [bins, frames]
    frames = spec.shape[1]
    steps = torch.arange(0, frames - 1, 1.0 / stretch) if frames > 1 else torch.zeros(1)
    k0 = steps.floor().long().clamp_max(frames - 1)
    k1 = (k0 + 1).clamp_max(frames - 1)
    frac = (steps - k0).unsqueeze(0)
    mag = spec.abs()
    mag_t = mag[:, k0] * (1 - frac) + mag[:, k1] * frac
    omega = (2 * math.pi * hop * torch.arange(spec.shape[0]) / n_fft).unsqueeze(1)          # expected advance per hop
    ang = spec.angle()
    dphi = ang[:, k1] - ang[:, k0] - omega
    dphi = dphi - 2 * math.pi * torch.round(dphi / (2 * math.pi)) + omega
    phase = torch.cat([ang[:, :1], ang[:, :1] + dphi[:, :-1].cumsum(1)], 1)
    out = torch.istft(torch.polar(mag_t, phase), n_fft, hop, window=win, length=int(round(x.shape[-1] * stretch)))
    return out


class PitchShift(Transform):
    """Pitch moved by ``semitones`` at the same length (transforms.rs:300-340): the clip is made
    ``2^(semitones/12)`` times longer at constant pitch by a phase vocoder and then played back at
    that speed (linear resampling to the original length), then scaled to the input's RMS level.
    Clips shorter than 64 samples come back unchanged."""

    def __init__(self, semitones: float): self.semitones = semitones
    @classmethod
    def new(cls, semitones: float): return cls(semitones)

    def apply(self, x):
        rate = 2.0 ** (self.semitones / 12.0)
        n = x.shape[-1]
        if n < 64 or abs(rate - 1.0) < 1e-9:
            return x
        n_fft = 1024 if n >= 4096 else 1 << max(5, (n // 4).bit_length() - 1)
        flat = x.reshape(-1, n)
        out = []
        for row in flat:
            long_ = _phase_vocoder(row, rate, n_fft)
            y = F.interpolate(long_.reshape(1, 1, -1), size=n, mode="linear", align_corners=False).reshape(n)
            gain = row.float().pow(2).mean().sqrt() / y.pow(2).mean().sqrt().clamp_min(1e-12)     # same loudness as the input
            out.append(y * gain)
        return torch.stack(out).reshape(x.shape).to(x.dtype)


class AddNoise(Transform):
    def __init__(self, snr_db: float = 20.0): self.snr_db = snr_db
    def apply(self, x):
        p = x.float().pow(2).mean().clamp_min(1e-12)
        return x + torch.randn_like(x.float()) * torch.sqrt(p / (10 ** (self.snr_db / 10)))


class NormalizeAudio(Transform):
    def __init__(self, peak: float = 1.0): self.peak = peak
    def apply(self, x): return x * (self.peak / x.abs().max().clamp_min(1e-12))


class TrimSilence(Transform):
    def __init__(self, threshold_db: float = -40.0): self.threshold_db, self.thr = threshold_db, 10 ** (threshold_db / 20.0)
    @classmethod
    def new(cls, threshold_db: float): return cls(threshold_db)
    @classmethod
    def default_threshold(cls):
        """-60 dB below the clip's peak."""
        return cls(-60.0)
    def apply(self, x):
        idx = (x.abs() > self.thr * x.abs().max().clamp_min(1e-12)).nonzero()
        if idx.numel() == 0:
            return x
        return x[..., int(idx[:, -1].min()): int(idx[:, -1].max()) + 1]
