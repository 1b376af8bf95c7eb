"""Synthetic audio datasets (crates/axonml-audio/src/datasets.rs:18-465): command words as tone
patterns, music genres as harmonic stacks, speakers as formant pairs."""
from __future__ import annotations

import math

import torch

from ..data.dataset import Dataset


class _Synthetic(Dataset):
    def __init__(self, num_samples, num_classes, sample_rate, duration, seed):
        self.n, self.classes, self.sr, self.len_s = num_samples, num_classes, sample_rate, int(sample_rate * duration)
        self.seed = seed

    def len(self) -> int: return self.n
    def num_classes(self) -> int: return self.classes
    def _wave(self, label, g): raise NotImplementedError

    def get(self, i: int):
        g = torch.Generator().manual_seed(self.seed + i)
        label = i % self.classes
        return self._wave(label, g), torch.tensor(label, dtype=torch.long)


class SyntheticCommandDataset(_Synthetic):
    def __init__(self, num_samples=1000, num_classes=10, sample_rate=16000, duration=1.0, seed=42):
        super().__init__(num_samples, num_classes, sample_rate, duration, seed)

    def _wave(self, label, g):
        t = torch.arange(self.len_s) / self.sr
        f = 200.0 + 80.0 * label
        env = torch.exp(-3.0 * t)
        return env * torch.sin(2 * math.pi * f * t) + 0.05 * torch.randn(self.len_s, generator=g)


class SyntheticMusicDataset(_Synthetic):
    def __init__(self, num_samples=500, num_classes=5, sample_rate=22050, duration=1.0, seed=42):
        super().__init__(num_samples, num_classes, sample_rate, duration, seed)

    def _wave(self, label, g):
        t = torch.arange(self.len_s) / self.sr
        base = 110.0 * (1 + label)
        w = sum(torch.sin(2 * math.pi * base * h * t) / h for h in range(1, 3 + label))
        return w / w.abs().max() + 0.02 * torch.randn(self.len_s, generator=g)


class SyntheticSpeakerDataset(_Synthetic):
    def __init__(self, num_samples=500, num_speakers=8, sample_rate=16000, duration=1.0, seed=42):
        super().__init__(num_samples, num_speakers, sample_rate, duration, seed)

    def _wave(self, label, g):
        t = torch.arange(self.len_s) / self.sr
        f1, f2 = 300.0 + 40 * label, 900.0 + 90 * label
        pitch = 100.0 + 10 * label
        src = torch.sign(torch.sin(2 * math.pi * pitch * t))
        return 0.5 * src * (torch.sin(2 * math.pi * f1 * t) + 0.6 * torch.sin(2 * math.pi * f2 * t)) + 0.03 * torch.randn(self.len_s, generator=g)
