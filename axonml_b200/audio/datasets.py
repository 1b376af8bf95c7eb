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
    def sample_rate(self) -> int: return self.sr

    @classmethod
    def new(cls, num_samples, sample_rate, duration, num_classes):
        """The reference's argument order: size, sample rate, seconds per clip, classes."""
        return cls(num_samples, num_classes, sample_rate, duration)

    def _wave(self, label, g): raise NotImplementedError

    def get(self, i: int):
        if not 0 <= i < self.n:
            raise IndexError(f"index {i} out of range for a dataset of {self.n} samples")
        g = torch.Generator().manual_seed(self.seed + i)
        label = i % self.classes
        return self._wave(label, g), torch.tensor(label, dtype=torch.long)


class SyntheticCommandDataset(_Synthetic):
    def __init__(self, num_samples=1000, num_classes=10, sample_rate=16000, duration=1.0, seed=42):
        super().__init__(num_samples, num_classes, sample_rate, duration, seed)

    # sizes of the reference's presets (datasets.rs:105-119)
    @classmethod
    def small(cls): return cls.new(100, 16000, 0.5, 10)
    @classmethod
    def medium(cls): return cls.new(1000, 16000, 0.5, 10)
    @classmethod
    def large(cls): return cls.new(10000, 16000, 0.5, 35)

    def _wave(self, label, g):
        t = torch.arange(self.len_s) / self.sr
        f = 200.0 + 80.0 * label
        env = torch.exp(-3.0 * t)
        return env * torch.sin(2 * math.pi * f * t) + 0.05 * torch.randn(self.len_s, generator=g)


class SyntheticMusicDataset(_Synthetic):
    def __init__(self, num_samples=500, num_classes=5, sample_rate=22050, duration=1.0, seed=42):
        super().__init__(num_samples, num_classes, sample_rate, duration, seed)

    @classmethod
    def small(cls): return cls.new(100, 22050, 1.0, 5)
    @classmethod
    def medium(cls): return cls.new(500, 22050, 2.0, 10)
    def num_genres(self) -> int: return self.classes

    def _wave(self, label, g):
        t = torch.arange(self.len_s) / self.sr
        base = 110.0 * (1 + label)
        w = sum(torch.sin(2 * math.pi * base * h * t) / h for h in range(1, 3 + label))
        return w / w.abs().max() + 0.02 * torch.randn(self.len_s, generator=g)


class SyntheticSpeakerDataset(_Synthetic):
    def __init__(self, num_samples=500, num_speakers=8, sample_rate=16000, duration=1.0, seed=42):
        super().__init__(num_samples, max(num_speakers, 2), sample_rate, duration, seed)

    @classmethod
    def small(cls): return cls.new(100, 16000, 0.5, 5)
    @classmethod
    def medium(cls): return cls.new(500, 16000, 1.0, 20)
    def num_speakers(self) -> int: return self.classes

    def _wave(self, label, g):
        t = torch.arange(self.len_s) / self.sr
        f1, f2 = 300.0 + 40 * label, 900.0 + 90 * label
        pitch = 100.0 + 10 * label
        src = torch.sign(torch.sin(2 * math.pi * pitch * t))
        return 0.5 * src * (torch.sin(2 * math.pi * f1 * t) + 0.6 * torch.sin(2 * math.pi * f2 * t)) + 0.03 * torch.randn(self.len_s, generator=g)


class AudioClassificationDataset(Dataset):
    """Waveforms with class labels held in memory (datasets.rs:18-75).  ``get`` returns the class
    index; ``one_hot=True`` gives the reference's one-hot float target instead."""

    def __init__(self, waveforms, labels, sample_rate: int, num_classes: int, one_hot: bool = False):
        if len(waveforms) != len(labels):
            raise ValueError(f"{len(waveforms)} waveforms but {len(labels)} labels")
        bad = [l for l in labels if not 0 <= int(l) < num_classes]
        if bad:
            raise ValueError(f"label {bad[0]} is outside 0..{num_classes - 1}")
        self.waveforms = [torch.as_tensor(w, dtype=torch.float32) for w in waveforms]
        self.labels = [int(l) for l in labels]
        self._sr, self._classes, self.one_hot = sample_rate, num_classes, one_hot

    @classmethod
    def new(cls, waveforms, labels, sample_rate, num_classes): return cls(waveforms, labels, sample_rate, num_classes)

    def len(self) -> int: return len(self.waveforms)
    def sample_rate(self) -> int: return self._sr
    def num_classes(self) -> int: return self._classes

    def get(self, i: int):
        if not 0 <= i < self.len():
            return None
        if self.one_hot:
            t = torch.zeros(self._classes)
            t[self.labels[i]] = 1.0
            return self.waveforms[i], t
        return self.waveforms[i], torch.tensor(self.labels[i], dtype=torch.long)


class AudioSeq2SeqDataset(Dataset):
    """Pairs of source and target waveforms (datasets.rs:451-505)."""

    def __init__(self, sources, targets):
        if len(sources) != len(targets):
            raise ValueError(f"{len(sources)} sources but {len(targets)} targets")
        self.sources = [torch.as_tensor(s, dtype=torch.float32) for s in sources]
        self.targets = [torch.as_tensor(t, dtype=torch.float32) for t in targets]

    @classmethod
    def new(cls, sources, targets): return cls(sources, targets)

    @classmethod
    def noise_reduction_task(cls, num_samples: int, sample_rate: int, duration: float):
        """Noisy sine -> clean sine: tone i has frequency 200 + (50 i mod 800) Hz and amplitude 0.5;
        the source adds uniform noise in [-0.2, 0.2) drawn from a generator seeded with i."""
        n = int(sample_rate * duration)
        t = torch.arange(n, dtype=torch.float32) / sample_rate
        sources, targets = [], []
        for i in range(num_samples):
            freq = 200.0 + (i * 50.0) % 800.0
            clean = 0.5 * torch.sin(2 * math.pi * freq * t)
            g = torch.Generator().manual_seed(i)
            sources.append(clean + (torch.rand(n, generator=g) * 0.4 - 0.2))
            targets.append(clean)
        return cls(sources, targets)

    def len(self) -> int: return len(self.sources)

    def get(self, i: int):
        if not 0 <= i < self.len():
            return None
        return self.sources[i], self.targets[i]
