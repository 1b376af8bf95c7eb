"""Tensor transforms (crates/axonml-data/src/transforms.rs:16-550)."""
from __future__ import annotations

import torch


class Transform:
    def apply(self, x): raise NotImplementedError
    def __call__(self, x): return self.apply(x)


class Compose(Transform):
    def __init__(self, transforms): self.transforms = list(transforms)
    @classmethod
    def new(cls, transforms): return cls(transforms)
    @classmethod
    def empty(cls): return cls([])
    def add(self, t): self.transforms.append(t); return self
    def len(self) -> int: return len(self.transforms)
    def is_empty(self) -> bool: return not self.transforms
    def apply(self, x):
        for t in self.transforms:
            x = t(x)
        return x


class ToTensor(Transform):
    def apply(self, x): return torch.as_tensor(x, dtype=torch.float32)


class Normalize(Transform):
    def __init__(self, mean, std): self.mean, self.std = mean, std
    @classmethod
    def new(cls, mean, std): return cls(mean, std)
    @classmethod
    def standard(cls): return cls(0.0, 1.0)
    @classmethod
    def zero_centered(cls):
        """[0, 1] -> [-1, 1]: mean 0.5, std 0.5."""
        return cls(0.5, 0.5)
    def apply(self, x):
        m, s = self.mean, self.std
        if isinstance(m, (list, tuple)):        # per-channel statistics: broadcast over [C, H, W]
            shape = [-1] + [1] * max(x.dim() - 1, 0) if len(m) > 1 else [1]
            m = torch.tensor(m, dtype=x.dtype, device=x.device).view(shape)
            s = torch.tensor(s, dtype=x.dtype, device=x.device).view(shape)
        return (x - m) / s


class RandomNoise(Transform):
    def __init__(self, std: float): self.std = std
    def apply(self, x): return x + torch.randn_like(x) * self.std


class RandomCrop(Transform):
    def __init__(self, size): self.size = (size, size) if isinstance(size, int) else tuple(size)
    @classmethod
    def new(cls, size): return cls(size)
    @classmethod
    def new_2d(cls, height: int, width: int): return cls((height, width))
    def apply(self, x):
        h, w = x.shape[-2:]
        th, tw = self.size
        i = int(torch.randint(0, h - th + 1, ())) if h > th else 0
        j = int(torch.randint(0, w - tw + 1, ())) if w > tw else 0
        return x[..., i:i + th, j:j + tw]


class RandomFlip(Transform):
    def __init__(self, dim: int = -1, p: float = 0.5): self.dim, self.p = dim, p
    @classmethod
    def new(cls, dim: int, probability: float): return cls(dim, probability)
    @classmethod
    def horizontal(cls):
        """Mirror left-right (the last dimension) half of the time."""
        return cls(-1, 0.5)
    @classmethod
    def vertical(cls):
        """Mirror top-bottom (the second to last dimension) half of the time."""
        return cls(-2, 0.5)
    def apply(self, x): return x.flip(self.dim) if float(torch.rand(())) < self.p else x


class Scale(Transform):
    def __init__(self, factor: float): self.factor = factor
    def apply(self, x): return x * self.factor


class Clamp(Transform):
    def __init__(self, lo: float, hi: float): self.lo, self.hi = lo, hi
    @classmethod
    def new(cls, lo: float, hi: float): return cls(lo, hi)
    @classmethod
    def zero_one(cls): return cls(0.0, 1.0)
    @classmethod
    def symmetric(cls): return cls(-1.0, 1.0)
    def apply(self, x): return x.clamp(self.lo, self.hi)


class Flatten(Transform):
    def apply(self, x): return x.flatten()


class Reshape(Transform):
    def __init__(self, shape): self.shape = tuple(shape)
    def apply(self, x): return x.reshape(self.shape)


class DropoutTransform(Transform):
    def __init__(self, p: float): self.p = p
    def apply(self, x): return torch.nn.functional.dropout(x, self.p, True)


class Lambda(Transform):
    def __init__(self, fn): self.fn = fn
    def apply(self, x): return self.fn(x)
