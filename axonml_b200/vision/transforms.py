"""Image transforms (crates/axonml-vision/src/transforms.rs:17-783) on ``[C, H, W]`` or
``[N, C, H, W]`` float tensors."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..data.transforms import Transform


def _b(x): return (x.unsqueeze(0), True) if x.dim() == 3 else (x, False)
def _u(x, s): return x.squeeze(0) if s else x


class Resize(Transform):
    def __init__(self, size, width: int | None = None):
        self.size = (size, width) if width is not None else (size, size) if isinstance(size, int) else tuple(size)
    @classmethod
    def new(cls, height: int, width: int): return cls((height, width))
    @classmethod
    def square(cls, size: int): return cls((size, size))
    def apply(self, x):
        y, s = _b(x)
        return _u(F.interpolate(y.float(), size=self.size, mode="bilinear", align_corners=False), s)


class CenterCrop(Transform):
    def __init__(self, size, width: int | None = None):
        self.size = (size, width) if width is not None else (size, size) if isinstance(size, int) else tuple(size)
    @classmethod
    def new(cls, height: int, width: int): return cls((height, width))
    @classmethod
    def square(cls, size: int): return cls((size, size))
    def apply(self, x):
        h, w = x.shape[-2:]
        th, tw = self.size
        i, j = max(0, (h - th) // 2), max(0, (w - tw) // 2)
        return x[..., i:i + th, j:j + tw]


class RandomHorizontalFlip(Transform):
    def __init__(self, p: float = 0.5): self.p = min(max(float(p), 0.0), 1.0)
    @classmethod
    def new(cls): return cls(0.5)
    @classmethod
    def with_probability(cls, probability: float):
        """Flip with this probability (clamped to [0, 1])."""
        return cls(probability)
    def apply(self, x): return x.flip(-1) if float(torch.rand(())) < self.p else x


class RandomVerticalFlip(Transform):
    def __init__(self, p: float = 0.5): self.p = min(max(float(p), 0.0), 1.0)
    @classmethod
    def new(cls): return cls(0.5)
    @classmethod
    def with_probability(cls, probability: float):
        """Flip with this probability (clamped to [0, 1])."""
        return cls(probability)
    def apply(self, x): return x.flip(-2) if float(torch.rand(())) < self.p else x


class RandomRotation(Transform):
    """Two forms: ``RandomRotation(degrees)`` turns by a uniformly drawn angle in [-degrees, degrees]
    (bilinear resampling); ``RandomRotation.new()`` / ``with_angles([...])`` picks one of the
    quarter turns 0 / 90 / 180 / 270 and rotates exactly, as the reference does
    (transforms.rs:391-470)."""

    def __init__(self, degrees: float = 0.0, angles=None):
        self.degrees, self.angles = degrees, angles

    @classmethod
    def new(cls): return cls(0.0, [0, 90, 180, 270])

    @classmethod
    def with_angles(cls, angles):
        """Quarter turns to choose from; anything else in the list is dropped (an empty choice means no rotation)."""
        valid = [int(a) for a in angles if int(a) in (0, 90, 180, 270)]
        return cls(0.0, valid or [0])

    def apply(self, x):
        if self.angles is not None:
            a = self.angles[int(torch.randint(0, len(self.angles), ()))]
            return torch.rot90(x, a // 90, dims=(-2, -1)) if a else x
        a = math.radians((float(torch.rand(())) * 2 - 1) * self.degrees)
        y, s = _b(x)
        theta = torch.tensor([[math.cos(a), -math.sin(a), 0.0], [math.sin(a), math.cos(a), 0.0]]).repeat(y.shape[0], 1, 1)
        grid = F.affine_grid(theta, list(y.shape), align_corners=False)
        return _u(F.grid_sample(y.float(), grid, align_corners=False), s)


class ColorJitter(Transform):
    def __init__(self, brightness: float = 0.0, contrast: float = 0.0, saturation: float = 0.0):
        self.b, self.c, self.s = brightness, contrast, saturation
    def apply(self, x):
        r = lambda a: 1.0 + (float(torch.rand(())) * 2 - 1) * a
        x = x * r(self.b)
        m = x.mean(dim=(-3, -2, -1), keepdim=True)
        x = (x - m) * r(self.c) + m
        g = x.mean(dim=-3, keepdim=True)
        return ((x - g) * r(self.s) + g).clamp(0, 1)


class Grayscale(Transform):
    def __init__(self, num_output_channels: int = 1): self.n = max(int(num_output_channels), 1)
    @classmethod
    def new(cls): return cls(1)
    @classmethod
    def with_channels(cls, num_output_channels: int):
        """Grey image repeated over this many channels (at least one)."""
        return cls(num_output_channels)
    def apply(self, x):
        w = torch.tensor([0.299, 0.587, 0.114], device=x.device).view(3, 1, 1)
        g = (x * w).sum(-3, keepdim=True)
        return g.expand(*g.shape[:-3], self.n, *g.shape[-2:]) if self.n > 1 else g


class ImageNormalize(Transform):
    def __init__(self, mean, std):
        self.mean, self.std = torch.tensor(mean).view(-1, 1, 1), torch.tensor(std).view(-1, 1, 1)
    @classmethod
    def imagenet(cls): return cls([0.485, 0.456, 0.406], [0.229, 0.224, 0.225])
    @classmethod
    def mnist(cls): return cls([0.1307], [0.3081])
    @classmethod
    def cifar10(cls): return cls([0.4914, 0.4822, 0.4465], [0.2470, 0.2435, 0.2616])
    def apply(self, x): return (x - self.mean.to(x.device)) / self.std.to(x.device)


class Pad(Transform):
    """Constant padding of the last two dimensions; ``padding`` = one width for every side or
    ``(left, right, top, bottom)``."""

    def __init__(self, padding, value: float = 0.0):
        self.padding = (padding,) * 4 if isinstance(padding, int) else tuple(int(p) for p in padding)
        if len(self.padding) != 4:
            raise ValueError("padding is one int or (left, right, top, bottom)")
        self.p, self.v = self.padding[0], value
    @classmethod
    def new(cls, padding: int): return cls(padding)
    @classmethod
    def asymmetric(cls, left: int, right: int, top: int, bottom: int): return cls((left, right, top, bottom))
    def with_fill(self, value: float):
        self.v = float(value)
        return self
    def apply(self, x): return F.pad(x, self.padding, value=self.v)


class ToTensorImage(Transform):
    """HWC uint8 -> CHW float in [0, 1]."""
    def apply(self, x):
        t = torch.as_tensor(x)
        if t.dim() == 3 and t.shape[-1] in (1, 3, 4):
            t = t.permute(2, 0, 1)
        return t.float() / 255.0 if t.dtype == torch.uint8 else t.float()
