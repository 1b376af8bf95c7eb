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
    def __init__(self, size): self.size = (size, size) if isinstance(size, int) else tuple(size)
    def apply(self, x):
        y, s = _b(x)
        return _u(F.interpolate(y.float(), size=self.size, mode="bilinear", align_corners=False), s)


class CenterCrop(Transform):
    def __init__(self, size): self.size = (size, size) if isinstance(size, int) else tuple(size)
    def apply(self, x):
        h, w = x.shape[-2:]
        th, tw = self.size
        i, j = max(0, (h - th) // 2), max(0, (w - tw) // 2)
        return x[..., i:i + th, j:j + tw]


class RandomHorizontalFlip(Transform):
    def __init__(self, p: float = 0.5): self.p = p
    def apply(self, x): return x.flip(-1) if float(torch.rand(())) < self.p else x


class RandomVerticalFlip(Transform):
    def __init__(self, p: float = 0.5): self.p = p
    def apply(self, x): return x.flip(-2) if float(torch.rand(())) < self.p else x


class RandomRotation(Transform):
    def __init__(self, degrees: float): self.degrees = degrees
    def apply(self, x):
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
    def __init__(self, num_output_channels: int = 1): self.n = num_output_channels
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
    def apply(self, x): return (x - self.mean.to(x.device)) / self.std.to(x.device)


class Pad(Transform):
    def __init__(self, padding: int, value: float = 0.0): self.p, self.v = padding, value
    def apply(self, x): return F.pad(x, (self.p,) * 4, value=self.v)


class ToTensorImage(Transform):
    """HWC uint8 -> CHW float in [0, 1]."""
    def apply(self, x):
        t = torch.as_tensor(x)
        if t.dim() == 3 and t.shape[-1] in (1, 3, 4):
            t = t.permute(2, 0, 1)
        return t.float() / 255.0 if t.dtype == torch.uint8 else t.float()
