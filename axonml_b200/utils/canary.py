"""Canary-padded tensors: a stand-in for a memory checker on a GPU pool where
``compute-sanitizer`` is not available.

``guarded(shape, dtype, device)`` carves the tensor out of the middle of a larger allocation whose
head and tail are filled with a byte pattern; ``Guarded.check()`` raises if a kernel wrote outside
the tensor.  The pads are multiples of 256 bytes, so the tensor keeps the 16-byte (TMA) and 256-byte
alignment the kernels expect.  Writes outside the tensor are detected, reads are not."""
from __future__ import annotations

import torch

_PATTERN = 0xA5


class CanaryViolation(AssertionError):
    pass


class Guarded:
    def __init__(self, shape, dtype=torch.float32, device="cuda", pad_bytes: int = 4096, fill=None,
                 memory_format=torch.contiguous_format):
        pad = (pad_bytes + 255) // 256 * 256
        self.pad = pad
        numel = 1
        for s in shape:
            numel *= int(s)
        esz = torch.empty((), dtype=dtype).element_size()
        body = (numel * esz + 255) // 256 * 256
        self.nbytes = numel * esz
        self.raw = torch.full((pad + body + pad,), _PATTERN, dtype=torch.uint8, device=device)
        view = self.raw[pad:pad + numel * esz].view(dtype)
        if memory_format == torch.channels_last and len(shape) == 4:
            n, c, h, w = shape
            self.tensor = view.view(n, h, w, c).permute(0, 3, 1, 2)
        else:
            self.tensor = view.view(*shape)
        if fill is not None:
            self.tensor.fill_(fill)

    def check(self, what: str = "tensor") -> None:
        head = self.raw[:self.pad]
        tail = self.raw[self.pad + self.nbytes:]
        bad_h = int((head != _PATTERN).sum())
        bad_t = int((tail != _PATTERN).sum())
        if bad_h or bad_t:
            first = None
            if bad_t:
                first = int((tail != _PATTERN).nonzero()[0]) + self.nbytes
            elif bad_h:
                first = int((head != _PATTERN).nonzero()[-1]) - self.pad
            raise CanaryViolation(f"{what}: {bad_h} byte(s) written before and {bad_t} after the buffer "
                                  f"(first at byte offset {first} relative to its start)")


def guarded(shape, dtype=torch.float32, device="cuda", **kw) -> Guarded:
    return Guarded(shape, dtype, device, **kw)
