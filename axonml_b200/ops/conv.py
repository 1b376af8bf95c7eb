"""Conv2d dispatch.  ``conv2d_supported`` tells the nn layer whether the hand-written
implicit-GEMM kernel takes this call; otherwise the layer uses the torch convolution."""
from __future__ import annotations

import torch


def conv2d_supported(x, weight, stride, padding) -> bool:
    from . import conv_igemm
    return conv_igemm.supported(x, weight, stride, padding) or conv_igemm.thin_supported(x, weight, stride, padding)


def conv2d(x, weight, bias, stride, padding):
    from . import conv_igemm
    return conv_igemm.conv2d(x, weight, bias, stride, padding)
