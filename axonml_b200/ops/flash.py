"""Flash attention on tcgen05 (``csrc/kernels/flash_fwd.cu``, ``flash_bwd.cu``)."""
from __future__ import annotations

import torch

from .. import _native as N


def supported(q, k, v, mask, dropout_p) -> bool:
    return False
