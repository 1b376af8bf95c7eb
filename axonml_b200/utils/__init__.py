"""Small helpers shared by tests and tools: canary-padded tensors (``canary``)."""
from .canary import CanaryViolation, Guarded, guarded

__all__ = ["CanaryViolation", "Guarded", "guarded"]
