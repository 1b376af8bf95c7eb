"""Error types, one class per variant of the reference's ``Error`` enum
(crates/axonml-core/src/error.rs, whole file)."""
from __future__ import annotations


class AxonmlError(Exception):
    """Base class of every framework error (the reference's ``Error``)."""


class ShapeMismatch(AxonmlError):
    def __init__(self, expected, actual):
        super().__init__(f"shape mismatch: expected {list(expected)}, got {list(actual)}")
        self.expected, self.actual = tuple(expected), tuple(actual)


class DTypeMismatch(AxonmlError):
    def __init__(self, expected, actual):
        super().__init__(f"dtype mismatch: expected {expected}, got {actual}")
        self.expected, self.actual = expected, actual


class DeviceMismatch(AxonmlError):
    def __init__(self, expected, actual):
        super().__init__(f"device mismatch: expected {expected}, got {actual}")
        self.expected, self.actual = expected, actual


class InvalidDimension(AxonmlError):
    def __init__(self, index, ndim):
        super().__init__(f"invalid dimension {index} for a tensor with {ndim} dimensions")
        self.index, self.ndim = index, ndim


class IndexOutOfBounds(AxonmlError):
    def __init__(self, index, size):
        super().__init__(f"index {index} out of bounds for size {size}")
        self.index, self.size = index, size


class AllocationFailed(AxonmlError):
    def __init__(self, size, device):
        super().__init__(f"failed to allocate {size} bytes on {device}")
        self.size, self.device = size, device


class DeviceNotAvailable(AxonmlError):
    def __init__(self, device):
        super().__init__(f"device not available: {device}")
        self.device = device


class InvalidOperation(AxonmlError):
    def __init__(self, message):
        super().__init__(f"invalid operation: {message}")


class BroadcastError(AxonmlError):
    def __init__(self, shape1, shape2):
        super().__init__(f"cannot broadcast {list(shape1)} with {list(shape2)}")
        self.shape1, self.shape2 = tuple(shape1), tuple(shape2)


class EmptyTensor(AxonmlError):
    def __init__(self):
        super().__init__("operation not supported on an empty tensor")


class NotContiguous(AxonmlError):
    def __init__(self):
        super().__init__("operation requires a contiguous tensor")


class GradientError(AxonmlError):
    def __init__(self, message):
        super().__init__(f"gradient error: {message}")


class SerializationError(AxonmlError):
    def __init__(self, message):
        super().__init__(f"serialization error: {message}")


class InternalError(AxonmlError):
    def __init__(self, message):
        super().__init__(f"internal error: {message}")


Error = AxonmlError


# constructor helpers of the reference's ``Error`` (error.rs ``Error::shape_mismatch`` ...)
def _as_static(fn):
    return staticmethod(fn)


AxonmlError.shape_mismatch = _as_static(lambda expected, actual: ShapeMismatch(expected, actual))
AxonmlError.invalid_operation = _as_static(lambda message: InvalidOperation(message))
AxonmlError.internal = _as_static(lambda message: InternalError(message))
