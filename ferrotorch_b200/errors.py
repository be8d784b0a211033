"""Error types of the framework.

The variants follow the reference's ``FerrotorchError`` enum
(ferrotorch-core/src/error.rs:8-89) and ``DistributedError``
(ferrotorch-distributed/src/error.rs:10-52): one Python exception class per
variant so callers can match on the failure kind instead of parsing messages.
"""
from __future__ import annotations


class FerrotorchError(RuntimeError):
    """Base class of every error raised by the framework."""


class ShapeMismatch(FerrotorchError):
    pass


class DeviceMismatch(FerrotorchError):
    def __init__(self, expected, got):
        super().__init__(f"device mismatch: expected {expected}, got {got}")
        self.expected, self.got = expected, got


class BackwardNonScalar(FerrotorchError):
    def __init__(self, shape):
        super().__init__(f"backward() on a non-scalar tensor of shape {list(shape)} needs an explicit gradient")
        self.shape = tuple(shape)


class NoGradFn(FerrotorchError):
    pass


class DtypeMismatch(FerrotorchError):
    def __init__(self, expected, got):
        super().__init__(f"dtype mismatch: expected {expected}, got {got}")
        self.expected, self.got = expected, got


class IndexOutOfBounds(FerrotorchError, IndexError):
    pass


class InvalidArgument(FerrotorchError, ValueError):
    pass


class LockPoisoned(FerrotorchError):
    pass


class Internal(FerrotorchError):
    pass


class DeviceUnavailable(FerrotorchError):
    pass


class GpuTensorNotAccessible(FerrotorchError):
    pass


class NotImplementedOnCuda(FerrotorchError, NotImplementedError):
    def __init__(self, op: str):
        super().__init__(f"{op} is not implemented on CUDA")
        self.op = op


class GpuError(FerrotorchError):
    pass


class WorkerPanic(FerrotorchError):
    pass


class NativeLibraryMissing(FerrotorchError, ImportError):
    """The in-tree native library has not been built."""


# ---------------------------------------------------------------------------
# distributed
# ---------------------------------------------------------------------------
class DistributedError(FerrotorchError):
    pass


class InvalidWorldSize(DistributedError):
    pass


class InvalidRank(DistributedError):
    pass


class SelfSend(DistributedError):
    pass


class SizeMismatch(DistributedError):
    pass


class IoError(DistributedError):
    pass


class ChannelClosed(DistributedError):
    pass


class UnsupportedOp(DistributedError):
    pass


class Timeout(DistributedError, TimeoutError):
    def __init__(self, seconds=None, message: str = ""):
        super().__init__(message or f"operation timed out after {seconds} s")
        self.seconds = seconds


class NoConnection(DistributedError):
    pass


class BackendUnavailable(DistributedError):
    pass
