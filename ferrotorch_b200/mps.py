"""Metal Performance Shaders backend: not part of this framework, which targets CUDA sm_100a only (ferrotorch-mps/src/lib.rs:101). The module exists so that code probing for
the backend gets a definite answer instead of an import error."""
from .errors import DeviceUnavailable


def is_available() -> bool:
    return False


def device_count() -> int:
    return 0


class MtlBackend:
    def __init__(self, *args, **kwargs):
        raise DeviceUnavailable("the mps backend is unavailable: this framework runs on CUDA devices only")


def is_mps_available() -> bool:
    return False


class MpsDevice(MtlBackend):
    @staticmethod
    def count() -> int:
        return 0
