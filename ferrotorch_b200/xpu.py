"""Intel XPU (Level Zero) backend: not part of this framework, which targets CUDA sm_100a only (ferrotorch-xpu/src/lib.rs). The module exists so that code probing for
the backend gets a definite answer instead of an import error."""
from .errors import DeviceUnavailable


def is_available() -> bool:
    return False


def device_count() -> int:
    return 0


class XpuDevice:
    def __init__(self, *args, **kwargs):
        raise DeviceUnavailable("the xpu backend is unavailable: this framework runs on CUDA devices only")


def make_xpu_tensor(*args, **kwargs):
    raise DeviceUnavailable("the xpu backend is unavailable: this framework runs on CUDA devices only")
