"""Loader for the in-tree native libraries.

``kernels()`` returns the ctypes handle of ``libft_kernels.so`` (sm_100a CUDA
kernels), ``runtime()`` the handle of ``libft_runtime.so`` (C++ host runtime).
Both are built by :mod:`ferrotorch_b200._build`. On a machine with a GPU a
missing kernel library is an error (there is no silent eager fallback); on a
CPU-only machine the library still loads because it has no link-time
dependency on the driver.
"""
from __future__ import annotations

import ctypes
import os
import re
import threading
from pathlib import Path

import torch

from .errors import FerrotorchError, NativeLibraryMissing

_DIR = Path(__file__).resolve().parent / "_C"
_lock = threading.Lock()
_kernels = None
_runtime = None

c_void_p, c_int, c_int64, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float

_ERR_NAMES = {-1: "invalid argument / unsupported shape or alignment", -2: "CUDA driver entry point unavailable",
              -3: "tensor-map encode refused", -4: "request exceeds a compiled-in maximum",
              -5: "guard bytes behind an allocation were overwritten"}


def _load(name: str):
    path = _DIR / name
    if not path.exists():
        if os.environ.get("FT_NO_AUTOBUILD") != "1":
            from . import _build
            _build.build_all()
    if not path.exists():
        raise NativeLibraryMissing(f"{path} is missing; run `python -m ferrotorch_b200._build`")
    # local binding: the kernels library carries its own static CUDA runtime, whose symbols must not interpose on the ones other
    # libraries in the process (cuDNN, NCCL) resolve lazily
    return ctypes.CDLL(str(path), mode=ctypes.RTLD_LOCAL)


def kernels():
    global _kernels
    if _kernels is None:
        with _lock:
            if _kernels is None:
                _kernels = _load("libft_kernels.so")
    return _kernels


def runtime():
    global _runtime
    if _runtime is None:
        with _lock:
            if _runtime is None:
                _runtime = _load("libft_runtime.so")
    return _runtime


def check(code: int, what: str) -> None:
    if code == 0:
        return
    if code < 0:
        raise FerrotorchError(f"{what}: {_ERR_NAMES.get(code, 'error')} (code {code})")
    raise FerrotorchError(f"{what}: CUDA error {code}")


def ptr(t) -> int:
    """Device (or host) address of a tensor, 0 for None."""
    return 0 if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


# Argument signatures of the exported launchers are read from the sources themselves
# (every `FT_EXPORT int name(args)` in csrc/kernels/*.cu): p = pointer, i = int, l = int64, f = float, d = double.
_SIGS: dict = {}
_EXPORT_RE = re.compile(r"FT_EXPORT\s+int\s+(\w+)\s*\(([^)]*)\)", re.S)


def _parse_sigs() -> None:
    src_dir = Path(__file__).resolve().parent / "csrc" / "kernels"
    for f in sorted(src_dir.glob("*.cu")):
        for name, args in _EXPORT_RE.findall(f.read_text()):
            sig = ""
            for a in [x.strip() for x in args.split(",") if x.strip()]:
                if "*" in a or "cudaStream_t" in a:
                    sig += "p"
                elif re.search(r"\b(int64_t|uint64_t|size_t)\b", a):
                    sig += "l"
                elif re.search(r"\bfloat\b", a):
                    sig += "f"
                elif re.search(r"\bdouble\b", a):
                    sig += "d"
                else:
                    sig += "i"
            _SIGS[name] = sig


_CT = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_int64, "f": ctypes.c_float, "d": ctypes.c_double}
_bound: dict = {}
launch_calls = 0  # number of native launcher calls made by this process (each launches >= 1 kernel)


def register_sigs(sigs: dict) -> None:
    _SIGS.update(sigs)


def _fn(fn_name: str):
    f = _bound.get(fn_name)
    if f is None:
        f = getattr(kernels(), fn_name)
        if not _SIGS:
            _parse_sigs()
        sig = _SIGS.get(fn_name)
        if sig is None:
            raise FerrotorchError(f"no signature registered for native function {fn_name}")
        f.argtypes = [_CT[c] for c in sig]
        f.restype = ctypes.c_int
        _bound[fn_name] = f
    return f


def _unwrap(a):
    if isinstance(a, torch.Tensor):
        return a.data_ptr()
    if isinstance(a, ctypes._SimpleCData):
        return a.value
    return a


_trace = None  # while a launch trace is open: {"events": [(label, start, end)], "classify": callable or None}


def trace_begin(classify=None) -> None:
    """Start timing every native launcher call with a CUDA event pair on its own stream. ``classify(fn_name, args)`` may map a call to a
    label (default: the launcher's name). Meant for step breakdowns: it adds two event records per launch, so a traced step is a little
    slower than an untraced one."""
    global _trace
    _trace = {"events": [], "classify": classify}


def trace_end() -> dict:
    """Stop the trace, synchronise and return ``{label: {"ms": total, "calls": n}}``."""
    global _trace
    t, _trace = _trace, None
    out: dict = {}
    if t is None:
        return out
    torch.cuda.synchronize()
    for label, e0, e1 in t["events"]:
        d = out.setdefault(label, {"ms": 0.0, "calls": 0})
        d["ms"] += e0.elapsed_time(e1)
        d["calls"] += 1
    return out


def call(fn_name: str, *args) -> None:
    """Call an exported launcher ``int fn(...)`` and raise on a non-zero return code.

    Tensors are passed as their data pointers, ``None`` as a null pointer.
    """
    global launch_calls
    fn = _fn(fn_name)
    launch_calls += 1
    if len(args) != len(fn.argtypes):
        raise FerrotorchError(f"{fn_name}: expected {len(fn.argtypes)} arguments, got {len(args)}")
    raw = [_unwrap(a) for a in args]
    if _trace is None:
        check(fn(*raw), fn_name)
        return
    label = _trace["classify"](fn_name, raw) if _trace["classify"] else fn_name
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    check(fn(*raw), fn_name)
    e1.record()
    _trace["events"].append((label or fn_name, e0, e1))


def read_status() -> int:
    """Synchronise the current device and return (and clear) the kernel status word.

    Non-zero means a bounded device-side wait ran out: bits [31:24] name the
    kernel, [23:16] the wait site, [15:0] a detail value.
    """
    out = ctypes.c_uint32(0)
    check(kernels().ft_status_read_clear(ctypes.byref(out)), "ft_status_read_clear")
    return out.value


def P(t):
    return c_void_p(ptr(t))


def S():
    return c_void_p(stream_ptr())
