"""ferrotorch_b200: a Blackwell-native deep-learning framework with the capability surface of ferrotorch.

Sub-packages: ``ops`` (sm_100a kernels), ``models``, ``parallel``, ``utils``; the framework layers
(``nn``, ``optim``, ``data``, ``train``, ``serialize``, ``jit``, ``distributions``, ``profiler`` ...) are imported lazily.
"""
from __future__ import annotations

import importlib

from . import errors
from .errors import FerrotorchError

__version__ = "0.1.0"

_LAZY = ("ops", "models", "parallel", "utils", "nn", "optim", "data", "train", "serialize", "jit", "distributions", "profiler",
         "core", "autograd", "hub", "tokenize", "grammar", "ml", "vision", "runtime", "distributed", "gpu", "cubecl", "mps", "xpu", "prelude")


def __getattr__(name):
    if name in _LAZY:
        mod = importlib.import_module(f"{__name__}.{name}")
        globals()[name] = mod
        return mod
    if name == "jit_script":                                  # the scripting front end lives in the jit package
        mod = importlib.import_module(f"{__name__}.jit.script")
        globals()[name] = mod
        return mod
    if not name.startswith("_"):                              # the core names are also reachable from the top level (``ferrotorch::*``)
        core = importlib.import_module(f"{__name__}.core")
        if hasattr(core, name):
            return getattr(core, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def build(verbose: bool = False):
    """Compile the in-tree native libraries (sm_100a kernels and the C++ runtime)."""
    from . import _build
    return _build.build_all(verbose)
