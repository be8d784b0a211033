"""Per-device scratch buffers reused across launches (grown on demand, never shrunk).

Kernels that need scratch memory beyond their inputs and outputs (per-CTA
partials of a two-stage reduction, split-K partial tiles) take it from here so
the steady state of a training step performs no allocation for scratch.
"""
from __future__ import annotations

import torch

_bufs: dict = {}


def workspace(device, tag: str, nbytes: int) -> torch.Tensor:
    key = (str(device), tag)
    buf = _bufs.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 16), device=device, dtype=torch.uint8)
        _bufs[key] = buf
    return buf


def release_all() -> None:
    _bufs.clear()
