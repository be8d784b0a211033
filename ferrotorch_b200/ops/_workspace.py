"""Per-device, per-stream scratch buffers reused across launches (grown on demand, never shrunk).

Kernels that need scratch memory beyond their inputs and outputs (per-CTA
partials of a two-stage reduction, split-K partial tiles) take it from here so
the steady state of a training step performs no allocation for scratch.

A buffer belongs to the stream that was current when it was requested: two
launches of the same operation on different streams (the FSDP side stream
beside the compute stream) get different buffers and cannot race on the
partials. Within one stream launches are ordered, so re-use is safe. When a
buffer has to grow, the old one is handed back to the caching allocator only
after ``record_stream``, so a kernel still writing to it keeps it alive.
"""
from __future__ import annotations

import torch

_bufs: dict = {}


def workspace(device, tag: str, nbytes: int) -> torch.Tensor:
    device = torch.device(device)
    stream = torch.cuda.current_stream(device) if device.type == "cuda" else None
    key = (str(device), tag, stream.cuda_stream if stream is not None else 0)
    buf = _bufs.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None and stream is not None:
            buf.record_stream(stream)
        buf = torch.empty(max(nbytes, 1 << 16), device=device, dtype=torch.uint8)
        _bufs[key] = buf
    return buf


def release_all() -> None:
    _bufs.clear()
