"""Flat parameter units.

A unit is one contiguous bf16 buffer holding several named tensors (for a
transformer: every weight of one decoder layer), plus the f32 master copy and
optimizer moments for the slice of it that this rank owns. Collectives and the
optimizer run once per unit on flat memory instead of once per parameter:

* world 1: the rank owns the whole buffer;
* world N (full shard): rank r owns ``[r*chunk, (r+1)*chunk)`` of the padded
  buffer; the full bf16 buffer is (re)materialised by an all-gather and the
  full bf16 gradient buffer is reduce-scattered into the owner's slice.

The reference shards per parameter with no padding and asserts divisibility
(ferrotorch-distributed/src/fsdp.rs:206-223); here the unit is padded to a
multiple of ``world * 128`` elements so any shape shards evenly and every shard
starts on a 256-byte boundary.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Tuple

import torch


@dataclass
class TensorSpec:
    name: str
    offset: int
    shape: Tuple[int, ...]

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class FlatUnit:
    """One flat bf16 parameter buffer with named views."""

    def __init__(self, name: str, shapes: List[Tuple[str, Tuple[int, ...]]], device, dtype=torch.bfloat16, world: int = 1,
                 rank: int = 0, align: int = 128):
        self.name = name
        self.world, self.rank = world, rank
        self.specs: Dict[str, TensorSpec] = {}
        off = 0
        for n, shp in shapes:
            self.specs[n] = TensorSpec(n, off, tuple(shp))
            off = _round_up(off + self.specs[n].numel, align)
        self.numel = off
        self.padded = _round_up(off, world * align)
        self.chunk = self.padded // world
        self.device, self.dtype = torch.device(device), dtype
        # the full compute-precision buffer (always resident at world 1; gathered on demand otherwise)
        self.full: torch.Tensor | None = torch.zeros(self.padded, device=device, dtype=dtype)
        self.grad: torch.Tensor | None = None          # full-size gradient buffer, supplied by the engine
        self.master: torch.Tensor | None = None        # f32 [chunk]
        self.exp_avg: torch.Tensor | None = None
        self.exp_avg_sq: torch.Tensor | None = None
        self.momentum: torch.Tensor | None = None
        self.step = 0

    def reshard(self, shard_align: int) -> None:
        """Re-pad the unit so that every rank's shard is a multiple of ``shard_align`` elements (the arrival granularity of the fully
        sharded engine's gather). Only before the optimizer state exists; the values are kept, the new tail is zero."""
        if self.master is not None:
            raise RuntimeError("FlatUnit.reshard must run before the optimizer state is created")
        chunk = _round_up(-(-self.numel // self.world), shard_align)
        padded = chunk * self.world
        if padded != self.padded:
            full = torch.zeros(padded, device=self.device, dtype=self.dtype)
            n = min(self.padded, padded)
            full[:n].copy_(self.full[:n])
            self.full = full
            self.padded, self.chunk = padded, chunk

    # -- views -------------------------------------------------------------
    def view(self, name: str, buf: torch.Tensor | None = None) -> torch.Tensor:
        s = self.specs[name]
        b = self.full if buf is None else buf
        return b[s.offset: s.offset + s.numel].view(s.shape)

    def views(self, buf: torch.Tensor | None = None) -> Dict[str, torch.Tensor]:
        return {n: self.view(n, buf) for n in self.specs}

    def shard_slice(self, buf: torch.Tensor, rank: int | None = None) -> torch.Tensor:
        r = self.rank if rank is None else rank
        return buf[r * self.chunk: (r + 1) * self.chunk]

    # -- optimizer state ---------------------------------------------------
    def init_master(self) -> None:
        """f32 master copy of this rank's slice, taken from the current bf16 values."""
        self.master = self.shard_slice(self.full).to(torch.float32, copy=True)

    def init_adam(self) -> None:
        if self.master is None:
            self.init_master()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)

    def nbytes_state(self) -> int:
        n = 0
        for t in (self.master, self.exp_avg, self.exp_avg_sq, self.momentum):
            if t is not None:
                n += t.numel() * t.element_size()
        return n
