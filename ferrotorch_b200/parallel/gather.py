"""Parameter gather of the fully sharded (ZeRO-3) engine: slots, arrival counters, prefetch and the consumer-side gate.

Every rank keeps only its own bf16 shard of each flat unit. A unit is materialised for one forward or backward pass in one of a few
full-size *slots* in symmetric memory: each rank pushes its shard into the slot of every rank (``ft_fsdp_push_shard``, 512 KiB pieces,
plain peer stores) from a side stream, one unit ahead of the compute stream, and marks every piece in the receiver's arrival
counters. Consumers never wait for "the gather" as a whole:

* the GEMM that reads a weight first waits *inside its TMA producer* for the pieces under the tile it is about to load
  (``ops.gemm(..., gate=...)`` -> ``ft_gemm_gated``), so it starts on what has landed;
* consumers that are not GEMMs (norm weights, the embedding table) put a small gate kernel on the compute stream.

A slot is recycled least-recently-used. Before a rank's slot is overwritten that rank *releases* it (a flag write on every peer, ordered
on its compute stream after the slot's last reader); pushers wait for the release of the previous occupant. A unit that is still resident
when it is needed again (the last layers between forward and backward) is not gathered twice.

Reference parity: ferrotorch-distributed/src/fsdp.rs:389-542 (forward gather of every parameter), :586-609 (restore_shards).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Tuple

import torch

from .. import _lib
from .symm import SymmetricBuffer

PIECE_BYTES = 512 << 10


class ParamViews(dict):
    """Named views of a gathered unit plus the gate its consumers wait on (``None`` when the values are simply resident)."""
    gate: Optional["GatherGate"] = None


class GatherGate:
    """Arrival state of one gather as seen by the consumers on the compute stream."""

    def __init__(self, counters_ptr: int, expected: int, slot_ptr: int, piece_bytes: int, nbytes: int):
        self.counters_ptr, self.expected, self.slot_ptr, self.piece_bytes, self.nbytes = counters_ptr, expected, slot_ptr, piece_bytes, nbytes
        self._ensured: List[Tuple[int, int]] = []       # piece ranges some kernel on the compute stream has already waited for

    def pieces_of(self, t: torch.Tensor) -> Tuple[int, int]:
        off = t.data_ptr() - self.slot_ptr
        if off < 0 or off + t.numel() * t.element_size() > self.nbytes:
            raise ValueError("tensor does not lie inside the gathered unit")
        if not t.is_contiguous():
            raise ValueError("gated tensors must be contiguous views of the unit")
        return off // self.piece_bytes, (off + t.numel() * t.element_size() - 1) // self.piece_bytes + 1

    def covered(self, t: torch.Tensor) -> bool:
        lo, hi = self.pieces_of(t)
        return any(a <= lo and hi <= b for a, b in self._ensured)

    def mark(self, t: torch.Tensor) -> None:
        lo, hi = self.pieces_of(t)
        merged = []
        for a, b in self._ensured:
            if a <= hi and lo <= b:
                lo, hi = min(a, lo), max(b, hi)
            else:
                merged.append((a, b))
        merged.append((lo, hi))
        self._ensured = merged

    def wait(self, t: torch.Tensor) -> None:
        """Put a gate kernel for the pieces under ``t`` on the current stream (nothing if an earlier kernel already waited for them)."""
        if self.covered(t):
            return
        lo, hi = self.pieces_of(t)
        _lib.call("ft_fsdp_gate", self.counters_ptr, int(lo), int(hi), self.expected, _lib.S())
        self.mark(t)


class ShardedParams:
    """Owns the bf16 shards, the gather slots and their flags for one engine."""

    def __init__(self, engine, slots: int = 3, piece_bytes: int = PIECE_BYTES):
        import torch.distributed as dist
        self.e = engine
        dev, group = engine.device, engine.pg
        self.world, self.rank = engine.world, engine.rank
        self.piece_bytes = piece_bytes
        self.nslots = max(2, int(os.environ.get("FT_FSDP_SLOTS", slots)))
        units = engine.units
        self.maxn = max(u.padded for u in units)
        self.geom: Dict[str, Tuple[int, int]] = {}       # unit -> (piece bytes, pieces per chunk)
        for u in units:
            cb = u.chunk * 2
            pb = piece_bytes if cb >= piece_bytes else cb
            if cb % pb:
                raise ValueError(f"unit {u.name}: shard of {cb} bytes is not a whole number of {pb}-byte pieces (FlatUnit.reshard was not applied)")
            self.geom[u.name] = (pb, cb // pb)
        self.max_pieces = max(self.world * ppc for _, ppc in self.geom.values())
        self.slot_buf = SymmetricBuffer(self.nslots * self.maxn, torch.bfloat16, dev, group)
        self.arrive = SymmetricBuffer(self.nslots * self.max_pieces, torch.int32, dev, group, zero=True)
        self.free = SymmetricBuffer(self.nslots * 8, torch.int32, dev, group, zero=True)
        # this rank's shard of every unit, in ordinary device memory (only the owner reads it)
        self.shard: Dict[str, torch.Tensor] = engine._shards
        self.gather_no = [0] * self.nslots
        self.resident: List[Optional[str]] = [None] * self.nslots
        self.where: Dict[str, int] = {}
        self.last_use = [0] * self.nslots
        self.clock = 0
        self.gates: Dict[str, GatherGate] = {}
        self.stream = torch.cuda.Stream(device=dev, priority=-1)
        self.push_done: Dict[str, torch.cuda.Event] = {}       # last push that read a unit's shard (the optimizer waits for it)
        self.shard_ready: Dict[str, torch.cuda.Event] = {}     # last optimizer update of a unit's shard (the next push waits for it)
        self.max_ctas = int(os.environ.get("FT_FSDP_PUSH_CTAS", "0"))
        # "dma": the shards travel by copy engine (cudaMemcpyAsync to the peer mapping); "sm": the push kernel (plain peer stores, per-piece arrival)
        self.mode = os.environ.get("FT_FSDP_PUSH", "dma")
        self.gathers = 0                                         # pushes issued (a resident unit needs none)
        torch.cuda.synchronize(dev)
        dist.barrier(group)

    # -- slot bookkeeping -------------------------------------------------------------------------------------------------
    def _slot_view(self, s: int, unit) -> torch.Tensor:
        return self.slot_buf.tensor[s * self.maxn: s * self.maxn + unit.padded]

    def _ptrs(self, buf: SymmetricBuffer, elem_offset: int):
        return buf.ptr_array(elem_offset)

    def prefetch(self, unit, reverse: bool = False) -> None:
        """Start gathering ``unit`` into the least recently used slot (nothing if it is resident). Called on the compute stream's thread:
        the release of the slot's previous occupant is ordered after everything enqueued on the compute stream so far."""
        self.clock += 1
        if unit.name in self.where:
            self.last_use[self.where[unit.name]] = self.clock
            return
        s = min(range(self.nslots), key=lambda i: self.last_use[i])
        n_prev = self.gather_no[s]
        if n_prev > 0:
            # this rank is done with the previous occupant: tell every pusher (flag free[s][rank] on each rank)
            _lib.call("ft_fsdp_release", self._ptrs(self.free, s * 8 + self.rank), self.world, n_prev, _lib.S())
        prev = self.resident[s]
        if prev is not None:
            self.where.pop(prev, None)
            self.gates.pop(prev, None)
        n = n_prev + 1
        pb, ppc = self.geom[unit.name]
        src = self.shard[unit.name]
        ready = self.shard_ready.get(unit.name)
        with torch.cuda.stream(self.stream):
            if ready is not None:
                self.stream.wait_event(ready)
            free_local = ctypes.c_void_p(self.free.ptrs[self.rank] + (s * 8) * 4)
            if self.mode == "sm":
                _lib.call("ft_fsdp_push_shard", src, self._ptrs(self.slot_buf, s * self.maxn), self._ptrs(self.arrive, s * self.max_pieces),
                          free_local, self.rank, self.world, ctypes.c_int64(unit.chunk * 2), ctypes.c_int64(pb), n, int(reverse), self.max_ctas,
                          _lib.S())
            else:
                # copy engines: no SM is taken from the GEMMs while the shard travels; arrival is marked per source rank
                _lib.call("ft_fsdp_wait_free", free_local, self.world, n_prev, _lib.S())
                for d in range(self.world):
                    q = (self.rank + 1 + d) % self.world            # peers first, rotated so that the ranks address distinct receivers
                    dst = self.slot_buf.ptrs[q] + (s * self.maxn + self.rank * unit.chunk) * 2
                    _lib.call("ft_memcpy_d2d_async", ctypes.c_void_p(dst), src, ctypes.c_int64(unit.chunk * 2), _lib.S())
                    _lib.call("ft_fsdp_signal", ctypes.c_void_p(self.arrive.ptrs[q] + (s * self.max_pieces + self.rank * ppc) * 4), ppc, n, _lib.S())
            ev = torch.cuda.Event()
            ev.record(self.stream)
            self.push_done[unit.name] = ev
        self.gathers += 1
        self.gather_no[s] = n
        self.resident[s] = unit.name
        self.where[unit.name] = s
        self.last_use[s] = self.clock
        self.gates[unit.name] = GatherGate(self.arrive.ptrs[self.rank] + s * self.max_pieces * 4, n,
                                           self.slot_buf.ptrs[self.rank] + s * self.maxn * 2, pb, unit.padded * 2)

    def invalidate(self, unit) -> None:
        """The unit's shards were updated: a copy that is still resident in a slot must not be used again (the slot becomes the preferred
        victim; it is released to the pushers when the next gather takes it)."""
        s = self.where.pop(unit.name, None)
        self.gates.pop(unit.name, None)
        if s is not None:
            self.resident[s] = None
            self.last_use[s] = 0

    def acquire(self, unit, reverse: bool = False) -> ParamViews:
        if unit.name not in self.where:
            self.prefetch(unit, reverse)
        s = self.where[unit.name]
        self.clock += 1
        self.last_use[s] = self.clock
        views = ParamViews(unit.views(self._slot_view(s, unit)))
        views.gate = self.gates[unit.name]
        return views

    def full_tensor(self, unit) -> torch.Tensor:
        """The whole gathered unit after waiting for all of it (state-dict export, tests)."""
        v = self.acquire(unit)
        buf = self._slot_view(self.where[unit.name], unit)
        v.gate.wait(buf)
        return buf
