"""Symmetric (peer-mapped) device memory and the NVLink collectives built on it.

``SymmetricBuffer`` allocates a buffer that every rank of the group maps into its own address space
(torch.distributed._symmetric_memory does the cuMem export/import and, where the fabric supports it, binds an
NVSwitch multicast address). ``SymmComm`` launches the hand-written collective kernels of ``csrc/kernels/comm.cu``
on such buffers: peers are addressed by plain loads/stores from inside the kernel, completion is signalled through
a flag block in symmetric memory, and every device-side wait has a deadline - a missing peer surfaces as
:class:`~ferrotorch_b200.errors.Timeout` from :meth:`SymmComm.check`, not as a hung GPU.

Reference parity: the TCP/NCCL transports under ferrotorch-distributed/src/{backend,nccl_backend,gpu_collective}.rs;
the reference has no peer-memory path at all.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch

from .. import _lib
from ..errors import DistributedError, Timeout


def _symm_mod():
    import torch.distributed._symmetric_memory as sm
    return sm


class SymmetricBuffer:
    """A 1-D buffer of ``numel`` elements of ``dtype`` mapped on every rank of ``group``."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group=None, zero: bool = False):
        import torch.distributed as dist
        sm = _symm_mod()
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        name = self.group.group_name
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")          # newer torch versions no longer need the call and say so for every buffer
            try:
                sm.enable_symm_mem_for_group(name)
            except Exception:
                pass
        self.tensor = sm.empty(numel, dtype=dtype, device=device)
        if zero:
            self.tensor.zero_()
        self.handle = sm.rendezvous(self.tensor, name)
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        mc = getattr(self.handle, "multicast_ptr", 0) or 0
        self.multicast_ptr = int(mc) if os.environ.get("FT_DISABLE_NVLS", "0") != "1" else 0
        self.itemsize = self.tensor.element_size()

    def ptr_array(self, elem_offset: int = 0):
        off = elem_offset * self.itemsize
        return (ctypes.c_void_p * self.world)(*[p + off for p in self.ptrs])

    def mc(self, elem_offset: int = 0) -> int:
        return self.multicast_ptr + elem_offset * self.itemsize if self.multicast_ptr else 0


class CommTrace:
    """Device-side phase stamps of the peer-memory collectives launched on one device: every launch writes, from inside the kernel, the
    ``globaltimer`` time at which it entered, saw all peers arrive, finished its own part and retired after the closing handshake. The ring
    keeps the last ``capacity`` launches (indexed by launch number). Used as a context manager::

        with CommTrace(device) as tr:
            ...training steps...
        for r in tr.records(): print(r["kind"], r["wait_peers_us"], r["body_us"], r["drain_us"])

    ``chrome_events`` renders the same records as Chrome-trace slices that can be merged into a profiler report (one row per phase)."""

    KINDS = {1: "all_reduce", 2: "all_reduce_1shot", 3: "reduce_scatter", 4: "all_gather", 5: "all_to_all", 6: "broadcast", 7: "barrier",
             8: "fsdp_rs_adamw_ag"}
    WORDS = 5

    def __init__(self, device, capacity: int = 4096):
        self.device = torch.device(device)
        self.capacity = int(capacity)
        self.ring = torch.zeros(self.capacity * self.WORDS, device=self.device, dtype=torch.int64)

    def enable(self) -> None:
        with torch.cuda.device(self.device):
            _lib.call("ft_comm_set_trace", self.ring, self.capacity)

    def disable(self) -> None:
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            _lib.call("ft_comm_set_trace", None, 0)

    def __enter__(self):
        self.enable()
        return self

    def __exit__(self, *exc):
        self.disable()
        return False

    @staticmethod
    def decode(words) -> List[dict]:
        """Records from the raw ring (a flat sequence of int64, five per record); empty and half-written records are skipped."""
        out = []
        w = [int(v) & 0xFFFFFFFFFFFFFFFF for v in words]
        for i in range(0, len(w) - CommTrace.WORDS + 1, CommTrace.WORDS):
            head, t_in, t_ready, t_body, t_out = w[i: i + CommTrace.WORDS]
            if head == 0 or not (0 < t_in <= t_ready <= t_body <= t_out):
                continue
            kind = head >> 32
            out.append({"seq": head & 0xFFFFFFFF, "kind": CommTrace.KINDS.get(kind, f"kind{kind}"), "start_ns": t_in,
                        "wait_peers_us": (t_ready - t_in) / 1e3, "body_us": (t_body - t_ready) / 1e3, "drain_us": (t_out - t_body) / 1e3,
                        "total_us": (t_out - t_in) / 1e3})
        out.sort(key=lambda r: r["start_ns"])
        return out

    def records(self) -> List[dict]:
        torch.cuda.synchronize(self.device)
        return self.decode(self.ring.cpu().tolist())

    @staticmethod
    def chrome_events(records: List[dict], pid: int = 0, tid: str = "comm kernels") -> List[dict]:
        ev = []
        for r in records:
            t = r["start_ns"] / 1e3
            for phase in ("wait_peers", "body", "drain"):
                d = r[phase + "_us"]
                ev.append({"name": f"{r['kind']}:{phase}", "ph": "X", "ts": t, "dur": d, "pid": pid, "tid": tid, "args": {"seq": r["seq"]}})
                t += d
        return ev


class SymmComm:
    """Launcher of the peer-memory collectives for one process group (at most 8 ranks on one NVSwitch domain)."""

    def __init__(self, device, group=None):
        import torch.distributed as dist
        self.device = torch.device(device)
        self.flags = SymmetricBuffer(_lib.kernels().ft_comm_flag_bytes() // 4, torch.int32, device, group, zero=True)
        self.group, self.world, self.rank = self.flags.group, self.flags.world, self.flags.rank
        self.flag_ptrs = self.flags.ptr_array()
        self.counter = torch.zeros(2, device=device, dtype=torch.int32)
        self.seq = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)        # every rank's flag block is zeroed before anybody signals into it

    def _next(self) -> int:
        self.seq += 1
        return self.seq

    def all_reduce_(self, buf: SymmetricBuffer, numel: int, elem_offset: int = 0, scale: float = 1.0, use_nvls: bool = True,
                    max_ctas: int = 0) -> None:
        """In-place sum (times ``scale``) across ranks of ``buf[elem_offset : elem_offset+numel]``."""
        dt = 0 if buf.tensor.dtype == torch.bfloat16 else 1
        mc = buf.mc(elem_offset) if use_nvls else 0
        _lib.call("ft_comm_allreduce", buf.ptr_array(elem_offset), self.flag_ptrs, self.counter, self.rank, self.world, self._next(),
                  numel, dt, float(scale), mc, max_ctas, _lib.S())

    def all_reduce_small(self, buf: SymmetricBuffer, out: torch.Tensor, numel: int, elem_offset: int = 0, scale: float = 1.0,
                         seq_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One-shot all-reduce into ``out``. With ``seq_dev`` (a device int32 scalar, zero-initialised, used by every rank for this
        communicator) the launch numbers itself on the device and can be captured in a CUDA graph and replayed."""
        dt = 0 if buf.tensor.dtype == torch.bfloat16 else 1
        seq = 0 if seq_dev is not None else self._next()
        _lib.call("ft_comm_allreduce_1shot", buf.ptr_array(elem_offset), out, self.flag_ptrs, self.counter, self.rank, self.world,
                  seq, numel, dt, float(scale), 0, seq_dev, _lib.S())
        return out

    def reduce_scatter(self, buf: SymmetricBuffer, out: torch.Tensor, chunk: int, elem_offset: int = 0, scale: float = 1.0,
                       use_nvls: bool = True) -> torch.Tensor:
        """``out[chunk]`` = ``scale`` x the sum over ranks of their ``buf[rank*chunk:(rank+1)*chunk]``. With a multicast mapping the sum is
        formed inside the switch (one ``multimem.ld_reduce`` per 16 bytes); otherwise the slice is pulled from every peer in fixed rank order
        (bit-identical on every run)."""
        dt = 0 if buf.tensor.dtype == torch.bfloat16 else 1
        mc = buf.mc(elem_offset) if use_nvls else 0
        if mc:
            _lib.call("ft_comm_reduce_scatter_nvls", ctypes.c_void_p(mc), out, self.flag_ptrs, self.counter, self.rank, self.world, self._next(), chunk, dt,
                      float(scale), 0, _lib.S())
            return out
        _lib.call("ft_comm_reduce_scatter", buf.ptr_array(elem_offset), out, self.flag_ptrs, self.counter, self.rank, self.world,
                  self._next(), chunk, dt, float(scale), 0, _lib.S())
        return out

    def all_gather(self, buf: SymmetricBuffer, src: torch.Tensor, chunk: int, elem_offset: int = 0) -> None:
        dt = 0 if buf.tensor.dtype == torch.bfloat16 else 1
        _lib.call("ft_comm_allgather", buf.ptr_array(elem_offset), src, self.flag_ptrs, self.counter, self.rank, self.world, self._next(),
                  chunk, dt, 0, _lib.S())

    def all_to_all(self, buf: SymmetricBuffer, out: torch.Tensor, chunk: int, elem_offset: int = 0) -> torch.Tensor:
        """``out[q*chunk:(q+1)*chunk]`` = rank q's ``buf[rank*chunk:(rank+1)*chunk]`` (every rank exposes ``world`` chunks, chunk q addressed to rank q)."""
        dt = 0 if buf.tensor.dtype == torch.bfloat16 else 1
        _lib.call("ft_comm_alltoall", buf.ptr_array(elem_offset), out, self.flag_ptrs, self.counter, self.rank, self.world, self._next(), chunk, dt, 0, _lib.S())
        return out

    def broadcast(self, buf: SymmetricBuffer, out: torch.Tensor, numel: int, root: int = 0, elem_offset: int = 0) -> torch.Tensor:
        dt = 0 if buf.tensor.dtype == torch.bfloat16 else 1
        _lib.call("ft_comm_broadcast", buf.ptr_array(elem_offset), out, self.flag_ptrs, self.counter, self.rank, self.world, self._next(), root, numel, dt, 0,
                  _lib.S())
        return out

    @staticmethod
    def set_timeout(seconds: float) -> None:
        """Deadline of the device-side waits on peers for collectives launched from now on (default 2 s, or ``FT_COMM_TIMEOUT_MS``). Every rank
        of a group should use the same value."""
        _lib.call("ft_comm_set_timeout_ms", max(1, int(seconds * 1000)))

    def barrier(self) -> None:
        _lib.call("ft_comm_barrier", self.flag_ptrs, self.counter, self.rank, self.world, self._next(), _lib.S())

    def check(self) -> None:
        """Synchronise and raise :class:`Timeout` if a device-side wait on a peer ran out since the last check."""
        st = _lib.read_status()
        if st:
            kernel, site, peer = st >> 24, (st >> 16) & 0xFF, st & 0xFFFF
            raise Timeout(message=f"device-side wait timed out: kernel {kernel}, site {site}, peer {peer}")


class SymmStatsReducer:
    """Sum of a small f32 vector over the ranks of a group by the one-shot peer-memory kernel: the producer kernel writes its partial
    vector straight into a staging slot in symmetric memory (:meth:`stage`), :meth:`reduce` then reads every peer's slot and returns
    the total in local memory. Used for the ``[sum, sum_sq]`` and ``[sum dy, sum dy*xhat]`` vectors of synchronised batch norm
    (ferrotorch-distributed/src/sync_batch_norm.rs:236,474).

    Four slots rotate: a rank can be at most one reduction ahead of its slowest peer (finishing a reduction needs every peer's arrival),
    so the slot a peer may still be reading is never the one being written."""

    SLOTS = 4

    def __init__(self, device, group=None, capacity: int = 8192):
        self.comm = SymmComm(device, group)
        self.group, self.world, self.rank = self.comm.group, self.comm.world, self.comm.rank
        self.capacity = (capacity + 3) // 4 * 4
        self.buf = SymmetricBuffer(self.SLOTS * self.capacity, torch.float32, device, group, zero=True)
        self._i = 0
        self._staged = None

    def stage(self, numel: int) -> torch.Tensor:
        if numel > self.capacity:
            raise ValueError(f"{numel} values exceed the staging capacity {self.capacity}")
        self._i = (self._i + 1) % self.SLOTS
        off = self._i * self.capacity
        self._staged = (off, numel)
        return self.buf.tensor[off: off + numel]

    def reduce(self) -> torch.Tensor:
        off, numel = self._staged
        out = torch.empty(numel, device=self.buf.tensor.device, dtype=torch.float32)
        return self.comm.all_reduce_small(self.buf, out, numel, off)


_stats_reducers: dict = {}


def stats_reducer(device, group=None) -> SymmStatsReducer:
    """One reducer per (device, group), created on first use (collective: every rank of the group must call it at the same point)."""
    import torch.distributed as dist
    g = group if group is not None else dist.group.WORLD
    key = (torch.device(device).index, g.group_name)
    if key not in _stats_reducers:
        _stats_reducers[key] = SymmStatsReducer(device, g)
    return _stats_reducers[key]


class FusedShardedAdamW:
    """Reduce-scatter + sharded AdamW (+ all-gather) of one flat unit in a single kernel over peer memory.

    Owns the symmetric arenas. The engine's rotating gradient buffers always live in one, so a peer can read any rank's gradients.
    ``full_shard=False`` (shard-grad-op): every unit's bf16 parameter buffer is moved into a second symmetric arena and the kernel pushes
    the refreshed slice into every rank's copy (the all-gather is part of the update). ``full_shard=True``: there is no replicated copy;
    the kernel writes the refreshed slice into this rank's shard only (``engine.sharded``, see ``parallel/gather.py``) and the parameters
    are gathered again when the next pass needs them.
    """

    def __init__(self, engine, full_shard: bool = False):
        self.e = engine
        self.full_shard = full_shard
        dev, group = engine.device, engine.pg
        self.comm = SymmComm(dev, group)
        units = engine.units
        self.offset = {}
        if not full_shard:
            total = sum(u.padded for u in units)
            self.params = SymmetricBuffer(total, torch.bfloat16, dev, group)
            off = 0
            name_to_param = _unit_params(engine.model)
            with torch.no_grad():
                for u in units:
                    view = self.params.tensor[off: off + u.padded]
                    view.copy_(u.full)
                    u.full = view
                    p = name_to_param.get(u.name)
                    if p is not None:
                        p.data = view
                    self.offset[u.name] = off
                    off += u.padded
        # CTAs of the fused reduce-scatter + AdamW (+ all-gather) launch (0 = the kernel's default of 96): it shares the SMs with the backward GEMMs
        self.max_ctas = int(os.environ.get("FT_FSDP_CTAS", "0"))
        nbuf = len(engine._grad_pool)
        self.maxn = max(u.padded for u in units)
        self.grads = SymmetricBuffer(nbuf * self.maxn, torch.bfloat16, dev, group)
        engine._grad_pool = [self.grads.tensor[i * self.maxn: (i + 1) * self.maxn] for i in range(nbuf)]
        torch.cuda.synchronize(dev)
        import torch.distributed as dist
        dist.barrier(group)

    def step(self, unit, slot: int) -> None:
        o = self.e.optim
        c = self.comm
        if self.full_shard:
            _lib.call("ft_fsdp_rs_adamw", self.grads.ptr_array(slot * self.maxn), self.e.sharded.shard[unit.name], c.flag_ptrs, c.counter, c.rank,
                      c.world, c._next(), unit.master, unit.exp_avg, unit.exp_avg_sq, unit.chunk, o.lr, o.betas[0], o.betas[1], o.eps,
                      o.weight_decay, unit.step, None, self.max_ctas, _lib.S())
            return
        _lib.call("ft_fsdp_rs_adamw_ag", self.grads.ptr_array(slot * self.maxn), self.params.ptr_array(self.offset[unit.name]),
                  c.flag_ptrs, c.counter, c.rank, c.world, c._next(), unit.master, unit.exp_avg, unit.exp_avg_sq, unit.chunk, o.lr,
                  o.betas[0], o.betas[1], o.eps, o.weight_decay, unit.step, None, self.max_ctas, _lib.S())


def _unit_params(model) -> dict:
    """``unit name -> the nn.Parameter that stands for the unit in the autograd graph``."""
    out = {}
    for mod in model.modules():
        for attr, unit_attr in (("flat", "unit"), ("embed_flat", "embed_unit"), ("norm_flat", "norm_unit"), ("head_flat", "head_unit")):
            if hasattr(mod, attr) and hasattr(mod, unit_attr):
                out[getattr(mod, unit_attr).name] = getattr(mod, attr)
    return out
