"""Collectives on CPU tensors over a :class:`~ferrotorch_b200.distributed.backend.Backend`.

Semantics follow the reference (ferrotorch-distributed/src/collective.rs): every function returns a new tensor;
``allreduce`` with ``Mean`` sums in rank order and then divides by the world size, so all ranks hold identical bits;
``all_gather`` concatenates on dim 0 (a 0-d input yields ``[world]``); ``reduce_scatter`` needs ``shape[0] % world == 0``;
world size 1 is the identity; zero-size tensors return a correctly shaped empty result. Every call has a timeout
(default 60 s) after which :class:`~ferrotorch_b200.errors.Timeout` is raised.
"""
from __future__ import annotations

import ctypes
import enum
import threading
from typing import List, Optional, Sequence

import torch

from .. import errors
from .backend import Backend, raise_for, rt, _ms

DEFAULT_COLLECTIVE_TIMEOUT = 60.0


class ReduceOp(enum.IntEnum):
    Sum = 0
    Mean = 1
    Max = 2
    Min = 3
    Prod = 4


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.float64:
        return 1
    raise errors.DtypeMismatch("float32 or float64", str(t.dtype))


def _cpu_contig(t: torch.Tensor) -> torch.Tensor:
    if t.is_cuda:
        raise errors.DeviceMismatch("cpu", str(t.device))
    return t.detach().contiguous()


def allreduce(tensor: torch.Tensor, backend: Backend, op: ReduceOp = ReduceOp.Sum, timeout: Optional[float] = DEFAULT_COLLECTIVE_TIMEOUT,
              algorithm: str = "star") -> torch.Tensor:
    """Reduce ``tensor`` across ranks. ``algorithm``: "star" (through rank 0) or "ring" (needs a full-mesh/simulated backend)."""
    orig_dtype = tensor.dtype
    work = _cpu_contig(tensor).clone()
    if work.dtype not in (torch.float32, torch.float64):
        work = work.to(torch.float32)
    if work.numel():
        raise_for(rt().ft_allreduce(backend._h, work.data_ptr(), work.numel(), _dtype_code(work), int(op), 1 if algorithm == "ring" else 0,
                                    _ms(timeout)), "allreduce", timeout)
    return work.to(orig_dtype)


def allreduce_with_timeout(tensor, backend, op, timeout):
    return allreduce(tensor, backend, op, timeout)


def broadcast(tensor: torch.Tensor, backend: Backend, root: int = 0, timeout: Optional[float] = DEFAULT_COLLECTIVE_TIMEOUT,
              algorithm: str = "star") -> torch.Tensor:
    if not 0 <= root < backend.world_size():
        raise errors.InvalidRank(f"root {root} out of range for world {backend.world_size()}")
    work = _cpu_contig(tensor).clone()
    nbytes = work.numel() * work.element_size()
    if nbytes:
        raise_for(rt().ft_broadcast(backend._h, work.data_ptr(), nbytes, root, 1 if algorithm == "tree" else 0, _ms(timeout)), "broadcast", timeout)
    return work


def all_gather(tensor: torch.Tensor, backend: Backend, timeout: Optional[float] = DEFAULT_COLLECTIVE_TIMEOUT) -> torch.Tensor:
    w = backend.world_size()
    mine = _cpu_contig(tensor)
    shape = (w,) if mine.dim() == 0 else (mine.shape[0] * w, *mine.shape[1:])
    out = torch.empty(shape, dtype=mine.dtype)
    nbytes = mine.numel() * mine.element_size()
    if nbytes:
        raise_for(rt().ft_all_gather(backend._h, mine.data_ptr(), nbytes, out.data_ptr(), _ms(timeout)), "all_gather", timeout)
    return out


def all_gather_with_timeout(tensor, backend, timeout):
    return all_gather(tensor, backend, timeout)


def reduce_scatter(tensor: torch.Tensor, backend: Backend, op: ReduceOp = ReduceOp.Sum,
                   timeout: Optional[float] = DEFAULT_COLLECTIVE_TIMEOUT) -> torch.Tensor:
    w = backend.world_size()
    full = _cpu_contig(tensor)
    if full.dim() == 0 or full.shape[0] % w or full.numel() % w:
        raise errors.ShapeMismatch(f"reduce_scatter needs shape[0] divisible by world size {w}, got {tuple(full.shape)}")
    out_shape = (full.shape[0] // w, *full.shape[1:])
    work = full if full.dtype in (torch.float32, torch.float64) else full.to(torch.float32)
    out = torch.empty(out_shape, dtype=work.dtype)
    if work.numel():
        raise_for(rt().ft_reduce_scatter(backend._h, work.data_ptr(), work.numel() // w, out.data_ptr(), _dtype_code(work), int(op),
                                         _ms(timeout)), "reduce_scatter", timeout)
    return out.to(tensor.dtype)


reduce_scatter_tensor = reduce_scatter


def reduce_scatter_with_timeout(tensor, backend, op, timeout):
    return reduce_scatter(tensor, backend, op, timeout)


def all_to_all(tensor: torch.Tensor, backend: Backend, timeout: Optional[float] = DEFAULT_COLLECTIVE_TIMEOUT) -> torch.Tensor:
    """Rank r sends chunk p of its tensor (split evenly on dim 0) to rank p and receives chunk r of every rank."""
    w = backend.world_size()
    src = _cpu_contig(tensor)
    if src.dim() == 0 or src.shape[0] % w:
        raise errors.ShapeMismatch(f"all_to_all needs shape[0] divisible by world size {w}")
    per = src.numel() // w * src.element_size()
    counts = (ctypes.c_int64 * w)(*([per] * w))
    out = torch.empty_like(src)
    if src.numel():
        raise_for(rt().ft_all_to_all(backend._h, src.data_ptr(), counts, out.data_ptr(), counts, _ms(timeout)), "all_to_all", timeout)
    return out


def all_to_all_with_timeout(tensor, backend, timeout):
    return all_to_all(tensor, backend, timeout)


def all_to_all_single_uneven(tensor: torch.Tensor, send_splits: Sequence[int], recv_splits: Sequence[int], backend: Backend,
                             timeout: Optional[float] = DEFAULT_COLLECTIVE_TIMEOUT) -> torch.Tensor:
    """Uneven all-to-all on dim 0: ``send_splits[p]`` rows go to rank p, ``recv_splits[p]`` rows arrive from rank p."""
    w = backend.world_size()
    src = _cpu_contig(tensor)
    if len(send_splits) != w or len(recv_splits) != w or sum(send_splits) != (src.shape[0] if src.dim() else 0):
        raise errors.ShapeMismatch("split sizes do not match the tensor / world size")
    row = (src.numel() // max(src.shape[0], 1)) * src.element_size() if src.dim() and src.shape[0] else src.element_size()
    sc = (ctypes.c_int64 * w)(*[s * row for s in send_splits])
    rc = (ctypes.c_int64 * w)(*[s * row for s in recv_splits])
    out = torch.empty((sum(recv_splits), *src.shape[1:]), dtype=src.dtype)
    raise_for(rt().ft_all_to_all(backend._h, src.data_ptr(), sc, out.data_ptr(), rc, _ms(timeout)), "all_to_all_single_uneven", timeout)
    return out


def barrier(backend: Backend, timeout: Optional[float] = DEFAULT_COLLECTIVE_TIMEOUT) -> None:
    backend.barrier(timeout)


# -- typed point-to-point (ferrotorch-distributed/src/p2p.rs:19-150) ---------------------------------------------------
def send(tensor: torch.Tensor, dst: int, backend: Backend) -> None:
    t = _cpu_contig(tensor)
    backend.send_ptr(t.data_ptr(), t.numel() * t.element_size(), dst)


def recv(shape, dtype: torch.dtype, src: int, backend: Backend, timeout: Optional[float] = DEFAULT_COLLECTIVE_TIMEOUT) -> torch.Tensor:
    out = torch.empty(tuple(shape), dtype=dtype)
    backend.recv_ptr(out.data_ptr(), out.numel() * out.element_size(), src, timeout)
    return out


def sendrecv(tensor: torch.Tensor, dst: int, src: int, backend: Backend, timeout: Optional[float] = DEFAULT_COLLECTIVE_TIMEOUT) -> torch.Tensor:
    """Send to ``dst`` and receive a same-shaped tensor from ``src``; the lower rank of a pair sends first."""
    if backend.rank() < dst:
        send(tensor, dst, backend)
        return recv(tensor.shape, tensor.dtype, src, backend, timeout)
    out = recv(tensor.shape, tensor.dtype, src, backend, timeout)
    send(tensor, dst, backend)
    return out


# -- async handles (ferrotorch-distributed/src/async_collective.rs:16-133) ----------------------------------------------
_turns_lock = threading.Lock()


def _turn_state(backend):
    """[tickets issued, tickets served, condition] of a backend, kept on the backend object."""
    with _turns_lock:
        st = getattr(backend, "_async_turns", None)
        if st is None:
            st = [0, 0, threading.Condition()]
            backend._async_turns = st
        return st


class PendingCollective:
    """A collective running on a background thread; ``wait()`` returns its result or re-raises its error.

    The channels of a backend are untagged, so two collectives must not interleave on one rank. Each handle takes a ticket from its backend
    when it is created (in the caller's thread, that is in program order) and its thread runs the collective when the ticket comes up:
    several handles may be outstanding at once, and they execute in the order they were issued, the same on every rank."""

    def __init__(self, fn, *args, _backend=None, **kwargs):
        self._result, self._error = None, None
        st = _turn_state(_backend) if _backend is not None else None
        if st is not None:
            with st[2]:
                ticket = st[0]
                st[0] += 1

        def run():
            if st is not None:
                with st[2]:
                    st[2].wait_for(lambda: st[1] == ticket)
            try:
                self._result = fn(*args, **kwargs)
            except BaseException as e:  # converted to an error for the waiter, as thread panics are in the reference
                self._error = e
            finally:
                if st is not None:
                    with st[2]:
                        st[1] += 1
                        st[2].notify_all()
        self._t = threading.Thread(target=run, daemon=True)
        self._t.start()

    def is_done(self) -> bool:
        return not self._t.is_alive()

    def wait(self, timeout: Optional[float] = None):
        self._t.join(timeout)
        if self._t.is_alive():
            raise errors.Timeout(timeout)
        if self._error is not None:
            if isinstance(self._error, errors.FerrotorchError):
                raise self._error
            raise errors.WorkerPanic(f"collective thread failed: {self._error!r}")
        return self._result


def async_all_gather(tensor, backend, timeout=DEFAULT_COLLECTIVE_TIMEOUT) -> PendingCollective:
    return PendingCollective(all_gather, tensor, backend, timeout, _backend=backend)


def async_reduce_scatter(tensor, backend, op=ReduceOp.Sum, timeout=DEFAULT_COLLECTIVE_TIMEOUT) -> PendingCollective:
    return PendingCollective(reduce_scatter, tensor, backend, op, timeout, _backend=backend)


def async_allreduce(tensor, backend, op=ReduceOp.Sum, timeout=DEFAULT_COLLECTIVE_TIMEOUT) -> PendingCollective:
    return PendingCollective(allreduce, tensor, backend, op, timeout, _backend=backend)
