"""Point-to-point backends over the C++ runtime (``libft_runtime.so``).

``TcpBackend`` (star or full mesh), ``SimulatedBackend`` (in-process fabric for thread ranks) and ``SubBackend``
(sub-group view) expose byte-level ``send`` / ``recv`` / ``recv_timeout`` / ``barrier``; the collectives of
:mod:`ferrotorch_b200.distributed.collective` are layered on top. Error codes from the runtime are raised as the
typed exceptions of :mod:`ferrotorch_b200.errors`.

Reference parity: ``Backend`` trait, ``TcpBackend``, ``SimulatedBackend``, ``SubBackend``
(ferrotorch-distributed/src/backend.rs:29-753).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

from .. import _lib, errors

_c = ctypes
_rt = None


def rt():
    global _rt
    if _rt is None:
        lib = _lib.runtime()
        i64, vp, ci = _c.c_int64, _c.c_void_p, _c.c_int
        lib.ft_tcp_backend_create.restype = i64
        lib.ft_tcp_backend_create.argtypes = [ci, ci, _c.c_char_p, ci, ci, i64, _c.POINTER(ci)]
        lib.ft_sim_fabric_create.restype = i64
        lib.ft_sim_fabric_create.argtypes = [ci]
        lib.ft_sim_backend_create.restype = i64
        lib.ft_sim_backend_create.argtypes = [i64, ci]
        lib.ft_sub_backend_create.restype = i64
        lib.ft_sub_backend_create.argtypes = [i64, _c.POINTER(ci), ci]
        lib.ft_backend_destroy.restype = None
        lib.ft_backend_destroy.argtypes = [i64]
        lib.ft_backend_rank.argtypes = [i64]
        lib.ft_backend_world.argtypes = [i64]
        lib.ft_backend_send.argtypes = [i64, vp, i64, ci]
        lib.ft_backend_recv.argtypes = [i64, vp, i64, ci, i64]
        lib.ft_backend_barrier.argtypes = [i64, i64]
        lib.ft_backend_set_fault.argtypes = [i64, ci, i64]
        lib.ft_allreduce.argtypes = [i64, vp, i64, ci, ci, ci, i64]
        lib.ft_broadcast.argtypes = [i64, vp, i64, ci, ci, i64]
        lib.ft_all_gather.argtypes = [i64, vp, i64, vp, i64]
        lib.ft_reduce_scatter.argtypes = [i64, vp, i64, vp, ci, ci, i64]
        lib.ft_all_to_all.argtypes = [i64, vp, _c.POINTER(i64), vp, _c.POINTER(i64), i64]
        lib.ft_ddp_plan_buckets.argtypes = [_c.POINTER(i64), ci, ci, i64, _c.POINTER(ci)]
        _rt = lib
    return _rt


_ERRS = {1: errors.InvalidWorldSize, 2: errors.InvalidRank, 3: errors.SelfSend, 4: errors.SizeMismatch, 5: errors.IoError,
         6: errors.LockPoisoned, 7: errors.ChannelClosed, 8: errors.UnsupportedOp, 10: errors.NoConnection,
         11: errors.BackendUnavailable, 12: errors.InvalidArgument}


def raise_for(code: int, what: str, timeout_s: Optional[float] = None) -> None:
    if code == 0:
        return
    if code == 9:
        raise errors.Timeout(timeout_s, f"{what}: timed out after {timeout_s} s")
    cls = _ERRS.get(code, errors.DistributedError)
    raise cls(f"{what}: runtime error {code} ({cls.__name__})")


def _ms(timeout) -> int:
    return -1 if timeout is None else max(0, int(float(timeout) * 1000))


FAULT_NONE, FAULT_DROP_NEXT_SEND, FAULT_DELAY_SEND_MS, FAULT_CORRUPT_LENGTH, FAULT_CLOSE = range(5)


class Backend:
    """Byte-level point-to-point transport between the ranks of a group."""

    def __init__(self, handle: int):
        if not handle:
            raise errors.BackendUnavailable("backend creation failed")
        self._h = handle

    def rank(self) -> int:
        return rt().ft_backend_rank(self._h)

    def world_size(self) -> int:
        return rt().ft_backend_world(self._h)

    def send(self, data: bytes, dst: int) -> None:
        buf = (_c.c_char * len(data)).from_buffer_copy(data) if len(data) else None
        raise_for(rt().ft_backend_send(self._h, buf, len(data), dst), f"send to rank {dst}")

    def send_ptr(self, ptr: int, nbytes: int, dst: int) -> None:
        raise_for(rt().ft_backend_send(self._h, ptr, nbytes, dst), f"send to rank {dst}")

    def recv(self, nbytes: int, src: int) -> bytes:
        return self.recv_timeout(nbytes, src, None)

    def recv_timeout(self, nbytes: int, src: int, timeout: Optional[float]) -> bytes:
        buf = (_c.c_char * max(nbytes, 1))()
        raise_for(rt().ft_backend_recv(self._h, buf, nbytes, src, _ms(timeout)), f"recv from rank {src}", timeout)
        return bytes(buf[:nbytes])

    def recv_ptr(self, ptr: int, nbytes: int, src: int, timeout: Optional[float] = None) -> None:
        raise_for(rt().ft_backend_recv(self._h, ptr, nbytes, src, _ms(timeout)), f"recv from rank {src}", timeout)

    def barrier(self, timeout: Optional[float] = 60.0) -> None:
        raise_for(rt().ft_backend_barrier(self._h, _ms(timeout)), "barrier", timeout)

    def inject_fault(self, kind: int, param: int = 0) -> None:
        """Host-side fault injection for failure-detection tests: drop / delay / corrupt the next send, or close the links."""
        raise_for(rt().ft_backend_set_fault(self._h, kind, param), "inject_fault")

    def as_nccl_backend(self):
        return None

    def close(self) -> None:
        if self._h:
            rt().ft_backend_destroy(self._h)
            self._h = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class TcpBackend(Backend):
    """TCP transport. ``address`` is ``"host:port"`` of rank 0 (star) or the base port of the mesh (``full_mesh=True``)."""

    def __init__(self, rank: int, world_size: int, address: str = "127.0.0.1:29500", full_mesh: bool = False, connect_timeout: float = 30.0):
        host, _, port = address.rpartition(":")
        err = _c.c_int(0)
        h = rt().ft_tcp_backend_create(rank, world_size, (host or "127.0.0.1").encode(), int(port), int(full_mesh), _ms(connect_timeout),
                                       _c.byref(err))
        if not h:
            raise_for(err.value or 11, f"TcpBackend(rank={rank}, world={world_size}, {address})", connect_timeout)
        super().__init__(h)

    @classmethod
    def from_env(cls, full_mesh: bool = False) -> "TcpBackend":
        import os
        return cls(int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]),
                   f'{os.environ.get("MASTER_ADDR", "127.0.0.1")}:{os.environ.get("MASTER_PORT", "29500")}', full_mesh)


class SimulatedBackend(Backend):
    """Rank view of an in-process fabric: ``SimulatedBackend.create_group(n)`` returns one backend per thread rank."""

    def __init__(self, fabric: int, rank: int, _keep=None):
        super().__init__(rt().ft_sim_backend_create(fabric, rank))
        self._fabric_keep = _keep

    @staticmethod
    def create_group(world_size: int) -> List["SimulatedBackend"]:
        if world_size < 1:
            raise errors.InvalidWorldSize(f"world size {world_size}")
        fab = rt().ft_sim_fabric_create(world_size)

        class _Fabric:
            def __init__(self, h):
                self.h = h

            def __del__(self):
                try:
                    rt().ft_backend_destroy(self.h)
                except Exception:
                    pass
        keep = _Fabric(fab)
        return [SimulatedBackend(fab, r, keep) for r in range(world_size)]


class SubBackend(Backend):
    """View of ``parent`` restricted to ``members`` (global ranks); ranks are renumbered 0..len-1 in the given order."""

    def __init__(self, parent: Backend, members: Sequence[int]):
        arr = (_c.c_int * len(members))(*members)
        h = rt().ft_sub_backend_create(parent._h, arr, len(members))
        if not h:
            raise errors.InvalidRank(f"rank {parent.rank()} is not a member of {list(members)} (or a member is out of range)")
        super().__init__(h)
        self._parent = parent
        self.members = list(members)
