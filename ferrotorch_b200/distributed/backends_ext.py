"""Process-group backends over ``torch.distributed`` (NCCL, gloo, MPI, UCC), the CPU + GPU hybrid, device-buffer collectives, bounded
point-to-point receives, the RPC byte transport and the distributed-checkpoint object.

The framework's own transports are :class:`TcpBackend` (host control plane, C++) and the peer-memory kernels of ``ferrotorch_b200.parallel``
(device data plane). The classes here give the same :class:`Backend` surface to a library process group, so code written against a backend
handle runs on whichever transport a deployment has; the device collectives run in place on CUDA tensors and never stage through the host
when the backend is NCCL.

Reference parity: ferrotorch-distributed/src/{nccl_backend.rs:45, nccl_sys.rs:39 (NcclUniqueId), nccl_collective.rs:75-260, gloo_backend.rs:52-78,
mpi_backend.rs:144-173, ucc_backend.rs, hybrid_backend.rs:39, gpu_collective.rs:276-400, p2p.rs:53-130, rpc.rs:45-330 (RpcError, TcpRpcBackend),
checkpoint.rs:35-130, 889-915}.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Optional, Sequence

import torch

from .. import errors
from ..errors import BackendUnavailable, FerrotorchError, InvalidArgument
from .backend import Backend
from .collective import DEFAULT_COLLECTIVE_TIMEOUT, ReduceOp, allreduce, broadcast
from .extras import MAX_RPC_BYTES, ShardMetadata, TensorShardSpec, load_distributed, save_distributed


def is_nccl_available() -> bool:
    import torch.distributed as dist
    return dist.is_available() and dist.is_nccl_available() and torch.cuda.is_available()


def is_gloo_available() -> bool:
    import torch.distributed as dist
    return dist.is_available() and dist.is_gloo_available()


def is_mpi_available() -> bool:
    import torch.distributed as dist
    return dist.is_available() and dist.is_mpi_available()


def is_ucc_available() -> bool:
    import torch.distributed as dist
    return dist.is_available() and getattr(dist, "is_ucc_available", lambda: False)()


@dataclass(frozen=True)
class NcclUniqueId:
    """The 128-byte rendezvous token every rank of an NCCL communicator must share (nccl_sys.rs:39). Rank 0 makes one with :meth:`generate`
    and hands ``to_bytes()`` to the others over any side channel (a :class:`TcpBackend` broadcast, a file, the launcher's store)."""
    internal: bytes

    def __post_init__(self):
        if len(self.internal) != 128:
            raise InvalidArgument(f"NcclUniqueId: expected 128 bytes, got {len(self.internal)}")

    @classmethod
    def generate(cls) -> "NcclUniqueId":
        if not is_nccl_available():
            raise BackendUnavailable("NCCL is not available in this process (no CUDA device or a torch build without NCCL)")
        from torch.cuda import nccl
        return cls(bytes(nccl.unique_id()))

    @classmethod
    def from_bytes(cls, b: bytes) -> "NcclUniqueId":
        return cls(bytes(b))

    def to_bytes(self) -> bytes:
        return self.internal


_TORCH_OP = None


def _torch_op(op: ReduceOp):
    import torch.distributed as dist
    global _TORCH_OP
    if _TORCH_OP is None:
        _TORCH_OP = {"sum": dist.ReduceOp.SUM, "mean": dist.ReduceOp.AVG, "avg": dist.ReduceOp.AVG, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN,
                     "product": dist.ReduceOp.PRODUCT, "prod": dist.ReduceOp.PRODUCT}
    name = getattr(op, "name", str(op)).lower()
    if name not in _TORCH_OP:
        raise errors.UnsupportedOp(f"reduce op {op} is not supported by this backend")
    return _TORCH_OP[name]


class _ProcessGroupBackend(Backend):
    """:class:`Backend` over one ``torch.distributed`` process group. Byte sends and receives go through uint8 tensors on the group's device;
    the tensor collectives (``allreduce_`` ...) run directly on the caller's tensors."""
    kind = "gloo"
    device = "cpu"

    def __init__(self, rank: Optional[int] = None, world_size: Optional[int] = None, init_method: Optional[str] = None, group=None,
                 timeout: float = DEFAULT_COLLECTIVE_TIMEOUT or 60.0):
        import torch.distributed as dist
        self._check_available()
        self._own = False
        if group is None and not dist.is_initialized():
            rank = int(os.environ.get("RANK", 0)) if rank is None else rank
            world_size = int(os.environ.get("WORLD_SIZE", 1)) if world_size is None else world_size
            if init_method is None:
                os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
                os.environ.setdefault("MASTER_PORT", "29500")
                init_method = "env://"
            try:
                dist.init_process_group(self.kind, init_method=init_method, rank=rank, world_size=world_size, timeout=datetime.timedelta(seconds=timeout))
            except Exception as e:
                raise BackendUnavailable(f"{type(self).__name__}: process-group rendezvous failed: {e}") from None
            self._own = True
        elif group is None and dist.get_backend() != self.kind and self.kind not in str(dist.get_backend()):
            group = dist.new_group(backend=self.kind, timeout=datetime.timedelta(seconds=timeout))
        self.group = group
        self._h = 1                                           # no native handle: the base class' close() must not call the C runtime
        self._rank, self._world = dist.get_rank(group), dist.get_world_size(group)

    @classmethod
    def _check_available(cls) -> None:
        ok = {"gloo": is_gloo_available, "nccl": is_nccl_available, "mpi": is_mpi_available, "ucc": is_ucc_available}[cls.kind]()
        if not ok:
            raise BackendUnavailable(f"the {cls.kind} backend is not available in this build / on this machine")

    def rank(self) -> int:
        return self._rank

    def world_size(self) -> int:
        return self._world

    def _peer(self, r: int, what: str) -> int:
        import torch.distributed as dist
        if not 0 <= r < self._world:
            raise errors.InvalidRank(f"{what}: rank {r} out of range for world size {self._world}")
        if r == self._rank:
            raise errors.SelfSend(f"{what}: rank {r} is this rank")
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def _wrap(self, fn, what: str):
        try:
            return fn()
        except FerrotorchError:
            raise
        except Exception as e:
            msg = str(e)
            if "timeout" in msg.lower() or "timed out" in msg.lower():
                raise errors.Timeout(f"{what} timed out: {msg}") from None
            raise errors.IoError(f"{what} failed: {msg}") from None

    def send(self, data: bytes, dst: int) -> None:
        import torch.distributed as dist
        t = torch.frombuffer(bytearray(data), dtype=torch.uint8).to(self.device) if len(data) else torch.empty(0, dtype=torch.uint8, device=self.device)
        d = self._peer(dst, "send")
        if len(data):
            self._wrap(lambda: dist.send(t, d, group=self.group), f"send to rank {dst}")

    def recv_timeout(self, nbytes: int, src: int, timeout: Optional[float]) -> bytes:
        import torch.distributed as dist
        s = self._peer(src, "recv")
        if nbytes == 0:
            return b""
        t = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self._wait(dist.irecv(t, s, group=self.group), timeout, f"recv from rank {src}")
        return t.cpu().numpy().tobytes()

    def _wait(self, work, timeout: Optional[float], what: str) -> None:
        def go():
            if timeout is None:
                work.wait()
            elif not work.wait(datetime.timedelta(seconds=timeout)):
                raise errors.Timeout(f"{what} timed out after {timeout} s")
        self._wrap(go, what)

    def send_ptr(self, ptr: int, nbytes: int, dst: int) -> None:
        import ctypes
        self.send(ctypes.string_at(ptr, nbytes), dst)

    def recv_ptr(self, ptr: int, nbytes: int, src: int, timeout: Optional[float] = None) -> None:
        import ctypes
        ctypes.memmove(ptr, self.recv_timeout(nbytes, src, timeout), nbytes)

    def send_tensor(self, t: torch.Tensor, dst: int) -> None:
        import torch.distributed as dist
        self._wrap(lambda: dist.send(t.contiguous().to(self.device), self._peer(dst, "send"), group=self.group), f"send to rank {dst}")

    def recv_tensor_(self, out: torch.Tensor, src: int, timeout: Optional[float] = None) -> torch.Tensor:
        import torch.distributed as dist
        buf = out if out.is_contiguous() and out.device.type == self.device else torch.empty(out.shape, dtype=out.dtype, device=self.device)
        self._wait(dist.irecv(buf, self._peer(src, "recv"), group=self.group), timeout, f"recv from rank {src}")
        if buf is not out:
            out.copy_(buf)
        return out

    def barrier(self, timeout: Optional[float] = 60.0) -> None:
        import torch.distributed as dist
        self._wait(dist.barrier(group=self.group, async_op=True), timeout, "barrier")

    # -- tensor collectives, in place ------------------------------------------------------------------------------------
    def allreduce_(self, t: torch.Tensor, op: ReduceOp = ReduceOp.Sum) -> torch.Tensor:
        import torch.distributed as dist
        self._wrap(lambda: dist.all_reduce(t, _torch_op(op), group=self.group), "allreduce")
        return t

    def broadcast_(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        import torch.distributed as dist
        if not 0 <= root < self._world:
            raise errors.InvalidRank(f"broadcast: root {root} out of range for world size {self._world}")
        src = dist.get_global_rank(self.group, root) if self.group is not None else root
        self._wrap(lambda: dist.broadcast(t, src, group=self.group), "broadcast")
        return t

    def all_gather_into(self, out: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        if out.numel() != t.numel() * self._world:
            raise errors.SizeMismatch(f"all_gather: output has {out.numel()} elements, expected {t.numel() * self._world}")
        self._wrap(lambda: dist.all_gather_into_tensor(out, t.contiguous(), group=self.group), "all_gather")
        return out

    def reduce_scatter_into(self, out: torch.Tensor, t: torch.Tensor, op: ReduceOp = ReduceOp.Sum) -> torch.Tensor:
        import torch.distributed as dist
        if t.numel() != out.numel() * self._world:
            raise errors.SizeMismatch(f"reduce_scatter: input has {t.numel()} elements, expected {out.numel() * self._world}")
        self._wrap(lambda: dist.reduce_scatter_tensor(out, t.contiguous(), _torch_op(op), group=self.group), "reduce_scatter")
        return out

    def inject_fault(self, kind: int, param: int = 0) -> None:
        raise errors.UnsupportedOp("fault injection exists on the TCP and simulated backends only")

    def close(self) -> None:
        import torch.distributed as dist
        if getattr(self, "_own", False) and dist.is_initialized():
            dist.destroy_process_group()
        self._own, self._h = False, 0


class GlooBackend(_ProcessGroupBackend):
    """CPU collectives over gloo (gloo_backend.rs:68)."""
    kind, device = "gloo", "cpu"


class MpiBackend(_ProcessGroupBackend):
    """MPI process group; constructing one without MPI support raises :class:`BackendUnavailable` (mpi_backend.rs:163)."""
    kind, device = "mpi", "cpu"


class UccBackend(_ProcessGroupBackend):
    """UCC process group (ucc_backend.rs); unavailable builds raise :class:`BackendUnavailable`."""
    kind, device = "ucc", "cpu"


class NcclBackend(_ProcessGroupBackend):
    """Device collectives over NCCL: every operation takes CUDA tensors and runs on the current stream without touching the host
    (nccl_backend.rs:45). ``torch.cuda.set_device`` must have been called with this rank's GPU."""
    kind, device = "nccl", "cuda"

    def as_nccl_backend(self):
        return self

    def _dev(self, t: torch.Tensor, what: str) -> None:
        if not t.is_cuda:
            raise InvalidArgument(f"{what}: NCCL operates on CUDA tensors, got a {t.device.type} tensor")

    def allreduce_(self, t, op=ReduceOp.Sum):
        self._dev(t, "allreduce")
        return super().allreduce_(t, op)

    def broadcast_(self, t, root=0):
        self._dev(t, "broadcast")
        return super().broadcast_(t, root)


class HybridBackend(Backend):
    """Host bytes and CPU tensors over a TCP (or any CPU) backend, CUDA tensors over NCCL (hybrid_backend.rs:39)."""

    def __init__(self, cpu: Backend, nccl: NcclBackend):
        if cpu.rank() != nccl.rank() or cpu.world_size() != nccl.world_size():
            raise InvalidArgument(f"HybridBackend: rank / world size differ (cpu {cpu.rank()}/{cpu.world_size()}, nccl {nccl.rank()}/{nccl.world_size()})")
        self.cpu, self.nccl, self._h = cpu, nccl, 1

    def rank(self): return self.cpu.rank()                                            # noqa: E704
    def world_size(self): return self.cpu.world_size()                                # noqa: E704
    def send(self, data, dst): return self.cpu.send(data, dst)                        # noqa: E704
    def send_ptr(self, ptr, nbytes, dst): return self.cpu.send_ptr(ptr, nbytes, dst)  # noqa: E704
    def recv_timeout(self, nbytes, src, timeout): return self.cpu.recv_timeout(nbytes, src, timeout)                 # noqa: E704
    def recv_ptr(self, ptr, nbytes, src, timeout=None): return self.cpu.recv_ptr(ptr, nbytes, src, timeout)          # noqa: E704
    def barrier(self, timeout=60.0): return self.cpu.barrier(timeout)                 # noqa: E704
    def inject_fault(self, kind, param=0): return self.cpu.inject_fault(kind, param)  # noqa: E704
    def as_nccl_backend(self): return self.nccl                                       # noqa: E704

    def close(self) -> None:
        self.cpu.close()
        self.nccl.close()
        self._h = 0


# -- device-buffer collectives --------------------------------------------------------------------------------------------
def _nccl_of(backend: Backend, what: str) -> NcclBackend:
    n = backend.as_nccl_backend()
    if n is None:
        raise InvalidArgument(f"{what} needs an NcclBackend (or a HybridBackend), got {type(backend).__name__}")
    return n


def nccl_allreduce(buffer: torch.Tensor, backend: Backend, op: ReduceOp = ReduceOp.Sum) -> None:
    """In-place all-reduce of a CUDA tensor (nccl_collective.rs:75)."""
    _nccl_of(backend, "nccl_allreduce").allreduce_(buffer, op)


def nccl_broadcast(buffer: torch.Tensor, backend: Backend, root: int) -> None:
    _nccl_of(backend, "nccl_broadcast").broadcast_(buffer, root)


def nccl_all_gather(send_buf: torch.Tensor, recv_buf: torch.Tensor, backend: Backend) -> None:
    _nccl_of(backend, "nccl_all_gather").all_gather_into(recv_buf, send_buf)


def nccl_reduce_scatter(send_buf: torch.Tensor, recv_buf: torch.Tensor, backend: Backend, op: ReduceOp = ReduceOp.Sum) -> None:
    _nccl_of(backend, "nccl_reduce_scatter").reduce_scatter_into(recv_buf, send_buf, op)


def gpu_allreduce(tensor: torch.Tensor, backend: Backend, op: ReduceOp = ReduceOp.Sum) -> torch.Tensor:
    """All-reduce of a device tensor, returning a new tensor on the same device: NCCL when the backend has it, otherwise one staged round
    trip through the host over the backend's own all-reduce (gpu_collective.rs:276)."""
    n = backend.as_nccl_backend()
    if n is not None and tensor.is_cuda:
        return n.allreduce_(tensor.clone(), op)
    if isinstance(backend, _ProcessGroupBackend):
        return backend.allreduce_(tensor.detach().cpu().clone(), op).to(tensor.device)
    return allreduce(tensor.detach().cpu(), backend, op).to(tensor.device)


def gpu_broadcast(tensor: torch.Tensor, backend: Backend, root: int = 0) -> torch.Tensor:
    n = backend.as_nccl_backend()
    if n is not None and tensor.is_cuda:
        return n.broadcast_(tensor.clone(), root)
    if isinstance(backend, _ProcessGroupBackend):
        return backend.broadcast_(tensor.detach().cpu().clone(), root).to(tensor.device)
    return broadcast(tensor.detach().cpu(), backend, root).to(tensor.device)


# -- bounded point-to-point receives (p2p.rs:53-130) ------------------------------------------------------------------------
def _check_src(src: int, backend: Backend) -> None:
    if not 0 <= src < backend.world_size():
        raise errors.InvalidRank(f"recv: src_rank {src} >= world_size {backend.world_size()}")
    if src == backend.rank():
        raise errors.SelfSend(f"recv: src_rank {src} is this rank")


def recv_with_timeout(shape: Sequence[int], dtype: torch.dtype, src: int, backend: Backend, timeout: Optional[float]) -> torch.Tensor:
    out = torch.empty(tuple(shape), dtype=dtype)
    recv_into_with_timeout(out, src, backend, timeout)
    return out


def recv_into_with_timeout(out: torch.Tensor, src: int, backend: Backend, timeout: Optional[float]) -> None:
    """Receives exactly ``out.numel()`` elements from ``src`` into ``out`` (any device: device tensors are filled from a host staging copy
    unless the backend receives tensors natively); nothing is written when the deadline passes first."""
    _check_src(src, backend)
    if isinstance(backend, _ProcessGroupBackend):
        backend.recv_tensor_(out, src, timeout)
        return
    host = out if (out.device.type == "cpu" and out.is_contiguous()) else torch.empty(out.shape, dtype=out.dtype)
    backend.recv_ptr(host.data_ptr(), host.numel() * host.element_size(), src, timeout)
    if host is not out:
        out.copy_(host)


def recv_into(out: torch.Tensor, src: int, backend: Backend) -> None:
    recv_into_with_timeout(out, src, backend, DEFAULT_COLLECTIVE_TIMEOUT)


# -- RPC transport (rpc.rs:45-330) --------------------------------------------------------------------------------------------
class RpcError(InvalidArgument):
    """``kind``: function_not_found | invalid_message | no_connection | internal | timeout."""

    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind

    @classmethod
    def function_not_found(cls, name: str): return cls("function_not_found", f"RPC function not found: {name}")                    # noqa: E704
    @classmethod
    def invalid_message(cls, reason: str): return cls("invalid_message", f"invalid RPC message: {reason}")                          # noqa: E704
    @classmethod
    def no_connection(cls, rank: int): return cls("no_connection", f"no connection to rank {rank} (star topology: non-zero ranks only connect to rank 0)")  # noqa: E704
    @classmethod
    def internal(cls, msg: str): return cls("internal", f"RPC internal error: {msg}")                                               # noqa: E704
    @classmethod
    def timeout(cls): return cls("timeout", "RPC timeout")                                                                          # noqa: E704


class TcpRpcBackend:
    """Byte transport of the RPC layer over any :class:`Backend`: refuses messages above 1 GiB before allocating for them and reports a missing
    link of the star topology as ``RpcError.no_connection`` (rpc.rs:263)."""

    def __init__(self, backend: Backend):
        self.backend = backend

    def rank(self) -> int:
        return self.backend.rank()

    def world_size(self) -> int:
        return self.backend.world_size()

    def send(self, data: bytes, dst_rank: int) -> None:
        if len(data) > MAX_RPC_BYTES:
            raise RpcError.invalid_message(f"RPC message size {len(data)} exceeds maximum allowed size {MAX_RPC_BYTES} (1 GiB)")
        try:
            self.backend.send(bytes(data), dst_rank)
        except errors.NoConnection:
            raise RpcError.no_connection(dst_rank) from None

    def recv(self, nbytes: int, src_rank: int, timeout: Optional[float] = DEFAULT_COLLECTIVE_TIMEOUT) -> bytes:
        if nbytes > MAX_RPC_BYTES:
            raise RpcError.invalid_message(f"RPC message size {nbytes} exceeds maximum allowed size {MAX_RPC_BYTES} (1 GiB)")
        try:
            return self.backend.recv_timeout(nbytes, src_rank, timeout)
        except errors.NoConnection:
            raise RpcError.no_connection(src_rank) from None
        except errors.Timeout:
            raise RpcError.timeout() from None


# -- distributed checkpoint object (checkpoint.rs:35-130, 889-915) -------------------------------------------------------------------
class DistCheckpointError(InvalidArgument):
    """``kind``: io | serialization | metadata | missing_shard | tensor | invalid_argument | async_failed."""

    def __init__(self, kind: str, message: str):
        prefix = {"io": "I/O error", "serialization": "serialization error", "metadata": "metadata error", "missing_shard": "shard file missing",
                  "tensor": "tensor error", "invalid_argument": "invalid argument", "async_failed": "async checkpoint failed"}[kind]
        super().__init__(f"{prefix}: {message}")
        self.kind = kind


def flat_shard_metadata(state_dict: Dict[str, torch.Tensor], world_size: int) -> ShardMetadata:
    """Metadata of FSDP-style flat shards: every local tensor counts as a 1-D chunk of ``numel`` elements, the full tensor is
    ``numel * world_size`` long and split evenly on dimension 0."""
    if world_size < 1:
        raise DistCheckpointError("invalid_argument", "world_size must be >= 1")
    return ShardMetadata(world_size, {k: TensorShardSpec([v.numel() * world_size], 0, [v.numel()] * world_size) for k, v in state_dict.items()})


@dataclass
class DistributedCheckpoint:
    """A checkpoint directory with its shard layout: ``save`` writes this rank's shard (rank 0 also the metadata), ``load`` returns the shard
    of ``rank`` for any world size, re-splitting when it differs from the one that wrote the files."""
    checkpoint_dir: Path
    shard_metadata: ShardMetadata

    @classmethod
    def open(cls, directory) -> "DistributedCheckpoint":
        p = Path(directory) / "metadata.json"
        try:
            return cls(Path(directory), ShardMetadata.from_json(p.read_text()))
        except OSError as e:
            raise DistCheckpointError("io", f"{p}: {e}") from None
        except (ValueError, KeyError, TypeError) as e:
            raise DistCheckpointError("metadata", f"{p}: {e}") from None

    def save(self, local_state: Dict[str, torch.Tensor], rank: int) -> None:
        world = self.shard_metadata.num_ranks
        if not 0 <= rank < world:
            raise DistCheckpointError("invalid_argument", f"rank {rank} out of range for {world} ranks")
        missing = [k for k in local_state if k not in self.shard_metadata.tensor_specs]
        if missing:
            raise DistCheckpointError("metadata", f"no shard spec for {missing[:3]}")
        for k, v in local_state.items():
            spec = self.shard_metadata.tensor_specs[k]
            want = spec.shard_sizes[rank]
            got = v.numel() if len(spec.full_shape) == 1 else (v.shape[spec.shard_dim] if v.dim() else 1)
            if got != want:
                raise DistCheckpointError("tensor", f"{k}: rank {rank} holds {got} along dim {spec.shard_dim}, the spec says {want}")
        try:
            save_distributed(self.checkpoint_dir, local_state, rank, world, {k: s.shard_dim for k, s in self.shard_metadata.tensor_specs.items()})
            if rank == 0:
                (Path(self.checkpoint_dir) / "metadata.json").write_text(self.shard_metadata.to_json())
        except OSError as e:
            raise DistCheckpointError("io", str(e)) from None

    def load(self, rank: int, world_size: Optional[int] = None) -> Dict[str, torch.Tensor]:
        world = world_size or self.shard_metadata.num_ranks
        if world < 1 or not 0 <= rank < world:
            raise DistCheckpointError("invalid_argument", f"rank {rank} / world size {world}")
        for r in range(self.shard_metadata.num_ranks if world != self.shard_metadata.num_ranks else 0):
            if not (Path(self.checkpoint_dir) / f"rank_{r}.safetensors").exists():
                raise DistCheckpointError("missing_shard", str(Path(self.checkpoint_dir) / f"rank_{r}.safetensors"))
        mine = Path(self.checkpoint_dir) / f"rank_{rank}.safetensors"
        if world == self.shard_metadata.num_ranks and not mine.exists():
            raise DistCheckpointError("missing_shard", str(mine))
        try:
            return load_distributed(self.checkpoint_dir, rank, world)
        except OSError as e:
            raise DistCheckpointError("io", str(e)) from None
