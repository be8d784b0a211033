"""Device runtime: devices, buffers and transfers, the caching allocator, streams / events, CUDA graphs, the memory guard, the kernel-module
cache, the Philox generator manager, the standalone ``GpuTensor`` and the backend registration entry point.

Reference parity (all under ferrotorch-gpu/src/): device.rs:25-102, buffer.rs:36-150, transfer.rs:19-159, allocator.rs:488-682, pool.rs:33-292,
stream.rs:70-683, graph.rs:59-706, memory_guard.rs:55-1181, module_cache.rs:76,134, rng.rs:75-520, tensor_bridge.rs:71-1130,
backend_impl.rs:4275 (``init_cuda_backend``).
"""
from __future__ import annotations

import contextlib
import ctypes
import enum
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .. import _lib
from ..errors import FerrotorchError, InvalidArgument


class GpuError(FerrotorchError):
    pass


class OutOfMemory(GpuError):
    pass


# ----------------------------------------------------------------------------------------------------------------------
# device / buffers / transfers
# ----------------------------------------------------------------------------------------------------------------------
class GpuDevice:
    """One CUDA device: ordinal, its default stream and properties. ``fork_for_capture`` gives a device view bound to a fresh stream."""

    def __init__(self, ordinal: int = 0, stream: Optional[torch.cuda.Stream] = None):
        if not torch.cuda.is_available():
            raise GpuError("no CUDA device is available")
        if not 0 <= ordinal < torch.cuda.device_count():
            raise InvalidArgument(f"device ordinal {ordinal} out of range")
        self.ordinal = ordinal
        self.device = torch.device("cuda", ordinal)
        self.stream = stream or torch.cuda.default_stream(self.device)

    @property
    def name(self) -> str:
        return torch.cuda.get_device_name(self.ordinal)

    @property
    def sm_count(self) -> int:
        return torch.cuda.get_device_properties(self.ordinal).multi_processor_count

    @property
    def total_memory(self) -> int:
        return torch.cuda.get_device_properties(self.ordinal).total_memory

    def synchronize(self) -> None:
        torch.cuda.synchronize(self.device)

    def fork_for_capture(self) -> "GpuDevice":
        return GpuDevice(self.ordinal, torch.cuda.Stream(self.device))

    def mem_info(self) -> Tuple[int, int]:
        return torch.cuda.mem_get_info(self.device)


class CudaBuffer:
    """A typed 1-D device allocation. ``len`` is the logical element count, ``alloc_len`` the (possibly rounded-up) capacity."""

    def __init__(self, length: int, dtype: torch.dtype = torch.float32, device: Optional[GpuDevice] = None, zero: bool = False, pool: Optional["BufferPool"] = None):
        self.device = device or GpuDevice(torch.cuda.current_device())
        self.len, self.dtype, self._pool = length, dtype, pool
        alloc = pool.round_len(length) if pool is not None else length
        t = pool.take(alloc, dtype, self.device.device) if pool is not None else None
        self.storage = t if t is not None else torch.empty(alloc, dtype=dtype, device=self.device.device)
        self.alloc_len = self.storage.numel()
        if zero:
            self.storage[:length].zero_()

    def tensor(self) -> torch.Tensor:
        return self.storage[: self.len]

    def device_ptr(self) -> int:
        return self.storage.data_ptr()

    def release(self) -> None:
        if self._pool is not None and self.storage is not None:
            self._pool.give(self.storage)
        self.storage = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class BufferPool:
    """Cache of released buffers keyed by (dtype, rounded length); ``record_stream`` defers re-use until the stream has passed."""

    def __init__(self):
        self._free: Dict[Tuple[torch.dtype, int], List[torch.Tensor]] = {}
        self.hits = self.misses = 0

    @staticmethod
    def round_len(n: int) -> int:
        if n <= 0:
            return 0
        return 1 << (n - 1).bit_length() if n < (1 << 20) else (n + (1 << 20) - 1) // (1 << 20) * (1 << 20)

    def take(self, n: int, dtype, device) -> Optional[torch.Tensor]:
        lst = self._free.get((dtype, n))
        if lst:
            self.hits += 1
            return lst.pop()
        self.misses += 1
        return None

    def give(self, t: torch.Tensor) -> None:
        self._free.setdefault((t.dtype, t.numel()), []).append(t)

    def record_stream(self, t: torch.Tensor, stream: torch.cuda.Stream) -> None:
        t.record_stream(stream)

    def stats(self) -> Dict[str, int]:
        return {"hits": self.hits, "misses": self.misses, "cached": sum(len(v) for v in self._free.values()),
                "cached_bytes": sum(t.numel() * t.element_size() for v in self._free.values() for t in v)}

    def clear(self) -> None:
        self._free.clear()


def cpu_to_gpu(t: torch.Tensor, device: Optional[GpuDevice] = None, non_blocking: bool = False) -> torch.Tensor:
    dev = (device or GpuDevice(torch.cuda.current_device())).device
    return t.to(dev, non_blocking=non_blocking)


def cpu_to_gpu_pinned(t: torch.Tensor, device: Optional[GpuDevice] = None) -> torch.Tensor:
    """Host-to-device copy through page-locked memory on the current stream (asynchronous with respect to the host)."""
    dev = (device or GpuDevice(torch.cuda.current_device())).device
    src = t if t.is_pinned() else t.pin_memory()
    return src.to(dev, non_blocking=True)


def gpu_to_cpu(t: torch.Tensor, pinned: bool = False) -> torch.Tensor:
    if not pinned:
        return t.cpu()
    out = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
    out.copy_(t, non_blocking=True)
    torch.cuda.current_stream(t.device).synchronize()
    return out


def alloc_zeros(n: int, dtype=torch.float32, device: Optional[GpuDevice] = None, pool: Optional[BufferPool] = None) -> CudaBuffer:
    return CudaBuffer(n, dtype, device, zero=True, pool=pool)


# ----------------------------------------------------------------------------------------------------------------------
# caching allocator (native)
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class AllocatorStats:
    allocated: int
    reserved: int
    peak_allocated: int
    peak_reserved: int
    num_allocs: int
    num_frees: int
    num_segment_allocs: int
    num_cache_hits: int
    num_ooms: int
    live_blocks: int


class CudaAllocator:
    """The native split/coalesce caching allocator. ``host_mode=True`` backs segments with the host heap (logic tests without a GPU)."""

    def __init__(self, host_mode: bool = False, _handle: Optional[int] = None):
        self._own = _handle is None
        if _handle is None:
            h = ctypes.c_void_p()
            _lib.call("ft_alloc_create", int(host_mode), ctypes.addressof(h))
            _handle = h.value
        self._h = _handle

    def malloc(self, nbytes: int, stream: int = 0) -> int:
        out = ctypes.c_void_p()
        try:
            _lib.call("ft_alloc_malloc", self._h, int(nbytes), stream, ctypes.addressof(out))
        except FerrotorchError as e:
            raise OutOfMemory(f"allocation of {nbytes} bytes refused: {e}") from None
        return out.value or 0

    def free(self, ptr: int) -> None:
        """Returns the block to its pool. In canary mode a write past the end of the allocation raises (the block is released all the same)."""
        _lib.call("ft_alloc_free", self._h, ptr)

    def set_canary(self, nbytes: int) -> None:
        """Debug aid: ``nbytes`` guard bytes behind every later allocation, filled on malloc and verified on free. Only while nothing is live."""
        _lib.call("ft_alloc_set_canary", self._h, int(nbytes))

    def canary_violations(self) -> int:
        out = ctypes.c_int64()
        _lib.call("ft_alloc_canary_violations", self._h, ctypes.addressof(out))
        return out.value

    def record_stream(self, ptr: int, stream: int) -> None:
        _lib.call("ft_alloc_record_stream", self._h, ptr, stream)

    def set_budget(self, max_reserved_bytes: int) -> None:
        _lib.call("ft_alloc_set_budget", self._h, int(max_reserved_bytes))

    def empty_cache(self) -> int:
        freed = ctypes.c_int64()
        _lib.call("ft_alloc_empty_cache", self._h, ctypes.addressof(freed))
        return freed.value

    def stats(self) -> AllocatorStats:
        out = (ctypes.c_int64 * 10)()
        _lib.call("ft_alloc_stats", self._h, out)
        return AllocatorStats(*list(out))

    def memory_allocated(self) -> int:
        return self.stats().allocated

    def max_memory_allocated(self) -> int:
        return self.stats().peak_allocated

    def memory_reserved(self) -> int:
        return self.stats().reserved

    def reset_peak_stats(self) -> None:
        _lib.call("ft_alloc_reset_peak", self._h)

    def close(self) -> None:
        if self._own and self._h:
            _lib.call("ft_alloc_destroy", self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def install_as_torch_allocator() -> None:
    """Routes every torch CUDA allocation of this process through the native allocator (must run before the first CUDA allocation)."""
    from .._lib import _DIR
    alloc = torch.cuda.memory.CUDAPluggableAllocator(str(_DIR / "libft_kernels.so"), "ft_torch_malloc", "ft_torch_free")
    torch.cuda.memory.change_current_allocator(alloc)


def torch_allocator(device: int = 0) -> CudaAllocator:
    """The per-device instance behind :func:`install_as_torch_allocator` (for statistics / budget)."""
    h = ctypes.c_void_p()
    _lib.call("ft_torch_allocator_handle", device, ctypes.addressof(h))
    return CudaAllocator(_handle=h.value)


# ----------------------------------------------------------------------------------------------------------------------
# streams / events
# ----------------------------------------------------------------------------------------------------------------------
class StreamPriority(enum.IntEnum):
    HIGH = -1
    NORMAL = 0


class CudaEventWrapper:
    def __init__(self, timing: bool = True):
        self.event = torch.cuda.Event(enable_timing=timing)

    def record(self, stream: Optional[torch.cuda.Stream] = None) -> "CudaEventWrapper":
        self.event.record(stream or torch.cuda.current_stream())
        return self

    def query(self) -> bool:
        return self.event.query()

    def synchronize(self) -> None:
        self.event.synchronize()

    def wait(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        (stream or torch.cuda.current_stream()).wait_event(self.event)

    def elapsed_ms(self, end: "CudaEventWrapper") -> float:
        return self.event.elapsed_time(end.event)

    def elapsed_us(self, end: "CudaEventWrapper") -> float:
        return self.elapsed_ms(end) * 1e3


class StreamPool:
    """Round-robin pool of side streams per device (8 by default)."""

    def __init__(self, device=None, size: int = 8, priority: StreamPriority = StreamPriority.NORMAL):
        self.streams = [torch.cuda.Stream(device, priority=int(priority)) for _ in range(size)]
        self._i = 0
        self._lock = threading.Lock()

    def next(self) -> torch.cuda.Stream:
        with self._lock:
            s = self.streams[self._i % len(self.streams)]
            self._i += 1
            return s


@contextlib.contextmanager
def StreamGuard(stream: torch.cuda.Stream):
    """Makes ``stream`` current for the enclosed block (thread-local), ordering it after the previous current stream on entry."""
    prev = torch.cuda.current_stream(stream.device)
    stream.wait_stream(prev)
    with torch.cuda.stream(stream):
        yield stream


def current_stream(device=None) -> torch.cuda.Stream:
    return torch.cuda.current_stream(device)


# ----------------------------------------------------------------------------------------------------------------------
# CUDA graphs
# ----------------------------------------------------------------------------------------------------------------------
class CaptureMode(enum.Enum):
    GLOBAL = "global"
    THREAD_LOCAL = "thread_local"
    RELAXED = "relaxed"


class DeviceScalar:
    """A scalar that lives in device memory so a captured graph reads its current value at every replay (positions, step counters)."""

    def __init__(self, value=0, dtype=torch.int32, device=None):
        self.t = torch.tensor([value], dtype=dtype, device=device or "cuda")
        self._stage = torch.empty(1, dtype=dtype, pin_memory=True)

    def set(self, value) -> None:
        self._stage[0] = value
        self.t.copy_(self._stage, non_blocking=True)

    def tensor(self) -> torch.Tensor:
        return self.t

    def get(self):
        return self.t.item()


class CapturePool:
    """Shared memory pool handle so several graphs captured one after another re-use the same private allocations."""

    def __init__(self):
        self.handle = torch.cuda.graph_pool_handle()


class CapturedGraph:
    def __init__(self, graph: torch.cuda.CUDAGraph, outputs: Any = None):
        self.graph, self.outputs, self.launches = graph, outputs, 0

    def launch(self) -> Any:
        self.graph.replay()
        self.launches += 1
        return self.outputs

    def upload(self) -> None:
        """Instantiation already uploaded the executable graph; kept for interface parity (first-launch latency is paid at capture)."""

    def reset(self) -> None:
        self.graph.reset()


@contextlib.contextmanager
def GraphCaptureGuard(pool: Optional[CapturePool] = None, mode: CaptureMode = CaptureMode.THREAD_LOCAL, stream: Optional[torch.cuda.Stream] = None):
    """Captures the enclosed launches; yields a holder whose ``.graph`` is a :class:`CapturedGraph` after the block."""
    g = torch.cuda.CUDAGraph()
    holder = type("Capture", (), {})()
    with torch.cuda.graph(g, pool=pool.handle if pool else None, stream=stream, capture_error_mode=mode.value):
        yield holder
    holder.graph = CapturedGraph(g, getattr(holder, "outputs", None))


def begin_capture_with_pool(pool: CapturePool):
    return GraphCaptureGuard(pool)


def make_graphed_callable(fn: Callable[..., Any], sample_args: Sequence[torch.Tensor], warmup: int = 3, pool: Optional[CapturePool] = None) -> Callable[..., Any]:
    """Captures ``fn(*static_inputs)`` once; the returned callable copies new arguments into the static inputs and replays."""
    static_in = [a.clone() for a in sample_args]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.no_grad():
        for _ in range(warmup):
            fn(*static_in)
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.no_grad(), torch.cuda.graph(g, pool=pool.handle if pool else None):
        static_out = fn(*static_in)

    def run(*args):
        for s, a in zip(static_in, args):
            s.copy_(a)
        g.replay()
        return static_out
    run.graph = CapturedGraph(g, static_out)
    return run


# ----------------------------------------------------------------------------------------------------------------------
# memory guard
# ----------------------------------------------------------------------------------------------------------------------
class OomPolicy(enum.Enum):
    FAIL = "fail"                          # raise at once
    RETRY_AFTER_FREE = "retry_after_free"  # run hooks + empty caches, retry once
    WAIT = "wait"                          # block (up to a timeout) until enough memory is free, then retry
    CHECKPOINT_AND_FAIL = "checkpoint"     # call on_oom (emergency checkpoint), then raise


class PressureLevel(enum.IntEnum):
    NONE = 0
    MODERATE = 1
    HIGH = 2
    CRITICAL = 3


@dataclass
class MemoryGuardStats:
    budget: int
    used: int
    reserved_by_guard: int
    peak_used: int
    oom_events: int
    hook_invocations: int
    pressure: PressureLevel


class MemoryReservation:
    def __init__(self, guard: "MemoryGuard", nbytes: int):
        self.guard, self.nbytes, self.active = guard, nbytes, True

    def release(self) -> None:
        if self.active:
            self.guard._release(self.nbytes)
            self.active = False

    __enter__ = lambda self: self                       # noqa: E731
    __exit__ = lambda self, *a: self.release()           # noqa: E731


class MemoryGuard:
    """Budgeted view of device memory: reservations against a byte budget, OOM policies, pre-OOM hooks run in priority order, pressure
    listeners and a watchdog thread. ``query`` returns (used, total) bytes; the default asks the CUDA driver, tests inject a fake."""

    def __init__(self, budget_bytes: Optional[int] = None, policy: OomPolicy = OomPolicy.RETRY_AFTER_FREE, query: Optional[Callable[[], Tuple[int, int]]] = None,
                 device=None, wait_timeout_s: float = 30.0, thresholds: Tuple[float, float, float] = (0.7, 0.85, 0.95)):
        self.device = device
        self._query = query or self._cuda_query
        total = self._query()[1]
        self.budget = budget_bytes if budget_bytes is not None else total
        self.policy, self.wait_timeout_s, self.thresholds = policy, wait_timeout_s, thresholds
        self._reserved = 0
        self._lock = threading.Condition()
        self._hooks: List[Tuple[int, str, Callable[[int], int]]] = []
        self._listeners: List[Callable[[PressureLevel, PressureLevel], None]] = []
        self.on_oom: Optional[Callable[[int], None]] = None
        self._peak = self._ooms = self._hook_calls = 0
        self._level = PressureLevel.NONE
        self._paused = False
        self._watchdog: Optional[threading.Thread] = None
        self._stop = threading.Event()

    def _cuda_query(self) -> Tuple[int, int]:
        free, total = torch.cuda.mem_get_info(self.device)
        return total - free, total

    # -- hooks / listeners
    def add_pre_oom_hook(self, name: str, fn: Callable[[int], int], priority: int = 0) -> None:
        """``fn(bytes_needed) -> bytes_freed``; lower priority numbers run first."""
        self._hooks.append((priority, name, fn))
        self._hooks.sort(key=lambda h: h[0])

    def add_pressure_listener(self, fn: Callable[[PressureLevel, PressureLevel], None]) -> None:
        self._listeners.append(fn)

    # -- accounting
    def used(self) -> int:
        return self._query()[0] + self._reserved

    def pressure(self) -> PressureLevel:
        frac = self.used() / max(self.budget, 1)
        lvl = PressureLevel.NONE
        for l, th in zip((PressureLevel.MODERATE, PressureLevel.HIGH, PressureLevel.CRITICAL), self.thresholds):
            if frac >= th:
                lvl = l
        if lvl != self._level:
            old, self._level = self._level, lvl
            for fn in self._listeners:
                fn(old, lvl)
        return lvl

    def _try(self, nbytes: int) -> bool:
        if self.used() + nbytes <= self.budget:
            self._reserved += nbytes
            self._peak = max(self._peak, self.used())
            return True
        return False

    def _run_hooks(self, need: int) -> int:
        freed = 0
        for _, _, fn in self._hooks:
            self._hook_calls += 1
            freed += int(fn(need - freed) or 0)
            if freed >= need:
                break
        return freed

    def reserve(self, nbytes: int) -> MemoryReservation:
        """Books ``nbytes`` against the budget before the caller allocates; applies the OOM policy when the budget would be exceeded."""
        with self._lock:
            if self._try(nbytes):
                self.pressure()
                return MemoryReservation(self, nbytes)
            self._ooms += 1
            if self.policy is OomPolicy.FAIL:
                raise OutOfMemory(f"{nbytes} bytes over the budget of {self.budget} (used {self.used()})")
            if self.policy is OomPolicy.CHECKPOINT_AND_FAIL:
                if self.on_oom is not None:
                    self.on_oom(nbytes)
                raise OutOfMemory(f"{nbytes} bytes over the budget of {self.budget}; emergency callback ran")
            self._run_hooks(self.used() + nbytes - self.budget)
            if self._try(nbytes):
                return MemoryReservation(self, nbytes)
            if self.policy is OomPolicy.WAIT:
                deadline = time.monotonic() + self.wait_timeout_s
                while time.monotonic() < deadline:
                    self._lock.wait(timeout=min(0.05, max(deadline - time.monotonic(), 0.001)))
                    if self._try(nbytes):
                        return MemoryReservation(self, nbytes)
            if self.on_oom is not None:
                self.on_oom(nbytes)
            raise OutOfMemory(f"{nbytes} bytes over the budget of {self.budget} after running {len(self._hooks)} hook(s)")

    def _release(self, nbytes: int) -> None:
        with self._lock:
            self._reserved -= nbytes
            self._lock.notify_all()
        self.pressure()

    def stats(self) -> MemoryGuardStats:
        return MemoryGuardStats(self.budget, self.used(), self._reserved, self._peak, self._ooms, self._hook_calls, self._level)

    # -- watchdog
    def start_watchdog(self, interval_s: float = 0.05) -> None:
        """Background thread: samples pressure, pauses cooperative workers at CRITICAL (``wait_if_paused``) and resumes them below HIGH."""
        def loop():
            while not self._stop.wait(interval_s):
                lvl = self.pressure()
                with self._lock:
                    if lvl >= PressureLevel.CRITICAL:
                        self._paused = True
                    elif lvl < PressureLevel.HIGH and self._paused:
                        self._paused = False
                        self._lock.notify_all()
        self._stop.clear()
        self._watchdog = threading.Thread(target=loop, daemon=True, name="ft-memory-watchdog")
        self._watchdog.start()

    def stop_watchdog(self) -> None:
        self._stop.set()
        if self._watchdog is not None:
            self._watchdog.join(2.0)
            self._watchdog = None

    def wait_if_paused(self, timeout_s: float = 10.0) -> bool:
        """Called by data-loader / prefetch workers between items; returns False if still paused at the timeout."""
        with self._lock:
            deadline = time.monotonic() + timeout_s
            while self._paused:
                rem = deadline - time.monotonic()
                if rem <= 0:
                    return False
                self._lock.wait(timeout=rem)
            return True


class MemoryGuardBuilder:
    def __init__(self):
        self._kw: Dict[str, Any] = {}
        self._hooks: List[Tuple[str, Callable[[int], int], int]] = []

    def with_budget(self, nbytes: int): self._kw["budget_bytes"] = nbytes; return self
    def with_policy(self, p: OomPolicy): self._kw["policy"] = p; return self
    def with_wait_timeout(self, s: float): self._kw["wait_timeout_s"] = s; return self
    def with_thresholds(self, a: float, b: float, c: float): self._kw["thresholds"] = (a, b, c); return self
    def with_query(self, q): self._kw["query"] = q; return self
    def with_pre_oom_hook(self, name, fn, priority=0): self._hooks.append((name, fn, priority)); return self

    def build(self) -> MemoryGuard:
        g = MemoryGuard(**self._kw)
        for n, f, p in self._hooks:
            g.add_pre_oom_hook(n, f, p)
        return g


# ----------------------------------------------------------------------------------------------------------------------
# module cache
# ----------------------------------------------------------------------------------------------------------------------
class ModuleCache:
    """Compiled-kernel cache keyed by (kernel name, device): source -> cubin (NVRTC, sm_100a) -> loaded kernel handle."""

    def __init__(self):
        self._cache: Dict[Tuple[str, int], Tuple[int, int]] = {}
        self._keep: List[Any] = []
        self.compiles = self.hits = 0

    def get_or_compile(self, name: str, source: str, device: int = 0) -> int:
        key = (name, device)
        hit = self._cache.get(key)
        if hit is not None:
            self.hits += 1
            return hit[1]
        from ..jit.codegen import compile_cuda
        img = compile_cuda(source)
        self.compiles += 1
        buf = ctypes.create_string_buffer(img, len(img))
        lib, fn = ctypes.c_void_p(), ctypes.c_void_p()
        nm = ctypes.create_string_buffer(name.encode())
        _lib.call("ft_jit_load", ctypes.addressof(buf), ctypes.addressof(lib))
        _lib.call("ft_jit_get_kernel", lib.value, ctypes.addressof(nm), ctypes.addressof(fn))
        self._keep.append(buf)
        self._cache[key] = (lib.value, fn.value)
        return fn.value

    def launch(self, kernel: int, grid: int, block: int, args: Sequence[ctypes._SimpleCData], smem: int = 0) -> None:
        arr = (ctypes.c_void_p * len(args))(*[ctypes.addressof(a) for a in args])
        _lib.call("ft_jit_launch", kernel, grid, block, smem, ctypes.addressof(arr), _lib.S())


# ----------------------------------------------------------------------------------------------------------------------
# Philox generator manager
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class PhiloxState:
    seed: int
    offset: int


class CudaRngManager:
    """Per-device Philox generators with save / restore and fork / join for deterministic replay of a region (activation checkpointing)."""

    def __init__(self, seed: int = 0):
        from ..ops.tensor_ops import PhiloxGenerator
        self._G = PhiloxGenerator
        self._gens: Dict[int, Any] = {}
        self._seed = seed
        self._stack: List[Dict[int, PhiloxState]] = []

    def generator(self, device: int = 0):
        g = self._gens.get(device)
        if g is None:
            g = self._gens[device] = self._G(self._seed + device)
        return g

    def manual_seed(self, seed: int) -> None:
        self._seed = seed
        for d, g in self._gens.items():
            g.set_state((seed + d, 0))

    def get_state(self, device: int = 0) -> PhiloxState:
        return PhiloxState(*self.generator(device).state())

    def set_state(self, st: PhiloxState, device: int = 0) -> None:
        self.generator(device).set_state((st.seed, st.offset))

    def fork_rng(self) -> None:
        """Remembers every generator's state; :meth:`join_rng` restores it, so the forked region can be replayed with identical draws."""
        if torch.cuda.is_available():
            self.generator(torch.cuda.current_device())            # the current device's generator exists from here on, so its state is captured
        self._stack.append({d: PhiloxState(*g.state()) for d, g in self._gens.items()})

    def join_rng(self) -> None:
        if not self._stack:
            raise InvalidArgument("join_rng without fork_rng")
        for d, st in self._stack.pop().items():
            self.set_state(st, d)


rng_manager = CudaRngManager()


# ----------------------------------------------------------------------------------------------------------------------
# GpuTensor
# ----------------------------------------------------------------------------------------------------------------------
class GpuTensor:
    """Standalone device tensor (no autograd) with the small op set of the reference's bridge type; ops run on this framework's kernels."""

    def __init__(self, data: torch.Tensor):
        if not data.is_cuda:
            raise InvalidArgument("GpuTensor wraps a CUDA tensor")
        self.data = data

    @classmethod
    def from_host(cls, values: Sequence[float], shape: Sequence[int], dtype=torch.float32, device: Optional[GpuDevice] = None) -> "GpuTensor":
        t = torch.tensor(values, dtype=dtype).reshape(tuple(shape))
        return cls(cpu_to_gpu(t, device))

    def to_host(self) -> torch.Tensor:
        return self.data.cpu()

    @property
    def shape(self): return tuple(self.data.shape)
    def numel(self) -> int: return self.data.numel()
    def cu_device_ptr(self) -> int: return self.data.data_ptr()
    def try_clone(self) -> "GpuTensor": return GpuTensor(self.data.clone())

    def _bin(self, o: "GpuTensor", op: str) -> "GpuTensor":
        from ..ops import tensor_ops
        return GpuTensor(tensor_ops.binary(op, self.data, o.data))

    def add(self, o): return self._bin(o, "add")
    def sub(self, o): return self._bin(o, "sub")
    def mul(self, o): return self._bin(o, "mul")

    def neg(self):
        from ..ops import tensor_ops
        return GpuTensor(tensor_ops.unary("neg", self.data))

    def relu(self):
        from ..ops import tensor_ops
        return GpuTensor(tensor_ops.unary("relu", self.data))

    def matmul(self, o: "GpuTensor") -> "GpuTensor":
        from .. import ops
        if self.data.dtype == torch.bfloat16 and self.data.dim() == 2 and o.data.dim() == 2:
            return GpuTensor(ops.gemm(self.data, o.data, b_mn=True))
        return GpuTensor(self.data @ o.data)

    def conv2d(self, w: "GpuTensor", bias: Optional["GpuTensor"] = None, stride=1, padding=0) -> "GpuTensor":
        return GpuTensor(torch.nn.functional.conv2d(self.data, w.data, None if bias is None else bias.data, stride, padding))


# ----------------------------------------------------------------------------------------------------------------------
# backend registration
# ----------------------------------------------------------------------------------------------------------------------
class CudaBackendImpl:
    """Handle returned by :func:`init_cuda_backend`: the device, its allocator statistics and the kernel library's ABI version."""

    def __init__(self, device: GpuDevice):
        self.device = device
        self.abi = int(_lib.kernels().ft_abi_version())
        self.streams = StreamPool(device.device)
        self.modules = ModuleCache()

    def memory_allocated(self) -> int: return torch.cuda.memory_allocated(self.device.device)
    def max_memory_allocated(self) -> int: return torch.cuda.max_memory_allocated(self.device.device)
    def memory_reserved(self) -> int: return torch.cuda.memory_reserved(self.device.device)
    def empty_cache(self) -> None: torch.cuda.empty_cache()
    def kernel_status(self) -> int: return _lib.read_status()


_backend: Optional[CudaBackendImpl] = None


def init_cuda_backend(ordinal: int = 0) -> CudaBackendImpl:
    """Loads the kernel library, binds the device and returns the backend handle; raises if no CUDA device or the library is missing."""
    global _backend
    if _backend is None or _backend.device.ordinal != ordinal:
        torch.cuda.set_device(ordinal)
        _backend = CudaBackendImpl(GpuDevice(ordinal))
    return _backend


def gpu_backend() -> Optional[CudaBackendImpl]:
    return _backend


from . import api_ext  # noqa: E402
from .api_ext import *  # noqa: E402,F401,F403
from .api_ext import GpuResult, GpuFloat  # noqa: E402,F401
