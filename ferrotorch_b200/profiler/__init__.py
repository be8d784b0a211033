"""Profiler: op / memory / CUDA-event recording, FLOP estimates, table + Chrome-trace + TensorBoard export, schedules.

``with_profiler(config, fn)`` installs a :class:`Profiler` as the thread's op hook (see ``core.profile_op_scope``), runs ``fn``
and returns ``(result, ProfileReport)``. GPU work is timed with CUDA event pairs on the launching stream and resolved lazily
(``flush_cuda_kernels``); every scope also opens an NVTX range so external tools see the same names.

Reference parity: ferrotorch-profiler/src/profiler.rs:53-437, event.rs:3-98, cuda_timing.rs:59-107, report.rs:58-500,
schedule.rs:53-179, flops.rs:41.
"""
from __future__ import annotations

import contextlib
import enum
import json
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..core import OpProfiler, set_current_profiler, current_profiler


class DeviceType(enum.Enum):
    Cpu = "cpu"
    Cuda = "cuda"


class MemoryCategory(enum.Enum):
    Parameter = "parameter"
    Activation = "activation"
    Gradient = "gradient"
    OptimizerState = "optimizer_state"
    Workspace = "workspace"
    Other = "other"


@dataclass
class ProfileEvent:
    name: str
    category: str
    start_us: float
    duration_us: float
    device: DeviceType = DeviceType.Cpu
    shapes: Any = None
    flops: Optional[float] = None
    thread: int = 0
    memory_bytes: Optional[int] = None
    memory_category: Optional[MemoryCategory] = None


@dataclass
class GpuTimingPair:
    name: str
    start: Any
    stop: Any
    host_start_us: float
    category: str = "kernel"


@dataclass
class ProfileConfig:
    record_shapes: bool = True
    profile_memory: bool = False
    with_flops: bool = True
    cuda_events: bool = True
    nvtx: bool = True


def estimate_flops(name: str, shapes) -> Optional[float]:
    """FLOP estimates for the common ops (matmul-like: 2*M*N*K; conv: 2*out_elems*k; attention: 4*B*H*S^2*D)."""
    try:
        if name in ("mm", "matmul", "linear", "gemm", "addmm") and shapes and len(shapes) >= 2:
            a, b = shapes[0], shapes[1]
            m = 1
            for d in a[:-1]:
                m *= d
            return 2.0 * m * a[-1] * (b[0] if name == "linear" else b[-1])
        if name == "bmm" and shapes:
            a, b = shapes[0], shapes[1]
            return 2.0 * a[0] * a[1] * a[2] * b[2]
        if name in ("conv2d",) and shapes and len(shapes) >= 3:
            out, w = shapes[2], shapes[1]
            n = 1
            for d in out:
                n *= d
            return 2.0 * n * w[1] * w[2] * w[3]
        if name in ("attention", "flash_attention") and shapes:
            B, H, S, D = shapes[0]
            return 4.0 * B * H * S * S * D
        if name in ("add", "mul", "sub", "div", "relu", "gelu", "silu") and shapes:
            n = 1
            for d in shapes[0]:
                n *= d
            return float(n)
    except Exception:
        return None
    return None


class Profiler(OpProfiler):
    def __init__(self, config: Optional[ProfileConfig] = None):
        self.config = config or ProfileConfig()
        self.events: List[ProfileEvent] = []
        self._gpu: List[GpuTimingPair] = []
        self._t0 = time.perf_counter()
        self._lock = threading.Lock()

    def _now_us(self) -> float:
        return (time.perf_counter() - self._t0) * 1e6

    # -- OpProfiler hook
    def on_op(self, name, category, shapes, seconds):
        self.record_with_duration(name, category, seconds * 1e6, shapes)

    def record(self, name: str, category: str = "op", shapes=None) -> None:
        self.record_with_duration(name, category, 0.0, shapes)

    def record_with_duration(self, name: str, category: str, duration_us: float, shapes=None, device: DeviceType = DeviceType.Cpu) -> None:
        ev = ProfileEvent(name, category, self._now_us() - duration_us, duration_us, device, shapes if self.config.record_shapes else None,
                          estimate_flops(name, shapes) if self.config.with_flops else None, threading.get_ident())
        with self._lock:
            self.events.append(ev)

    def record_memory(self, name: str, nbytes: int, category: MemoryCategory = MemoryCategory.Other) -> None:
        with self._lock:
            self.events.append(ProfileEvent(name, "memory", self._now_us(), 0.0, memory_bytes=nbytes, memory_category=category))

    record_memory_categorized = record_memory

    def push_gpu_event(self, pair: GpuTimingPair) -> None:
        with self._lock:
            self._gpu.append(pair)

    @contextlib.contextmanager
    def scope(self, name: str, category: str = "scope", shapes=None):
        """CPU timing + (on CUDA) an event pair on the current stream + an NVTX range."""
        cuda = self.config.cuda_events and torch.cuda.is_available()
        if cuda and self.config.nvtx:
            torch.cuda.nvtx.range_push(name)
        pair = None
        if cuda:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            pair = GpuTimingPair(name, s, e, self._now_us(), category)
        t0 = time.perf_counter()
        try:
            yield
        finally:
            dur = (time.perf_counter() - t0) * 1e6
            if pair is not None:
                pair.stop.record()
                self.push_gpu_event(pair)
                if self.config.nvtx:
                    torch.cuda.nvtx.range_pop()
            self.record_with_duration(name, category, dur, shapes)

    def flush_cuda_kernels(self) -> None:
        """Resolve pending event pairs into GPU-duration events (synchronises on each stop event)."""
        with self._lock:
            pend, self._gpu = self._gpu, []
        for p in pend:
            p.stop.synchronize()
            self.events.append(ProfileEvent(p.name, p.category, p.host_start_us, p.start.elapsed_time(p.stop) * 1e3, DeviceType.Cuda))

    def report(self) -> "ProfileReport":
        self.flush_cuda_kernels()
        return ProfileReport(list(self.events))


class CudaKernelScope:
    """RAII-style start/stop event pair on the current stream, pushed to the profiler on exit (cuda_timing.rs:59-107)."""

    def __init__(self, profiler: Profiler, name: str):
        self.p, self.name = profiler, name

    def __enter__(self):
        self.s, self.e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.t = self.p._now_us()
        self.s.record()
        return self

    def __exit__(self, *a):
        self.e.record()
        self.p.push_gpu_event(GpuTimingPair(self.name, self.s, self.e, self.t))


@dataclass
class OpSummary:
    name: str
    count: int
    total_us: float
    mean_us: float
    flops: float
    device: str


class ProfileReport:
    def __init__(self, events: List[ProfileEvent]):
        self.events = events

    def summaries(self) -> List[OpSummary]:
        agg: Dict[Tuple[str, str], List[float]] = {}
        for e in self.events:
            if e.category == "memory":
                continue
            k = (e.name, e.device.value)
            a = agg.setdefault(k, [0, 0.0, 0.0])
            a[0] += 1
            a[1] += e.duration_us
            a[2] += e.flops or 0.0
        return sorted((OpSummary(n, int(c), t, t / max(c, 1), f, d) for (n, d), (c, t, f) in agg.items()), key=lambda s: -s.total_us)

    def top_ops(self, k: int = 10) -> List[OpSummary]:
        return self.summaries()[:k]

    def table(self, k: int = 30) -> str:
        rows = ["{:<40} {:>6} {:>8} {:>12} {:>12} {:>10}".format("name", "dev", "calls", "total_us", "mean_us", "GFLOP")]
        for s in self.top_ops(k):
            rows.append("{:<40} {:>6} {:>8} {:>12.1f} {:>12.1f} {:>10.2f}".format(s.name[:40], s.device, s.count, s.total_us, s.mean_us, s.flops / 1e9))
        return "\n".join(rows)

    def total_flops(self) -> float:
        return sum(e.flops or 0.0 for e in self.events)

    def memory_by_category(self) -> Dict[str, int]:
        out: Dict[str, int] = {}
        for e in self.events:
            if e.memory_bytes is not None:
                out[e.memory_category.value] = out.get(e.memory_category.value, 0) + e.memory_bytes
        return out

    def chrome_trace_json(self) -> str:
        tr = []
        for e in self.events:
            if e.category == "memory":
                tr.append({"name": e.name, "ph": "C", "ts": e.start_us, "pid": 0, "tid": 0, "args": {"bytes": e.memory_bytes}})
            else:
                tr.append({"name": e.name, "cat": e.category, "ph": "X", "ts": e.start_us, "dur": max(e.duration_us, 0.001),
                           "pid": 1 if e.device == DeviceType.Cuda else 0, "tid": e.thread % 100000,
                           "args": {"shapes": str(e.shapes) if e.shapes is not None else None, "flops": e.flops}})
        return json.dumps({"traceEvents": tr, "displayTimeUnit": "us"})

    def save_chrome_trace(self, path) -> None:
        with open(path, "w") as f:
            f.write(self.chrome_trace_json())

    def save_tensorboard_trace(self, log_dir, step: int = 0) -> None:
        from ..train import TensorBoardWriter
        w = TensorBoardWriter(log_dir)
        for s in self.top_ops(50):
            w.add_scalar(f"profile/{s.device}/{s.name}_total_us", s.total_us, step)
        w.close()


def with_profiler(config: Optional[ProfileConfig], fn: Callable[[], Any]):
    prof = Profiler(config)
    prev = current_profiler()
    set_current_profiler(prof)
    try:
        out = fn()
    finally:
        set_current_profiler(prev)
    return out, prof.report()


class ScheduleAction(enum.Enum):
    Skip = "skip"
    Warmup = "warmup"
    Record = "record"
    RecordAndSave = "record_and_save"


class SchedulePhase(enum.Enum):
    """Where a step falls in the wait / warmup / active cycle; ``Done`` after the last repeat (ferrotorch-profiler/src/schedule.rs:5)."""
    Waiting = "Waiting"
    Warmup = "Warmup"
    Active = "Active"
    Done = "Done"

    def __str__(self):
        return self.value


class ProfileSchedule:
    """wait / warmup / active / repeat step schedule with an ``on_trace_ready`` callback (schedule.rs:53-179)."""

    def __init__(self, wait: int = 1, warmup: int = 1, active: int = 3, repeat: int = 1, on_trace_ready: Optional[Callable[[ProfileReport], None]] = None):
        self.wait, self.warmup, self.active, self.repeat, self.on_trace_ready = wait, warmup, active, repeat, on_trace_ready
        self.step_num = 0
        self.profiler: Optional[Profiler] = None

    def action(self, step: int) -> ScheduleAction:
        cycle = self.wait + self.warmup + self.active
        if self.repeat and step >= cycle * self.repeat:
            return ScheduleAction.Skip
        s = step % cycle
        if s < self.wait:
            return ScheduleAction.Skip
        if s < self.wait + self.warmup:
            return ScheduleAction.Warmup
        return ScheduleAction.RecordAndSave if s == cycle - 1 else ScheduleAction.Record

    def phase(self, step: Optional[int] = None) -> SchedulePhase:
        """Phase of ``step`` (default: the step about to run)."""
        step = self.step_num if step is None else step
        cycle = self.wait + self.warmup + self.active
        if self.repeat and step >= cycle * self.repeat:
            return SchedulePhase.Done
        s = step % cycle
        return SchedulePhase.Waiting if s < self.wait else (SchedulePhase.Warmup if s < self.wait + self.warmup else SchedulePhase.Active)

    def step(self) -> None:
        a = self.action(self.step_num)
        if a in (ScheduleAction.Record, ScheduleAction.RecordAndSave) and self.profiler is None:
            self.profiler = Profiler()
            set_current_profiler(self.profiler)
        if a == ScheduleAction.RecordAndSave and self.profiler is not None:
            rep = self.profiler.report()
            set_current_profiler(None)
            self.profiler = None
            if self.on_trace_ready:
                self.on_trace_ready(rep)
        self.step_num += 1


class flops:  # noqa: N801  (namespace: ``profiler.flops.estimate(op, shapes)``, ferrotorch-profiler/src/flops.rs:41)
    @staticmethod
    def estimate(op_name: str, input_shapes):
        """Integer FLOP estimate of one operation, ``None`` for an operation without a rule."""
        v = estimate_flops(op_name, [list(s) for s in input_shapes])
        return None if v is None else int(v)


estimate = flops.estimate
