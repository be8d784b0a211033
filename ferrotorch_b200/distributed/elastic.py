"""Failure detection and stop-the-world elastic recovery on the host, plus the distributed throughput monitor.

* :class:`KeyValueStore` / :class:`MemoryStore` / :class:`TcpStoreAdapter`: the small store the control plane needs (set / get / add / wait).
* :class:`HeartbeatMonitor`: every rank bumps ``hb/<rank>`` from a thread; a watchdog thread compares the peers' counters against a timeout and
  reports ranks that stopped. Nothing here touches a GPU: a rank is declared failed between steps, from host state only.
* :class:`ElasticCoordinator`: survivors agree on a new generation (``rendezvous``), get new contiguous ranks, and resume from a distributed
  checkpoint that is re-sharded for the new world size (``ferrotorch_b200.distributed.load_distributed``).
* :class:`DistributedMonitor`: per-step throughput, device-timed collective / compute spans, communication-to-compute ratio and achieved
  fraction of a roofline, aggregated as the max over ranks.

The reference has no elastic membership, heartbeat or monitor (ferrotorch-distributed: "design only", .design/phase-7-distributed.md:17,19); its
failure handling is per-receive timeouts and typed errors (backend.rs:282-357, error.rs:8-52), which the transport layer here keeps.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from ..errors import DistributedError, Timeout


class RankFailure(DistributedError):
    def __init__(self, ranks: Sequence[int]):
        super().__init__(f"ranks {sorted(ranks)} stopped sending heartbeats")
        self.ranks = sorted(ranks)


class KeyValueStore:
    def set(self, key: str, value: bytes) -> None: raise NotImplementedError      # noqa: E704
    def get(self, key: str) -> Optional[bytes]: raise NotImplementedError         # noqa: E704
    def add(self, key: str, amount: int) -> int: raise NotImplementedError        # noqa: E704

    def wait(self, key: str, timeout_s: float) -> bytes:
        deadline = time.monotonic() + timeout_s
        while time.monotonic() < deadline:
            v = self.get(key)
            if v is not None:
                return v
            time.sleep(0.005)
        raise Timeout(message=f"store key {key!r} not set within {timeout_s}s")


class MemoryStore(KeyValueStore):
    """In-process store shared by rank threads (tests, single-node simulations)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, key, value):
        with self._lock:
            self._d[key] = bytes(value)

    def get(self, key):
        with self._lock:
            return self._d.get(key)

    def add(self, key, amount):
        with self._lock:
            v = int(self._d.get(key, b"0")) + amount
            self._d[key] = str(v).encode()
            return v


class TcpStoreAdapter(KeyValueStore):
    """The same interface over ``torch.distributed.TCPStore`` (one process hosts it, the rest connect to 127.0.0.1 / MASTER_ADDR)."""

    def __init__(self, host: str, port: int, is_master: bool, world_size: Optional[int] = None, timeout_s: float = 30.0):
        import datetime
        from torch.distributed import TCPStore
        self._s = TCPStore(host, port, world_size, is_master, timeout=datetime.timedelta(seconds=timeout_s), wait_for_workers=False)

    def set(self, key, value):
        self._s.set(key, value)

    def get(self, key):
        return self._s.get(key) if self._s.check([key]) else None

    def add(self, key, amount):
        return self._s.add(key, amount)


class HeartbeatMonitor:
    def __init__(self, store: KeyValueStore, rank: int, world: int, interval_s: float = 0.05, timeout_s: float = 0.5, on_failure: Optional[Callable[[List[int]], None]] = None,
                 generation: int = 0):
        self.store, self.rank, self.world, self.interval_s, self.timeout_s = store, rank, world, interval_s, timeout_s
        self.on_failure, self.generation = on_failure, generation
        self._stop = threading.Event()
        self._threads: List[threading.Thread] = []
        self._failed: List[int] = []
        self._lock = threading.Lock()

    def _key(self, r: int) -> str:
        return f"g{self.generation}/hb/{r}"

    def start(self) -> "HeartbeatMonitor":
        self.store.set(self._key(self.rank), b"0")

        def beat():
            n = 0
            while not self._stop.wait(self.interval_s):
                n += 1
                self.store.set(self._key(self.rank), str(n).encode())

        def watch():
            last: Dict[int, Tuple[bytes, float]] = {}
            start = time.monotonic()
            while not self._stop.wait(self.interval_s):
                now = time.monotonic()
                dead = []
                for r in range(self.world):
                    if r == self.rank:
                        continue
                    v = self.store.get(self._key(r))
                    prev = last.get(r)
                    if v is not None and (prev is None or prev[0] != v):
                        last[r] = (v, now)
                    elif now - (prev[1] if prev else start) > self.timeout_s:
                        dead.append(r)
                if dead:
                    with self._lock:
                        new = [r for r in dead if r not in self._failed]
                        self._failed += new
                    if new and self.on_failure is not None:
                        self.on_failure(new)
        for fn, name in ((beat, "ft-heartbeat"), (watch, "ft-heartbeat-watchdog")):
            t = threading.Thread(target=fn, daemon=True, name=name)
            t.start()
            self._threads.append(t)
        return self

    def failed_ranks(self) -> List[int]:
        with self._lock:
            return list(self._failed)

    def check(self) -> None:
        """Called between steps, with no kernel or collective of this rank in flight: raises :class:`RankFailure` if a peer stopped."""
        f = self.failed_ranks()
        if f:
            raise RankFailure(f)

    def stop(self) -> None:
        self._stop.set()
        for t in self._threads:
            t.join(2.0)
        self._threads.clear()


@dataclass
class Membership:
    generation: int
    rank: int
    world: int
    old_ranks: List[int]          # old rank of each new rank


class ElasticCoordinator:
    """Stop-the-world recovery: every survivor calls :meth:`rendezvous` with the same failed set; they get the next generation and new ranks
    ordered by old rank. ``min_world`` guards against continuing with too few ranks."""

    def __init__(self, store: KeyValueStore, min_world: int = 1, timeout_s: float = 10.0):
        self.store, self.min_world, self.timeout_s = store, min_world, timeout_s

    def rendezvous(self, old_rank: int, old_world: int, failed: Sequence[int], generation: int) -> Membership:
        survivors = [r for r in range(old_world) if r not in set(failed)]
        if old_rank not in survivors:
            raise DistributedError(f"rank {old_rank} is in the failed set")
        if len(survivors) < self.min_world:
            raise DistributedError(f"{len(survivors)} survivors, fewer than min_world={self.min_world}")
        gen = generation + 1
        self.store.set(f"g{gen}/join/{old_rank}", b"1")
        deadline = time.monotonic() + self.timeout_s
        while True:
            present = [r for r in survivors if self.store.get(f"g{gen}/join/{r}") is not None]
            if len(present) == len(survivors):
                break
            if time.monotonic() > deadline:
                missing = sorted(set(survivors) - set(present))
                raise Timeout(message=f"re-rendezvous for generation {gen}: ranks {missing} did not join")
            time.sleep(0.005)
        return Membership(gen, survivors.index(old_rank), len(survivors), survivors)


def resume_from_checkpoint(directory: str, membership: Membership):
    """Loads this (new) rank's shards of a distributed checkpoint written by any earlier world size."""
    from .extras import load_distributed
    return load_distributed(directory, membership.rank, membership.world)


# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class StepRecord:
    step: int
    units: float                 # tokens / images processed by the whole job
    ms: float                    # device-timed, max over ranks
    comm_ms: float = 0.0
    compute_ms: float = 0.0


class DistributedMonitor:
    """Aggregates per-step timings. ``span(kind)`` brackets device work with CUDA events (host clocks on CPU); ``end_step`` resolves the
    events and, when a process group is given, reduces with MAX so the record is the slowest rank's."""

    def __init__(self, unit: str = "tokens", group=None, roofline_ms: Optional[float] = None):
        self.unit, self.group, self.roofline_ms = unit, group, roofline_ms
        self.records: List[StepRecord] = []
        self._spans: Dict[str, List[Tuple[object, object]]] = {"comm": [], "compute": [], "step": []}
        self._step = 0

    def span(self, kind: str):
        import contextlib
        import torch
        mon = self

        @contextlib.contextmanager
        def ctx():
            if torch.cuda.is_available():
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                yield
                e1.record()
                mon._spans[kind].append((e0, e1))
            else:
                t0 = time.perf_counter()
                yield
                mon._spans[kind].append((t0, time.perf_counter()))
        return ctx()

    def _resolve(self, kind: str) -> float:
        import torch
        total = 0.0
        for a, b in self._spans[kind]:
            if isinstance(a, float):
                total += (b - a) * 1e3
            else:
                b.synchronize()
                total += a.elapsed_time(b)
        self._spans[kind] = []
        return total

    def end_step(self, units: float) -> StepRecord:
        import torch
        vals = [self._resolve("step"), self._resolve("comm"), self._resolve("compute")]
        if self.group is not None:
            import torch.distributed as dist
            t = torch.tensor(vals, dtype=torch.float64, device="cuda" if torch.cuda.is_available() and dist.get_backend(self.group) == "nccl" else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            vals = t.tolist()
        self._step += 1
        r = StepRecord(self._step, units, vals[0], vals[1], vals[2])
        self.records.append(r)
        return r

    def summary(self, skip: int = 0) -> Dict[str, float]:
        rs = self.records[skip:]
        if not rs:
            return {}
        ms = sum(r.ms for r in rs)
        out = {f"{self.unit}_per_s": sum(r.units for r in rs) / (ms / 1e3) if ms > 0 else 0.0, "ms_per_step": ms / len(rs),
               "comm_ms_per_step": sum(r.comm_ms for r in rs) / len(rs), "compute_ms_per_step": sum(r.compute_ms for r in rs) / len(rs)}
        out["comm_to_compute"] = out["comm_ms_per_step"] / out["compute_ms_per_step"] if out["compute_ms_per_step"] > 0 else 0.0
        if self.roofline_ms:
            out["fraction_of_roofline"] = self.roofline_ms / out["ms_per_step"] if out["ms_per_step"] > 0 else 0.0
        return out
