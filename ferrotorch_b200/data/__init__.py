"""Datasets, samplers, collation and the DataLoader (API names follow ferrotorch-data).

The loader prefetches batches on worker threads, gathers in-memory datasets with the native multi-threaded row gather,
stages through pinned host memory and copies to the device on a side stream so the copy overlaps the previous step.

Reference parity: dataset.rs:8-356, sampler.rs:2-459 (DistributedSampler semantics :129-188), dataloader.rs:34-1255,
collate / transforms / interop modules.
"""
from __future__ import annotations

import ctypes
import enum
import math
import queue
import threading
from dataclasses import dataclass
from typing import Any, Callable, Iterable, Iterator, List, Optional, Sequence

import numpy as np
import torch

from .. import _lib
from ..errors import InvalidArgument, IndexOutOfBounds


# ----------------------------------------------------------------------------------------------------------------------
# datasets
# ----------------------------------------------------------------------------------------------------------------------
class Dataset:
    """Map-style dataset: ``len`` and ``get(index)`` (``__getitem__``)."""

    def len(self) -> int:  # noqa: A003
        return len(self)

    def get(self, index: int):
        return self[index]

    def is_empty(self) -> bool:
        return len(self) == 0


class IterableDataset:
    """Stream-style dataset: ``iter(worker_info)`` yields samples; workers shard the stream themselves."""

    def iter(self, worker_info: Optional["WorkerInfo"] = None) -> Iterator:  # noqa: A003
        raise NotImplementedError

    def __iter__(self):
        return self.iter(None)


@dataclass
class WorkerInfo:
    worker_id: int
    num_workers: int
    seed: int = 0


class VecDataset(Dataset):
    def __init__(self, items: Sequence):
        self.items = list(items)

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        if not -len(self.items) <= i < len(self.items):
            raise IndexOutOfBounds(f"index {i} out of range for dataset of length {len(self.items)}")
        return self.items[i]


class MappedDataset(Dataset):
    def __init__(self, inner: Dataset, fn: Callable):
        self.inner, self.fn = inner, fn

    def __len__(self):
        return len(self.inner)

    def __getitem__(self, i):
        return self.fn(self.inner[i])


class TensorDataset(Dataset):
    """Rows of one or more tensors sharing dim 0."""

    def __init__(self, *tensors: torch.Tensor):
        if not tensors or any(t.shape[0] != tensors[0].shape[0] for t in tensors):
            raise InvalidArgument("TensorDataset needs tensors with equal first dimension")
        self.tensors = tensors

    def __len__(self):
        return self.tensors[0].shape[0]

    def __getitem__(self, i):
        if not -len(self) <= i < len(self):
            raise IndexOutOfBounds(f"index {i} out of range")
        return tuple(t[i] for t in self.tensors)

    def gather(self, indices: Sequence[int], pin: bool = False, threads: int = 8):
        """Batch rows ``indices`` of every tensor at once with the native row gather."""
        idx = np.ascontiguousarray(np.asarray(indices, dtype=np.int64))
        outs = []
        for t in self.tensors:
            if t.is_cuda or not t.is_contiguous():
                outs.append(t[torch.as_tensor(idx, device=t.device)])
                continue
            out = torch.empty((len(idx), *t.shape[1:]), dtype=t.dtype, pin_memory=pin and torch.cuda.is_available())
            row = t[0].numel() * t.element_size() if t.dim() > 1 else t.element_size()
            rc = _lib.runtime().ft_gather_rows(ctypes.c_void_p(t.data_ptr()), ctypes.c_int64(row), idx.ctypes.data_as(ctypes.c_void_p),
                                               ctypes.c_int64(len(idx)), ctypes.c_int64(t.shape[0]), ctypes.c_void_p(out.data_ptr()), threads)
            if rc:
                raise IndexOutOfBounds("gather index out of range")
            outs.append(out)
        return tuple(outs)


class ConcatDataset(Dataset):
    def __init__(self, datasets: Sequence[Dataset]):
        self.datasets = list(datasets)
        self.cum = np.cumsum([len(d) for d in self.datasets]).tolist()

    def __len__(self):
        return self.cum[-1] if self.cum else 0

    def __getitem__(self, i):
        if i < 0:
            i += len(self)
        if not 0 <= i < len(self):
            raise IndexOutOfBounds(f"index {i} out of range")
        k = int(np.searchsorted(self.cum, i, side="right"))
        return self.datasets[k][i - (self.cum[k - 1] if k else 0)]


class ChainDataset(IterableDataset):
    def __init__(self, datasets: Sequence[IterableDataset]):
        self.datasets = list(datasets)

    def iter(self, worker_info=None):  # noqa: A003
        for d in self.datasets:
            yield from d.iter(worker_info)


class SyntheticTokenDataset(Dataset):
    """Uniform random token ids of shape ``[seq_len+1]`` (inputs and shifted targets), reproducible per index."""

    def __init__(self, n: int, seq_len: int, vocab: int, seed: int = 0):
        self.n, self.seq_len, self.vocab, self.seed = n, seq_len, vocab, seed

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 1000003 + i)
        return torch.randint(0, self.vocab, (self.seq_len + 1,), generator=g)


# ----------------------------------------------------------------------------------------------------------------------
# samplers
# ----------------------------------------------------------------------------------------------------------------------
def _permutation(n: int, seed: int) -> List[int]:
    out = (ctypes.c_int64 * n)()
    _lib.runtime().ft_permutation(ctypes.c_int64(n), ctypes.c_uint64(seed & 0xFFFFFFFFFFFFFFFF), out)
    return list(out)


class Sampler:
    def indices(self, epoch: int = 0) -> List[int]:
        raise NotImplementedError

    def __iter__(self):
        return iter(self.indices(getattr(self, "epoch", 0)))

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch


class SequentialSampler(Sampler):
    def __init__(self, n: int):
        self.n = n

    def indices(self, epoch: int = 0):
        return list(range(self.n))

    def __len__(self):
        return self.n


class RandomSampler(Sampler):
    def __init__(self, n: int, seed: int = 0, replacement: bool = False, num_samples: Optional[int] = None):
        self.n, self.seed, self.replacement, self.num_samples = n, seed, replacement, num_samples or n

    def indices(self, epoch: int = 0):
        s = self.seed ^ ((epoch * 0x9e3779b97f4a7c15) & 0xFFFFFFFFFFFFFFFF)
        if self.replacement:
            g = torch.Generator().manual_seed(s & 0x7FFFFFFFFFFFFFFF)
            return torch.randint(0, self.n, (self.num_samples,), generator=g).tolist()
        return _permutation(self.n, s)[: self.num_samples]

    def __len__(self):
        return self.num_samples


class DistributedSampler(Sampler):
    """Shuffle with ``seed ^ epoch*0x9e3779b97f4a7c15``, pad by wrap-around to a multiple of ``num_replicas``, then take the
    interleaved slice ``rank, rank+R, rank+2R, ...`` (``len = ceil(n/R)``); defaults ``shuffle=True, seed=0``."""

    def __init__(self, n: int, num_replicas: int, rank: int, shuffle: bool = True, seed: int = 0, drop_last: bool = False):
        if not 0 <= rank < num_replicas:
            raise InvalidArgument(f"rank {rank} out of range for {num_replicas} replicas")
        self.n, self.num_replicas, self.rank, self.shuffle, self.seed, self.drop_last = n, num_replicas, rank, shuffle, seed, drop_last
        self.epoch = 0

    def __len__(self):
        return self.n // self.num_replicas if self.drop_last else math.ceil(self.n / self.num_replicas)

    def indices(self, epoch: Optional[int] = None):
        epoch = self.epoch if epoch is None else epoch
        idx = _permutation(self.n, self.seed ^ ((epoch * 0x9e3779b97f4a7c15) & 0xFFFFFFFFFFFFFFFF)) if self.shuffle else list(range(self.n))
        total = len(self) * self.num_replicas
        if self.drop_last:
            idx = idx[:total]
        else:
            i = 0
            while len(idx) < total and self.n:
                idx.append(idx[i])
                i += 1
        return idx[self.rank:: self.num_replicas]


class WeightedRandomSampler(Sampler):
    def __init__(self, weights: Sequence[float], num_samples: int, replacement: bool = True, seed: int = 0):
        self.weights, self.num_samples, self.replacement, self.seed = torch.as_tensor(weights, dtype=torch.double), num_samples, replacement, seed

    def indices(self, epoch: int = 0):
        g = torch.Generator().manual_seed((self.seed + epoch) & 0x7FFFFFFFFFFFFFFF)
        return torch.multinomial(self.weights, self.num_samples, self.replacement, generator=g).tolist()

    def __len__(self):
        return self.num_samples


class BatchSampler(Sampler):
    def __init__(self, sampler: Sampler, batch_size: int, drop_last: bool = False):
        self.sampler, self.batch_size, self.drop_last = sampler, batch_size, drop_last

    def batches(self, epoch: int = 0) -> List[List[int]]:
        idx = self.sampler.indices(epoch)
        out = [idx[i: i + self.batch_size] for i in range(0, len(idx), self.batch_size)]
        if self.drop_last and out and len(out[-1]) < self.batch_size:
            out.pop()
        return out

    def indices(self, epoch: int = 0):
        return self.batches(epoch)

    def __len__(self):
        n = len(self.sampler)
        return n // self.batch_size if self.drop_last else math.ceil(n / self.batch_size)


# ----------------------------------------------------------------------------------------------------------------------
# collate + loader
# ----------------------------------------------------------------------------------------------------------------------
def default_collate(samples: List[Any]):
    e = samples[0]
    if isinstance(e, torch.Tensor):
        return torch.stack(samples)
    if isinstance(e, np.ndarray):
        return torch.from_numpy(np.stack(samples))
    if isinstance(e, (int, float, bool)):
        return torch.tensor(samples)
    if isinstance(e, (tuple, list)):
        parts = [default_collate([s[i] for s in samples]) for i in range(len(e))]
        return type(e)(*parts) if hasattr(e, "_fields") else type(e)(parts)          # a named tuple takes its fields one by one
    if isinstance(e, dict):
        return {k: default_collate([s[k] for s in samples]) for k in e}
    return samples


class WorkerMode(enum.Enum):
    Sync = "sync"            # load on the caller's thread
    Threads = "threads"      # worker threads (GIL released in the native gather, pin and copy paths)


@dataclass
class ToDevice:
    device: Any
    non_blocking: bool = True


class DataLoader:
    """``for batch in loader``: batches are produced ``prefetch`` ahead by ``num_workers`` threads, optionally pinned and
    copied to ``device`` on a side stream (the consumer's stream waits on the copy's event, not on the host)."""

    def __init__(self, dataset, batch_size: int = 1, shuffle: bool = False, sampler: Optional[Sampler] = None, drop_last: bool = False,
                 num_workers: int = 0, prefetch: int = 2, pin_memory: bool = False, device=None, collate_fn: Optional[Callable] = None,
                 seed: int = 0, worker_mode: Optional[WorkerMode] = None):
        self.dataset, self.batch_size, self.drop_last = dataset, batch_size, drop_last
        self.num_workers, self.prefetch, self.pin_memory = num_workers, max(1, prefetch), pin_memory
        self.device = torch.device(device) if device is not None else None
        self.collate_fn = collate_fn or default_collate
        self.iterable = isinstance(dataset, IterableDataset)
        self.worker_mode = worker_mode or (WorkerMode.Threads if num_workers > 0 else WorkerMode.Sync)
        if not self.iterable:
            base = sampler or (RandomSampler(len(dataset), seed) if shuffle else SequentialSampler(len(dataset)))
            self.batch_sampler = BatchSampler(base, batch_size, drop_last)
        self.epoch = 0
        self._copy_stream = None

    # builder-style setters (ferrotorch-data/src/dataloader.rs:195-364)
    def with_workers(self, n: int) -> "DataLoader":
        self.num_workers = n
        self.worker_mode = WorkerMode.Threads if n > 0 else WorkerMode.Sync
        return self

    def with_prefetch(self, n: int) -> "DataLoader":
        self.prefetch = max(1, n)
        return self

    def with_pin_memory(self, flag: bool = True) -> "DataLoader":
        self.pin_memory = flag
        return self

    def with_device(self, device) -> "DataLoader":
        self.device = torch.device(device)
        return self

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def __len__(self):
        if self.iterable:
            raise TypeError("an iterable dataset has no length")
        return len(self.batch_sampler)

    def _load(self, idx: List[int]):
        fast = isinstance(self.dataset, TensorDataset) and self.collate_fn is default_collate
        b = self.dataset.gather(idx, pin=self.pin_memory) if fast else self.collate_fn([self.dataset[i] for i in idx])
        if self.pin_memory and not fast and torch.cuda.is_available():
            b = _map(b, lambda t: t.pin_memory())
        return b

    def _to_device(self, b):
        if self.device is None:
            return b
        if self.device.type != "cuda":
            return _map(b, lambda t: t.to(self.device))
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(self.device)
        with torch.cuda.stream(self._copy_stream):
            out = _map(b, lambda t: t.to(self.device, non_blocking=True))
            ev = torch.cuda.Event()
            ev.record(self._copy_stream)
        torch.cuda.current_stream(self.device).wait_event(ev)
        _map(out, lambda t: (t.record_stream(torch.cuda.current_stream(self.device)), t)[1])
        return out

    def iter(self):  # noqa: A003
        return iter(self)

    def __iter__(self):
        if self.iterable:
            yield from self._iter_stream()
            return
        batches = self.batch_sampler.batches(self.epoch)
        self.epoch += 1
        if self.worker_mode == WorkerMode.Sync or self.num_workers == 0:
            for idx in batches:
                yield self._to_device(self._load(idx))
            return
        results: "queue.Queue" = queue.Queue()
        slots = threading.Semaphore(self.prefetch + self.num_workers)
        nxt = [0]
        lock = threading.Lock()
        done: dict = {}
        stop = threading.Event()

        def worker():
            while not stop.is_set():
                slots.acquire()
                with lock:
                    i = nxt[0]
                    nxt[0] += 1
                if i >= len(batches):
                    slots.release()
                    return
                try:
                    results.put((i, self._load(batches[i]), None))
                except BaseException as e:  # surfaced on the consumer thread
                    results.put((i, None, e))
        ts = [threading.Thread(target=worker, daemon=True) for _ in range(self.num_workers)]
        [t.start() for t in ts]
        try:
            for want in range(len(batches)):
                while want not in done:
                    i, b, e = results.get()
                    done[i] = (b, e)
                b, e = done.pop(want)
                slots.release()
                if e is not None:
                    from ..errors import WorkerPanic
                    raise WorkerPanic(f"data worker failed on batch {want}: {e!r}") from e
                yield self._to_device(b)
        finally:
            stop.set()
            for _ in ts:
                slots.release()

    def _iter_stream(self):
        buf = []
        for s in self.dataset.iter(WorkerInfo(0, 1)):
            buf.append(s)
            if len(buf) == self.batch_size:
                yield self._to_device(self.collate_fn(buf))
                buf = []
        if buf and not self.drop_last:
            yield self._to_device(self.collate_fn(buf))


def _map(b, fn):
    if isinstance(b, torch.Tensor):
        return fn(b)
    if isinstance(b, (tuple, list)):
        return type(b)(_map(x, fn) for x in b)
    if isinstance(b, dict):
        return {k: _map(v, fn) for k, v in b.items()}
    return b


PrefetchIter = MultiWorkerIter = CollatedIter = DataLoader  # iteration strategies are modes of the one loader


# ----------------------------------------------------------------------------------------------------------------------
# interop
# ----------------------------------------------------------------------------------------------------------------------
def from_numpy(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a))


def to_numpy(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def load_npy(path: str) -> torch.Tensor:
    return from_numpy(np.load(path))


def save_npy(path: str, t: torch.Tensor) -> None:
    np.save(path, to_numpy(t))


def from_arrow(array) -> torch.Tensor:
    """Zero-copy where possible from a pyarrow Array / ChunkedArray of a primitive type."""
    import pyarrow as pa
    if isinstance(array, pa.ChunkedArray):
        array = array.combine_chunks()
    return torch.from_numpy(array.to_numpy(zero_copy_only=False))


def shuffle_with_seed(indices: List[int], seed: int) -> None:
    """In-place Fisher-Yates shuffle driven by xorshift64 (13 / 7 / 17; seed 0 becomes 0xdeadbeefcafe) with unbiased bounded draws (128-bit
    multiply, rejection below ``2^64 mod bound``), walking ``i`` from the last index down (ferrotorch-data/src/sampler.rs:17-69): the shuffle
    primitive shared by the random and distributed samplers, so a given seed orders a dataset the same way everywhere."""
    M = (1 << 64) - 1
    state = (int(seed) & M) or 0xDEADBEEFCAFE

    def nxt():
        nonlocal state
        x = state
        x ^= (x << 13) & M
        x ^= x >> 7
        x ^= (x << 17) & M
        state = x
        return x
    for i in range(len(indices) - 1, 0, -1):
        bound = i + 1
        prod = nxt() * bound
        if (prod & M) < bound:
            t = ((1 << 64) - bound) % bound
            while (prod & M) < t:
                prod = nxt() * bound
        j = prod >> 64
        indices[i], indices[j] = indices[j], indices[i]


def default_collate_pair(samples: Sequence):
    """``[(input, target), ...]`` -> ``(stack(inputs), stack(targets))`` (ferrotorch-data/src/collate.rs:32)."""
    if len(samples) == 0:
        raise InvalidArgument("default_collate_pair: empty sample list")
    xs, ys = zip(*samples)
    return torch.stack([torch.as_tensor(x) for x in xs], 0), torch.stack([torch.as_tensor(y) for y in ys], 0)


class BatchIter:
    """Iterator over the raw (uncollated) batches of a dataset: each item is the list of samples of one batch, in sampler order
    (ferrotorch-data/src/dataloader.rs, ``BatchIter``)."""

    def __init__(self, dataset, batches: Iterable[Sequence[int]]):
        self.dataset, self._it = dataset, iter(batches)

    def __iter__(self):
        return self

    def __next__(self):
        return [self.dataset[i] for i in next(self._it)]


# -- transforms with their own counter-based random stream (ferrotorch-data/src/transforms.rs) ------------------------------------------
class Transform:
    """Base of the tensor transforms: ``apply(x)`` (also ``__call__``)."""

    def apply(self, x):
        raise NotImplementedError

    def __call__(self, x):
        return self.apply(x)


class _SplitMixCounter:
    _M = (1 << 64) - 1

    def __init__(self):
        self.seed, self.counter, self._lock = 0, 0, threading.Lock()

    def manual_seed(self, seed: int) -> None:
        with self._lock:
            self.seed, self.counter = int(seed) & self._M, 0

    def random(self) -> float:
        with self._lock:
            c = self.counter
            self.counter += 1
        z = (self.seed + c * 0x9E3779B97F4A7C15) & self._M
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & self._M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & self._M
        return (z ^ (z >> 31)) / float(self._M)


_transform_rng = _SplitMixCounter()


def manual_seed(seed: int) -> None:
    """Seeds the transforms' random stream and restarts its counter: draw ``n`` afterwards is splitmix64 of ``seed + n * golden``
    (transforms.rs:331-350)."""
    _transform_rng.manual_seed(seed)


class ToTensor(Transform):
    """Image (PIL image, ``[H, W, C]`` uint8 array) -> float ``[C, H, W]`` in [0, 1]; a tensor passes through unchanged, as the reference's
    tensor-to-tensor form does (transforms.rs:221-270)."""

    def apply(self, x):
        if torch.is_tensor(x):
            return x
        a = np.asarray(x.convert("RGB") if hasattr(x, "convert") else x)
        if a.ndim == 2:
            a = a[:, :, None]
        if a.ndim != 3 or 0 in a.shape:
            raise InvalidArgument(f"ToTensor: expected an [H, W, C] image with non-zero sides, got shape {list(a.shape)}")
        return torch.from_numpy(np.ascontiguousarray(a)).permute(2, 0, 1).float().div(255.0)


class RandomHorizontalFlip(Transform):
    """Reverses the last dimension with probability ``p`` (transforms.rs:288-390)."""

    def __init__(self, p: float = 0.5):
        if not 0.0 <= p <= 1.0:
            raise InvalidArgument(f"RandomHorizontalFlip: p must be in [0, 1], got {p}")
        self.p = p

    def apply(self, x):
        if x.dim() == 0:
            raise InvalidArgument("RandomHorizontalFlip: input must be at least 1-D")
        if _transform_rng.random() >= self.p or x.shape[-1] <= 1:
            return x
        return x.detach().flip(-1)


class RandomCrop(Transform):
    """A ``height x width`` window of the last two dimensions at a random origin ``floor(u * (in - crop))`` per axis (no draw for an axis that
    already fits) (transforms.rs:403-470)."""

    def __init__(self, height: int, width: Optional[int] = None):
        self.height, self.width = int(height), int(width if width is not None else height)

    def apply(self, x):
        if x.dim() < 2:
            raise InvalidArgument(f"RandomCrop: input must be at least 2-D, got shape {list(x.shape)}")
        H, W = x.shape[-2:]
        if self.height > H or self.width > W:
            raise InvalidArgument(f"RandomCrop: crop size ({self.height}x{self.width}) is larger than input spatial size ({H}x{W})")
        top = 0 if H == self.height else int(_transform_rng.random() * (H - self.height))
        left = 0 if W == self.width else int(_transform_rng.random() * (W - self.width))
        return x.detach()[..., top: top + self.height, left: left + self.width].contiguous()


class Compose:
    def __init__(self, fns: Sequence[Callable]):
        self.fns = list(fns)

    def __call__(self, x):
        for f in self.fns:
            x = f(x)
        return x

    apply = __call__


class Normalize:
    def __init__(self, mean, std):
        self.mean, self.std = torch.as_tensor(mean), torch.as_tensor(std)

    def __call__(self, x):
        shp = (-1,) + (1,) * (x.dim() - 1)
        return (x - self.mean.view(shp).to(x)) / self.std.view(shp).to(x)


class ToFloat:
    def __call__(self, x):
        return x.float()


class Lambda:
    def __init__(self, fn):
        self.fn = fn

    def __call__(self, x):
        return self.fn(x)
