"""DistributedDataParallel over a byte-level backend (CPU tensors) - the control-plane / CPU path.

Buckets are built in reverse parameter order with a 25 MiB cap; ``sync_gradients`` flattens each bucket (a missing
gradient counts as zeros), all-reduces it with ``Mean`` and scatters the result back into ``.grad``;
``overlapped_sync_gradients`` runs one thread per bucket. On CUDA tensors with an NCCL process group the GPU reducer of
:mod:`ferrotorch_b200.parallel.ddp` (fused cast/scale + peer-memory all-reduce, overlapped with backward) is used instead.

Reference parity: ferrotorch-distributed/src/ddp.rs:18 (DEFAULT_BUCKET_SIZE_BYTES), :38-205 (DDP), :213-241 (compute_buckets),
:248-294 (sync_one_bucket).
"""
from __future__ import annotations

import ctypes
import threading
from typing import List, Optional

import torch

from .backend import Backend, rt
from .collective import ReduceOp, allreduce, broadcast, DEFAULT_COLLECTIVE_TIMEOUT

DEFAULT_BUCKET_SIZE_BYTES = 25 * 1024 * 1024


def compute_buckets(params: List[torch.Tensor], bucket_size_bytes: int = DEFAULT_BUCKET_SIZE_BYTES) -> List[List[int]]:
    """Parameter indices per bucket; bucket 0 holds the *last* parameters (their gradients are ready first)."""
    n = len(params)
    if n == 0:
        return []
    numels = (ctypes.c_int64 * n)(*[p.numel() for p in params])
    out = (ctypes.c_int * n)()
    elem = params[0].element_size()
    nb = rt().ft_ddp_plan_buckets(numels, n, elem, bucket_size_bytes, out)
    buckets: List[List[int]] = [[] for _ in range(nb)]
    for i in range(n - 1, -1, -1):
        buckets[out[i]].append(i)
    return buckets


class DDP:
    """Wraps a module; gradients are averaged across ranks by :meth:`sync_gradients` after ``backward``."""

    def __init__(self, module: torch.nn.Module, backend: Backend, bucket_size_bytes: int = DEFAULT_BUCKET_SIZE_BYTES,
                 timeout: Optional[float] = DEFAULT_COLLECTIVE_TIMEOUT, algorithm: str = "star"):
        """``algorithm``: "star" (the reference's gather-to-rank-0 all-reduce, works on every backend) or "ring" (needs links between
        neighbours: a full-mesh TCP backend or the simulated fabric)."""
        self._module, self.backend, self.timeout, self.algorithm = module, backend, timeout, algorithm
        self.params = [p for p in module.parameters() if p.requires_grad]
        self.buckets = compute_buckets(self.params, bucket_size_bytes)

    def module(self) -> torch.nn.Module:
        return self._module

    def forward(self, *a, **k):
        return self._module(*a, **k)

    __call__ = forward

    def parameters(self):
        return self._module.parameters()

    def train(self, mode: bool = True):
        self._module.train(mode)
        return self

    def eval(self):
        return self.train(False)

    def broadcast_parameters(self, root: int = 0) -> None:
        with torch.no_grad():
            for p in self._module.parameters():
                p.copy_(broadcast(p.data, self.backend, root, self.timeout))
            for b in self._module.buffers():
                if b.is_floating_point():
                    b.copy_(broadcast(b.data, self.backend, root, self.timeout))

    def _sync_one_bucket(self, idx: List[int]) -> None:
        ps = [self.params[i] for i in idx]
        flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in ps])
        red = allreduce(flat, self.backend, ReduceOp.Mean, self.timeout, self.algorithm)
        off = 0
        for p in ps:
            n = p.numel()
            p.grad = red[off: off + n].view_as(p).clone()
            off += n

    def sync_gradients(self) -> None:
        for b in self.buckets:
            self._sync_one_bucket(b)

    def overlapped_sync_gradients(self) -> None:
        """One thread per bucket. The transport serialises frames per peer, so buckets are issued in order under a lock
        on untagged channels: the overlap is between a bucket's host-side flatten/scatter and the next bucket's transfer."""
        errs: List[BaseException] = []
        lock = threading.Lock()

        def work(b):
            try:
                with lock:
                    self._sync_one_bucket(b)
            except BaseException as e:
                errs.append(e)
        ts = [threading.Thread(target=work, args=(b,)) for b in self.buckets]
        for t in ts:
            t.start()
            t.join()   # untagged channels carry one message stream per peer: keep bucket order identical on every rank
        if errs:
            raise errs[0]


class NativeDDP:
    """The same bucketed gradient averaging for a model built on the native core (:mod:`ferrotorch_b200.native`): parameters are native
    tensors, buckets are flattened from zero-copy NumPy views of their ``.grad`` and the reduced values are written back in place."""

    class _Meta:
        def __init__(self, t):
            self.t = t

        def numel(self):
            return self.t.numel()

        def element_size(self):
            return 4

    def __init__(self, module, backend: Backend, bucket_size_bytes: int = DEFAULT_BUCKET_SIZE_BYTES,
                 timeout: Optional[float] = DEFAULT_COLLECTIVE_TIMEOUT, algorithm: str = "star"):
        self._module, self.backend, self.timeout, self.algorithm = module, backend, timeout, algorithm
        self.params = list(module.parameters())
        self.buckets = compute_buckets([self._Meta(p) for p in self.params], bucket_size_bytes)

    def __call__(self, *a):
        return self._module(*a)

    def module(self):
        return self._module

    def parameters(self):
        return self.params

    def broadcast_parameters(self, root: int = 0) -> None:
        for p in self.params:
            v = p.numpy()
            v[...] = broadcast(torch.from_numpy(v), self.backend, root, self.timeout).numpy()

    def sync_gradients(self) -> None:
        import numpy as np
        for idx in self.buckets:
            ps = [self.params[i] for i in idx]
            grads = [p.grad for p in ps]
            flat = np.concatenate([(g.numpy() if g is not None else np.zeros(p.shape, np.float32)).reshape(-1) for p, g in zip(ps, grads)])
            red = allreduce(torch.from_numpy(flat), self.backend, ReduceOp.Mean, self.timeout, self.algorithm).numpy()
            off = 0
            for p, g in zip(ps, grads):
                n = p.numel()
                if g is not None:
                    g.numpy().reshape(-1)[:] = red[off: off + n]
                off += n
