#!/usr/bin/env python
"""CPU DDP plumbing benchmark (no GPU): world size 2 over the TCP backend, MLP 784 -> 256 (ReLU) -> 10 in f32 with Kaiming-uniform init from
seed 0, batch 64 per rank (x ~ N(0,1), labels uniform in [0,10)), cross-entropy, SGD lr 0.01 momentum 0.9, 100 steps.

    python bench_cpu_ddp.py [--world 2] [--steps 100] [--algo star|ring] [--framework native|torch]

``--framework native`` (default) builds the model, the backward pass and the optimizer on this repository's native C++ core
(``ferrotorch_b200.native``: ft::Tensor, the Kahn-ordered autograd engine, ft::Sgd); ``torch`` uses torch.nn / torch.autograd / torch.optim
for the same numbers (A/B).

Prints one JSON line: milliseconds per step (max over ranks, wall clock around the timed steps after ``--warmup`` untimed ones), the share of
the step spent in the gradient all-reduce, and the two checks of the configuration: gradients and parameters bit-identical across ranks, and
parameters within 1e-5 of single-process batch-128 training. ``star`` is the reference's algorithm (rank 0 gathers, reduces in rank order
and sends back: ferrotorch-distributed/src/collective.rs:64-132 over backend.rs:92-378); ``ring`` is the full-mesh ring all-reduce.
"""
from __future__ import annotations

import argparse
import json
import multiprocessing as mp
import os
import time

import numpy as np
import torch


def _mlp():
    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Linear(784, 256), torch.nn.ReLU(), torch.nn.Linear(256, 10))
    for l in (m[0], m[2]):
        torch.nn.init.kaiming_uniform_(l.weight, nonlinearity="relu")
        torch.nn.init.zeros_(l.bias)
    return m


def _data(steps, world):
    g = torch.Generator().manual_seed(1234)
    return torch.randn(steps, 64 * world, 784, generator=g), torch.randint(0, 10, (steps, 64 * world), generator=g)


def _native_mlp():
    """The same network on the native core, with the same initial values as ``_mlp()`` (taken from it, so both frameworks start identically)."""
    from ferrotorch_b200 import native as N
    ref = _mlp()
    return N.Sequential(N.Linear(784, 256, weight=ref[0].weight.detach().numpy(), bias_value=ref[0].bias.detach().numpy()), N.ReLU(),
                        N.Linear(256, 10, weight=ref[2].weight.detach().numpy(), bias_value=ref[2].bias.detach().numpy()))


def _native_worker(rank, world, port, steps, warmup, algo, q):
    from ferrotorch_b200 import distributed as fd, native as N
    from ferrotorch_b200.distributed.ddp import NativeDDP
    torch.set_num_threads(1)
    backend = fd.TcpBackend(rank, world, f"127.0.0.1:{port}", full_mesh=(algo == "ring"))
    model = _native_mlp()
    ddp = NativeDDP(model, backend, algorithm=algo)
    ddp.broadcast_parameters(0)
    opt = N.Sgd(model.parameters(), lr=0.01, momentum=0.9)
    X, Y = _data(steps + warmup, world)
    X, Y = X.numpy(), Y.numpy()
    comm_s, t0, grads = 0.0, None, None
    for step in range(steps + warmup):
        if step == warmup:
            backend.barrier()
            t0 = time.perf_counter()
            comm_s = 0.0
        x, y = X[step, rank * 64:(rank + 1) * 64], Y[step, rank * 64:(rank + 1) * 64]
        opt.zero_grad()
        N.cross_entropy(ddp(N.Tensor(x)), y).backward()
        c0 = time.perf_counter()
        ddp.sync_gradients()
        comm_s += time.perf_counter() - c0
        if step == steps + warmup - 1:
            grads = [p.grad.numpy().copy() for p in model.parameters()]
        opt.step()
    total = time.perf_counter() - t0
    q.put((rank, total, comm_s, [p.numpy().copy() for p in model.parameters()], grads))
    backend.barrier()


def _worker(rank, world, port, steps, warmup, algo, q):
    from ferrotorch_b200 import distributed as fd
    torch.set_num_threads(1)
    backend = fd.TcpBackend(rank, world, f"127.0.0.1:{port}", full_mesh=(algo == "ring"))
    model = _mlp()
    ddp = fd.DDP(model, backend, algorithm=algo)
    ddp.broadcast_parameters(0)
    opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
    X, Y = _data(steps + warmup, world)
    comm_s, t0, grads = 0.0, None, None
    for step in range(steps + warmup):
        if step == warmup:
            backend.barrier()
            t0 = time.perf_counter()
            comm_s = 0.0
        x, y = X[step, rank * 64:(rank + 1) * 64], Y[step, rank * 64:(rank + 1) * 64]
        opt.zero_grad()
        torch.nn.functional.cross_entropy(ddp(x), y).backward()
        c0 = time.perf_counter()
        ddp.sync_gradients()
        comm_s += time.perf_counter() - c0
        if step == steps + warmup - 1:
            grads = [p.grad.numpy().copy() for p in model.parameters()]
        opt.step()
    total = time.perf_counter() - t0
    q.put((rank, total, comm_s, [p.detach().numpy().copy() for p in model.parameters()], grads))
    backend.barrier()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--algo", default="star", choices=["star", "ring"])
    ap.add_argument("--framework", default="native", choices=["native", "torch"])
    a = ap.parse_args()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + os.getpid() % 90
    target = _native_worker if a.framework == "native" else _worker
    ps = [ctx.Process(target=target, args=(r, a.world, port, a.steps, a.warmup, a.algo, q)) for r in range(a.world)]
    [p.start() for p in ps]
    got = {}
    for _ in range(a.world):
        r, total, comm, params, grads = q.get(timeout=600)
        got[r] = (total, comm, params, grads)
    [p.join(30) for p in ps]
    identical = all(np.array_equal(x, y) for r in range(1, a.world) for x, y in zip(got[0][2] + got[0][3], got[r][2] + got[r][3]))
    torch.set_num_threads(1)
    X, Y = _data(a.steps + a.warmup, a.world)
    if a.framework == "native":
        from ferrotorch_b200 import native as N
        model = _native_mlp()
        opt = N.Sgd(model.parameters(), lr=0.01, momentum=0.9)
        Xn, Yn = X.numpy(), Y.numpy()
        t0 = time.perf_counter()
        for step in range(a.steps + a.warmup):
            opt.zero_grad()
            N.cross_entropy(model(N.Tensor(Xn[step])), Yn[step]).backward()
            opt.step()
        single_ms = (time.perf_counter() - t0) / (a.steps + a.warmup) * 1e3
        single = [p.numpy() for p in model.parameters()]
    else:
        model = _mlp()
        opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
        t0 = time.perf_counter()
        for step in range(a.steps + a.warmup):
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(X[step]), Y[step]).backward()
            opt.step()
        single_ms = (time.perf_counter() - t0) / (a.steps + a.warmup) * 1e3
        single = [p.detach().numpy() for p in model.parameters()]
    err = max(float(np.abs(x - p).max()) for x, p in zip(got[0][2], single))
    ms = max(v[0] for v in got.values()) / a.steps * 1e3
    print(json.dumps({"metric": "cpu_ddp_tcp_ms_per_step", "value": round(ms, 3), "unit": "ms/step", "higher_is_better": False, "world": a.world,
                      "steps": a.steps, "warmup": a.warmup, "algo": a.algo, "framework": "native C++ core (ft::Tensor, autograd engine, ft::Sgd)" if a.framework == "native" else "torch.nn / torch.autograd / torch.optim", "allreduce_share": round(max(v[1] for v in got.values()) / max(v[0] for v in got.values()), 3),
                      "single_process_batch%d_ms_per_step" % (64 * a.world): round(single_ms, 3), "ranks_bit_identical": bool(identical),
                      "max_abs_diff_vs_single_process": err, "matches_single_process_1e-5": bool(err < 1e-5),
                      "config": {"model": "mlp-784-256-10", "dtype": "f32", "batch_per_rank": 64, "optimizer": "SGD(lr=0.01,momentum=0.9)", "transport": "tcp loopback"}}))


if __name__ == "__main__":
    main()
