#!/usr/bin/env python
"""The reference's published micro-benchmark table (benchmarks/RESULTS.md:10-40 of the reference: tensor creation, elementwise, matmul, and a
784 -> 256 -> 10 MLP at batch 32) measured through this framework's public API, on the CPU and, with ``--device cuda``, on the GPU.

    python benchmarks/micro_bench.py [--device cpu|cuda] [--json out.json]

Every row prints the median time in microseconds next to the two published columns (ferrotorch and PyTorch on the reference's machine:
an AMD CPU under WSL2 / an RTX 3090), so the ratio is indicative only across machines. Timing: 10 warm-up calls, then the median of
``--iters`` calls (``time.perf_counter``; on CUDA a synchronize before and after each call).
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
from pathlib import Path

import torch

PUBLISHED_CPU = {  # name -> (ferrotorch us, pytorch us)
    "zeros [1000,1000]": (74.5, 73.5), "rand [1000,1000]": (1189.0, 1907.0), "add [1000,1000]": (211.5, 32.2), "mul [1000,1000]": (178.6, 51.5),
    "relu [1000,1000]": (120.0, 69.6), "sigmoid [1000,1000]": (1447.6, 168.7), "matmul [64,64]": (108.0, 5.6), "matmul [256,256]": (7329.0, 92.5),
    "matmul [1024,1024]": (2106087.0, 2860.0), "mlp forward B=32": (3320.0, 51.2), "mlp backward B=32": (8348.0, 393.2),
    "mlp training step B=32": (6978.0, 535.1),
}
PUBLISHED_GPU = {"add [1000,1000]": (None, 17.0), "matmul [1024,1024]": (35.0, 521.7), "matmul [4096,4096]": (None, 5248.0), "mlp forward B=32": (None, 73.4)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))          # run from a checkout without installing the package
    from ferrotorch_b200 import core, nn, optim
    dev = torch.device(a.device)
    cuda = dev.type == "cuda"

    def timeit(fn, iters=a.iters):
        for _ in range(10):
            fn()
        ts = []
        for _ in range(iters):
            if cuda:
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            fn()
            if cuda:
                torch.cuda.synchronize()
            ts.append((time.perf_counter() - t0) * 1e6)
        return statistics.median(ts)

    x, y = core.rand([1000, 1000], device=dev), core.rand([1000, 1000], device=dev)
    rows = {
        "zeros [1000,1000]": lambda: core.zeros([1000, 1000], device=dev),
        "rand [1000,1000]": lambda: core.rand([1000, 1000], device=dev),
        "add [1000,1000]": lambda: x + y,
        "mul [1000,1000]": lambda: x * y,
        "relu [1000,1000]": lambda: torch.relu(x),
        "sigmoid [1000,1000]": lambda: torch.sigmoid(x),
    }
    for n in (64, 256, 1024) + ((4096,) if cuda else ()):
        p, q = core.rand([n, n], device=dev), core.rand([n, n], device=dev)
        rows[f"matmul [{n},{n}]"] = (lambda p=p, q=q: p @ q)
    model = nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Linear(256, 10)).to(dev)
    opt = optim.Sgd(model.parameters(), lr=0.01)
    lossf = nn.CrossEntropyLoss()
    xb, yb = core.randn([32, 784], device=dev), torch.randint(0, 10, (32,), device=dev)

    def fwd():
        with core.no_grad():
            return model(xb)

    def bwd():
        model.zero_grad()
        lossf(model(xb), yb).backward()

    def step():
        bwd()
        opt.step()
    rows["mlp forward B=32"] = fwd
    rows["mlp backward B=32"] = bwd
    rows["mlp training step B=32"] = step
    published = PUBLISHED_GPU if cuda else PUBLISHED_CPU
    out = []
    print(f"{'operation':28s} {'ours us':>12s} {'ref ferrotorch us':>18s} {'ref pytorch us':>15s} {'ferrotorch / ours':>18s}")
    for name, fn in rows.items():
        us = timeit(fn, max(5, a.iters // 20) if name.startswith("matmul [1024") and not cuda else a.iters)
        ref, pt = published.get(name, (None, None))
        ratio = (ref / us) if ref else None
        out.append({"operation": name, "device": a.device, "ours_us": round(us, 2), "reference_ferrotorch_us": ref, "reference_pytorch_us": pt,
                    "speedup_vs_reference": round(ratio, 2) if ratio else None})
        print(f"{name:28s} {us:12.1f} {ref if ref else '-':>18} {pt if pt else '-':>15} {f'{ratio:.1f}x' if ratio else '-':>18}")
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"device": a.device, "torch": torch.__version__, "threads": torch.get_num_threads(), "rows": out}, f, indent=1)


if __name__ == "__main__":
    main()
