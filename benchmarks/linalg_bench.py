#!/usr/bin/env python
"""Host linear algebra: this package's factorisations (``csrc/runtime/linalg.cpp`` behind ``core.linalg``) against LAPACK through the substrate.

    python benchmarks/linalg_bench.py [--sizes 32 128 256] [--repeat 3]

One JSON line per matrix size (milliseconds, best of ``repeat``, f64, one matrix) and one for a batch of 512 matrices of 16 x 16.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path


def best(fn, *args, repeat=3):
    fn(*args)
    ts = []
    for _ in range(repeat):
        t0 = time.perf_counter()
        fn(*args)
        ts.append(time.perf_counter() - t0)
    return round(min(ts) * 1e3, 3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", type=int, nargs="+", default=[32, 128, 256])
    ap.add_argument("--repeat", type=int, default=3)
    a = ap.parse_args()
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import torch
    from ferrotorch_b200 import core as X
    L = torch.linalg
    torch.manual_seed(0)
    for n in a.sizes:
        m = torch.randn(n, n, dtype=torch.float64)
        spd = m @ m.mT + n * torch.eye(n, dtype=torch.float64)
        rhs = torch.randn(n, 4, dtype=torch.float64)
        row = {"bench": "host_linalg", "n": n, "unit": "ms", "ours_vs_lapack": {}}
        for name, args in (("cholesky", (spd,)), ("solve", (m, rhs)), ("qr", (m,)), ("eigh", (spd,)), ("svd", (m,)), ("eig", (m,))):
            row["ours_vs_lapack"][name] = [best(getattr(X.linalg, name), *args, repeat=a.repeat), best(getattr(L, name), *args, repeat=a.repeat)]
        print(json.dumps(row))
    b = torch.randn(512, 16, 16, dtype=torch.float64)
    sym = b + b.mT
    row = {"bench": "host_linalg_batch", "shape": [512, 16, 16], "unit": "ms", "ours_vs_lapack": {}}
    for name, arg in (("inv", b), ("svd", b), ("eigh", sym), ("eig", b)):
        row["ours_vs_lapack"][name] = [best(getattr(X.linalg, name), arg, repeat=a.repeat), best(getattr(L, name), arg, repeat=a.repeat)]
    print(json.dumps(row))


if __name__ == "__main__":
    main()
