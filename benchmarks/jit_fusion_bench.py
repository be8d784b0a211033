#!/usr/bin/env python
"""Fused elementwise chain: ``jit.compile`` against eager execution of the same function (the reference claims a 2-5x speedup for fused
elementwise chains, README.md:31 of the reference, without a table).

    python benchmarks/jit_fusion_bench.py [--device cpu|cuda] [--numel 4000000]

The function is a 12-operation chain over two inputs (sigmoid, tanh, relu, exp and arithmetic). Host: one threaded, vectorised C++ loop compiled
by the JIT; device: one NVRTC-compiled sm_100a kernel. Median of 20 calls after warm-up (CUDA: events).
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
from pathlib import Path

import torch


def chain(x, y):
    t = torch.sigmoid(x) * y + torch.tanh(x * 0.5)
    t = torch.relu(t - 0.1) * torch.exp(-y * y)
    return t * t + x


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--numel", type=int, default=4_000_000)
    a = ap.parse_args()
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    from ferrotorch_b200 import jit
    dev = torch.device(a.device)
    x, y = torch.randn(a.numel, device=dev), torch.randn(a.numel, device=dev)
    compiled = jit.compile(chain, example_inputs=[x, y], backend="auto")

    def timed(fn):
        for _ in range(3):
            fn(x, y)
        ts = []
        for _ in range(20):
            if dev.type == "cuda":
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn(x, y)
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            else:
                t0 = time.perf_counter()
                fn(x, y)
                ts.append((time.perf_counter() - t0) * 1e3)
        return statistics.median(ts)
    eager_ms, jit_ms = timed(chain), timed(compiled)
    err = float((chain(x, y) - compiled(x, y)).abs().max())
    print(json.dumps({"bench": "jit_fused_chain", "device": a.device, "numel": a.numel, "ops_in_chain": 12, "eager_ms": round(eager_ms, 3),
                      "jit_ms": round(jit_ms, 3), "speedup": round(eager_ms / jit_ms, 2), "max_abs_diff": err,
                      "fused_kernels": compiled.stats.fused_kernels, "reference_claim": "2-5x"}))


if __name__ == "__main__":
    main()
