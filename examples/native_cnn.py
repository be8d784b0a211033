#!/usr/bin/env python
"""Train a small convolutional network with the native C++ tensor / autograd core only: no torch.nn, torch.autograd or torch.optim on the
path (NumPy is the interchange format). Synthetic digits: each class is a fixed random 14 x 14 template plus noise.

    python examples/native_cnn.py [--steps 60] [--threads 4]

Counterpart of the reference's ferrotorch/examples/train_mnist.rs on the host path of its own tensor core.
"""
import argparse
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import numpy as np

from ferrotorch_b200 import native as N


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--threads", type=int, default=4, help="worker threads of the backward sweep (same bits as one thread)")
    a = ap.parse_args()
    rng = np.random.default_rng(0)
    templates = rng.standard_normal((10, 1, 14, 14)).astype(np.float32)

    def batch(n):
        y = rng.integers(0, 10, n)
        return templates[y] + 0.8 * rng.standard_normal((n, 1, 14, 14)).astype(np.float32), y
    net = N.Sequential(N.Conv2d(1, 8, 3, padding=1, rng=rng), N.ReLU(), N.MaxPool2d(2), N.Conv2d(8, 16, 3, padding=1, rng=rng), N.GELU(), N.MaxPool2d(2),
                       N.Flatten(), N.Linear(16 * 3 * 3, 10, rng=rng))
    opt = N.AdamW(net.parameters(), lr=3e-3, weight_decay=0.01)
    t0 = time.perf_counter()
    for step in range(a.steps):
        x, y = batch(a.batch)
        opt.zero_grad()
        loss = N.cross_entropy(net(N.Tensor(x)), y)
        loss.backward(threads=a.threads)
        opt.step()
        if step % 10 == 0 or step == a.steps - 1:
            print(f"step {step:3d}  loss {loss.item():.4f}")
    x, y = batch(512)
    with N.no_grad():
        acc = float((net(N.Tensor(x)).numpy().argmax(1) == y).mean())
    print(f"accuracy on 512 fresh samples: {acc:.3f}   ({(time.perf_counter() - t0) / a.steps * 1e3:.1f} ms per step)")


if __name__ == "__main__":
    main()
