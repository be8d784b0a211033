#!/usr/bin/env python
"""Train a small CNN on (synthetic) MNIST with the Learner: data loader, AdamW, cosine schedule, accuracy metric, checkpoints, TensorBoard.

    python examples/train_mnist.py [--epochs 3] [--device cuda] [--out DIR]

Counterpart of the reference's ferrotorch/examples/train_mnist.rs.
"""
import argparse
import sys
import tempfile
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch

from ferrotorch_b200 import data, nn, optim, train
from ferrotorch_b200.vision import Mnist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--epochs", type=int, default=3)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--samples", type=int, default=2048)
    ap.add_argument("--out", default=None, help="directory for checkpoints and TensorBoard events (default: a new temporary directory)")
    a = ap.parse_args()
    torch.manual_seed(0)
    ds = Mnist.synthetic(a.samples)
    loader = data.DataLoader(ds, batch_size=64, shuffle=True, seed=0)
    model = nn.Sequential(nn.Conv2d(1, 16, 3, padding=1), nn.BatchNorm2d(16), nn.ReLU(), nn.MaxPool2d(2), nn.Conv2d(16, 32, 3, padding=1), nn.ReLU(),
                          nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(32, 10)).to(a.device)
    opt = optim.AdamW(model.parameters(), lr=3e-3)
    out = Path(a.out) if a.out else Path(tempfile.mkdtemp(prefix="ft_mnist_"))
    out.mkdir(parents=True, exist_ok=True)
    learner = train.Learner(model, opt, nn.CrossEntropyLoss(), device=a.device, metrics=[train.AccuracyMetric()],
                            callbacks=[train.ProgressLogger(), train.TensorBoardCallback(str(out / "tb"))]).with_checkpointing(str(out / "ckpt"))
    hist = learner.fit(loader, epochs=a.epochs)
    print("final:", hist.epochs[-1] if hasattr(hist, "epochs") else hist, "artifacts in", out)


if __name__ == "__main__":
    main()
