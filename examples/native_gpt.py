#!/usr/bin/env python
"""A two-layer causal transformer language model trained and sampled with the native C++ tensor / autograd core alone (embedding, layer
norm, multi-head attention with a causal mask, GELU MLP, cross-entropy, AdamW): no torch on the path.

    python examples/native_gpt.py [--steps 150] [--threads 4]

The corpus is a short sentence repeated; after a few dozen steps the model continues it letter by letter.
"""
import argparse
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import numpy as np

from ferrotorch_b200 import native as N

TEXT = "the quick brown fox jumps over the lazy dog. " * 40


class Block(N.Module):
    def __init__(self, dim: int, heads: int, rng):
        self.heads = heads
        self.ln1, self.ln2 = N.LayerNorm(dim), N.LayerNorm(dim)
        self.qkv, self.out = N.Linear(dim, 3 * dim, rng=rng), N.Linear(dim, dim, rng=rng)
        self.up, self.down = N.Linear(dim, 4 * dim, rng=rng), N.Linear(4 * dim, dim, rng=rng)

    def forward(self, x, mask):
        B, S, D = x.shape
        H, hd = self.heads, D // self.heads
        qkv = self.qkv(self.ln1(x).reshape(B * S, D)).reshape(B, S, 3, H, hd).permute(2, 0, 3, 1, 4)        # [3, B, H, S, hd]
        q, k, v = qkv[0], qkv[1], qkv[2]
        att = ((q @ k.transpose(2, 3)) * (1.0 / np.sqrt(hd)) + mask).softmax()
        o = (att @ v).permute(0, 2, 1, 3).reshape(B * S, D)
        x = x + self.out(o).reshape(B, S, D)
        return x + self.down(self.up(self.ln2(x).reshape(B * S, D)).gelu()).reshape(B, S, D)


class TinyGPT(N.Module):
    def __init__(self, vocab: int, dim: int = 48, heads: int = 4, layers: int = 2, ctx: int = 32, seed: int = 0):
        rng = np.random.default_rng(seed)
        self.tok, self.pos = N.Embedding(vocab, dim, rng=rng), N.Embedding(ctx, dim, rng=rng)
        self.blocks = [Block(dim, heads, rng) for _ in range(layers)]
        self.ln, self.head = N.LayerNorm(dim), N.Linear(dim, vocab, rng=rng)
        for p in (self.tok.weight, self.pos.weight):                      # small embeddings start the residual stream near zero
            p.numpy()[...] *= 0.1

    def forward(self, ids):
        B, S = ids.shape
        x = self.tok(ids) + self.pos(np.arange(S))
        mask = N.Tensor(np.triu(np.full((S, S), -1e4, np.float32), 1))
        for b in self.blocks:
            x = b(x, mask)
        return self.head(self.ln(x).reshape(B * S, x.shape[2]))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=150)
    ap.add_argument("--threads", type=int, default=4)
    a = ap.parse_args()
    chars = sorted(set(TEXT))
    stoi = {c: i for i, c in enumerate(chars)}
    data = np.array([stoi[c] for c in TEXT])
    ctx, batch = 32, 16
    model = TinyGPT(len(chars), ctx=ctx)
    opt = N.AdamW(model.parameters(), lr=3e-3, weight_decay=0.01)
    rng = np.random.default_rng(1)
    t0 = time.perf_counter()
    for step in range(a.steps):
        starts = rng.integers(0, len(data) - ctx - 1, batch)
        x = np.stack([data[s: s + ctx] for s in starts])
        y = np.stack([data[s + 1: s + ctx + 1] for s in starts]).reshape(-1)
        opt.zero_grad()
        loss = N.cross_entropy(model(x), y)
        loss.backward(threads=a.threads)
        opt.step()
        if step % 25 == 0 or step == a.steps - 1:
            print(f"step {step:3d}  loss {loss.item():.4f}")
    print(f"{(time.perf_counter() - t0) / a.steps * 1e3:.1f} ms per step, {len(model.parameters())} parameter tensors")
    seq = [stoi[c] for c in "the quick "]
    with N.no_grad():
        for _ in range(35):
            logits = model(np.array([seq[-ctx:]])).numpy()
            seq.append(int(logits[-1].argmax()))
    print("sample:", "".join(chars[i] for i in seq))


if __name__ == "__main__":
    main()
