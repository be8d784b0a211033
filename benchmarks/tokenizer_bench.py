#!/usr/bin/env python
"""Tokenizer throughput: the native merge engine against the direct Python loop and the HF ``tokenizers`` library (what the reference wraps,
ferrotorch-tokenize/src/lib.rs:85-131), on a byte-level BPE trained on this package's own sources.

    python benchmarks/tokenizer_bench.py [--vocab 8000] [--repeat 3]

Prints one JSON line: MB/s of one long text (`encode`) and of a batch of files (`encode_batch`, threads), best of ``repeat`` runs; the Python loop
is timed with an empty per-word cache (first pass over new text) and with a warm one.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import sys
import tempfile
import time
from pathlib import Path


def best(fn, repeat):
    ts = []
    for _ in range(repeat):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    return min(ts)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--vocab", type=int, default=8000)
    ap.add_argument("--repeat", type=int, default=3)
    a = ap.parse_args()
    root = Path(__file__).resolve().parent.parent
    sys.path.insert(0, str(root))
    import tokenizers as tk
    from tokenizers import decoders, models, pre_tokenizers, trainers
    from ferrotorch_b200 import tokenize
    files = sorted(glob.glob(str(root / "ferrotorch_b200" / "**" / "*.py"), recursive=True))
    hf = tk.Tokenizer(models.BPE())
    hf.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    hf.decoder = decoders.ByteLevel()
    hf.train(files[::2], trainers.BpeTrainer(vocab_size=a.vocab, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False))
    with tempfile.TemporaryDirectory() as d:
        hf.save(str(Path(d) / "tokenizer.json"))
        ours = tokenize.load_tokenizer(d)
        os.environ["FT_TOKENIZE_NATIVE"] = "0"
        loop = tokenize.load_tokenizer(d)
        del os.environ["FT_TOKENIZE_NATIVE"]
    texts = [Path(f).read_text() for f in files]
    one = "\n".join(texts)
    mb = len(one.encode()) / 1e6
    assert ours._native is not None and loop._native is None
    assert ours.encode(one) == hf.encode(one).ids
    assert ours.encode_batch(texts) == [e.ids for e in hf.encode_batch(texts)]

    def cold():
        loop._cache.clear()
        loop.encode(one)
    res = {"bench": "tokenizer", "corpus_mb": round(mb, 2), "files": len(texts), "vocab": a.vocab, "cpus": os.cpu_count(),
           "python_loop_cold_mb_s": round(mb / best(cold, a.repeat), 2),
           "python_loop_warm_mb_s": round(mb / best(lambda: loop.encode(one), a.repeat), 2),
           "native_encode_mb_s": round(mb / best(lambda: ours.encode(one), a.repeat), 2),
           "native_encode_batch_mb_s": round(mb / best(lambda: ours.encode_batch(texts), a.repeat), 2),
           "hf_encode_mb_s": round(mb / best(lambda: hf.encode(one), a.repeat), 2),
           "hf_encode_batch_mb_s": round(mb / best(lambda: hf.encode_batch(texts), a.repeat), 2)}
    print(json.dumps(res))


if __name__ == "__main__":
    main()
