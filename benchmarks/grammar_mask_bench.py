#!/usr/bin/env python
"""Per-step cost of the JSON-schema token mask: native walk over the vocabulary against the Python matcher.

    python benchmarks/grammar_mask_bench.py [--vocab 128256]

The vocabulary is synthetic but shaped like a byte-level BPE one: every printable character, JSON fragments, and random short strings of
letters, digits, blanks and punctuation. The mask is computed at four positions of a growing document (inside a key, inside a string, after
a number, between elements); one JSON line with milliseconds per mask.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import statistics
import sys
import time
from pathlib import Path


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--threads", type=int, default=1, help="worker threads of the native walk")
    ap.add_argument("--python-vocab", type=int, default=8192, help="entries the Python matcher is timed on (scaled to --vocab in the output)")
    a = ap.parse_args()
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    from ferrotorch_b200 import grammar as G
    rng = random.Random(0)
    alphabet = "abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789      .,:;-_\"'{}[]()\n"
    vocab = [chr(c) for c in range(32, 127)] + ["{\"", "\":", "\": ", "\",", "\", \"", "},", "],", "true", "false", "null"]
    seen = set(vocab)
    while len(vocab) < a.vocab - 1:
        t = "".join(rng.choice(alphabet) for _ in range(rng.randint(2, 8)))
        if t not in seen:
            seen.add(t)
            vocab.append(t)
    vocab.append("<eos>")
    schema = {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"}, "scores": {"type": "array", "items": {"type": "number"}},
                                               "address": {"type": "object", "properties": {"city": {"type": "string"}, "zip": {"type": "string"}}, "required": ["city"]}},
              "required": ["name", "age"]}
    texts = ['{"na', '{"name": "Ada Lovelace, first of her', '{"name": "Ada", "age": 36', '{"name": "Ada", "age": 36, "scores": [1.5, 2.25, ',
             '{"name": "Ada", "age": 36, "scores": [1.5, 2.25, 3], "address": {"city": "London", "zip": "N1 9GU"}}']
    proc = G.JsonSchemaProcessor(schema, vocab, eos_id=len(vocab) - 1)
    assert proc._native is not None
    proc.threads = a.threads
    os.environ["FT_GRAMMAR_NATIVE"] = "0"
    small = G.JsonSchemaProcessor(schema, vocab[: a.python_vocab] + ["<eos>"], eos_id=a.python_vocab)
    nat, py, allowed = [], [], []
    for t in texts:
        proc.text = small.text = t
        ts = []
        for _ in range(5):
            t0 = time.perf_counter()
            m = proc.mask()
            ts.append(time.perf_counter() - t0)
        nat.append(statistics.median(ts) * 1e3)
        allowed.append(m.count())
        t0 = time.perf_counter()
        mp = small._mask_py()
        py.append((time.perf_counter() - t0) * 1e3 * a.vocab / (a.python_vocab + 1))
        assert bool((mp.allowed[: a.python_vocab] == m.allowed[: a.python_vocab]).all())
    print(json.dumps({"bench": "json_schema_token_mask", "vocab": len(vocab), "cpus": os.cpu_count(), "threads": a.threads, "positions": len(texts), "allowed": allowed,
                      "native_ms_per_mask": [round(x, 2) for x in nat], "python_ms_per_mask_scaled": [round(x, 1) for x in py],
                      "speedup_median": round(statistics.median(p / n for p, n in zip(py, nat)), 1)}))


if __name__ == "__main__":
    main()
