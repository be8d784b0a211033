#!/usr/bin/env python
"""SafeTensors load times for the two cases the reference publishes (CHANGELOG.md:36-40 of the reference: a 3.4 GB f32 file, 315-379 s; a
300 MB bf16 file, 0.205 s parallel / 0.237 s serial, on a 16-core machine): synthetic files of those sizes, written and read back through
``ferrotorch_b200.serialize``. A load is timed until every tensor is materialised in ordinary (non-mapped) memory and checksummed, so a lazy
mapping does not count as loaded.

    python benchmarks/safetensors_bench.py [--dir /tmp] [--skip-large]
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dir", default="/tmp")
    ap.add_argument("--skip-large", action="store_true")
    a = ap.parse_args()
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    from ferrotorch_b200.serialize import load_safetensors, save_safetensors
    cases = [("bf16 300 MB", torch.bfloat16, 150, (1024, 1024), 0.205)]
    if not a.skip_large:
        cases.append(("f32 3.4 GB (UNet-sized)", torch.float32, 212, (2048, 2048), 315.0))
    out = []
    for name, dtype, n, shape, ref_s in cases:
        g = torch.Generator().manual_seed(0)
        state = {f"block{i}.weight": torch.randn(*shape, generator=g).to(dtype) for i in range(n)}
        path = os.path.join(a.dir, f"ft_bench_{dtype}.safetensors".replace("torch.", ""))
        t0 = time.perf_counter()
        save_safetensors(state, path)
        save_s = time.perf_counter() - t0
        want = {k: int(v.view(torch.int16 if dtype == torch.bfloat16 else torch.int32)[0, 0]) for k, v in state.items()}
        del state
        best = {}
        for parallel in (True, False):
            ts = []
            for _ in range(3):
                t0 = time.perf_counter()
                d = load_safetensors(path, parallel=parallel)
                d = {k: v.clone() for k, v in d.items()}                 # off the mapping, into ordinary memory
                ts.append(time.perf_counter() - t0)
                assert all(int(v.view(torch.int16 if dtype == torch.bfloat16 else torch.int32)[0, 0]) == want[k] for k, v in d.items())
                del d
            best[parallel] = min(ts)
        r = {"case": name, "file_mb": round(os.path.getsize(path) / 1e6, 1), "save_s": round(save_s, 3), "load_parallel_s": round(best[True], 4),
             "load_serial_s": round(best[False], 4), "reference_published_s": ref_s, "speedup_vs_reference": round(ref_s / min(best.values()), 1)}
        out.append(r)
        print(json.dumps(r), flush=True)
        os.remove(path)


if __name__ == "__main__":
    main()
