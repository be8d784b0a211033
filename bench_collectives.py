#!/usr/bin/env python
"""Collective sweep: all-reduce, reduce-scatter and all-gather, bf16 and f32, 1 KB - 1 GB in powers of two, peer-memory kernels vs NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench_collectives.py

Values ~U(-1, 1) from seed 0 (+ rank). Sizes are nccl-tests sizes: the whole vector for all-reduce, the gathered / scattered vector
(world x chunk) for all-gather / reduce-scatter. Bus bandwidth = size x f / time with f = 2(n-1)/n for all-reduce and (n-1)/n for the
other two, reported against 900 GB/s per direction (nominal) and 770 GB/s (peer copy measured on this pool). Every time is device-timed
with CUDA events around ``iters`` back-to-back launches after ``warmup`` launches, and is the maximum over ranks.

This framework's side: one-shot all-reduce (every rank reads all peers' vectors) up to ``--oneshot-bytes``, the two-shot kernel
(NVLS multimem for bf16 when the buffer has a multicast mapping) above it; reduce-scatter pulls its slice from every peer in fixed rank
order; all-gather pushes the local chunk into every peer's buffer. One JSON line per (collective, dtype, size), then one summary line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", type=int, default=1 << 10)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--oneshot-bytes", type=int, default=256 << 10)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--ops", default="all_reduce,reduce_scatter,all_gather")
    ap.add_argument("--dtypes", default="bf16,f32")
    ap.add_argument("--no-nvls", action="store_true")
    a = ap.parse_args()
    import torch
    import torch.distributed as dist
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        print(json.dumps({"bench": "collectives", "unavailable": "needs at least 2 ranks (launch with torch.distributed.run)"}))
        return 0
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    from ferrotorch_b200 import _lib
    from ferrotorch_b200.parallel.symm import SymmComm, SymmetricBuffer
    comm = SymmComm(dev)
    results = []

    def timed(fn, iters):
        for _ in range(a.warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    for dname in a.dtypes.split(","):
        dtype = {"bf16": torch.bfloat16, "f32": torch.float32}[dname]
        isz = 2 if dtype == torch.bfloat16 else 4
        nmax = a.max_bytes // isz
        g = torch.Generator(device=dev).manual_seed(rank)
        buf = SymmetricBuffer(nmax, dtype, dev)
        src = (torch.rand(nmax, device=dev, generator=g) * 2 - 1).to(dtype)
        out = torch.empty(nmax, device=dev, dtype=dtype)
        lib_in = src.clone()
        lib_out = torch.empty(nmax, device=dev, dtype=dtype)
        for op in a.ops.split(","):
            size = a.min_bytes
            while size <= a.max_bytes:
                n = size // isz
                chunk = n // world
                vec = 16 // isz
                if chunk % vec or chunk == 0:
                    size *= 2
                    continue
                iters = 50 if size <= (1 << 20) else (20 if size <= (64 << 20) else 5)
                buf.tensor[:n].copy_(src[:n])
                if op == "all_reduce":
                    form = "one-shot" if size <= a.oneshot_bytes else ("two-shot" + ("" if (a.no_nvls or not buf.multicast_ptr) else " nvls"))
                    if size <= a.oneshot_bytes:
                        ours = lambda: comm.all_reduce_small(buf, out, n)
                    else:
                        ours = lambda: comm.all_reduce_(buf, n, use_nvls=not a.no_nvls)
                    lib = lambda: dist.all_reduce(lib_in[:n])
                    factor = 2.0 * (world - 1) / world
                elif op == "reduce_scatter":
                    form = "pull" if (a.no_nvls or not buf.multicast_ptr) else "nvls"
                    ours = lambda: comm.reduce_scatter(buf, out[:chunk], chunk, use_nvls=not a.no_nvls)
                    lib = lambda: dist.reduce_scatter_tensor(lib_out[:chunk], lib_in[:n])
                    factor = (world - 1) / world
                else:
                    form = "push"
                    ours = lambda: comm.all_gather(buf, src[:chunk], chunk)
                    lib = lambda: dist.all_gather_into_tensor(lib_out[:n], lib_in[:chunk])
                    factor = (world - 1) / world
                t_ours = timed(ours, iters)
                lib_in[:n].copy_(src[:n])          # the in-place library all-reduce grows its input: start every size from the same values
                t_lib = timed(lib, iters)
                r = {"bench": "collectives", "op": op, "dtype": dname, "bytes": size, "n_gpus": world, "form": form,
                     "ours_us": round(t_ours * 1e3, 2), "nccl_us": round(t_lib * 1e3, 2),
                     "ours_busbw_gbs": round(size * factor / (t_ours * 1e-3) / 1e9, 2), "nccl_busbw_gbs": round(size * factor / (t_lib * 1e-3) / 1e9, 2),
                     "speedup_vs_nccl": round(t_lib / t_ours, 3)}
                r["ours_frac_of_900"] = round(r["ours_busbw_gbs"] / 900.0, 3)
                r["ours_frac_of_measured_770"] = round(r["ours_busbw_gbs"] / 770.0, 3)
                results.append(r)
                if rank == 0:
                    print(json.dumps(r), flush=True)
                size *= 2
        del buf, src, out, lib_in, lib_out
        torch.cuda.empty_cache()
    status = _lib.read_status()
    if rank == 0:
        best = {}
        for r in results:
            k = f"{r['op']}/{r['dtype']}"
            if k not in best or r["ours_busbw_gbs"] > best[k]["ours_busbw_gbs"]:
                best[k] = r
        print(json.dumps({"bench": "collectives_summary", "n_gpus": world, "kernel_status": status,
                          "peak_busbw_gbs": {k: {"ours": v["ours_busbw_gbs"], "nccl_same_size": v["nccl_busbw_gbs"], "bytes": v["bytes"]} for k, v in best.items()},
                          "sizes_where_ours_is_faster": sum(1 for r in results if r["speedup_vs_nccl"] > 1.0), "sizes": len(results),
                          "timing": "CUDA events, max over ranks; sizes above 126 MB exceed L2, smaller ones are deliberately latency-regime"}))
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
