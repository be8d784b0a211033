#!/usr/bin/env python
"""Fused tensor-parallel GEMMs vs the unfused library sequence, device-timed (max over ranks), against the roofline
max(FLOPs / measured GEMM peak, NVLink bytes / measured peer bandwidth).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench_tp_gemm.py [--tokens 8192 --hidden 8192]

Shapes: all-gather->GEMM  x[tokens/N, hidden] shards, w[hidden/N, hidden]  -> y[tokens, hidden/N]
        GEMM->reduce-scatter x[tokens, hidden/N], w[hidden, hidden/N]       -> y[tokens/N, hidden]
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--ncopy", type=int, default=0, help="copier CTAs of the all-gather GEMM (0 = kernel default)")
    a = ap.parse_args()
    import torch
    import torch.distributed as dist
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29631")
    dist.init_process_group("nccl", device_id=dev, rank=rank, world_size=world)
    from ferrotorch_b200 import _lib, ops
    from ferrotorch_b200.parallel.tp import TpGemmContext
    from ferrotorch_b200.utils.kbench import flush_l2, peaks
    pk = peaks()
    M, H = a.tokens, a.hidden
    torch.manual_seed(rank)
    xs = (torch.randn(M // world, H, device=dev) * 0.1).bfloat16()
    w_col = (torch.randn(H // world, H, device=dev) * 0.02).bfloat16()
    x_row = (torch.randn(M, H // world, device=dev) * 0.1).bfloat16()
    w_row = (torch.randn(H, H // world, device=dev) * 0.02).bfloat16()
    ag = TpGemmContext("ag_gemm", M, H // world, H, dev, ncopy=a.ncopy)
    rs = TpGemmContext("gemm_rs", M, H, H // world, dev)
    ag.shard_view().copy_(xs)
    gathered, y_rs = torch.empty(M, H, device=dev, dtype=torch.bfloat16), torch.empty(M // world, H, device=dev, dtype=torch.bfloat16)
    y_col, part = torch.empty(M, H // world, device=dev, dtype=torch.bfloat16), torch.empty(M, H, device=dev, dtype=torch.bfloat16)

    def lib_ag():
        dist.all_gather_into_tensor(gathered, xs)
        ops.gemm(gathered, w_col, out=y_col)

    def lib_rs():
        ops.gemm(x_row, w_row, out=part)
        dist.reduce_scatter_tensor(y_rs, part)

    def timeit(fn):
        for _ in range(a.warmup):
            fn()
        ts = []
        for _ in range(a.iters):
            flush_l2()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts.append(float(t))
        ts.sort()
        return ts[len(ts) // 2]
    res = {"fused_ag_gemm_ms": timeit(lambda: ag.ag_gemm(None, w_col, y_col)), "nccl_ag_then_gemm_ms": timeit(lib_ag),
           "fused_gemm_rs_ms": timeit(lambda: rs.gemm_rs(x_row, w_row, y_rs)), "gemm_then_nccl_rs_ms": timeit(lib_rs),
           "gemm_only_col_ms": timeit(lambda: ops.gemm(gathered, w_col, out=y_col)), "gemm_only_row_ms": timeit(lambda: ops.gemm(x_row, w_row, out=part))}
    flops = 2.0 * M * H * H / world
    link = 770e9
    nv_bytes = (world - 1) / world * M * H * 2
    roof = max(flops / (pk["bf16_tflops"] * 1e12), nv_bytes / link) * 1e3
    st = _lib.read_status()
    if rank == 0:
        print(json.dumps({"bench": "tp_fused_gemm", "n_gpus": world, "tokens": M, "hidden": H, **{k: round(v, 4) for k, v in res.items()},
                          "roofline_ms": round(roof, 4), "compute_ms_at_measured_peak": round(flops / (pk["bf16_tflops"] * 1e12) * 1e3, 4),
                          "nvlink_ms_at_770GBs": round(nv_bytes / link * 1e3, 4), "ag_gemm_frac_of_roofline": round(roof / res["fused_ag_gemm_ms"], 3),
                          "gemm_rs_frac_of_roofline": round(roof / res["fused_gemm_rs_ms"], 3), "speedup_ag": round(res["nccl_ag_then_gemm_ms"] / res["fused_ag_gemm_ms"], 3),
                          "speedup_rs": round(res["gemm_then_nccl_rs_ms"] / res["fused_gemm_rs_ms"], 3), "kernel_status": st, "peaks": pk}))
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
