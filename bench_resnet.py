#!/usr/bin/env python
"""ResNet-50 DDP training throughput (images/s over all GPUs).

    python bench_resnet.py --gpus 1
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench_resnet.py --gpus N

bf16 autocast with f32 master weights, 224x224x3 synthetic images ~N(0,1), batch 256 per GPU, labels uniform in [0,1000),
SGD lr 0.1 momentum 0.9 weight decay 1e-4 (fused flat kernel). Gradients are all-reduced in 25 MiB buckets by the peer-memory
all-reduce kernel, overlapped with backward. 1x1 convolutions run on the tcgen05 GEMM (channels-last, split-K weight gradients), batch norm
(+ residual + ReLU) and max pooling on the channels-last kernels, stride-1 3x3 convolutions (forward, input gradient) on the implicit-GEMM
kernel; what still goes through a library is listed in `config.library_ops` (it shrinks with FT_CONV_WGRAD / FT_CONV_ROWS).
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--comm", default=None)
    ap.add_argument("--compute-copies", action="store_true", help="bf16 weight copies maintained by the optimizer instead of a cast per forward")
    a = ap.parse_args()
    import torch
    import torch.distributed as dist
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    from ferrotorch_b200 import _lib, nn, optim
    from ferrotorch_b200.parallel import DDP
    from ferrotorch_b200.vision import resnet50
    torch.manual_seed(0)
    model = resnet50().to(dev).to(memory_format=torch.channels_last)
    if a.compute_copies:
        nn.attach_compute_copies(model)
    ddp = DDP(model, comm=a.comm)
    opt = optim.Sgd(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
    lossf = nn.CrossEntropyLoss()
    g = torch.Generator().manual_seed(rank)
    hx = [torch.randn(a.batch, 3, 224, 224, generator=g).pin_memory() for _ in range(2)]
    hy = [torch.randint(0, 1000, (a.batch,), generator=g).pin_memory() for _ in range(2)]
    dx = [t.to(dev).contiguous(memory_format=torch.channels_last) for t in hx]
    dy = [t.to(dev) for t in hy]

    def step(x, y):
        ddp.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = lossf(ddp(x), y)
        loss.backward()
        opt.step()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    for i in range(a.warmup):
        step(dx[i % 2], dy[i % 2])
    barrier()

    copy_stream = torch.cuda.Stream(device=dev)

    def fetch(i: int):
        with torch.cuda.stream(copy_stream):
            x = hx[i % 2].to(dev, non_blocking=True)
            y = hy[i % 2].to(dev, non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(copy_stream)
        return x, y, ready

    from bench import ClockSampler          # nvidia-smi sampling of SM clock and throttle reasons during the timed region

    def timed(e2e: bool):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = _lib.launch_calls
        barrier()
        sampler = ClockSampler(local)
        sampler.start()
        e0.record()
        last = None
        nxt = fetch(0) if e2e else None
        for i in range(a.steps):
            if e2e:
                # every step's batch crosses PCIe inside the timed region; the copy of batch i+1 is queued on the copy stream before step i
                # is launched, so it runs under step i's kernels
                x, y, ready = nxt
                torch.cuda.current_stream().wait_event(ready)
                x.record_stream(torch.cuda.current_stream())
                y.record_stream(torch.cuda.current_stream())
                if i + 1 < a.steps:
                    nxt = fetch(i + 1)
                last = float(step(x.contiguous(memory_format=torch.channels_last), y).cpu())
            else:
                last = step(dx[i % 2], dy[i % 2])
        e1.record()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms, _lib.launch_calls - l0, last, clocks
    ms, launches, last, clocks = timed(False)
    ms2, _, last2, clocks2 = timed(True)
    from ferrotorch_b200.ops import conv as _conv
    library_ops = []
    if _conv._STEM_MODE != "gemm":
        library_ops.insert(0, "conv 7x7 stem (cuDNN)")
    if _conv._ROWS_MODE not in ("1", "all"):
        library_ops.insert(1, "conv 3x3 stride 2: forward and both gradients (cuDNN)")
    if _conv._WGRAD_MODE not in ("gemm", "fused") and _conv._ROWS_MODE != "all":
        library_ops.insert(1, "conv 3x3 stride 1: weight gradient (cuDNN)")
    if rank == 0:
        print(json.dumps({
            "metric": "resnet50_ddp_train_images_per_s", "value": round(a.batch * world * a.steps / (ms / 1e3), 1), "unit": "images/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms / a.steps, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 autocast, f32 master", "data": "synthetic (N(0,1) images, uniform labels)",
            "config": {"model": "resnet50", "global_batch": a.batch * world, "image": "224x224x3", "parallelism": f"ddp{world}",
                       "optimizer": "SGD(lr=0.1,momentum=0.9,wd=1e-4)", "bucket_mb": 25, "compute_copies": bool(a.compute_copies), "comm": ddp.comm_mode if world > 1 else "none",
                       "library_ops": library_ops, "l2": "inputs_larger_than_L2 (154 MB of images per step)"},
            "e2e": {"value": round(a.batch * world * a.steps / (ms2 / 1e3), 1), "unit": "images/s", "h2d_bytes_per_step": a.batch * (3 * 224 * 224 * 4 + 8),
                    "d2h_bytes_per_step": 4},
            "clocks": clocks, "clocks_e2e": clocks2,
            "gpu_launches": int(launches), "last_loss": float(last), "kernel_status": _lib.read_status(), "impl": "ours"}))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
