#!/usr/bin/env python
"""Data-parallel ResNet training step loop (bf16 autocast, channels-last, fused bucket all-reduce overlapped with backward).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 examples/ddp_resnet.py [--model resnet18 --steps 20]

Counterpart of the reference's DDP example path (ferrotorch-distributed/src/ddp.rs:38) on the vision zoo.
"""
import argparse
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="resnet18")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--batch", type=int, default=64)
    a = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from ferrotorch_b200 import nn, optim, vision
    from ferrotorch_b200.parallel import DDP
    torch.manual_seed(0)
    model = vision.get_model(a.model, num_classes=100).to(dev).to(memory_format=torch.channels_last)
    ddp = DDP(model)
    opt = optim.Sgd(model.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4)
    g = torch.Generator(device=dev).manual_seed(rank)
    x = torch.randn(a.batch, 3, 128, 128, device=dev, generator=g).contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 100, (a.batch,), device=dev, generator=g)
    for step in range(a.steps):
        ddp.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(ddp(x).float(), y)
        loss.backward()
        opt.step()
        if rank == 0 and step % 5 == 0:
            print(f"step {step}: loss {float(loss.detach()):.4f}")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
