#!/usr/bin/env python
"""Same-box yardstick: the library path (PyTorch eager + cuBLAS / cuDNN / SDPA + NCCL) on the configurations of the headline benchmarks.

This is NOT the reference arm of ``bench.py`` (the reference is a Rust workspace and cannot be built here); it answers a different question:
what does a stock PyTorch program reach on this box for the same model, shapes, synthetic data and optimizer, with nothing of this
repository on the path?

    python bench_library.py llama  --steps 5 --warmup 3                       # Llama-3-8B, 1 GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P bench_library.py llama --gpus 8
    python bench_library.py resnet --steps 10 --warmup 3                      # ResNet-50, batch 256 per GPU
    python -m torch.distributed.run ... bench_library.py resnet --gpus 8

llama:  transformers.LlamaForCausalLM (random N(0, 0.02) init, SDPA attention), seq 4096, micro-batch 1 per GPU, AdamW lr 3e-4 betas 0.9/0.95.
        N > 1: FSDP2 ``fully_shard`` per decoder layer, f32 sharded parameters, bf16 compute (MixedPrecisionPolicy), fused AdamW.
        N = 1: ``--master f32`` (f32 parameters + autocast, the closest match to the engine's f32 master weights) needs ~170 GB and is refused by
        default; the default ``--master bf16`` keeps bf16 parameters and bf16 AdamW state (less memory traffic than the engine's step).
resnet: torchvision-style ResNet-50 (the repository's model definition is not used: ``torch.nn`` layers only), channels-last, bf16 autocast,
        SGD lr 0.1 momentum 0.9 wd 1e-4, DistributedDataParallel with 25 MB buckets for N > 1.

Timing as in bench.py: W warm-up steps, K steps between CUDA events after a barrier + synchronize, max over ranks. One JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")


def _setup():
    import torch
    import torch.distributed as dist
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    return torch, dist, world, rank, dev


def _timed(torch, dist, world, dev, step, K):
    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    last = None
    for i in range(K):
        last = step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    barrier()
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, float(last)


def llama(args):
    torch, dist, world, rank, dev = _setup()
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=args.layers or 32, num_attention_heads=32,
                      num_key_value_heads=8, rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8192, tie_word_embeddings=False,
                      attn_implementation="sdpa", use_cache=False)
    B, S = 1, 4096
    torch.manual_seed(0)
    master = args.master if world == 1 else "f32"
    pdt = torch.float32 if master == "f32" else torch.bfloat16
    with torch.device(dev):
        model = LlamaForCausalLM(cfg).to(pdt)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() > 1:
                p.normal_(0.0, 0.02)
    model.train()
    if world > 1:
        from torch.distributed.fsdp import fully_shard, MixedPrecisionPolicy
        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16)
        for layer in model.model.layers:
            fully_shard(layer, mp_policy=mp)
        fully_shard(model, mp_policy=mp)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True)
    g = torch.Generator().manual_seed(1234 + rank)
    batches = [torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g).to(dev) for _ in range(4)]
    autocast = world == 1 and master == "f32"

    def step(i):
        t = batches[i % 4]
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=autocast):
            loss = model(input_ids=t[:, :-1], labels=None).logits
            loss = torch.nn.functional.cross_entropy(loss.float().view(-1, cfg.vocab_size), t[:, 1:].reshape(-1))
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss.detach()
    for i in range(args.warmup):
        step(i)
    ms, last = _timed(torch, dist, world, dev, step, args.steps)
    if rank == 0:
        full = args.layers is None
        print(json.dumps({"impl": "library (PyTorch eager, transformers LlamaForCausalLM, SDPA, cuBLAS, " + ("FSDP2 fully_shard + NCCL" if world > 1 else "single GPU") + ")",
                          "metric": "llama3_8b_fsdp_train_tokens_per_s" if full else "DEBUG_reduced_config_tokens_per_s",
                          "value": round(B * S * world * args.steps / (ms / 1e3), 2), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3), "dtype": "bf16",
                          "config": {"model": "llama-3-8b", "seq_len": S, "global_batch": B * world,
                                     "parameters": "f32 master, bf16 compute" if master == "f32" else "bf16 parameters and bf16 AdamW state (no f32 master)",
                                     "optimizer": "torch.optim.AdamW(fused=True)", "parallelism": f"fsdp2-{world}" if world > 1 else "none"},
                          "last_loss": last, "mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 2), "torch": torch.__version__}))
    if world > 1:
        dist.destroy_process_group()
    return 0


def _resnet50(nn):
    class Bottleneck(nn.Module):
        def __init__(self, cin, width, stride):
            super().__init__()
            cout = width * 4
            self.c1, self.b1 = nn.Conv2d(cin, width, 1, bias=False), nn.BatchNorm2d(width)
            self.c2, self.b2 = nn.Conv2d(width, width, 3, stride, 1, bias=False), nn.BatchNorm2d(width)
            self.c3, self.b3 = nn.Conv2d(width, cout, 1, bias=False), nn.BatchNorm2d(cout)
            self.down = None
            if stride != 1 or cin != cout:
                self.down = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False), nn.BatchNorm2d(cout))
            self.relu = nn.ReLU(inplace=True)

        def forward(self, x):
            idt = x if self.down is None else self.down(x)
            y = self.relu(self.b1(self.c1(x)))
            y = self.relu(self.b2(self.c2(y)))
            return self.relu(self.b3(self.c3(y)) + idt)

    class ResNet50(nn.Module):
        def __init__(self):
            super().__init__()
            self.stem = nn.Sequential(nn.Conv2d(3, 64, 7, 2, 3, bias=False), nn.BatchNorm2d(64), nn.ReLU(inplace=True), nn.MaxPool2d(3, 2, 1))
            layers, cin = [], 64
            for width, n, stride in ((64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2)):
                for i in range(n):
                    layers.append(Bottleneck(cin, width, stride if i == 0 else 1))
                    cin = width * 4
            self.layers = nn.Sequential(*layers)
            self.fc = nn.Linear(2048, 1000)

        def forward(self, x):
            x = self.layers(self.stem(x))
            return self.fc(x.mean((2, 3)))
    return ResNet50()


def resnet(args):
    torch, dist, world, rank, dev = _setup()
    nn = torch.nn
    torch.backends.cudnn.benchmark = True
    torch.manual_seed(0)
    model = _resnet50(nn).to(dev).to(memory_format=torch.channels_last)
    if world > 1:
        model = nn.parallel.DistributedDataParallel(model, device_ids=[dev.index], bucket_cap_mb=25, gradient_as_bucket_view=True)
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
    B = 256
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    xs = [torch.randn(B, 3, 224, 224, device=dev, generator=g).contiguous(memory_format=torch.channels_last) for _ in range(2)]
    ys = [torch.randint(0, 1000, (B,), device=dev, generator=g) for _ in range(2)]

    def step(i):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = nn.functional.cross_entropy(model(xs[i % 2]).float(), ys[i % 2])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss.detach()
    for i in range(args.warmup):
        step(i)
    ms, last = _timed(torch, dist, world, dev, step, args.steps)
    if rank == 0:
        print(json.dumps({"impl": "library (PyTorch eager, cuDNN, cuBLAS" + (", DistributedDataParallel + NCCL)" if world > 1 else ")"),
                          "metric": "resnet50_ddp_train_images_per_s", "value": round(B * world * args.steps / (ms / 1e3), 1), "unit": "images/s",
                          "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3),
                          "dtype": "bf16 autocast, f32 parameters", "config": {"model": "resnet50", "global_batch": B * world, "image": "224x224x3",
                                                                              "memory_format": "channels_last", "optimizer": "SGD(lr=0.1,momentum=0.9,wd=1e-4)"},
                          "last_loss": last, "torch": torch.__version__}))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["llama", "resnet"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=None, help="debug only")
    ap.add_argument("--master", default="bf16", choices=["bf16", "f32"])
    a = ap.parse_args()
    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "library", "unavailable": "no CUDA device"}))
        return 0
    try:
        return llama(a) if a.what == "llama" else resnet(a)
    except torch.cuda.OutOfMemoryError as e:
        print(json.dumps({"impl": "library", "unavailable": f"out of memory: {str(e)[:200]}"}))
        return 0


if __name__ == "__main__":
    sys.exit(main())
