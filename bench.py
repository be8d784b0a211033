#!/usr/bin/env python
"""Headline benchmark: Llama-3-8B FSDP (full-shard) pretraining throughput in tokens/s.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Model: 32 layers, d_model 4096, 32 query / 8 KV heads (head_dim 128), SwiGLU FFN 14336, vocab 128256, RoPE theta 5e5,
RMSNorm eps 1e-5, random N(0, 0.02) weights, bf16 compute with f32 master weights and AdamW moments
(lr 3e-4, betas 0.9/0.95). Data: synthetic token ids uniform in [0, 128256), seq 4096, micro-batch 1 per GPU (weak scaling).
One step = forward + backward + gradient reduce-scatter + sharded AdamW + parameter all-gather.

Rank 0 prints one JSON line. `value` is device-timed (CUDA events, max over ranks) with the inputs resident on the
device; `e2e` times the same steps through the public API with the per-step host->device copy of the inputs from
pinned memory and the device->host read of the loss inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")


def _parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (the JSON line then says so and is not a headline number)")
    ap.add_argument("--comm", default=None, choices=[None, "nccl", "fused"])
    ap.add_argument("--strategy", default="full_shard", choices=["full_shard", "shard_grad_op"],
                    help="full_shard (ZeRO-3, the configuration the headline names): bf16 parameters sharded and gathered per unit for forward "
                         "and backward; shard_grad_op (ZeRO-2): a replicated bf16 copy stays resident and is refreshed by the update kernel")
    ap.add_argument("--breakdown", action="store_true",
                    help="after the timed runs, time every kernel class of one step with CUDA events (optimizer serialised on the compute "
                         "stream so that the classes add up to the step) and add the table to the JSON line")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "power_w_max": max(power) if power else None, "samples": len(sm)}


def reference_arm(args):
    # The reference is a Rust/Cargo workspace: pip cannot install it ("Neither 'setup.py' nor 'pyproject.toml' found") and
    # neither cargo nor rustc exists in this image; it also has no GPU FSDP path (its FSDP runs on host vectors over TCP).
    print(json.dumps({"impl": "reference", "unavailable": "reference is a Rust workspace: not pip-installable "
                      "(no setup.py/pyproject.toml), no cargo/rustc offline, and it has no GPU FSDP/bf16 training path"}))
    return 0


def _classify(name, raw):
    """Kernel class of one native launcher call (GEMMs are split by operand layout: NT = forward, NN = data gradient, TN = weight gradient)."""
    if name in ("ft_gemm_bf16", "ft_gemm_ex"):
        a_mn, b_mn = (raw[10], raw[11]) if name == "ft_gemm_bf16" else (raw[12], raw[13])
        return {(0, 0): "gemm forward", (0, 1): "gemm dgrad", (1, 1): "gemm wgrad", (1, 0): "gemm other"}[(a_mn, b_mn)]
    if name.startswith("ft_flash_fwd"):
        return "attention forward"
    if name.startswith("ft_flash_bwd"):
        return "attention backward"
    if "rmsnorm" in name:
        return "rmsnorm"
    if "rope" in name:
        return "rope"
    if "swiglu" in name:
        return "swiglu"
    if "cross_entropy" in name:
        return "cross entropy"
    if "adamw" in name or "fsdp" in name:
        return "optimizer (+collectives)"
    if "embedding" in name:
        return "embedding"
    return "other kernels (" + name + ")"


def step_breakdown(engine, step_fn, barrier, _lib, torch):
    """One step with every launch of this library bracketed by CUDA events. The side stream is switched off for it, so the classes run one
    after the other and their sum plus the remainder (PyTorch element-wise kernels, allocator, host gaps) is the serialised step time."""
    side, engine.side = engine.side, None
    try:
        for i in range(2):
            step_fn(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step_fn(2)
        e1.record()
        torch.cuda.synchronize()
        plain_ms = e0.elapsed_time(e1)
        _lib.trace_begin(_classify)
        e0.record()
        step_fn(3)
        e1.record()
        table = _lib.trace_end()
        traced_ms = e0.elapsed_time(e1)
    finally:
        engine.side = side
    barrier()
    total = sum(v["ms"] for v in table.values())
    rows = {k: {"ms": round(v["ms"], 3), "calls": v["calls"], "share": round(v["ms"] / traced_ms, 4)}
            for k, v in sorted(table.items(), key=lambda kv: -kv[1]["ms"])}
    rows["remainder (torch element-wise, allocator, host gaps)"] = {"ms": round(traced_ms - total, 3), "calls": None,
                                                                   "share": round((traced_ms - total) / traced_ms, 4)}
    return {"serialised_step_ms": round(plain_ms, 3), "traced_step_ms": round(traced_ms, 3), "classes": rows}


def main():
    args = _parse()
    if args.impl == "reference":
        return reference_arm(args)
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    import ferrotorch_b200 as ft
    from ferrotorch_b200 import _lib
    from ferrotorch_b200.models import LlamaConfig, LlamaForCausalLM
    from ferrotorch_b200.parallel import FSDP, AdamWConfig, ShardingStrategy

    cfg = LlamaConfig.llama3_8b()
    if args.layers is not None:
        cfg.num_hidden_layers = args.layers
    B, S = args.micro_batch, args.seq
    model = LlamaForCausalLM(cfg, device=dev, world=world, rank=rank, seed=0)
    engine = FSDP(model, AdamWConfig(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1), comm=args.comm,
                  strategy=ShardingStrategy(args.strategy))
    torch.cuda.synchronize()
    init_peak_gb = torch.cuda.max_memory_allocated() / 2**30      # includes the unsharded bf16 initialisation every rank starts from
    torch.cuda.reset_peak_memory_stats()

    # synthetic data: a few distinct pinned host batches per rank, cycled
    g = torch.Generator().manual_seed(1234 + rank)
    nb = 4
    host_ids = [torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g).pin_memory() for _ in range(nb)]
    dev_ids = [h.to(dev) for h in host_ids]

    def step_device(i):
        t = dev_ids[i % nb]
        return engine.train_step(t[:, :-1], t[:, 1:])

    def step_e2e(i):
        t = host_ids[i % nb].to(dev, non_blocking=True)
        loss = engine.train_step(t[:, :-1], t[:, 1:])
        return float(loss.cpu())      # device -> host read of the step's result

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    first_loss = None
    for i in range(args.warmup):
        l = step_e2e(i)
        first_loss = l if first_loss is None else first_loss
    engine.synchronize()
    barrier()

    def timed(fn, K):
        sampler = ClockSampler(local)
        sampler.start()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = _lib.launch_calls
        w0 = time.perf_counter()
        e0.record()
        last = None
        for i in range(K):
            last = fn(i)
        engine.synchronize()
        e1.record()
        torch.cuda.synchronize()
        w1 = time.perf_counter()
        ms = e0.elapsed_time(e1)
        launches = _lib.launch_calls - l0
        barrier()
        clocks = sampler.stop()
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, (w1 - w0) * 1e3, launches, clocks, last

    K = args.steps
    ms_dev, _, launches, clocks, last_loss = timed(step_device, K)
    ms_e2e, wall_e2e, _, clocks_e2e, last_e2e = timed(step_e2e, K)
    ms_e2e = max(ms_e2e, wall_e2e) if world == 1 else ms_e2e

    breakdown = None
    if args.breakdown:
        breakdown = step_breakdown(engine, step_device, barrier, _lib, torch)

    tokens_per_step = B * S * world
    value = tokens_per_step * K / (ms_dev / 1e3)
    e2e_value = tokens_per_step * K / (ms_e2e / 1e3)
    status = _lib.read_status()
    import math
    finite = all(v is None or math.isfinite(float(v)) for v in (first_loss, last_loss, last_e2e))
    if world > 1:
        f = torch.tensor([1.0 if finite else 0.0], device=dev)
        dist.all_reduce(f, op=dist.ReduceOp.MIN)
        finite = bool(f.item() > 0.5)
    if not finite or status != 0:
        if rank == 0:
            print(json.dumps({"error": "training diverged or a device-side wait timed out: no headline number", "first_loss": first_loss,
                              "last_loss": float(last_loss) if last_loss is not None else None, "kernel_status": status, "impl": "ours"}))
        if world > 1:
            dist.destroy_process_group()
        return 1
    if world == 1:
        sharding = "single GPU: parameters, gradients and optimizer state whole on the one rank (nothing to shard or gather)"
    elif args.strategy == "full_shard":
        sharding = ("full_shard (ZeRO-3): bf16 parameters, f32 master weights, AdamW moments and reduced gradients sharded over all ranks; every unit is "
                    "gathered into a slot for its forward and again for its backward pass")
    else:
        sharding = ("shard_grad_op (ZeRO-2): f32 master weights, AdamW moments and reduced gradients sharded; a replicated bf16 parameter copy stays "
                    "resident and is refreshed by the all-gather that is part of the update kernel")
    if rank == 0:
        full = args.layers is None and S == 4096 and B == 1
        out = {
            "metric": "llama3_8b_fsdp_train_tokens_per_s" if full else "DEBUG_reduced_config_tokens_per_s",
            "value": round(value, 2), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": args.warmup,
            "ms_per_step": round(ms_dev / K, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init N(0,0.02) weights)",
            "config": {"model": "llama-3-8b" if args.layers is None else f"llama-3-8b-{args.layers}layers", "global_batch": B * world,
                       "seq_len": S, "parallelism": f"fsdp{world}-{args.strategy.replace('_', '-')}", "strategy": args.strategy, "optimizer": "AdamW(lr=3e-4,betas=0.9/0.95), f32 master+moments",
                       "sharding": sharding,
                       "l2": "inputs_larger_than_L2 (16 GB of weights streamed per step)", "comm": engine.comm if world > 1 else "none",
                       "attention_backend": ft.ops.attention.backend()},
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 2), "unit": "tokens/s", "ms_per_step": round(ms_e2e / K, 3),
                    "h2d_bytes_per_step": int(B * (S + 1) * 8), "d2h_bytes_per_step": 4, "clocks": clocks_e2e},
            "gpu_launches": int(launches), "first_loss": first_loss, "last_loss": float(last_loss) if last_loss is not None else None,
            "kernel_status": status, "impl": "ours",
            "mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 2), "mem_gb_during_init": round(init_peak_gb, 2),
            "mem_gb_device_in_use": round((torch.cuda.mem_get_info()[1] - torch.cuda.mem_get_info()[0]) / 2**30, 2),
        }
        if breakdown is not None:
            out["breakdown"] = breakdown
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
