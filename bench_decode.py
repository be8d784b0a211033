#!/usr/bin/env python
"""Serving benchmark: Llama-3-70B tensor-parallel greedy decoding throughput (tokens/s over the whole batch).

    python bench_decode.py --gpus 1 --decode 64
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P bench_decode.py --gpus 8

Model: 80 layers, d_model 8192, 64 query / 8 KV heads (head_dim 128), SwiGLU FFN 28672, vocab 128256, random N(0,0.02) bf16 weights.
Workload: batch 8 prompts of 2048 uniform-random token ids, prefill, then greedy decode of 256 tokens with a paged KV cache
(block 16). The decode loop replays one captured CUDA graph per token. `value` = batch * decoded tokens / device time of the
decode loop (CUDA events, max over ranks); prefill time is reported separately. The tensor-parallel degree is the number of GPUs.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--model", default="70b", choices=["70b", "8b"])
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--decode", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--ab-ar", action="store_true", help="after the timed run, time the same steps again with the other all-reduce+norm kernel form")
    ap.add_argument("--profile", action="store_true", help="after the timed run, report eager per-kernel-class device time per step")
    a = ap.parse_args()
    import torch
    import torch.distributed as dist
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    from ferrotorch_b200 import _lib
    from ferrotorch_b200.models import LlamaConfig
    from ferrotorch_b200.models.llama_infer import LlamaTPEngine, TPContext
    cfg = LlamaConfig.llama3_70b() if a.model == "70b" else LlamaConfig.llama3_8b()
    if a.layers is not None:
        cfg.num_hidden_layers = a.layers
    eng = LlamaTPEngine(cfg, TPContext(dev), max_batch=a.batch, max_seq=a.prompt + (a.decode + a.warmup) * (2 if a.ab_ar else 1) + 8, device=dev, seed=0, use_graph=not a.no_graph)
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, cfg.vocab_size, (a.batch, a.prompt), generator=g).to(dev)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    eng.prefill(ids)
    e1.record()
    sync()
    prefill_ms = e0.elapsed_time(e1)
    for _ in range(a.warmup):
        eng.decode_step()
    sync()
    l0 = _lib.launch_calls
    e0.record()
    for _ in range(a.decode):
        eng.decode_step()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms, prefill_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, prefill_ms = float(t[0]), float(t[1])
    alt = None
    if a.ab_ar:
        eng.ar_cluster, eng.graph = not eng.ar_cluster, None
        for _ in range(a.warmup):
            eng.decode_step()
        sync()
        e0.record()
        for _ in range(a.decode):
            eng.decode_step()
        e1.record()
        sync()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        alt = {"ar_form": "cluster" if eng.ar_cluster else "grid-barrier", "ms_per_step": round(float(t[0]) / a.decode, 4)}
        eng.ar_cluster, eng.graph = not eng.ar_cluster, None
    breakdown = None
    if a.profile:
        prof = eng.profile_decode(8)                     # eager launches with CUDA events around each kernel class (after the timed region)
        breakdown = {k: round(v, 1) for k, v in sorted(prof.items(), key=lambda kv: -kv[1])}
    status = _lib.read_status()
    if rank == 0:
        full = a.layers is None and a.model == "70b" and a.batch == 8 and a.prompt == 2048
        weight_bytes = sum(L[k].numel() * 2 for L in eng.layers for k in ("wqkv", "wo", "wgu", "wd")) + eng.lm_head.numel() * 2
        print(json.dumps({
            "metric": "llama3_70b_tp_decode_tokens_per_s" if full else "DEBUG_reduced_config_decode_tokens_per_s",
            "value": round(a.batch * a.decode / (ms / 1e3), 2), "unit": "tokens/s", "n_gpus": world, "steps": a.decode, "warmup": a.warmup,
            "ms_per_step": round(ms / a.decode, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (uniform random prompt ids, random-init N(0,0.02) weights)",
            "config": {"model": f"llama-3-{a.model}" + (f"-{a.layers}layers" if a.layers else ""), "batch": a.batch, "prompt_len": a.prompt,
                       "decode_len": a.decode, "parallelism": f"tp{world}", "kv_cache": "paged, block 16", "cuda_graph": not a.no_graph,
                       "l2": "weights streamed per step exceed L2"},
            "prefill_ms": round(prefill_ms, 2), "prefill_tokens_per_s": round(a.batch * a.prompt / (prefill_ms / 1e3), 1),
            "weight_bytes_per_gpu": weight_bytes, "hbm_gbs_streamed": round(weight_bytes / (ms / a.decode / 1e3) / 1e9, 1),
            "gpu_launches": (_lib.launch_calls - l0) if a.no_graph else "graph replay", "kernel_status": status, "impl": "ours",
            **({"eager_us_per_step_by_kernel": breakdown} if breakdown else {}), **({"other_allreduce_form": alt} if alt else {}),
        }))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
