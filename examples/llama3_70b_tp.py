#!/usr/bin/env python
"""Llama-3 70B across the GPUs of one node, tensor parallel, bf16. Counterpart of ferrotorch-llama/examples/llama3_70b_gpu.rs, which
places the whole model on one device; here every rank holds 1/N of each projection (heads, FFN columns and vocabulary split), the
all-reduces run over NVLink peer memory, and decode steps replay a CUDA graph.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/llama3_70b_tp.py \
        "The meaning of life is" --model-dir /path/to/Llama-3.3-70B-Instruct --new 64
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/llama3_70b_tp.py --preset tiny

Without ``--model-dir`` the weights are random (identical on every rank before slicing). 70B in bf16 is 141 GB: 17.6 GB per GPU at N = 8."""
import argparse
import os
import time

from _model_dir import PRESETS, load_config, load_tok, load_weights, torch

from ferrotorch_b200.models.llama_infer import LlamaTPEngine, TPContext


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("prompt", nargs="?", default="The meaning of life is")
    ap.add_argument("--model-dir")
    ap.add_argument("--preset", choices=sorted(PRESETS), default="llama3.3-70b-instruct")
    ap.add_argument("--new", type=int, default=32)
    ap.add_argument("--batch", type=int, default=1)
    a = ap.parse_args()
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rank = dist.get_rank() if world > 1 else 0
    cfg = load_config(a.model_dir, a.preset)
    tok = load_tok(a.model_dir, cfg)
    ids = tok.encode(a.prompt)
    W = load_weights(a.model_dir, cfg, "cpu", mmap=True) if a.model_dir else None        # random weights are drawn on the device, shard by shard
    t0 = time.time()
    eng = LlamaTPEngine(cfg, TPContext(dev), max_batch=a.batch, max_seq=len(ids) + a.new + 16, device=dev, weights=W)
    torch.cuda.synchronize()
    if rank == 0:
        print(f"tp={world}: weights resident in {time.time() - t0:.1f} s, {torch.cuda.memory_allocated() / 2**30:.1f} GiB on this rank")
    prompt = torch.tensor([ids] * a.batch, device=dev)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    out = eng.generate(prompt, a.new)
    ev1.record()
    torch.cuda.synchronize()
    eng.check()
    if rank == 0:
        ms = ev0.elapsed_time(ev1)
        print(f"{a.new} new tokens x batch {a.batch} in {ms:.1f} ms ({a.batch * a.new / ms * 1e3:.1f} tok/s incl. prefill)")
        print("continuation:", tok.decode(out[0, len(ids):].tolist()))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
