#!/usr/bin/env python
"""Llama-3-8B on one GPU in bf16: whole-prompt forward, arg-max of the last position, then greedy decoding through the paged-KV engine
(CUDA-graph decode steps). Counterpart of ferrotorch-llama/examples/llama3_8b_gpu.rs.

    python examples/llama3_8b_gpu.py "The meaning of life is" --model-dir /path/to/Meta-Llama-3-8B --new 32
    python examples/llama3_8b_gpu.py --preset tiny            # random weights, no checkpoint needed

Steps: parse ``config.json`` -> ``LlamaConfig``; load ``tokenizer.json``; load the safetensors shards; ``LlamaGpuInferencer`` keeps every
tensor on the device in bf16 and runs the decoder; ``LlamaTPEngine`` (tensor-parallel degree 1 here) continues the prompt."""
import argparse
import time

from _model_dir import PRESETS, load_config, load_tok, load_weights, torch

from ferrotorch_b200.models import LlamaGpuInferencer
from ferrotorch_b200.models.llama_infer import LlamaTPEngine, TPContext


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("prompt", nargs="?", default="The meaning of life is")
    ap.add_argument("--model-dir")
    ap.add_argument("--preset", choices=sorted(PRESETS), default="llama3-8b")
    ap.add_argument("--new", type=int, default=16)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args()
    cfg = load_config(a.model_dir, a.preset)
    tok = load_tok(a.model_dir, cfg)
    ids = tok.encode(a.prompt)
    t0 = time.time()
    W = load_weights(a.model_dir, cfg, "cpu")
    print(f"config: {cfg.num_hidden_layers} layers, hidden {cfg.hidden_size}, vocab {cfg.vocab_size}; {len(W)} tensors in {time.time() - t0:.1f} s")
    inf = LlamaGpuInferencer(cfg, W, device=a.device, dtype=torch.bfloat16 if a.device != "cpu" else torch.float32)
    t0 = time.time()
    logits = inf.forward_from_ids(ids)
    nxt = int(logits.argmax())
    print(f"prefill of {len(ids)} tokens: {1e3 * (time.time() - t0):.1f} ms; next token {nxt} -> {tok.decode([nxt])!r}")
    if a.device == "cpu" or a.new <= 0:
        return
    del inf
    eng = LlamaTPEngine(cfg, TPContext(a.device), max_batch=1, max_seq=len(ids) + a.new + 16, device=a.device, weights=W)
    out = eng.generate(torch.tensor([ids], device=a.device), a.new)
    eng.check()
    new = out[0, len(ids):].tolist()
    print("continuation:", tok.decode(new))


if __name__ == "__main__":
    main()
