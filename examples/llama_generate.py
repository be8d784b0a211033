#!/usr/bin/env python
"""Generate with a (randomly initialised or safetensors-loaded) Llama model: KV-cached decoding, sampling, beam search, speculative decoding.

    python examples/llama_generate.py --prompt-len 16 --new 32 [--weights /path/to/model.safetensors --config /path/to/config.json]

On a B200 the same model runs through the tensor-parallel engine (`LlamaTPEngine`: paged KV cache, CUDA-graph decode) with `--engine tp`
(launch with torch.distributed.run for more than one GPU). Counterpart of ferrotorch-llama/examples/llama3_8b.rs and llama3_8b_gpu.rs.
"""
import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch

from ferrotorch_b200.models import CachedLlama, GenerationConfig, LlamaConfig, SpecDecodeConfig, generate, speculative_generate
from ferrotorch_b200.models.llama_infer import random_hf_weights


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--prompt-len", type=int, default=16)
    ap.add_argument("--new", type=int, default=32)
    ap.add_argument("--weights")
    ap.add_argument("--config")
    ap.add_argument("--engine", choices=["cached", "tp"], default="cached")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args()
    if a.config:
        cfg = LlamaConfig.from_hf(json.load(open(a.config)))
    else:
        cfg = LlamaConfig(vocab_size=4096, hidden_size=256, intermediate_size=512, num_hidden_layers=4, num_attention_heads=8, num_key_value_heads=2,
                          max_position_embeddings=2048)
    if a.weights:
        from ferrotorch_b200.serialize import load_safetensors
        W = {k: v.to(a.device) for k, v in load_safetensors(a.weights).items()}
    else:
        W = random_hf_weights(cfg, a.device, 0, 0.05)
    ids = torch.randint(0, cfg.vocab_size, (1, a.prompt_len), device=a.device, generator=torch.Generator(device=a.device).manual_seed(0))
    if a.engine == "tp":
        from ferrotorch_b200.models.llama_infer import LlamaTPEngine, TPContext
        eng = LlamaTPEngine(cfg, TPContext(a.device), max_batch=1, max_seq=a.prompt_len + a.new + 16, device=a.device, weights=W)
        print("tp engine:", eng.generate(ids, a.new)[0].tolist())
        return
    Wf = {k: v.float() for k, v in W.items()}
    m = CachedLlama(cfg, Wf)
    print("greedy :", generate(m, m.new_cache, ids, GenerationConfig(max_new_tokens=a.new))[0, a.prompt_len:].tolist())
    sampled = GenerationConfig(max_new_tokens=a.new, seed=0).with_temperature(0.8).with_top_k(50).with_top_p(0.95)
    print("sampled:", generate(m, m.new_cache, ids, sampled)[0, a.prompt_len:].tolist())
    print("beam   :", generate(m, m.new_cache, ids, GenerationConfig(max_new_tokens=min(a.new, 16), num_beams=4))[0, a.prompt_len:].tolist())
    draft = CachedLlama(cfg, {k: v.float() for k, v in random_hf_weights(cfg, a.device, 1, 0.05).items()})
    seq, stats = speculative_generate(m, m.new_cache, draft, draft.new_cache, ids, SpecDecodeConfig(4, a.new))
    print("spec   :", seq[0, a.prompt_len:].tolist(), f"(acceptance {stats.acceptance_rate():.2f})")


if __name__ == "__main__":
    main()
