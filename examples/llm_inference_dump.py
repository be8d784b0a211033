#!/usr/bin/env python
"""Run one prefill of a causal LM on a fixed prompt and write the logits to disk as ``[u32 ndim][u32 x ndim shape][f32 data]`` (little
endian), for comparison by ``verify_llm_inference.py``. Counterpart of ferrotorch-llama/examples/llm_inference_dump.rs.

    python examples/llm_inference_dump.py --model-dir /path/to/SmolLM-135M --device gpu --output /tmp/llm_dump.bin
    python examples/llm_inference_dump.py --write-random /tmp/tiny_llama && python examples/llm_inference_dump.py --model-dir /tmp/tiny_llama \
        --output /tmp/llm_dump.bin

``--device cpu`` evaluates the module graph in f32, ``--device gpu`` the bf16 inferencer. ``--write-random DIR`` writes a small random
checkpoint in the Hugging Face layout (for boxes with no network)."""
import argparse
import struct

from _model_dir import PRESETS, load_config, load_weights, torch, write_checkpoint

from ferrotorch_b200.models import LlamaGpuInferencer
from ferrotorch_b200.models.llama_infer import random_hf_weights

PROMPT_IDS = [1, 15, 27, 42, 99, 7, 3, 250, 17, 64, 5, 128]


def dump(path, t: torch.Tensor) -> None:
    t = t.detach().float().cpu().contiguous()
    with open(path, "wb") as f:
        f.write(struct.pack("<I", t.dim()))
        f.write(struct.pack(f"<{t.dim()}I", *t.shape))
        f.write(t.numpy().tobytes())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model-dir")
    ap.add_argument("--preset", choices=sorted(PRESETS), default="tiny")
    ap.add_argument("--device", choices=["cpu", "gpu"], default="cpu")
    ap.add_argument("--output", default="llm_dump.bin")
    ap.add_argument("--write-random")
    a = ap.parse_args()
    if a.write_random:
        cfg = PRESETS[a.preset]()
        write_checkpoint(a.write_random, cfg, {k: v.float() for k, v in random_hf_weights(cfg, "cpu", 0, 0.05).items()})
        print("wrote", a.write_random)
        return
    cfg = load_config(a.model_dir, a.preset)
    W = load_weights(a.model_dir, cfg, "cpu")
    ids = [i % cfg.vocab_size for i in PROMPT_IDS]
    dev, dt = ("cuda", torch.bfloat16) if a.device == "gpu" else ("cpu", torch.float32)
    logits = LlamaGpuInferencer(cfg, W, device=dev, dtype=dt).forward_logits_from_ids_all(ids)
    dump(a.output, logits)
    print(f"logits {list(logits.shape)} -> {a.output}; last-position arg-max {int(logits[-1].argmax())}")


if __name__ == "__main__":
    main()
