#!/usr/bin/env python
"""Compare a logits dump written by ``llm_inference_dump.py`` with the same checkpoint evaluated by the ``transformers`` library in f32
(the role of the reference's scripts/verify_causal_lm_inference.py and verify_causal_lm_gpu_inference.py).

    python examples/verify_llm_inference.py --model-dir /tmp/tiny_llama --dump /tmp/llm_dump.bin [--tolerance 2e-3]

Exit status 0 when the cosine similarity of the logits is at least 0.999 (0.99 for a bf16 dump with ``--bf16``) and the largest absolute
difference is below the tolerance."""
import argparse
import struct
import sys

from _model_dir import torch

from llm_inference_dump import PROMPT_IDS


def load_dump(path) -> torch.Tensor:
    raw = open(path, "rb").read()
    (nd,) = struct.unpack_from("<I", raw, 0)
    shape = struct.unpack_from(f"<{nd}I", raw, 4)
    return torch.frombuffer(bytearray(raw[4 + 4 * nd:]), dtype=torch.float32).view(*shape).clone()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model-dir", required=True)
    ap.add_argument("--dump", required=True)
    ap.add_argument("--tolerance", type=float, default=2e-3)
    ap.add_argument("--bf16", action="store_true", help="the dump came from the bf16 device path: compare with the looser bounds")
    a = ap.parse_args()
    from transformers import AutoConfig, AutoModelForCausalLM
    cfg = AutoConfig.from_pretrained(a.model_dir)
    model = AutoModelForCausalLM.from_pretrained(a.model_dir, dtype=torch.float32).eval()
    ids = torch.tensor([[i % cfg.vocab_size for i in PROMPT_IDS]])
    with torch.no_grad():
        ref = model(ids).logits[0].float()
    got = load_dump(a.dump)
    if got.shape != ref.shape:
        print(f"FAIL: shape {list(got.shape)} vs {list(ref.shape)}")
        return 1
    cos = torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0).item()
    err = (got - ref).abs().max().item()
    same_top = (got.argmax(-1) == ref.argmax(-1)).float().mean().item()
    min_cos, tol = (0.99, max(a.tolerance, 0.25)) if a.bf16 else (0.999, a.tolerance)
    ok = cos >= min_cos and err <= tol
    print(f"{'OK' if ok else 'FAIL'}: cosine {cos:.6f}, max |diff| {err:.3e}, arg-max agreement {100 * same_top:.0f} %")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
