#!/usr/bin/env python
"""Activation sparsity of a ProSparse-style Llama (FATReLU gate: ``x if x >= threshold else 0``), per layer. Counterpart of
ferrotorch-llama/examples/prosparse_7b_gpu.rs: load the checkpoint, run one forward with a tap on every MLP's gated activation and print
the share of exact zeros (the published ProSparse-Llama-2-7B reaches about 89 %).

    python examples/prosparse_sparsity.py --model-dir /path/to/prosparse-llama-2-7b
    python examples/prosparse_sparsity.py --preset tiny --threshold 0.01     # random weights: about half the gate inputs are negative"""
import argparse

from _model_dir import PRESETS, load_config, load_tok, load_weights, torch

from ferrotorch_b200.models import LlamaGpuInferencer


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("prompt", nargs="?", default="The quick brown fox jumps over the lazy dog.")
    ap.add_argument("--model-dir")
    ap.add_argument("--preset", choices=sorted(PRESETS), default="tiny")
    ap.add_argument("--threshold", type=float, default=None, help="FATReLU threshold (default: the checkpoint's hidden_act_param, else 0.01)")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args()
    cfg = load_config(a.model_dir, a.preset)
    if cfg.hidden_act not in ("fatrelu", "relu"):
        cfg.hidden_act = "fatrelu"
    if a.threshold is not None or cfg.hidden_act_param is None:
        cfg.hidden_act_param = 0.01 if a.threshold is None else a.threshold
    tok = load_tok(a.model_dir, cfg)
    ids = tok.encode(a.prompt)
    inf = LlamaGpuInferencer(cfg, load_weights(a.model_dir, cfg), device=a.device, dtype=torch.bfloat16 if a.device != "cpu" else torch.float32)
    zeros = []
    hooks = []
    for layer in inf.layers:
        orig = layer.mlp.gated

        def tapped(h, _orig=orig):
            g = _orig(h)
            zeros.append((g == 0).float().mean().item())
            return g
        layer.mlp.gated = tapped
        hooks.append((layer.mlp, orig))
    inf.forward_from_ids(ids)
    for mlp, orig in hooks:
        mlp.gated = orig
    print(f"activation {cfg.activation!r}, {len(ids)} tokens")
    for i, z in enumerate(zeros):
        print(f"layer {i:3d}: {100 * z:5.1f} % zeros")
    print(f"mean MLP sparsity: {100 * sum(zeros) / len(zeros):.1f} %")


if __name__ == "__main__":
    main()
