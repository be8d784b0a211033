"""Shared by the Llama entry points: resolve a checkpoint directory (``config.json``, ``tokenizer.json``, safetensors shards) or fall back
to a named preset with random weights and a byte-level stand-in tokenizer, so every script also runs on a box with no checkpoint."""
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch  # noqa: E402

from ferrotorch_b200.models import LlamaConfig  # noqa: E402
from ferrotorch_b200.models.llama_infer import random_hf_weights  # noqa: E402

PRESETS = {"llama3-8b": LlamaConfig.llama3_8b, "llama3-70b": LlamaConfig.llama3_70b, "llama3.3-70b-instruct": LlamaConfig.llama3_3_70b_instruct,
           "tiny": lambda: LlamaConfig.tiny(layers=2, hidden=256, heads=2, kv_heads=1, ffn=512, vocab=1024)}


class ByteTokenizer:
    """Stand-in used when no ``tokenizer.json`` is at hand: UTF-8 bytes folded into the vocabulary."""

    def __init__(self, vocab: int):
        self.vocab = vocab

    def encode(self, text: str):
        return [b % self.vocab for b in text.encode()] or [0]

    def decode(self, ids):
        return " ".join(f"<{int(i)}>" for i in ids)


def load_config(model_dir, preset: str) -> LlamaConfig:
    if model_dir:
        return LlamaConfig.from_hf(Path(model_dir) / "config.json")
    return PRESETS[preset]()


def load_tok(model_dir, cfg):
    if model_dir and (Path(model_dir) / "tokenizer.json").exists():
        from ferrotorch_b200.tokenize import load_tokenizer, encode, decode
        tok = load_tokenizer(Path(model_dir) / "tokenizer.json")

        class _T:
            def encode(self, text):
                return encode(tok, text, add_special_tokens=True)

            def decode(self, ids):
                return decode(tok, list(map(int, ids)))
        return _T()
    return ByteTokenizer(cfg.vocab_size)


def load_weights(model_dir, cfg, device="cpu", mmap: bool = True):
    """HF-named bf16 tensors. Sharded checkpoints are memory-mapped so that a rank which slices its part touches only those pages."""
    if not model_dir:
        return random_hf_weights(cfg, device, 0, 0.02)
    d = Path(model_dir)
    from ferrotorch_b200 import serialize
    idx = d / "model.safetensors.index.json"
    if idx.exists():
        return (serialize.load_safetensors_sharded_mmap(idx) if mmap else serialize.load_safetensors_sharded(idx))
    return serialize.load_safetensors(d / "model.safetensors")


def write_checkpoint(out_dir, cfg: LlamaConfig, weights) -> None:
    """``config.json`` + ``model.safetensors`` in the Hugging Face layout (what :func:`load_config` / :func:`load_weights` read back)."""
    from ferrotorch_b200.serialize import save_safetensors
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    fields = {k: getattr(cfg, k) for k in cfg.__dataclass_fields__}
    fields.update(architectures=["LlamaForCausalLM"], model_type="llama", torch_dtype="float32")
    (out / "config.json").write_text(json.dumps(fields, indent=1))
    save_safetensors({k: v.detach().cpu().contiguous() for k, v in weights.items()}, out / "model.safetensors")
