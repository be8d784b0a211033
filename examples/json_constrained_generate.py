#!/usr/bin/env python
"""Schema-constrained generation end to end: a byte-level tokenizer, a (randomly initialised or loaded) Llama model with a KV cache, and the
JSON-schema logits processor. Whatever the model would like to say, the output parses and matches the schema.

    python examples/json_constrained_generate.py [--model-dir DIR] [--new 96] [--seed 0]

Without ``--model-dir`` the vocabulary is the 256 byte stand-ins plus an end token and the weights are random, so the text is noise that is
valid JSON. With a model directory (``config.json``, ``tokenizer.json``, ``model.safetensors``) the same code constrains a real checkpoint.
Counterpart of the reference's grammar-constrained sampling (ferrotorch-grammar/src/lib.rs:58-85 driving ferrotorch-llama generation).
"""
import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch

from ferrotorch_b200 import grammar, tokenize
from ferrotorch_b200.models import CachedLlama, GenerationConfig, LlamaConfig, generate
from ferrotorch_b200.models.llama_infer import random_hf_weights

SCHEMA = {"type": "object",
          "properties": {"name": {"type": "string"}, "age": {"type": "integer"}, "tags": {"type": "array", "items": {"enum": ["a", "b", "c"]}},
                         "note": {"type": ["string", "null"]}},
          "required": ["name", "age"]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model-dir")
    ap.add_argument("--new", type=int, default=96)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--prompt", default="Describe a person as JSON: ")
    a = ap.parse_args()
    def byte_tokenizer():
        b2u = tokenize._bytes_to_unicode()
        return tokenize.Tokenizer({b2u[b]: b for b in range(256)}, [], {"<eos>": 256}, eos_token="<eos>"), 256
    if a.model_dir:
        from ferrotorch_b200.serialize import load_safetensors
        d = Path(a.model_dir)
        cfg = LlamaConfig.from_hf(json.load(open(d / "config.json")))
        if (d / "tokenizer.json").exists():
            tok = tokenize.load_tokenizer(d)
            eos = tok.vocab.get(tok.eos_token) if tok.eos_token else None
        elif cfg.vocab_size >= 257:                        # a checkpoint without a tokenizer file: bytes plus an end token
            tok, eos = byte_tokenizer()
        else:
            raise SystemExit("the model directory has no tokenizer.json and its vocabulary is too small for the byte tokenizer")
        W = {k: v.float() for k, v in load_safetensors(d / "model.safetensors").items()}
    else:
        tok, eos = byte_tokenizer()
        cfg = LlamaConfig(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                          max_position_embeddings=1024)
        W = {k: v.float() for k, v in random_hf_weights(cfg, "cpu", a.seed, 0.08).items()}
    texts = [tok.decode([i], skip_special_tokens=True) if i in tok.inv else "" for i in range(cfg.vocab_size)]
    proc = grammar.JsonSchemaProcessor(SCHEMA, texts, eos_id=eos)
    model = CachedLlama(cfg, W)
    ids = torch.tensor([tok.encode(a.prompt)])
    gcfg = GenerationConfig(max_new_tokens=a.new, seed=a.seed, eos_token_id=eos).with_temperature(1.0)
    seq = generate(model, model.new_cache, ids, gcfg, logits_processor=proc.as_logits_processor(ids.shape[1]))
    out = tok.decode(seq[0, ids.shape[1]:].tolist())
    print("generated:", out)
    ok, done = proc.grammar.accepts_prefix(out), proc.grammar.is_complete(out)
    print("valid prefix:", ok, "| complete document:", done)
    if done:
        print("parsed:", json.loads(out))


if __name__ == "__main__":
    main()
