"""The example entry points run end to end on CPU with the tiny preset; the logits dump agrees with the ``transformers`` evaluation of the
same checkpoint."""
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _run(*args, timeout=300):
    r = subprocess.run([sys.executable, *map(str, args)], cwd=ROOT, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout


def test_inference_dump_matches_transformers(tmp_path):
    pytest.importorskip("transformers")
    ckpt, dump = tmp_path / "tiny_llama", tmp_path / "dump.bin"
    _run(ROOT / "examples/llm_inference_dump.py", "--write-random", ckpt)
    assert (ckpt / "config.json").exists() and (ckpt / "model.safetensors").exists()
    out = _run(ROOT / "examples/llm_inference_dump.py", "--model-dir", ckpt, "--output", dump)
    assert "logits [12, 1024]" in out
    out = _run(ROOT / "examples/verify_llm_inference.py", "--model-dir", ckpt, "--dump", dump, "--tolerance", "1e-4")
    assert out.strip().splitlines()[-1].startswith("OK"), out
    # a corrupted dump is rejected
    raw = bytearray(dump.read_bytes())
    raw[-4000:] = bytes(4000)
    dump.write_bytes(bytes(raw))
    r = subprocess.run([sys.executable, str(ROOT / "examples/verify_llm_inference.py"), "--model-dir", str(ckpt), "--dump", str(dump), "--tolerance", "1e-4"],
                       cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert r.returncode == 1 and "FAIL" in r.stdout


def test_llama_entry_point_and_sparsity_report_run_on_cpu():
    out = _run(ROOT / "examples/llama3_8b_gpu.py", "--preset", "tiny", "--device", "cpu", "hello world")
    assert "prefill of 11 tokens" in out and "next token" in out
    out = _run(ROOT / "examples/prosparse_sparsity.py", "--preset", "tiny", "--device", "cpu", "--threshold", "0.02")
    assert "FatRelu(0.02)" in out and "mean MLP sparsity" in out
    share = float(out.strip().splitlines()[-1].split(":")[1].split("%")[0])
    assert 40.0 < share < 65.0          # random weights: about half of the gate pre-activations fall below the threshold


def test_constrained_generation_example_emits_a_document_of_the_schema():
    import json
    out = _run(ROOT / "examples/json_constrained_generate.py", "--new", "160", "--seed", "1")
    assert "valid prefix: True" in out
    line = next(l for l in out.splitlines() if l.startswith("generated: "))
    if "complete document: True" in out:
        doc = json.loads(line[len("generated: "):])
        assert isinstance(doc["name"], str) and isinstance(doc["age"], int) and set(doc) <= {"name", "age", "tags", "note"}


def test_native_core_cnn_example_learns():
    out = _run(ROOT / "examples/native_cnn.py", "--steps", "60")
    acc = float(out.split("accuracy on 512 fresh samples:")[1].split()[0])
    first, last = (float(l.split("loss")[1]) for l in (out.splitlines()[0], [l for l in out.splitlines() if l.startswith("step")][-1]))
    assert acc > 0.8 and last < 0.5 * first


def test_native_core_transformer_example_learns_its_corpus():
    out = _run(ROOT / "examples/native_gpt.py", "--steps", "90")
    losses = [float(l.split("loss")[1]) for l in out.splitlines() if l.startswith("step")]
    assert losses[-1] < 0.2 < losses[0]
    assert "sample: the quick brown fox jumps over the lazy dog." in out


def test_constrained_generation_with_a_checkpoint_directory_and_its_tokenizer_file(tmp_path):
    """A random checkpoint in the Hugging Face layout plus a byte-level BPE ``tokenizer.json`` trained with the HF library: the example loads
    both and its output stays a valid prefix of the schema."""
    tk = pytest.importorskip("tokenizers")
    import glob
    import json
    from tokenizers import decoders, models, pre_tokenizers, trainers
    ckpt = tmp_path / "ckpt"
    _run(ROOT / "examples/llm_inference_dump.py", "--write-random", ckpt)
    vocab = json.loads((ckpt / "config.json").read_text())["vocab_size"]
    out = _run(ROOT / "examples/json_constrained_generate.py", "--model-dir", ckpt, "--new", "40")          # no tokenizer file yet: the byte tokenizer
    assert "valid prefix: True" in out
    hf = tk.Tokenizer(models.BPE())
    hf.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    hf.decoder = decoders.ByteLevel()
    files = sorted(glob.glob(str(ROOT / "ferrotorch_b200" / "*.py")))[:6]
    hf.train(files, trainers.BpeTrainer(vocab_size=min(vocab, 400), special_tokens=["<|end|>"], initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False))
    hf.save(str(ckpt / "tokenizer.json"))
    (ckpt / "tokenizer_config.json").write_text(json.dumps({"eos_token": "<|end|>"}))
    out = _run(ROOT / "examples/json_constrained_generate.py", "--model-dir", ckpt, "--new", "40")
    assert "valid prefix: True" in out and out.splitlines()[0].startswith("generated: {")


def test_learner_example_trains_on_synthetic_digits(tmp_path):
    out = _run(ROOT / "examples/train_mnist.py", "--epochs", "3", "--device", "cpu", "--samples", "512", "--out", tmp_path / "run")
    losses = [float(l.split("train_loss")[1].split()[0]) for l in out.splitlines() if l.startswith("epoch")]
    assert len(losses) == 3 and losses[-1] < losses[0]
    assert any((tmp_path / "run").rglob("*")), "checkpoints / event files were written"
