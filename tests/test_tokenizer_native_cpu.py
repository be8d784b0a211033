"""The native merge engine of the tokenizer (``csrc/runtime/tokenizer.cpp``) against the direct Python loop and against the HF ``tokenizers``
library: byte-level and plain BPE, whole-piece vocabulary hits (``ignore_merges``), special tokens, batches spread over threads, and the
fall-back for pieces the engine cannot take."""
import glob
from pathlib import Path

import pytest

from ferrotorch_b200 import tokenize

tk = pytest.importorskip("tokenizers")
ROOT = Path(__file__).resolve().parents[1] / "ferrotorch_b200"


def _corpus(n=30):
    return sorted(glob.glob(str(ROOT / "**" / "*.py"), recursive=True))[:n]


def _train_byte_level(tmp_path, vocab_size=3000, ignore_merges=False):
    from tokenizers import decoders, models, pre_tokenizers, trainers
    hf = tk.Tokenizer(models.BPE())
    hf.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    hf.decoder = decoders.ByteLevel()
    hf.train(_corpus(), trainers.BpeTrainer(vocab_size=vocab_size, special_tokens=["<|begin|>", "<|end|>"],
                                            initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False))
    path = tmp_path / "tokenizer.json"
    hf.save(str(path))
    if ignore_merges:
        import json
        j = json.loads(path.read_text())
        j["model"]["ignore_merges"] = True
        # an entry that the merges cannot produce: only the whole-piece lookup can emit it
        j["model"]["vocab"]["Ġzyxwvut"] = max(j["model"]["vocab"].values()) + 3
        path.write_text(json.dumps(j))
        hf = tk.Tokenizer.from_file(str(path))
    return hf, path


TEXTS = ["hello world", "def f(x):\n    return x + 1  # comment", "naïve café — ünïcödé ✓ 你好 🙂", "  multiple   spaces\tand\ttabs\n\nnewlines", "",
         "<|begin|>special<|end|> tokens<|end|>", "12345 67890 3.14159", "a" * 300 + " " + "ab" * 200, "x"]


def test_native_engine_is_active_and_matches_python_loop_and_hf(tmp_path, monkeypatch):
    hf, path = _train_byte_level(tmp_path)
    ours = tokenize.load_tokenizer(path)
    assert ours._native is not None
    monkeypatch.setenv("FT_TOKENIZE_NATIVE", "0")
    plain = tokenize.load_tokenizer(path)
    assert plain._native is None
    texts = TEXTS + [Path(f).read_text()[:6000] for f in _corpus(6)]
    for t in texts:
        a = ours.encode(t)
        assert a == plain.encode(t) == hf.encode(t).ids, t[:40]
        assert ours.decode(a, skip_special_tokens=False) == hf.decode(a, skip_special_tokens=False)


def test_batch_encoding_over_threads_equals_text_by_text(tmp_path):
    hf, path = _train_byte_level(tmp_path)
    ours = tokenize.load_tokenizer(path)
    texts = [Path(f).read_text() for f in _corpus(12)] + TEXTS                # several hundred KB: the threaded split is taken
    assert sum(len(t) for t in texts) > (1 << 16)
    got = ours.encode_batch(texts)
    assert got == [ours.encode(t) for t in texts]
    assert got == [e.ids for e in hf.encode_batch(texts)]
    with_bos = tokenize.Tokenizer(ours.model_vocab, sorted(ours.ranks, key=ours.ranks.get), ours.added, bos_token="<|begin|>")
    assert with_bos.encode_batch(["hi there", ""], add_special_tokens=True) == [with_bos.encode("hi there", True), with_bos.encode("", True)]
    assert with_bos.encode_batch(["hi"], add_special_tokens=True)[0][0] == ours.added["<|begin|>"]


def test_whole_piece_vocabulary_hits_skip_the_merges(tmp_path, monkeypatch):
    hf, path = _train_byte_level(tmp_path, ignore_merges=True)
    ours = tokenize.load_tokenizer(path)
    assert ours.ignore_merges and ours._native is not None
    monkeypatch.setenv("FT_TOKENIZE_NATIVE", "0")
    plain = tokenize.load_tokenizer(path)
    for t in TEXTS + ["the zyxwvut entry", Path(_corpus(2)[1]).read_text()[:5000]]:
        assert ours.encode(t) == plain.encode(t) == hf.encode(t).ids, t[:40]
    assert ours.vocab["Ġzyxwvut"] in ours.encode("the zyxwvut entry")


def test_plain_bpe_with_unknown_characters_falls_back_to_the_python_rule():
    vocab = {"<unk>": 0, "h": 1, "e": 2, "l": 3, "o": 4, "he": 5, "ll": 6, "hell": 7, "hello": 8, " ": 9, "é": 10, "lé": 11}
    merges = [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o"), ("l", "é")]
    tok = tokenize.Tokenizer(vocab, merges, byte_level=False, unk_token="<unk>")
    assert tok._native is not None
    assert tok.encode("hello") == [8] and tok.encode("helé") == [5, 11]
    assert tok.encode("hello z") == [8, 9, 0]                                  # "z" has no token: the engine declines, the Python rule maps it to <unk>
    strict = tokenize.Tokenizer(vocab, merges, byte_level=False)
    with pytest.raises(Exception):
        strict.encode("z")
    # a merge whose result is not a vocabulary entry keeps the tokenizer on the Python loop
    assert tokenize.Tokenizer(vocab, merges + [("o", "o")], byte_level=False, unk_token="<unk>")._native is None


def test_equal_rank_ties_merge_leftmost_first():
    vocab = {c: i for i, c in enumerate("ab")}
    vocab.update({"aa": 2, "aaa": 3, "ab": 4})
    tok = tokenize.Tokenizer(vocab, [("a", "a"), ("aa", "a"), ("a", "b")], byte_level=False)
    ref = tokenize.Tokenizer(vocab, [("a", "a"), ("aa", "a"), ("a", "b")], byte_level=False)
    ref._native = None
    for w in ("aaa", "aaaa", "aaaaa", "aaab", "aabaaab", "baaaab"):
        assert tok.encode(w) == ref.encode(w), w


@pytest.mark.parametrize("pattern,regex_src", [("gpt2", tokenize._GPT2_SPLIT), ("llama3", tokenize._LLAMA3_SPLIT)])
def test_native_splitter_cuts_where_the_regular_expression_cuts(pattern, regex_src):
    """Random strings over an alphabet chosen to hit every branch of the two patterns: contraction suffixes in both cases (and U+017F, which
    the case-insensitive form accepts for "s"), runs of blanks before letters / digits / punctuation / the end, carriage returns and line
    feeds inside and after runs, non-ASCII letters, numbers and spaces."""
    import random
    import regex
    rx = regex.compile(regex_src)
    alphabet = [" ", " ", " ", "\t", "\n", "\r", "\u00a0", "\u2028", "\u3000", "'", "'", "s", "S", "t", "T", "r", "e", "E", "v", "m", "l", "L", "d", "D", "\u017f",
                "a", "Z", "é", "ß", "你", "я", "1", "2", "9", "²", "٣", "Ⅷ", ".", ",", "!", "-", "_", "(", "#", "🙂", "\u200d", "\u0301", "x"]
    rng = random.Random(0)
    for n in [0, 1, 2, 3] + [rng.randint(1, 40) for _ in range(3000)]:
        t = "".join(rng.choice(alphabet) for _ in range(n))
        assert tokenize.pre_tokenize(t, pattern) == rx.findall(t), repr(t)
    for t in ["I'm sure they'LL say it'S fine, won'T they? 'RE: 've", "x  \n\n  y", "a\r\n\r\nb   ", "   ", "1234567 12 1", "tab\tsep\t\tend\t",
              "(hello)[world]{!}", " \u00a0x", "\n x", "foo'", "'"]:
        assert tokenize.pre_tokenize(t, pattern) == rx.findall(t), repr(t)
    with pytest.raises(Exception):
        tokenize.pre_tokenize("x", "other")


def test_llama3_pattern_tokenizer_matches_hf_with_the_same_split(tmp_path):
    """A tokenizer file with the Llama-3 pre-tokeniser (Split by that pattern, then ByteLevel without its own regex) and whole-piece lookups,
    as the Llama-3 checkpoints ship it: native splitting + merging against the HF library."""
    import json
    from tokenizers import Regex, decoders, models, pre_tokenizers, trainers
    hf = tk.Tokenizer(models.BPE())
    hf.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(tokenize._LLAMA3_SPLIT), behavior="isolated", invert=False),
                                                pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    hf.decoder = decoders.ByteLevel()
    hf.train(_corpus(), trainers.BpeTrainer(vocab_size=2500, special_tokens=["<|begin_of_text|>", "<|eot_id|>"],
                                            initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False))
    path = tmp_path / "tokenizer.json"
    hf.save(str(path))
    j = json.loads(path.read_text())
    j["model"]["ignore_merges"] = True
    path.write_text(json.dumps(j))
    hf = tk.Tokenizer.from_file(str(path))
    ours = tokenize.load_tokenizer(path)
    assert ours._kind == 1 and ours._native is not None and ours.ignore_merges
    texts = TEXTS + ["<|begin_of_text|>It's 12345 o'clock\r\n\r\n  done<|eot_id|>", Path(_corpus(3)[2]).read_text()[:8000]]
    for t in texts:
        assert ours.encode(t) == hf.encode(t).ids, t[:40]
    assert ours.encode_batch(texts) == [e.ids for e in hf.encode_batch(texts)]
