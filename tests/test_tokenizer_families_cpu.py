"""The five tokenizer families the reference pins against the HF library (Llama-3, CLIP, BERT, GPT-2, SmolLM;
ferrotorch-tokenize/tests/conformance_hf_parity.rs:43), rebuilt here with the same pipeline stages (normalizer, pre-tokenizer, model,
post-processor, decoder) as the published files, trained on this package's sources, saved as ``tokenizer.json`` and read back: ids with and
without special tokens, and decoding with special tokens kept and skipped, must equal the HF library's."""
import glob
from pathlib import Path

import pytest

from ferrotorch_b200 import tokenize

tk = pytest.importorskip("tokenizers")
from tokenizers import Regex, decoders, models, normalizers, pre_tokenizers, processors, trainers  # noqa: E402

ROOT = Path(__file__).resolve().parents[1] / "ferrotorch_b200"
CORPUS = sorted(glob.glob(str(ROOT / "**" / "*.py"), recursive=True))[:25]
TEXTS = ["Hello, World! It's 12345 o'clock.", "def f(x):\n    return x + 1  # comment", "naïve café — Ünïcödé ✓ 你好 世界", "  multiple   spaces\tand\ttabs\n\nnewlines ",
         "", "don't you think we've done it? I'm sure they'll say: \"3.14159\"!", "UPPER lower MiXeD 007", "a", "emoji 🙂 and symbols ©®™ ½",
         "unknownwordthatisverylongandcertainlynotinthevocabulary" * 3, Path(CORPUS[3]).read_text()[:3000]]


def _check(hf, tmp_path, texts=TEXTS, expect_native=None):
    path = tmp_path / "tokenizer.json"
    hf.save(str(path))
    ours = tokenize.load_tokenizer(path)
    if expect_native is not None:
        assert (ours._native is not None) == expect_native
    for t in texts:
        for special in (False, True):
            want = hf.encode(t, add_special_tokens=special).ids
            got = ours.encode(t, add_special_tokens=special)
            assert got == want, (special, t[:50], got[:12], want[:12])
        ids = hf.encode(t, add_special_tokens=True).ids
        for skip in (False, True):
            assert ours.decode(ids, skip_special_tokens=skip) == hf.decode(ids, skip_special_tokens=skip), (skip, t[:50])
    assert ours.encode_batch(texts) == [e.ids for e in hf.encode_batch(texts, add_special_tokens=False)]
    return ours


def test_bert_wordpiece_family(tmp_path):
    hf = tk.Tokenizer(models.WordPiece(unk_token="[UNK]"))
    hf.normalizer = normalizers.BertNormalizer(clean_text=True, handle_chinese_chars=True, strip_accents=None, lowercase=True)
    hf.pre_tokenizer = pre_tokenizers.BertPreTokenizer()
    hf.decoder = decoders.WordPiece(prefix="##", cleanup=True)
    hf.train(CORPUS, trainers.WordPieceTrainer(vocab_size=2500, special_tokens=["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"], show_progress=False))
    hf.post_processor = processors.TemplateProcessing(single="[CLS] $A [SEP]", pair="[CLS] $A [SEP] $B:1 [SEP]:1",
                                                      special_tokens=[("[CLS]", hf.token_to_id("[CLS]")), ("[SEP]", hf.token_to_id("[SEP]"))])
    ours = _check(hf, tmp_path, TEXTS + ["control\x00chars\x07and​zero width", "accénts ÀÉÎÕÜ stripped", "[CLS] inline [MASK] specials [SEP]"])
    assert ours.model_type == "WordPiece"
    ids = ours.encode("hello", add_special_tokens=True)
    assert ids[0] == ours.vocab["[CLS]"] and ids[-1] == ours.vocab["[SEP]"]
    cased = tk.Tokenizer(models.WordPiece(unk_token="[UNK]"))
    cased.normalizer = normalizers.BertNormalizer(lowercase=False, strip_accents=False)
    cased.pre_tokenizer = pre_tokenizers.BertPreTokenizer()
    cased.decoder = decoders.WordPiece()
    cased.train(CORPUS, trainers.WordPieceTrainer(vocab_size=1500, special_tokens=["[UNK]", "[CLS]", "[SEP]"], show_progress=False))
    cased.post_processor = processors.BertProcessing(("[SEP]", cased.token_to_id("[SEP]")), ("[CLS]", cased.token_to_id("[CLS]")))
    _check(cased, tmp_path)


def test_clip_family_lowercase_bpe_with_end_of_word_suffix(tmp_path):
    hf = tk.Tokenizer(models.BPE(unk_token="<|endoftext|>", continuing_subword_prefix="", end_of_word_suffix="</w>"))
    hf.normalizer = normalizers.Sequence([normalizers.NFC(), normalizers.Replace(Regex(r"\s+"), " "), normalizers.Lowercase()])
    hf.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split(Regex(r"<\|startoftext\|>|<\|endoftext\|>|'s|'t|'re|'ve|'m|'ll|'d|[\p{L}]+|[\p{N}]|[^\s\p{L}\p{N}]+"), behavior="removed", invert=True),
        pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    hf.decoder = decoders.ByteLevel()
    hf.train(CORPUS, trainers.BpeTrainer(vocab_size=2500, special_tokens=["<|startoftext|>", "<|endoftext|>"], initial_alphabet=pre_tokenizers.ByteLevel.alphabet(),
                                        end_of_word_suffix="</w>", show_progress=False))
    hf.post_processor = processors.RobertaProcessing(sep=("<|endoftext|>", hf.token_to_id("<|endoftext|>")), cls=("<|startoftext|>", hf.token_to_id("<|startoftext|>")),
                                                     add_prefix_space=False, trim_offsets=False)
    ours = _check(hf, tmp_path, expect_native=False)
    assert ours.suffix == "</w>"
    ids = ours.encode("a photo of a cat", add_special_tokens=True)
    assert ids[0] == ours.vocab["<|startoftext|>"] and ids[-1] == ours.vocab["<|endoftext|>"]


def test_gpt2_family_with_byte_level_post_processor(tmp_path):
    hf = tk.Tokenizer(models.BPE())
    hf.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    hf.decoder = decoders.ByteLevel()
    hf.post_processor = processors.ByteLevel(trim_offsets=False)
    hf.train(CORPUS, trainers.BpeTrainer(vocab_size=2500, special_tokens=["<|endoftext|>"], initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False))
    ours = _check(hf, tmp_path, TEXTS + ["two<|endoftext|>documents"], expect_native=True)
    assert ours._kind == 0
    prefixed = tk.Tokenizer(models.BPE())
    prefixed.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=True, use_regex=True)
    prefixed.decoder = decoders.ByteLevel()
    prefixed.train(CORPUS, trainers.BpeTrainer(vocab_size=1500, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False))
    _check(prefixed, tmp_path)


def test_smollm_family_individual_digits_then_byte_level(tmp_path):
    hf = tk.Tokenizer(models.BPE())
    hf.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Digits(individual_digits=True), pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)])
    hf.decoder = decoders.ByteLevel()
    hf.train(CORPUS, trainers.BpeTrainer(vocab_size=2500, special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"],
                                        initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False))
    ours = _check(hf, tmp_path, TEXTS + ["<|im_start|>user\n2024 was 366 days<|im_end|>"], expect_native=True)
    assert ours._kind is None                       # the digit stage runs in Python, the merges in the library
    assert len(ours.encode("2024")) == 4


def test_llama3_family_with_template(tmp_path):
    hf = tk.Tokenizer(models.BPE(ignore_merges=True))
    hf.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(tokenize._LLAMA3_SPLIT), behavior="isolated", invert=False),
                                                pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    hf.decoder = decoders.ByteLevel()
    hf.train(CORPUS, trainers.BpeTrainer(vocab_size=2500, special_tokens=["<|begin_of_text|>", "<|end_of_text|>", "<|eot_id|>"],
                                        initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False))
    hf.post_processor = processors.Sequence([processors.ByteLevel(trim_offsets=False),
                                             processors.TemplateProcessing(single="<|begin_of_text|> $A", special_tokens=[("<|begin_of_text|>", hf.token_to_id("<|begin_of_text|>"))])])
    ours = _check(hf, tmp_path, TEXTS + ["turn one<|eot_id|>turn two"], expect_native=True)
    assert ours._kind == 1 and ours.ignore_merges
    assert ours.encode("hi", add_special_tokens=True)[0] == ours.vocab["<|begin_of_text|>"]


def test_other_stages_follow_the_hf_library(tmp_path):
    """Whitespace / punctuation / metaspace pre-tokenizers, NFKC + strip normalizers, byte fallback with the fuse / replace / strip decoder chain of
    sentencepiece-style files."""
    for pre in (pre_tokenizers.Whitespace(), pre_tokenizers.Sequence([pre_tokenizers.WhitespaceSplit(), pre_tokenizers.Punctuation()]),
                pre_tokenizers.Sequence([pre_tokenizers.WhitespaceSplit(), pre_tokenizers.Digits(individual_digits=False)])):
        hf = tk.Tokenizer(models.BPE(unk_token="<unk>"))
        hf.normalizer = normalizers.Sequence([normalizers.NFKC(), normalizers.Strip()])
        hf.pre_tokenizer = pre
        hf.train(CORPUS, trainers.BpeTrainer(vocab_size=1500, special_tokens=["<unk>"], show_progress=False))
        path = tmp_path / "tokenizer.json"
        hf.save(str(path))
        ours = tokenize.load_tokenizer(path)
        for t in TEXTS:
            assert ours.encode(t) == hf.encode(t, add_special_tokens=False).ids, t[:40]
    sp = tk.Tokenizer(models.BPE(unk_token="<unk>", byte_fallback=True, fuse_unk=False))
    sp.normalizer = normalizers.Sequence([normalizers.Prepend("▁"), normalizers.Replace(" ", "▁")])
    sp.decoder = decoders.Sequence([decoders.Replace("▁", " "), decoders.ByteFallback(), decoders.Fuse(), decoders.Strip(" ", 1, 0)])
    sp.train_from_iterator([Path(f).read_text().replace(" ", "▁") for f in CORPUS[:8]],
                           trainers.BpeTrainer(vocab_size=1500, special_tokens=["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)], show_progress=False))
    path = tmp_path / "tokenizer.json"
    sp.save(str(path))
    ours = tokenize.load_tokenizer(path)
    for t in ["hello world", "def f(x): return x", "snowman ☃ and 你好", " leading space"]:
        want = sp.encode(t, add_special_tokens=False).ids
        assert ours.encode(t) == want, t
        assert ours.decode(want) == sp.decode(want), t


def test_sentence_embeddings_from_strings_match_the_hf_stack(tmp_path):
    """Strings -> WordPiece ids with [CLS] / [SEP] -> padded batch -> BERT -> masked mean pool -> unit vectors: this package's tokenizer and
    model against the HF tokenizer feeding transformers' BertModel with the same weights."""
    import torch
    import transformers
    from ferrotorch_b200.models import bert
    hf = tk.Tokenizer(models.WordPiece(unk_token="[UNK]"))
    hf.normalizer = normalizers.BertNormalizer()
    hf.pre_tokenizer = pre_tokenizers.BertPreTokenizer()
    hf.train(CORPUS, trainers.WordPieceTrainer(vocab_size=800, special_tokens=["[PAD]", "[UNK]", "[CLS]", "[SEP]"], show_progress=False))
    hf.post_processor = processors.TemplateProcessing(single="[CLS] $A [SEP]", special_tokens=[("[CLS]", hf.token_to_id("[CLS]")), ("[SEP]", hf.token_to_id("[SEP]"))])
    hf.save(str(tmp_path / "tokenizer.json"))
    ours_tok = tokenize.load_tokenizer(tmp_path)
    torch.manual_seed(0)
    kw = dict(vocab_size=hf.get_vocab_size(), hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64, max_position_embeddings=64)
    hm, m = transformers.BertModel(transformers.BertConfig(**kw)).eval(), bert.BertModel(bert.BertConfig(**kw)).eval()
    m.load_state_dict(hm.state_dict(), strict=False)
    texts = ["return the tensor", "def forward(self, x): pass", "a much longer sentence about kernels, streams and graphs " * 3]
    emb = bert.SentenceTransformer(m).encode_texts(ours_tok, texts, max_length=48, pad_id=hf.token_to_id("[PAD]"))
    hf.enable_truncation(48)
    hf.enable_padding(pad_id=hf.token_to_id("[PAD]"), pad_token="[PAD]")
    enc = hf.encode_batch(texts)
    ids, mask = torch.tensor([e.ids for e in enc]), torch.tensor([e.attention_mask for e in enc])
    with torch.no_grad():
        h = hm(input_ids=ids, attention_mask=mask).last_hidden_state
    ref = torch.nn.functional.normalize((h * mask[..., None]).sum(1) / mask.sum(1, keepdim=True), dim=-1)
    assert emb.shape == (3, 32) and (emb - ref).abs().max() < 1e-5


def test_unigram_and_word_level_models(tmp_path):
    """A Unigram model (Viterbi over entry scores, unknown characters fused or spelled as byte tokens) with the metaspace stages of
    sentencepiece-style files, and a WordLevel model with an unknown token: ids and decoding against the HF library."""
    for byte_fallback in (False, True):
        hf = tk.Tokenizer(models.Unigram())
        hf.normalizer = normalizers.Sequence([normalizers.NFKC(), normalizers.Replace(Regex(" {2,}"), " ")])
        hf.pre_tokenizer = pre_tokenizers.Metaspace(replacement="▁", prepend_scheme="always")
        hf.decoder = decoders.Metaspace(replacement="▁", prepend_scheme="always")
        extra = [f"<0x{b:02X}>" for b in range(256)] if byte_fallback else []
        hf.train(CORPUS[:12], trainers.UnigramTrainer(vocab_size=1400, special_tokens=["<unk>", "<s>", "</s>"] + extra, unk_token="<unk>", show_progress=False))
        path = tmp_path / "tokenizer.json"
        hf.save(str(path))
        if byte_fallback:
            import json
            j = json.loads(path.read_text())
            j["model"]["byte_fallback"] = True
            path.write_text(json.dumps(j))
            hf = tk.Tokenizer.from_file(str(path))
        ours = tokenize.load_tokenizer(path)
        assert ours.model_type == "Unigram" and ours.unk_token == "<unk>"
        for t in ["hello world", "def forward(self, x): return self.proj(x)", "the tensor is contiguous", "snowman ☃☃ and 你好 unknown", "  two  spaces ", "x",
                  Path(CORPUS[2]).read_text()[:1500]]:
            want = hf.encode(t, add_special_tokens=False).ids
            assert ours.encode(t) == want, (byte_fallback, t[:40])
            assert ours.decode(want) == hf.decode(want), (byte_fallback, t[:40])
    wl = tk.Tokenizer(models.WordLevel(unk_token="[UNK]"))
    wl.normalizer = normalizers.Lowercase()
    wl.pre_tokenizer = pre_tokenizers.Whitespace()
    wl.train(CORPUS[:6], trainers.WordLevelTrainer(vocab_size=500, special_tokens=["[UNK]"], show_progress=False))
    path = tmp_path / "tokenizer.json"
    wl.save(str(path))
    ours = tokenize.load_tokenizer(path)
    assert ours.model_type == "WordLevel"
    for t in ["import torch", "Return SELF.value + zzzunknownzzz", "def f(x): pass"]:
        assert ours.encode(t) == wl.encode(t).ids, t
