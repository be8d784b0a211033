"""Tokenizer: a self-contained reader of HF ``tokenizer.json`` (BPE, WordPiece, WordLevel and Unigram models with the file's normalizer,
pre-tokenizer, post-processor and decoder stages, added / special tokens) plus chat templates.

Reference parity: ferrotorch-tokenize/src/lib.rs:59 (load_tokenizer), :85 (encode), :104 (encode_batch), :131 (decode),
:225 (apply_chat_template) - a wrapper over the HF ``tokenizers`` crate there; here the BPE merge loop is implemented directly: in
the host runtime library (``csrc/runtime/tokenizer.cpp``: heap-ordered merges, the pieces of a call spread over threads) with the
direct Python loop as the fallback for vocabularies the native engine cannot take (a merge whose halves are not vocabulary entries)
and for texts that need the unknown-token rule. ``FT_TOKENIZE_NATIVE=0`` keeps everything on the Python loop.
"""
from __future__ import annotations

import ctypes
import json
import os
from functools import lru_cache
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import regex as _re

from dataclasses import dataclass

from ..errors import Internal, InvalidArgument
from . import pipeline as _pl

_GPT2_SPLIT = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""
_LLAMA3_SPLIT = r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"""


_classes_installed = False


def _install_classes(rt) -> None:
    """Gives the runtime library the class of every code point (letter, number, white space) as the regular-expression engine used by
    the Python route sees it, so the native splitter and ``regex`` cut at the same places. Once per process (about 0.2 s)."""
    global _classes_installed
    if _classes_installed:
        return
    table = np.zeros(0x110000, np.uint8)
    allc = "".join(map(chr, range(0xD800))) + "".join(map(chr, range(0xE000, 0x110000)))

    def cp(i):                                          # index in ``allc`` -> code point (the surrogate block is left out of the string)
        return i if i < 0xD800 else i + 0x800
    for bit, pat in ((1, r"\p{L}+"), (2, r"\p{N}+"), (4, r"\s+")):
        for m in _re.finditer(pat, allc):
            table[cp(m.start()): cp(m.end() - 1) + 1] |= bit
    rt.ft_tok_set_classes.restype = None
    rt.ft_tok_set_classes(table.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(table.size))
    _classes_installed = True


def pre_tokenize(text: str, pattern: str = "gpt2") -> List[str]:
    """The pieces the pre-tokeniser cuts ``text`` into, by the native matcher of the ``"gpt2"`` or ``"llama3"`` split pattern (the same
    cuts as ``regex.findall`` with that pattern)."""
    kind = {"gpt2": 0, "llama3": 1}.get(pattern)
    if kind is None:
        raise InvalidArgument(f"pattern must be 'gpt2' or 'llama3', got {pattern!r}")
    from .. import _lib
    rt = _lib.runtime()
    _install_classes(rt)
    rt.ft_tok_split.restype = ctypes.c_int64
    raw = text.encode("utf-8")
    ends = np.empty(max(len(raw), 1), np.int64)
    n = rt.ft_tok_split(ctypes.c_int(kind), ctypes.c_char_p(raw), ctypes.c_int64(len(raw)), ends.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(ends.size))
    if n < 0:
        raise Internal(f"native splitter failed with code {n}")
    out, a = [], 0
    for b in ends[:n].tolist():
        out.append(raw[a:b].decode("utf-8"))
        a = b
    return out


@lru_cache(maxsize=1)
def _bytes_to_unicode() -> Dict[int, str]:
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return dict(zip(bs, map(chr, cs)))


class Tokenizer:
    def __init__(self, vocab: Dict[str, int], merges: Sequence[Tuple[str, str]], added_tokens: Optional[Dict[str, int]] = None,
                 byte_level: bool = True, split_pattern: Optional[str] = None, bos_token: Optional[str] = None, eos_token: Optional[str] = None,
                 unk_token: Optional[str] = None, ignore_merges: bool = False, model_type: str = "BPE", normalizer=None, pre_tokenizer=None,
                 post_processor=None, decoder=None, continuing_subword_prefix: str = "", end_of_word_suffix: str = "", byte_fallback: bool = False,
                 max_input_chars_per_word: int = 100, special_tokens: Optional[Iterable[str]] = None, scores: Optional[Sequence[float]] = None,
                 unk_id: Optional[int] = None):
        """``vocab`` / ``merges`` / ``added_tokens`` with the GPT-2 split (or ``split_pattern``) is the short form; ``load_tokenizer`` passes
        the stages of a ``tokenizer.json`` (``normalizer``: str -> str; ``pre_tokenizer``: ``pipeline.PreTokenizer``; ``post_processor``: ids ->
        ids with the special tokens of one sequence; ``decoder``: token strings -> strings) and the model's type and affixes."""
        if model_type not in ("BPE", "WordPiece", "WordLevel", "Unigram"):
            raise InvalidArgument(f"unsupported tokenizer model {model_type}")
        self.model_type = model_type
        self.normalizer, self.pre_tokenizer, self.post_processor, self.decoder_chain = normalizer, pre_tokenizer, post_processor, decoder
        self.prefix, self.suffix, self.byte_fallback, self.max_chars = continuing_subword_prefix or "", end_of_word_suffix or "", byte_fallback, max_input_chars_per_word
        self.scores = {t: float(sc) for t, sc in zip(vocab, scores)} if scores is not None else None     # Unigram: log-probability per entry
        if model_type == "Unigram":
            if self.scores is None:
                raise InvalidArgument("a Unigram model needs one score per vocabulary entry")
            self._max_piece = max((len(t) for t in vocab), default=1)
            self._unk_score = min(self.scores.values(), default=0.0) - 10.0
            if unk_id is not None and unk_token is None:
                unk_token = next((t for t, i in vocab.items() if i == unk_id), None)
        self.vocab = dict(vocab)
        self.model_vocab = dict(vocab)                 # without the added tokens: what ``ignore_merges`` looks whole pieces up in
        self.ignore_merges = bool(ignore_merges)
        self.added = dict(added_tokens or {})
        self.vocab.update(self.added)
        self.inv = {i: t for t, i in self.vocab.items()}
        self.ranks = {tuple(m): i for i, m in enumerate(merges)}
        self.byte_level = pre_tokenizer.byte_level if pre_tokenizer is not None else byte_level
        self.special = set(self.added) if special_tokens is None else set(special_tokens)        # what ``skip_special_tokens`` drops
        if pre_tokenizer is not None and pre_tokenizer.regex_source is not None:
            split_pattern = pre_tokenizer.regex_source
        self.split = _re.compile(split_pattern or _GPT2_SPLIT)
        self.bos_token, self.eos_token, self.unk_token = bos_token, eos_token, unk_token
        self._b2u = _bytes_to_unicode()
        self._u2b = {v: k for k, v in self._b2u.items()}
        self._special_re = _re.compile("|".join(_re.escape(t) for t in sorted(self.added, key=len, reverse=True))) if self.added else None
        self._cache: Dict[str, List[str]] = {}
        self._native = None
        pat = split_pattern or _GPT2_SPLIT
        self._kind = 0 if pat == _GPT2_SPLIT else 1 if pat == _LLAMA3_SPLIT else None      # patterns the native splitter restates
        if normalizer is not None or (pre_tokenizer is not None and pre_tokenizer.regex_source is None):
            self._kind = None                          # other stages run in Python; the merges may still be native
        if os.environ.get("FT_TOKENIZE_NATIVE", "1") != "0" and model_type == "BPE" and not self.prefix and not self.suffix and not byte_fallback:
            self._build_native()

    # ------------------------------------------------------------------ native merge engine
    def _build_native(self) -> None:
        """Hands the merge table to the runtime library as id triples. Left alone (Python loop) when the library is missing or a merge
        names a string that is not a vocabulary entry."""
        try:
            from .. import _lib
            rt = _lib.runtime()
            rt.ft_bpe_create.restype = ctypes.c_void_p
            rt.ft_bpe_encode.restype = ctypes.c_int64
            rt.ft_bpe_destroy.restype = None
        except Exception:
            return
        v = self.model_vocab
        pairs = sorted(self.ranks.items(), key=lambda kv: kv[1])
        left, right, merged = np.empty(len(pairs), np.int32), np.empty(len(pairs), np.int32), np.empty(len(pairs), np.int32)
        for r, ((a, b), _) in enumerate(pairs):
            ia, ib, iab = v.get(a), v.get(b), v.get(a + b)
            if ia is None or ib is None or iab is None:
                return
            left[r], right[r], merged[r] = ia, ib, iab
        null = ctypes.c_void_p(None)
        if self.byte_level:
            byte_sym = np.array([v.get(self._b2u[b], -1) for b in range(256)], np.int32)
            chars = (null, null, 0)
        else:
            single = [(ord(t), i) for t, i in v.items() if len(t) == 1]
            cp, cid = np.array([c for c, _ in single], np.uint32), np.array([i for _, i in single], np.int32)
            byte_sym = None
            chars = (cp.ctypes.data_as(ctypes.c_void_p), cid.ctypes.data_as(ctypes.c_void_p), len(single))
        whole = (null, null, null, 0)
        if self.ignore_merges:
            raw, ids = [], []
            for t, i in v.items():
                if self.byte_level:
                    try:
                        raw.append(bytes(self._u2b[ch] for ch in t))
                    except KeyError:
                        continue
                else:
                    raw.append(t.encode("utf-8"))
                ids.append(i)
            blob = np.frombuffer(b"".join(raw) or b"\0", np.uint8)
            woff = np.zeros(len(raw) + 1, np.int64)
            np.cumsum([len(x) for x in raw], out=woff[1:])
            wid = np.array(ids, np.int32)
            whole = (blob.ctypes.data_as(ctypes.c_void_p), woff.ctypes.data_as(ctypes.c_void_p), wid.ctypes.data_as(ctypes.c_void_p), len(raw))
        h = rt.ft_bpe_create(left.ctypes.data_as(ctypes.c_void_p), right.ctypes.data_as(ctypes.c_void_p), merged.ctypes.data_as(ctypes.c_void_p),
                             ctypes.c_int64(len(pairs)), byte_sym.ctypes.data_as(ctypes.c_void_p) if byte_sym is not None else null,
                             chars[0], chars[1], ctypes.c_int64(chars[2]), whole[0], whole[1], whole[2], ctypes.c_int64(whole[3]))
        if h:
            self._native, self._rt = ctypes.c_void_p(h), rt
            if self._kind is not None:
                rt.ft_bpe_encode_texts.restype = ctypes.c_int64
                _install_classes(rt)

    def __del__(self):
        h, self._native = getattr(self, "_native", None), None
        if h is not None:
            try:
                self._rt.ft_bpe_destroy(h)
            except Exception:
                pass

    def _native_pieces(self, pieces: Sequence[str], threads: int = 1):
        """ids (int32 array) and the running id count after each piece for ``pieces``; None when a piece needs the Python path."""
        raw = [p.encode("utf-8") for p in pieces]
        off = np.zeros(len(raw) + 1, np.int64)
        if raw:
            np.cumsum([len(x) for x in raw], out=off[1:])
        blob = b"".join(raw)
        out = np.empty(max(int(off[-1]), 1), np.int32)
        out_off = np.empty(len(raw) + 1, np.int64)
        n = self._rt.ft_bpe_encode(self._native, ctypes.c_char_p(blob), off.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(len(raw)),
                                   out.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(out.size), out_off.ctypes.data_as(ctypes.c_void_p),
                                   ctypes.c_int(threads))
        if n < 0:
            return None
        return out[:n], out_off

    def _native_texts(self, texts: Sequence[str], threads: int = 1):
        """Splits and encodes ``texts`` in the runtime library: ids and the running id count after each text; None when the split
        pattern is not one of the two restated ones or a text needs the Python path."""
        if self._native is None or self._kind is None:
            return None
        try:
            raw = [t.encode("utf-8") for t in texts]
        except UnicodeEncodeError:                     # lone surrogates
            return None
        off = np.zeros(len(raw) + 1, np.int64)
        if raw:
            np.cumsum([len(x) for x in raw], out=off[1:])
        out = np.empty(max(int(off[-1]), 1), np.int32)
        out_off = np.empty(len(raw) + 1, np.int64)
        n = self._rt.ft_bpe_encode_texts(self._native, ctypes.c_int(self._kind), ctypes.c_char_p(b"".join(raw)), off.ctypes.data_as(ctypes.c_void_p),
                                         ctypes.c_int64(len(raw)), out.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(out.size),
                                         out_off.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(threads))
        if n < 0:
            return None
        return out[:n], out_off

    def vocab_size(self) -> int:
        return len(self.vocab)

    def token_to_id(self, tok: str) -> Optional[int]:
        return self.vocab.get(tok)

    def id_to_token(self, i: int) -> Optional[str]:
        return self.inv.get(i)

    def _bpe(self, word: str) -> List[str]:
        if word in self._cache:
            return self._cache[word]
        if self.ignore_merges and word in self.model_vocab:
            self._cache[word] = [word]
            return [word]
        parts = list(word)
        if self.prefix:
            parts = parts[:1] + [self.prefix + c for c in parts[1:]]
        if self.suffix and parts:
            parts[-1] += self.suffix
        while len(parts) > 1:
            best, bi = None, -1
            for i in range(len(parts) - 1):
                r = self.ranks.get((parts[i], parts[i + 1]))
                if r is not None and (best is None or r < best):
                    best, bi = r, i
            if best is None:
                break
            parts[bi: bi + 2] = [parts[bi] + parts[bi + 1]]
        self._cache[word] = parts
        return parts

    def _encode_plain(self, text: str) -> List[int]:
        if self.normalizer is not None:
            text = self.normalizer(text)
        got = self._native_texts([text])
        if got is not None:
            return got[0].tolist()
        if self._native is not None:
            raw = self.pre_tokenizer.pieces(text, mapped=False) if self.pre_tokenizer is not None else self.split.findall(text)
            got = self._native_pieces(raw)
            if got is not None:
                return got[0].tolist()
        return self._encode_plain_py(text)

    def _lookup(self, tok: str, ids: List[int]) -> None:
        i = self.vocab.get(tok)
        if i is None and self.byte_fallback:
            fb = [self.vocab.get(f"<0x{b:02X}>") for b in tok.encode("utf-8")]
            if all(x is not None for x in fb):
                ids += fb
                return
        if i is None:
            if self.unk_token is None:
                raise InvalidArgument(f"token {tok!r} not in vocabulary and no unk token configured")
            i = self.vocab[self.unk_token]
        ids.append(i)

    def _wordpiece(self, word: str) -> List[str]:
        """Greedy longest match from the left; pieces after the first carry the continuing prefix; a word with a part that matches nothing
        is the unknown token as a whole."""
        unk = [self.unk_token or "[UNK]"]
        if len(word) > self.max_chars:
            return unk
        out, start = [], 0
        while start < len(word):
            end, cur = len(word), None
            while start < end:
                sub = word[start:end] if start == 0 else self.prefix + word[start:end]
                if sub in self.model_vocab:
                    cur = sub
                    break
                end -= 1
            if cur is None:
                return unk
            out.append(cur)
            start = end
        return out

    def _unigram(self, word: str) -> List[str]:
        """Best segmentation of ``word`` under the entry scores (Viterbi over end positions; ties keep the path found first, from the
        earlier start); a character that starts no entry costs the lowest score minus ten, and runs of such characters come out as one
        piece (which the lookup maps to the unknown token or to byte tokens)."""
        n = len(word)
        best = [float("-inf")] * (n + 1)
        back = [-1] * (n + 1)
        best[0] = 0.0
        scores = self.scores
        for a in range(n):
            if best[a] == float("-inf"):
                continue
            single = False
            for e in range(a + 1, min(n, a + self._max_piece) + 1):
                sc = scores.get(word[a:e])
                if sc is None:
                    continue
                if e == a + 1:
                    single = True
                if back[e] < 0 or best[a] + sc > best[e]:
                    best[e], back[e] = best[a] + sc, a
            if not single and (back[a + 1] < 0 or best[a] + self._unk_score > best[a + 1]):
                best[a + 1], back[a + 1] = best[a] + self._unk_score, a
        out, e = [], n
        while e > 0:
            out.append(word[back[e]: e])
            e = back[e]
        out.reverse()
        fused: List[str] = []
        for t in out:
            if t not in scores and fused and fused[-1] not in scores:
                fused[-1] += t
            else:
                fused.append(t)
        return fused

    def _encode_plain_py(self, text: str) -> List[int]:
        """``text`` is already normalised."""
        ids: List[int] = []
        if self.pre_tokenizer is not None:
            pieces = self.pre_tokenizer.pieces(text)
        else:
            pieces = ["".join(self._b2u[b] for b in p.encode("utf-8")) if self.byte_level else p for p in self.split.findall(text)]
        for w in pieces:
            mt = self.model_type
            for tok in (self._bpe(w) if mt == "BPE" else self._wordpiece(w) if mt == "WordPiece" else self._unigram(w) if mt == "Unigram" else [w]):
                self._lookup(tok, ids)
        return ids

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        """Ids of ``text``. ``add_special_tokens``: wrap them the way the file's post-processor does for one sequence (without one: the
        beginning-of-sequence token in front, if the tokenizer names one)."""
        if add_special_tokens and self.post_processor is not None:
            return self.post_processor(self.encode(text, False))
        ids: List[int] = []
        if add_special_tokens and self.bos_token:
            ids.append(self.vocab[self.bos_token])
        if self._special_re is None:
            ids += self._encode_plain(text)
        else:
            pos = 0
            for m in self._special_re.finditer(text):
                if m.start() > pos:
                    ids += self._encode_plain(text[pos: m.start()])
                ids.append(self.added[m.group(0)])
                pos = m.end()
            if pos < len(text):
                ids += self._encode_plain(text[pos:])
        return ids

    def _segments(self, text: str):
        """(plain text | None, special id | None) runs of ``text`` in order."""
        if self._special_re is None:
            if text:
                yield text, None
            return
        pos = 0
        for m in self._special_re.finditer(text):
            if m.start() > pos:
                yield text[pos: m.start()], None
            yield None, self.added[m.group(0)]
            pos = m.end()
        if pos < len(text):
            yield text[pos:], None

    def encode_batch(self, texts: Iterable[str], add_special_tokens: bool = False) -> List[List[int]]:
        """All texts in one call of the native engine (their pieces spread over the host's cores); a batch that holds a piece the engine
        cannot take goes text by text."""
        texts = list(texts)
        if self._native is None or not texts or self.normalizer is not None or self.post_processor is not None \
                or (self.pre_tokenizer is not None and self._kind is None):
            return [self.encode(t, add_special_tokens) for t in texts]
        threads = min(os.cpu_count() or 1, 16)
        bos = [self.vocab[self.bos_token]] if add_special_tokens and self.bos_token else []
        if self._kind is not None:                     # splitting and merging both in the library: one run of plain text = one unit of work
            runs: List[str] = []
            plan = []
            for t in texts:
                items = []
                for plain, special in self._segments(t):
                    if plain is None:
                        items.append(special)
                    else:
                        items.append((len(runs),))
                        runs.append(plain)
                plan.append(items)
            got = self._native_texts(runs, threads)
            if got is not None:
                ids, off = got
                out = []
                for items in plan:
                    if len(items) == 1 and isinstance(items[0], tuple) and not bos:
                        out.append(ids[off[items[0][0]]: off[items[0][0] + 1]].tolist())
                        continue
                    row = list(bos)
                    for it in items:
                        if isinstance(it, tuple):
                            row += ids[off[it[0]]: off[it[0] + 1]].tolist()
                        else:
                            row.append(it)
                    out.append(row)
                return out
        pieces: List[str] = []
        plan = []                                      # per text: list of (first piece, end piece) ranges or special ids
        for t in texts:
            items = []
            for plain, special in self._segments(t):
                if plain is None:
                    items.append(special)
                else:
                    ps = self.split.findall(plain)
                    items.append((len(pieces), len(pieces) + len(ps)))
                    pieces += ps
            plan.append(items)
        got = self._native_pieces(pieces, threads=threads)
        if got is None:
            return [self.encode(t, add_special_tokens) for t in texts]
        ids, off = got
        out = []
        for items in plan:
            row = list(bos)
            for it in items:
                if isinstance(it, tuple):
                    row += ids[off[it[0]]: off[it[1]]].tolist()
                else:
                    row.append(it)
            out.append(row)
        return out

    def decode(self, ids: Iterable[int], skip_special_tokens: bool = True) -> str:
        if self.decoder_chain is not None:
            toks = [self.inv[int(i)] for i in ids if int(i) in self.inv]
            if skip_special_tokens:
                toks = [t for t in toks if t not in self.special]
            return "".join(self.decoder_chain(toks))
        out, buf = [], bytearray()

        def flush():
            if buf:
                out.append(buf.decode("utf-8", "replace"))
                buf.clear()
        for i in ids:
            tok = self.inv.get(int(i))
            if tok is None:
                continue
            if tok in self.added:
                flush()
                if not skip_special_tokens:
                    out.append(tok)
                continue
            if self.byte_level:
                buf.extend(self._u2b.get(ch, ord("?")) for ch in tok)
            else:
                flush()
                out.append(tok)
        flush()
        return "".join(out)


def load_tokenizer(path) -> Tokenizer:
    """Load ``tokenizer.json`` (a file, or a directory containing one; ``tokenizer_config.json`` beside it supplies bos/eos)."""
    p = Path(path)
    if p.is_dir():
        p = p / "tokenizer.json"
    j = json.loads(p.read_text())
    model = j.get("model", {})
    mtype = model.get("type") or ("Unigram" if isinstance(model.get("vocab"), list) else "BPE" if "merges" in model else
                                  "WordPiece" if "continuing_subword_prefix" in model else "WordLevel")
    if mtype not in ("BPE", "WordPiece", "WordLevel", "Unigram"):
        raise InvalidArgument(f"unsupported tokenizer model {mtype}")
    merges = [tuple(m.split(" ", 1)) if isinstance(m, str) else tuple(m) for m in model.get("merges", [])]
    added = {a["content"]: a["id"] for a in j.get("added_tokens", [])}
    special = [a["content"] for a in j.get("added_tokens", []) if a.get("special", False)]
    b2u = _bytes_to_unicode()
    pre = _pl.PreTokenizer(j.get("pre_tokenizer"), b2u) if j.get("pre_tokenizer") else None
    vocab = model.get("vocab", {})
    scores = None
    if mtype == "Unigram":                             # a list of [entry, score]; the id is the position
        scores = [sc for _, sc in vocab]
        vocab = {t: i for i, (t, _) in enumerate(vocab)}
    full = dict(vocab)
    full.update(added)
    bos = eos = None
    cfg = p.parent / "tokenizer_config.json"
    if cfg.exists():
        c = json.loads(cfg.read_text())
        def tok(v):
            return v.get("content") if isinstance(v, dict) else v
        bos, eos = tok(c.get("bos_token")), tok(c.get("eos_token"))
    byte_level = (pre is not None and pre.byte_level) or (j.get("decoder") or {}).get("type") == "ByteLevel"
    if pre is None and mtype == "BPE" and byte_level:                       # a byte-level decoder without a pre-tokenizer entry: the GPT-2 form
        pre = _pl.PreTokenizer({"type": "ByteLevel", "add_prefix_space": False, "use_regex": True}, b2u)
    if pre is None:
        pre = _pl.PreTokenizer({"type": "Sequence", "pretokenizers": []}, b2u)     # the model sees the whole normalised text
    return Tokenizer(vocab, merges, added, byte_level, None, bos, eos, model.get("unk_token"), ignore_merges=bool(model.get("ignore_merges", False)),
                     model_type=mtype, normalizer=_pl.build_normalizer(j.get("normalizer")), pre_tokenizer=pre,
                     post_processor=_pl.build_post_processor(j.get("post_processor"), full), decoder=_pl.build_decoder(j.get("decoder"), {v: k for k, v in b2u.items()}),
                     continuing_subword_prefix=model.get("continuing_subword_prefix") or "", end_of_word_suffix=model.get("end_of_word_suffix") or "",
                     byte_fallback=bool(model.get("byte_fallback", False)), max_input_chars_per_word=int(model.get("max_input_chars_per_word", 100)),
                     special_tokens=special, scores=scores, unk_id=model.get("unk_id"))


def encode(tok: Tokenizer, text: str, add_special_tokens: bool = False) -> List[int]:
    return tok.encode(text, add_special_tokens)


def encode_batch(tok: Tokenizer, texts, add_special_tokens: bool = False):
    return tok.encode_batch(texts, add_special_tokens)


def decode(tok: Tokenizer, ids, skip_special_tokens: bool = True) -> str:
    return tok.decode(ids, skip_special_tokens)


@dataclass
class ChatMessage:
    """One turn of a conversation (ferrotorch-tokenize/src/lib.rs:167)."""
    role: str
    content: str

    def __getitem__(self, k):                                 # the built-in templates index messages like dicts
        return getattr(self, k)


def vocab_size(tok: Tokenizer, with_added_tokens: bool = True) -> int:
    return len(tok.vocab) if with_added_tokens else len(tok.vocab) - len(tok.added)


def token_to_id(tok: Tokenizer, token: str) -> Optional[int]:
    return tok.token_to_id(token)


def id_to_token(tok: Tokenizer, i: int) -> Optional[str]:
    return tok.id_to_token(i)


def _render_jinja(template: str, messages, add_generation_prompt: bool, bos_token: Optional[str], eos_token: Optional[str]) -> str:
    """Hugging Face chat templates are Jinja2: rendered in a sandbox with ``messages``, ``add_generation_prompt``, ``bos_token``, ``eos_token``
    and ``raise_exception(msg)`` (lib.rs:225-300). Undefined variables are errors, as in the reference."""
    try:
        import jinja2
        from jinja2.sandbox import ImmutableSandboxedEnvironment
    except ImportError:
        raise InvalidArgument("Jinja chat templates need the jinja2 package") from None

    def raise_exception(msg):
        raise jinja2.exceptions.TemplateError(msg)
    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, undefined=jinja2.StrictUndefined)
    env.globals["raise_exception"] = raise_exception
    msgs = [{"role": m["role"], "content": m["content"]} for m in messages]
    try:
        return env.from_string(template).render(messages=msgs, add_generation_prompt=add_generation_prompt, bos_token=bos_token or "", eos_token=eos_token or "")
    except jinja2.exceptions.TemplateError as e:
        raise InvalidArgument(f"chat template failed to render: {e}") from None


def apply_chat_template(messages, template="llama3", add_generation_prompt: bool = True, bos_token: Optional[str] = None, eos_token: Optional[str] = None) -> str:
    """Render a conversation. ``template``: "llama3", "chatml", "llama2", "plain", a Jinja2 template (the ``chat_template`` string of a
    ``tokenizer_config.json``), or a format string with ``{role}`` / ``{content}``. The reference's argument order
    ``(template, messages, ...)`` is accepted too."""
    if isinstance(messages, str) and not isinstance(template, str):
        messages, template = template, messages
    if "{%" in template or "{{" in template:
        return _render_jinja(template, messages, add_generation_prompt, bos_token, eos_token)
    if template == "llama3":
        s = "<|begin_of_text|>" + "".join(f"<|start_header_id|>{m['role']}<|end_header_id|>\n\n{m['content']}<|eot_id|>" for m in messages)
        return s + ("<|start_header_id|>assistant<|end_header_id|>\n\n" if add_generation_prompt else "")
    if template == "chatml":
        s = "".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in messages)
        return s + ("<|im_start|>assistant\n" if add_generation_prompt else "")
    if template == "llama2":
        sys = next((m["content"] for m in messages if m["role"] == "system"), None)
        out, first = "", True
        for m in messages:
            if m["role"] == "user":
                c = f"<<SYS>>\n{sys}\n<</SYS>>\n\n{m['content']}" if (sys and first) else m["content"]
                out += f"<s>[INST] {c} [/INST]"
                first = False
            elif m["role"] == "assistant":
                out += f" {m['content']} </s>"
        return out
    if template == "plain":
        return "\n".join(f"{m['role']}: {m['content']}" for m in messages) + ("\nassistant:" if add_generation_prompt else "")
    return "".join(template.format(role=m["role"], content=m["content"]) for m in messages)


def apply_chat_template_to_ids(tok: Tokenizer, template: str, messages, add_generation_prompt: bool = True, bos_token: Optional[str] = None,
                               eos_token: Optional[str] = None, add_special_tokens: bool = False):
    """``(rendered text, token ids)``. Templates normally write the BOS token themselves, hence ``add_special_tokens=False`` by default
    (lib.rs:313)."""
    text = apply_chat_template(messages, template, add_generation_prompt, bos_token if bos_token is not None else tok.bos_token,
                               eos_token if eos_token is not None else tok.eos_token)
    return text, tok.encode(text, add_special_tokens)


def load_chat_template(tokenizer_config_path) -> Optional[str]:
    """The ``chat_template`` of a ``tokenizer_config.json``: a string, or the first ``template`` of a list of named templates; ``None`` when the
    file has none. An unreadable file is an :class:`Internal` error, malformed content an :class:`InvalidArgument` (lib.rs:349)."""
    import json
    try:
        raw = open(tokenizer_config_path, "rb").read()
    except OSError as e:
        raise Internal(f"failed to read tokenizer_config {tokenizer_config_path}: {e!r}") from None
    try:
        value = json.loads(raw)
    except ValueError as e:
        raise InvalidArgument(f"failed to parse tokenizer_config {tokenizer_config_path}: {e}") from None
    ct = value.get("chat_template") if isinstance(value, dict) else None
    if ct is None:
        return None
    if isinstance(ct, str):
        return ct
    if isinstance(ct, list):
        return next((e["template"] for e in ct if isinstance(e, dict) and isinstance(e.get("template"), str)), None)
    raise InvalidArgument(f"tokenizer_config {tokenizer_config_path} has chat_template of unexpected type")
