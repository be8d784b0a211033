"""The stages of a ``tokenizer.json`` pipeline around the model: normalizers, pre-tokenizers, post-processors and decoders, each built from
its JSON description and following the behaviour of the HF ``tokenizers`` library for that ``type``.

Reference parity: the reference loads any ``tokenizer.json`` through that library (ferrotorch-tokenize/src/lib.rs:59-83) and pins five
families (Llama-3, CLIP, BERT, GPT-2, SmolLM; ferrotorch-tokenize/tests/conformance_hf_parity.rs:43); the stage types those files use,
and the common ones beside them, are implemented here.
"""
from __future__ import annotations

import unicodedata
from typing import Callable, Dict, List, Optional, Tuple

import regex as _re

from ..errors import InvalidArgument

GPT2_SPLIT = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""


# ---------------------------------------------------------------------------------------------------------------------
# character classes
# ---------------------------------------------------------------------------------------------------------------------
_WS = set("\t\n\x0b\x0c\r \x85\xa0\u1680\u2028\u2029\u202f\u205f\u3000") | {chr(c) for c in range(0x2000, 0x200B)}      # Unicode White_Space


def _is_ws(c: str) -> bool:
    return c in _WS


def _is_control(c: str) -> bool:
    if c in "\t\n\r":
        return False
    return unicodedata.category(c) in ("Cc", "Cf", "Cn", "Co")


def _is_punct(c: str) -> bool:
    o = ord(c)
    if 33 <= o <= 47 or 58 <= o <= 64 or 91 <= o <= 96 or 123 <= o <= 126:
        return True
    return unicodedata.category(c).startswith("P")


def _is_cjk(c: str) -> bool:
    o = ord(c)
    return (0x4E00 <= o <= 0x9FFF or 0x3400 <= o <= 0x4DBF or 0x20000 <= o <= 0x2A6DF or 0x2A700 <= o <= 0x2B73F or 0x2B740 <= o <= 0x2B81F
            or 0x2B920 <= o <= 0x2CEAF or 0xF900 <= o <= 0xFAFF or 0x2F800 <= o <= 0x2FA1F)


def _pattern(p) -> "_re.Pattern":
    """``{"String": s}`` (literal) or ``{"Regex": r}`` of a Split / Replace stage."""
    if isinstance(p, dict):
        if "Regex" in p:
            return _re.compile(p["Regex"])
        if "String" in p:
            return _re.compile(_re.escape(p["String"]))
    if isinstance(p, str):
        return _re.compile(_re.escape(p))
    raise InvalidArgument(f"unsupported pattern {p!r}")


# ---------------------------------------------------------------------------------------------------------------------
# normalizers: str -> str
# ---------------------------------------------------------------------------------------------------------------------
def _bert_normalizer(j) -> Callable[[str], str]:
    clean, chinese, lower = j.get("clean_text", True), j.get("handle_chinese_chars", True), j.get("lowercase", True)
    strip = j.get("strip_accents")
    strip = lower if strip is None else strip

    def run(t: str) -> str:
        if clean:
            t = "".join(" " if _is_ws(c) else c for c in t if not (ord(c) == 0 or ord(c) == 0xFFFD or _is_control(c)))
        if chinese:
            t = "".join(f" {c} " if _is_cjk(c) else c for c in t)
        if strip:
            t = "".join(c for c in unicodedata.normalize("NFD", t) if unicodedata.category(c) != "Mn")
        if lower:
            t = t.lower()
        return t
    return run


def build_normalizer(j) -> Optional[Callable[[str], str]]:
    if not j:
        return None
    t = j.get("type")
    if t == "Sequence":
        stages = [s for s in (build_normalizer(x) for x in j.get("normalizers", [])) if s is not None]

        def run(text: str) -> str:
            for s in stages:
                text = s(text)
            return text
        return run
    if t in ("NFC", "NFD", "NFKC", "NFKD"):
        return lambda text: unicodedata.normalize(t, text)
    if t == "Lowercase":
        return str.lower
    if t == "Strip":
        left, right = j.get("strip_left", True), j.get("strip_right", True)
        return lambda text: (text.lstrip() if left else text).rstrip() if right else (text.lstrip() if left else text)
    if t == "StripAccents":
        return lambda text: "".join(c for c in text if not unicodedata.category(c).startswith("M"))
    if t == "Replace":
        rx, content = _pattern(j.get("pattern")), j.get("content", "")
        return lambda text: rx.sub(lambda m: content, text)
    if t == "Prepend":
        pre = j.get("prepend", "")
        return lambda text: pre + text if text else text
    if t == "BertNormalizer":
        return _bert_normalizer(j)
    raise InvalidArgument(f"unsupported normalizer {t}")


# ---------------------------------------------------------------------------------------------------------------------
# pre-tokenizers: list of pieces -> list of pieces
# ---------------------------------------------------------------------------------------------------------------------
def _split(rx, text: str, behavior: str, invert: bool) -> List[str]:
    """Cuts ``text`` at the matches of ``rx`` (at the gaps between them when ``invert``) the way ``Split`` does for ``behavior``."""
    spans: List[Tuple[int, int, bool]] = []                # (start, end, is_delimiter)
    pos = 0
    for m in rx.finditer(text):
        if m.end() == m.start():
            continue
        if m.start() > pos:
            spans.append((pos, m.start(), False))
        spans.append((m.start(), m.end(), True))
        pos = m.end()
    if pos < len(text):
        spans.append((pos, len(text), False))
    if invert:
        spans = [(a, b, not d) for a, b, d in spans]
    b = behavior.lower().replace("_", "")
    out: List[str] = []
    if b == "removed":
        out = [text[a:e] for a, e, d in spans if not d]
    elif b == "isolated":
        out = [text[a:e] for a, e, _ in spans]
    elif b == "mergedwithprevious":
        for a, e, d in spans:
            if d and out:
                out[-1] += text[a:e]
            else:
                out.append(text[a:e])
    elif b == "mergedwithnext":
        carry = ""
        for a, e, d in spans:
            if d:
                carry += text[a:e]
            else:
                out.append(carry + text[a:e])
                carry = ""
        if carry:
            out.append(carry)
    elif b == "contiguous":
        prev = None
        for a, e, d in spans:
            if d and prev is True:
                out[-1] += text[a:e]
            else:
                out.append(text[a:e])
            prev = d
    else:
        raise InvalidArgument(f"unsupported split behaviour {behavior}")
    return [p for p in out if p]


_WHITESPACE_RX = _re.compile(r"\w+|[^\w\s]+")
_GPT2_RX = _re.compile(GPT2_SPLIT)
_DIGIT_RX, _DIGITS_RX = _re.compile(r"\p{N}"), _re.compile(r"\p{N}+")


def _bert_pre(text: str) -> List[str]:
    out: List[str] = []
    for word in text.split():
        cur = ""
        for c in word:
            if _is_punct(c):
                if cur:
                    out.append(cur)
                    cur = ""
                out.append(c)
            else:
                cur += c
        if cur:
            out.append(cur)
    return out


class PreTokenizer:
    """``pieces(text)``: the pieces the model sees. ``byte_level`` is set when a ByteLevel stage maps the bytes of every piece to printable
    stand-ins (the model's vocabulary is written in them); ``regex_source`` is the pattern of a pipeline that is nothing but one split by a
    regular expression followed by the byte mapping (what the native splitter can take over), else None."""

    def __init__(self, j, byte_to_unicode: Dict[int, str]):
        self.byte_level = False
        self.regex_source: Optional[str] = None
        self._b2u = byte_to_unicode
        self._stages = self._build(j) if j else []
        kinds = self._kinds(j) if j else []
        if kinds == ["ByteLevel:regex"]:
            self.regex_source = GPT2_SPLIT
        elif len(kinds) == 2 and kinds[0].startswith("Split:isolated:") and kinds[1] == "ByteLevel:plain":
            self.regex_source = kinds[0][len("Split:isolated:"):]

    def _kinds(self, j) -> List[str]:
        t = j.get("type")
        if t == "Sequence":
            return [k for x in j.get("pretokenizers", []) for k in self._kinds(x)]
        if t == "ByteLevel":
            return ["ByteLevel:prefix" if j.get("add_prefix_space", True) else "ByteLevel:regex" if j.get("use_regex", True) else "ByteLevel:plain"]
        if t == "Split" and isinstance(j.get("pattern"), dict) and "Regex" in j["pattern"] and not j.get("invert", False) \
                and j.get("behavior", "").lower() == "isolated":
            return ["Split:isolated:" + j["pattern"]["Regex"]]
        return [str(t)]

    def _build(self, j) -> List[Callable[[List[str]], List[str]]]:
        t = j.get("type")
        if t == "Sequence":
            return [s for x in j.get("pretokenizers", []) for s in self._build(x)]
        if t == "ByteLevel":
            self.byte_level = True
            prefix, use_regex = j.get("add_prefix_space", True), j.get("use_regex", True)

            def run(pieces: List[str]) -> List[str]:
                out = []
                for p in pieces:
                    if prefix and not p.startswith(" "):
                        p = " " + p
                    out += _GPT2_RX.findall(p) if use_regex else [p]
                return out
            return [run]
        if t == "Split":
            rx, behavior, invert = _pattern(j.get("pattern")), j.get("behavior", "Isolated"), j.get("invert", False)
            return [lambda pieces: [q for p in pieces for q in _split(rx, p, behavior, invert)]]
        if t == "Whitespace":
            return [lambda pieces: [q for p in pieces for q in _WHITESPACE_RX.findall(p)]]
        if t == "WhitespaceSplit":
            return [lambda pieces: [q for p in pieces for q in p.split()]]
        if t == "BertPreTokenizer":
            return [lambda pieces: [q for p in pieces for q in _bert_pre(p)]]
        if t == "Digits":
            rx = _DIGIT_RX if j.get("individual_digits", False) else _DIGITS_RX
            return [lambda pieces: [q for p in pieces for q in _split(rx, p, "isolated", False)]]
        if t == "Punctuation":
            behavior = j.get("behavior", "Isolated")
            rx = _re.compile(r"[!-/:-@\[-`{-~\p{P}]")
            return [lambda pieces: [q for p in pieces for q in _split(rx, p, behavior, False)]]
        if t == "Metaspace":
            rep = j.get("replacement", "▁")
            scheme = j.get("prepend_scheme", "always" if j.get("add_prefix_space", True) else "never")
            do_split = j.get("split", True)

            def run(pieces: List[str]) -> List[str]:
                out = []
                for k, p in enumerate(pieces):
                    p = p.replace(" ", rep)
                    if (scheme == "always" or (scheme == "first" and k == 0)) and not p.startswith(rep):
                        p = rep + p
                    out += [q for q in _re.split(f"(?={_re.escape(rep)})", p) if q] if do_split else [p]
                return out
            return [run]
        raise InvalidArgument(f"unsupported pre-tokenizer {t}")

    def pieces(self, text: str, mapped: bool = True) -> List[str]:
        """``mapped=False`` leaves the bytes of a byte-level pipeline as they are (the native merge engine maps them itself)."""
        ps = [text] if text else []
        for s in self._stages:
            ps = s(ps)
        if self.byte_level and mapped:
            b2u = self._b2u
            ps = ["".join(b2u[b] for b in p.encode("utf-8")) for p in ps]
        return ps


# ---------------------------------------------------------------------------------------------------------------------
# post-processors: ids -> ids with the special tokens of a single sequence
# ---------------------------------------------------------------------------------------------------------------------
def build_post_processor(j, vocab: Dict[str, int]) -> Optional[Callable[[List[int]], List[int]]]:
    if not j:
        return None
    t = j.get("type")
    if t == "Sequence":
        stages = [s for s in (build_post_processor(x, vocab) for x in j.get("processors", [])) if s is not None]
        if not stages:
            return None

        def run(ids: List[int]) -> List[int]:
            for s in stages:
                ids = s(ids)
            return ids
        return run
    if t == "ByteLevel":
        return None
    if t in ("BertProcessing", "RobertaProcessing"):
        cls_id, sep_id = int(j["cls"][1]), int(j["sep"][1])
        return lambda ids: [cls_id] + ids + [sep_id]
    if t == "TemplateProcessing":
        special = j.get("special_tokens", {})
        plan: List[Optional[List[int]]] = []
        for item in j.get("single", []):
            if "Sequence" in item:
                plan.append(None)
            else:
                name = item["SpecialToken"]["id"]
                plan.append([int(i) for i in special[name]["ids"]] if name in special else [vocab[name]])
        return lambda ids: [i for part in plan for i in (ids if part is None else part)]
    raise InvalidArgument(f"unsupported post-processor {t}")


# ---------------------------------------------------------------------------------------------------------------------
# decoders: list of token strings -> list of strings (joined by the caller)
# ---------------------------------------------------------------------------------------------------------------------
def _cleanup(s: str) -> str:
    for a, b in ((" .", "."), (" ?", "?"), (" !", "!"), (" ,", ","), (" ' ", "'"), (" n't", "n't"), (" 'm", "'m"), (" do not", " don't"), (" 's", "'s"),
                 (" 've", "'ve"), (" 're", "'re")):
        s = s.replace(a, b)
    return s


def build_decoder(j, unicode_to_byte: Dict[str, int]) -> Optional[Callable[[List[str]], List[str]]]:
    if not j:
        return None
    t = j.get("type")
    if t == "Sequence":
        stages = [s for s in (build_decoder(x, unicode_to_byte) for x in j.get("decoders", [])) if s is not None]

        def run(toks: List[str]) -> List[str]:
            for s in stages:
                toks = s(toks)
            return toks
        return run
    if t == "ByteLevel":
        def run(toks: List[str]) -> List[str]:
            buf = bytearray()
            for tok in toks:
                for ch in tok:
                    b = unicode_to_byte.get(ch)
                    if b is None:
                        buf.extend(ch.encode("utf-8"))
                    else:
                        buf.append(b)
            return [buf.decode("utf-8", "replace")]
        return run
    if t == "WordPiece":
        prefix, clean = j.get("prefix", "##"), j.get("cleanup", True)

        def run(toks: List[str]) -> List[str]:
            out = []
            for k, tok in enumerate(toks):
                if k:
                    tok = tok[len(prefix):] if tok.startswith(prefix) else " " + tok
                out.append(_cleanup(tok) if clean else tok)
            return out
        return run
    if t == "BPEDecoder":
        suffix = j.get("suffix", "</w>")
        return lambda toks: [tok.replace(suffix, "" if k == len(toks) - 1 else " ") for k, tok in enumerate(toks)]
    if t == "Metaspace":
        rep = j.get("replacement", "▁")
        scheme = j.get("prepend_scheme", "always" if j.get("add_prefix_space", True) else "never")

        def run(toks: List[str]) -> List[str]:
            out = []
            for k, tok in enumerate(toks):
                tok = tok.replace(rep, " ")
                if k == 0 and scheme != "never" and tok.startswith(" "):
                    tok = tok[1:]
                out.append(tok)
            return out
        return run
    if t == "Replace":
        rx, content = _pattern(j.get("pattern")), j.get("content", "")
        return lambda toks: [rx.sub(lambda m: content, tok) for tok in toks]
    if t == "Fuse":
        return lambda toks: ["".join(toks)]
    if t == "Strip":
        content, start, stop = j.get("content", " "), j.get("start", 0), j.get("stop", 0)

        def run(toks: List[str]) -> List[str]:
            out = []
            for tok in toks:
                a = 0
                while a < start and a < len(tok) and tok[a] == content:
                    a += 1
                e = len(tok)
                while len(tok) - e < stop and e > a and tok[e - 1] == content:
                    e -= 1
                out.append(tok[a:e])
            return out
        return run
    if t == "ByteFallback":
        def run(toks: List[str]) -> List[str]:
            out: List[str] = []
            buf = bytearray()

            def flush():
                if buf:
                    out.append(buf.decode("utf-8", "replace"))
                    buf.clear()
            for tok in toks:
                if len(tok) == 6 and tok.startswith("<0x") and tok.endswith(">"):
                    try:
                        buf.append(int(tok[3:5], 16))
                        continue
                    except ValueError:
                        pass
                flush()
                out.append(tok)
            flush()
            return out
        return run
    raise InvalidArgument(f"unsupported decoder {t}")
