"""Tokenizer: a self-contained reader of HF ``tokenizer.json`` (byte-level BPE and plain BPE models, added/special tokens,
pre-tokenisation by the GPT-2 / Llama-3 split pattern) plus chat templates.

Reference parity: ferrotorch-tokenize/src/lib.rs:59 (load_tokenizer), :85 (encode), :104 (encode_batch), :131 (decode),
:225 (apply_chat_template) - a wrapper over the HF ``tokenizers`` crate there; here the BPE merge loop is implemented directly.
"""
from __future__ import annotations

import json
from functools import lru_cache
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import regex as _re

from dataclasses import dataclass

from ..errors import Internal, InvalidArgument

_GPT2_SPLIT = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""
_LLAMA3_SPLIT = r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"""


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
                 unk_token: Optional[str] = None):
        self.vocab = dict(vocab)
        self.added = dict(added_tokens or {})
        self.vocab.update(self.added)
        self.inv = {i: t for t, i in self.vocab.items()}
        self.ranks = {tuple(m): i for i, m in enumerate(merges)}
        self.byte_level = byte_level
        self.split = _re.compile(split_pattern or _GPT2_SPLIT)
        self.bos_token, self.eos_token, self.unk_token = bos_token, eos_token, unk_token
        self._b2u = _bytes_to_unicode()
        self._u2b = {v: k for k, v in self._b2u.items()}
        self._special_re = _re.compile("|".join(_re.escape(t) for t in sorted(self.added, key=len, reverse=True))) if self.added else None
        self._cache: Dict[str, List[str]] = {}

    def vocab_size(self) -> int:
        return len(self.vocab)

    def token_to_id(self, tok: str) -> Optional[int]:
        return self.vocab.get(tok)

    def id_to_token(self, i: int) -> Optional[str]:
        return self.inv.get(i)

    def _bpe(self, word: str) -> List[str]:
        if word in self._cache:
            return self._cache[word]
        parts = list(word)
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
        ids: List[int] = []
        for piece in self.split.findall(text):
            w = "".join(self._b2u[b] for b in piece.encode("utf-8")) if self.byte_level else piece
            for tok in self._bpe(w):
                i = self.vocab.get(tok)
                if i is None:
                    if self.unk_token is None:
                        raise InvalidArgument(f"token {tok!r} not in vocabulary and no unk token configured")
                    i = self.vocab[self.unk_token]
                ids.append(i)
        return ids

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
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

    def encode_batch(self, texts: Iterable[str], add_special_tokens: bool = False) -> List[List[int]]:
        return [self.encode(t, add_special_tokens) for t in texts]

    def decode(self, ids: Iterable[int], skip_special_tokens: bool = True) -> str:
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
    if model.get("type", "BPE") != "BPE":
        raise InvalidArgument(f"unsupported tokenizer model {model.get('type')}")
    merges = [tuple(m.split(" ", 1)) if isinstance(m, str) else tuple(m) for m in model.get("merges", [])]
    added = {a["content"]: a["id"] for a in j.get("added_tokens", [])}
    pre = j.get("pre_tokenizer") or {}
    kinds = [pre.get("type")] + [x.get("type") for x in pre.get("pretokenizers", [])]
    byte_level = "ByteLevel" in kinds or (j.get("decoder") or {}).get("type") == "ByteLevel"
    pattern = None
    for x in [pre] + pre.get("pretokenizers", []):
        if x.get("type") == "Split" and isinstance(x.get("pattern"), dict):
            pattern = x["pattern"].get("Regex")
    bos = eos = None
    cfg = p.parent / "tokenizer_config.json"
    if cfg.exists():
        c = json.loads(cfg.read_text())
        def tok(v):
            return v.get("content") if isinstance(v, dict) else v
        bos, eos = tok(c.get("bos_token")), tok(c.get("eos_token"))
    return Tokenizer(model.get("vocab", {}), merges, added, byte_level, pattern, bos, eos, model.get("unk_token"))


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
