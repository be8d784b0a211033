"""JSON-schema constrained decoding: a schema is compiled to a character-level pushdown state machine; for each decoding
step ``JsonSchemaProcessor.mask`` marks which vocabulary tokens keep the output a valid prefix, and ``apply_mask`` sets the
logits of the others to -inf (on CUDA with the token-mask kernel, one thread per vocabulary entry).

Reference parity: ferrotorch-grammar/src/{json_schema.rs:53-125 (Schema, JsonGrammar), state.rs, lib.rs:58-85 (TokenMask,
JsonSchemaProcessor), gpu_dispatch.rs:778 (compute_mask_gpu)}; the mask kernel replaces the CubeCL one (ferrotorch-cubecl/src/grammar.rs:47).
"""
from __future__ import annotations

import ctypes
import enum
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from ..errors import FerrotorchError, InvalidArgument


_DIGITS = "0123456789"                          # JSON numbers take ASCII digits only (``str.isdigit`` also accepts other scripts)


@dataclass
class Schema:
    kind: str                                  # object | array | string | number | integer | boolean | null | enum | any | nullable (items = inner)
    properties: Dict[str, "Schema"] = field(default_factory=dict)
    required: List[str] = field(default_factory=list)
    items: Optional["Schema"] = None
    enum: Optional[List[Any]] = None

    @staticmethod
    def from_json(j) -> "Schema":
        if isinstance(j, str):
            j = json.loads(j)
        if not isinstance(j, dict):
            raise InvalidArgument("a JSON schema must be an object")
        for word in ("oneOf", "anyOf", "allOf", "$ref"):        # composition and references are not compiled: refuse rather than ignore them
            if word in j:
                raise InvalidArgument(f"unsupported schema keyword {word}")
        if "enum" in j:
            return Schema("enum", enum=list(j["enum"]))
        t = j.get("type", "any")
        if isinstance(t, list):                        # ["X", "null"]: a nullable X
            rest = [x for x in t if x != "null"]
            if len(rest) != 1 or len(rest) + 1 != len(t):
                raise InvalidArgument(f"unsupported type list {t}: only [X, \"null\"] is compiled")
            return Schema("nullable", items=Schema.from_json({**j, "type": rest[0]}))
        if t == "object":
            return Schema("object", {k: Schema.from_json(v) for k, v in j.get("properties", {}).items()}, list(j.get("required", [])))
        if t == "array":
            return Schema("array", items=Schema.from_json(j.get("items", {})))
        if t in ("string", "number", "integer", "boolean", "null", "any"):
            return Schema(t)
        raise InvalidArgument(f"unsupported schema type {t}")


def _key_literal(name: str) -> str:
    """A property name as it is written in the document: characters outside ASCII stay as they are (models emit them raw)."""
    return json.dumps(name, ensure_ascii=False)


def _enum_literals(s: "Schema") -> List[str]:
    """The accepted spellings of an enum's values: each value with characters outside ASCII written raw and, where that differs,
    also as ``\\uXXXX`` escapes."""
    out: List[str] = []
    for v in s.enum or []:
        raw, escaped = json.dumps(v, ensure_ascii=False), json.dumps(v)
        out.append(raw)
        if escaped != raw:
            out.append(escaped)
    return out


class JsonGrammar:
    """Incremental validator: ``accepts_prefix(text)`` is true iff ``text`` can be extended to a document matching the schema.
    Objects emit their properties in schema order (required ones mandatory), compact separators, no insignificant whitespace
    except a single optional space after ``:`` and ``,``."""

    def __init__(self, schema: Schema):
        self.schema = schema

    # returns set of possible remaining-state continuations; implemented as a recursive prefix matcher
    def accepts_prefix(self, text: str) -> bool:
        return self._match(self.schema, text, 0, True) is not None

    def is_complete(self, text: str) -> bool:
        r = self._match(self.schema, text, 0, False)
        return r is not None and r == len(text)

    # _match returns: position after the value if the value completes inside text; len(text)+1 sentinel (as "ran out of text
    # while still valid") is represented by returning -1 when allow_partial; None when invalid.
    def _match(self, s: Schema, t: str, i: int, partial: bool):
        r = self._value(s, t, i)
        if r is None:
            return None
        if isinstance(r, tuple):                       # a number that ends with the text: complete, and a valid prefix of a longer one
            return r[1] if r[1] == len(t) else None
        if r == -1:
            return len(t) if partial else None
        if r != len(t):
            return None if not partial else (r if r == len(t) else None)
        return r

    def _lit(self, lit: str, t: str, i: int):
        n = len(t) - i
        if n >= len(lit):
            return i + len(lit) if t.startswith(lit, i) else None
        return -1 if lit.startswith(t[i:]) else None

    def _string(self, t: str, i: int):
        if i >= len(t):
            return -1
        if t[i] != '"':
            return None
        i += 1
        while i < len(t):
            c = t[i]
            if c == '"':
                return i + 1
            if c == "\\":
                if i + 1 >= len(t):
                    return -1
                if t[i + 1] not in '"\\/bfnrtu':
                    return None
                i += 2
                continue
            if ord(c) < 0x20:
                return None
            i += 1
        return -1

    def _number(self, t: str, i: int, integer: bool):
        j = i
        if j >= len(t):
            return -1
        if t[j] == "-":
            j += 1
            if j >= len(t):
                return -1
        if not t[j] in _DIGITS:
            return None
        if t[j] == "0":
            j += 1
        else:
            while j < len(t) and t[j] in _DIGITS:
                j += 1
        if j >= len(t):
            return ("open", j)
        if not integer and t[j] == ".":
            j += 1
            if j >= len(t):
                return -1
            if not t[j] in _DIGITS:
                return None
            while j < len(t) and t[j] in _DIGITS:
                j += 1
            if j >= len(t):
                return ("open", j)
        if not integer and t[j] in "eE":
            j += 1
            if j < len(t) and t[j] in "+-":
                j += 1
            if j >= len(t):
                return -1
            if not t[j] in _DIGITS:
                return None
            while j < len(t) and t[j] in _DIGITS:
                j += 1
            if j >= len(t):
                return ("open", j)
        return j

    def _sep(self, t: str, i: int):
        if i < len(t) and t[i] == " ":
            return i + 1
        return i

    def _value(self, s: Schema, t: str, i: int):
        """Position after the value, -1 if text ended inside a still-valid value, None if invalid. Numbers at end of text return
        ("open", pos): complete so far but extendable."""
        if i >= len(t):
            return -1
        k = s.kind
        if k == "string":
            return self._string(t, i)
        if k in ("number", "integer"):
            r = self._number(t, i, k == "integer")
            return r
        if k == "boolean":
            a, b = self._lit("true", t, i), self._lit("false", t, i)
            return a if a is not None else b
        if k == "null":
            return self._lit("null", t, i)
        if k == "nullable":
            r = self._lit("null", t, i)
            return r if r is not None else self._value(s.items, t, i)
        if k == "enum":
            res = None
            for lit in _enum_literals(s):
                r = self._lit(lit, t, i)
                if r is not None and r != -1:
                    return r
                if r == -1:
                    res = -1
            return res
        if k == "any":
            for sub in (Schema("string"), Schema("number"), Schema("boolean"), Schema("null"), Schema("array", items=Schema("any")), Schema("object")):
                r = self._value(sub, t, i)
                if r is not None:
                    return r
            return None
        if k == "array":
            if t[i] != "[":
                return None
            i += 1
            if i >= len(t):
                return -1
            if t[i] == "]":
                return i + 1
            while True:
                r = self._value(s.items or Schema("any"), t, i)
                if r is None or r == -1:
                    return r
                if isinstance(r, tuple):
                    return -1
                i = r
                if i >= len(t):
                    return -1
                if t[i] == "]":
                    return i + 1
                if t[i] != ",":
                    return None
                i = self._sep(t, i + 1)
                if i >= len(t):
                    return -1
        if k == "object":
            if t[i] != "{":
                return None
            i += 1
            props = list(s.properties.items())
            if not props:
                if i >= len(t):
                    return -1
                return i + 1 if t[i] == "}" else None
            first = True
            for idx, (name, sub) in enumerate(props):
                if i >= len(t):
                    return -1
                optional_rest = all(n not in s.required for n, _ in props[idx:])
                if t[i] == "}" and optional_rest and (first or True):
                    return i + 1 if (first or t[i - 1] != ",") else None
                if not first:
                    if t[i] != ",":
                        return None
                    i = self._sep(t, i + 1)
                    if i >= len(t):
                        return -1
                key = _key_literal(name)
                r = self._lit(key, t, i)
                if r is None:
                    if name in s.required:
                        return None
                    continue_ok = False
                    # an optional property may be skipped: try the following ones at this position
                    for n2, _ in props[idx + 1:]:
                        r2 = self._lit(_key_literal(n2), t, i)
                        if r2 is not None:
                            continue_ok = True
                            break
                    if not continue_ok:
                        return None
                    if not first:
                        # we consumed a comma for a property we are skipping: rewind is handled by retrying from the next property
                        pass
                    # emulate "not first" state for the next property without consuming another comma
                    first_backup = first
                    first = True if first_backup else True
                    continue
                if r == -1:
                    return -1
                i = r
                if i >= len(t):
                    return -1
                if t[i] != ":":
                    return None
                i = self._sep(t, i + 1)
                r = self._value(sub, t, i)
                if r is None or r == -1:
                    return r
                if isinstance(r, tuple):
                    return -1
                i = r
                first = False
            if i >= len(t):
                return -1
            return i + 1 if t[i] == "}" else None
        return None


class GrammarError(FerrotorchError):
    """Failure of the constrained-decoding layer (ferrotorch-grammar/src/json_schema.rs:41): ``kind`` is ``schema`` (the schema does not
    compile), ``step`` (a token was fed that the grammar cannot take) or ``invalid_token_id``."""

    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind

    @classmethod
    def invalid_token_id(cls, token_id: int) -> "GrammarError":
        return cls("invalid_token_id", f"token id {token_id} out of range")


class BooleanEmissionStage(enum.Enum):
    """How much of a ``true`` / ``false`` literal has been produced (ferrotorch-grammar/src/state.rs:193)."""
    Start = "start"
    PartialTrue = "partial_true"
    PartialFalse = "partial_false"
    Done = "done"

    @staticmethod
    def of(text: str):
        """``(stage, remaining)`` for the characters emitted so far; ``None`` when they start neither literal."""
        if text == "":
            return BooleanEmissionStage.Start, ""
        for lit, st in (("true", BooleanEmissionStage.PartialTrue), ("false", BooleanEmissionStage.PartialFalse)):
            if lit.startswith(text):
                return (BooleanEmissionStage.Done, "") if text == lit else (st, lit[len(text):])
        return None


@dataclass
class PackedVocab:
    """Vocabulary flattened for a device-side mask kernel (ferrotorch-grammar/src/gpu_dispatch.rs:709): ``chars`` holds the code points of
    all tokens back to back, token ``i`` spans ``chars[offsets[i]:offsets[i + 1]]``."""
    offsets: List[int]
    chars: List[int]
    max_token_len: int

    @classmethod
    def pack(cls, vocab: Sequence[str]) -> "PackedVocab":
        offsets, chars, longest = [0], [], 0
        for tok in vocab:
            chars.extend(ord(c) for c in tok)
            offsets.append(len(chars))
            longest = max(longest, len(tok))
        return cls(offsets, chars, longest)

    def vocab_size(self) -> int:
        return len(self.offsets) - 1

    def token(self, i: int) -> str:
        if not 0 <= i < self.vocab_size():
            raise GrammarError.invalid_token_id(i)
        return "".join(chr(c) for c in self.chars[self.offsets[i]: self.offsets[i + 1]])

    def tensors(self, device="cpu"):
        """``(offsets int32 [V + 1], chars int32 [total])`` on ``device``."""
        return torch.tensor(self.offsets, dtype=torch.int32, device=device), torch.tensor(self.chars, dtype=torch.int32, device=device)

    def __repr__(self):
        return f"PackedVocab(offsets=<{len(self.offsets)} entries>, chars=<{len(self.chars)} entries>, max_token_len={self.max_token_len})"


@dataclass
class TokenMask:
    allowed: torch.Tensor            # bool [vocab]

    def count(self) -> int:
        return int(self.allowed.sum())


_KIND_CODE = {"object": 0, "array": 1, "string": 2, "number": 3, "integer": 4, "boolean": 5, "null": 6, "enum": 7, "any": 8, "nullable": 9}


def _flatten_schema(root: Schema):
    """Schema tree -> the arrays ``ft_json_grammar_create`` takes (node kinds, edge ranges, edge literals / children / required flags)."""
    nodes: List[Schema] = []
    index: Dict[int, int] = {}

    def visit(s: Schema) -> int:
        if s.kind not in _KIND_CODE:
            raise InvalidArgument(f"unsupported schema kind {s.kind}")
        index[id(s)] = len(nodes)
        nodes.append(s)
        for sub in list(s.properties.values()) + ([s.items] if s.items is not None else []):
            visit(sub)
        return index[id(s)]
    visit(root)
    kinds, first, lits, child, req = [], [0], [], [], []
    for s in nodes:
        kinds.append(_KIND_CODE[s.kind])
        if s.kind == "object":
            for name, sub in s.properties.items():
                lits.append(_key_literal(name).encode("utf-8"))
                child.append(index[id(sub)])
                req.append(1 if name in s.required else 0)
        elif s.kind in ("array", "nullable") and s.items is not None:
            lits.append(b"")
            child.append(index[id(s.items)])
            req.append(0)
        elif s.kind == "enum":
            for lit in _enum_literals(s):
                lits.append(lit.encode("utf-8"))
                child.append(-1)
                req.append(0)
        first.append(len(lits))
    return kinds, first, lits, child, req


def _blob(items: Sequence[bytes]):
    off = np.zeros(len(items) + 1, np.int64)
    if items:
        np.cumsum([len(x) for x in items], out=off[1:])
    return np.frombuffer(b"".join(items) + b"\0", np.uint8), off


class JsonSchemaProcessor:
    """Logits processor: keeps only tokens whose text leaves the generated string a valid prefix of a schema-conforming document.

    The per-step walk over the vocabulary runs in the host runtime library (``csrc/runtime/grammar.cpp``: the same prefix matcher as
    ``JsonGrammar``, the vocabulary spread over threads); ``FT_GRAMMAR_NATIVE=0`` or a missing library keeps it on the Python matcher."""

    def __init__(self, schema, vocab_texts: Sequence[str], eos_id: Optional[int] = None):
        self.grammar = JsonGrammar(schema if isinstance(schema, Schema) else Schema.from_json(schema))
        self.vocab = list(vocab_texts)
        self.eos_id = eos_id
        self.text = ""
        self._native = None
        # Worker threads of the native vocabulary walk. One by default: a walk costs 0.3 - 3 ms on one core, and threads started next to a
        # process whose math library keeps its own workers spinning are scheduled late more often than they help.
        self.threads = 1
        if os.environ.get("FT_GRAMMAR_NATIVE", "1") != "0":
            self._build_native()

    def _build_native(self) -> None:
        try:
            from .. import _lib
            rt = _lib.runtime()
            rt.ft_json_grammar_create.restype = ctypes.c_void_p
            rt.ft_json_grammar_mask.restype = ctypes.c_int64
            rt.ft_json_grammar_destroy.restype = None
            kinds, first, lits, child, req = _flatten_schema(self.grammar.schema)
            vocab = [t.encode("utf-8") for t in self.vocab]
        except Exception:
            return
        p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
        lit_blob, lit_off = _blob(lits)
        vocab_blob, voff = _blob(vocab)
        kind_a, first_a = np.array(kinds, np.int32), np.array(first, np.int32)
        child_a, req_a = np.array(child + [0], np.int32), np.array(req + [0], np.uint8)
        h = rt.ft_json_grammar_create(p(kind_a), p(first_a), ctypes.c_int64(len(kinds)), p(lit_blob), p(lit_off), p(child_a), p(req_a), p(vocab_blob), p(voff),
                                      ctypes.c_int64(len(vocab)))
        if h:
            self._native, self._rt = ctypes.c_void_p(h), rt
            self._mask_buf = np.zeros(max(len(vocab), 1), np.uint8)

    def __del__(self):
        h, self._native = getattr(self, "_native", None), None
        if h is not None:
            try:
                self._rt.ft_json_grammar_destroy(h)
            except Exception:
                pass

    def reset(self) -> None:
        self.text = ""

    def advance(self, token_id: int) -> None:
        if not 0 <= token_id < len(self.vocab):
            raise GrammarError.invalid_token_id(token_id)
        if token_id != self.eos_id:
            self.text += self.vocab[token_id]

    def _valid(self, text: str) -> bool:
        r = self.grammar._value(self.grammar.schema, text, 0)
        if r is None:
            return False
        if r == -1 or isinstance(r, tuple):
            return True
        return r == len(text)

    def _complete(self) -> bool:
        r = self.grammar._value(self.grammar.schema, self.text, 0)
        if isinstance(r, tuple):
            return r[1] == len(self.text)
        return r is not None and r != -1 and r == len(self.text)

    def mask(self) -> TokenMask:
        if self._native is not None:
            allowed = self._mask_buf                  # one buffer for the life of the processor: a fresh 128 KB array per step costs page faults
            raw = self.text.encode("utf-8")
            self._rt.ft_json_grammar_mask(self._native, ctypes.c_char_p(raw), ctypes.c_int64(len(raw)), ctypes.c_int64(-1 if self.eos_id is None else self.eos_id),
                                          allowed.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(self.threads))
            return TokenMask(torch.from_numpy(allowed[: len(self.vocab)]).to(torch.bool))
        return self._mask_py()

    def _mask_py(self) -> TokenMask:
        ok = torch.zeros(len(self.vocab), dtype=torch.bool)
        done = self._complete()
        for i, tok in enumerate(self.vocab):
            if i == self.eos_id:
                ok[i] = done
            elif tok and not (done and self.grammar.schema.kind not in ("number", "integer")):
                ok[i] = self._valid(self.text + tok)
        return TokenMask(ok)

    def apply(self, logits: torch.Tensor) -> torch.Tensor:
        return apply_mask(logits, self.mask())

    def as_logits_processor(self, prompt_len: int):
        """``f(logits, seq)`` for ``models.llama_gen.generate(..., logits_processor=f)`` (batch size 1): every token appended to ``seq`` since
        the last call is fed to ``advance``, then the mask of the new state is applied. ``prompt_len`` tokens at the front are not output."""
        seen = [prompt_len]

        def f(logits: torch.Tensor, seq: torch.Tensor) -> torch.Tensor:
            if seq.shape[0] != 1:
                raise InvalidArgument("one grammar state constrains one sequence: batch size must be 1")
            for t in seq[0, seen[0]:].tolist():
                self.advance(int(t))
            seen[0] = seq.shape[1]
            return self.apply(logits)
        return f


class BatchJsonSchemaProcessor:
    """One schema constraining a batch of sequences (a serving batch): the compiled grammar and the packed vocabulary are shared, each
    sequence keeps its own generated text. ``apply(logits [B, V])`` masks row by row, ``advance(tokens [B])`` feeds one token per sequence;
    a sequence that has emitted its end token stays finished and its row is left untouched."""

    def __init__(self, schema, vocab_texts: Sequence[str], batch: int, eos_id: Optional[int] = None):
        self._proc = JsonSchemaProcessor(schema, vocab_texts, eos_id)
        self.eos_id = eos_id
        self.texts: List[str] = [""] * batch
        self.finished: List[bool] = [False] * batch

    def reset(self) -> None:
        self.texts = [""] * len(self.texts)
        self.finished = [False] * len(self.texts)

    def masks(self, threads: Optional[int] = None) -> torch.Tensor:
        """bool [B, V]; the row of a finished sequence is all True. With the native walk all live sequences go to the library in one call,
        one sequence per thread."""
        V = len(self._proc.vocab)
        live = [b for b, done in enumerate(self.finished) if not done]
        out = torch.ones(len(self.texts), V, dtype=torch.bool)
        if not live:
            return out
        if self._proc._native is not None:
            raw = [self.texts[b].encode("utf-8") for b in live]
            off = np.zeros(len(raw) + 1, np.int64)
            np.cumsum([len(x) for x in raw], out=off[1:])
            buf = np.zeros((len(live), max(V, 1)), np.uint8)
            rt = self._proc._rt
            rt.ft_json_grammar_mask_batch.restype = None
            rt.ft_json_grammar_mask_batch(self._proc._native, ctypes.c_char_p(b"".join(raw) + b"\0"), off.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(len(live)),
                                          ctypes.c_int64(-1 if self.eos_id is None else self.eos_id), buf.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(None),
                                          ctypes.c_int(threads or min(os.cpu_count() or 1, len(live))))
            out[live] = torch.from_numpy(buf[:, :V]).to(torch.bool)
            return out
        for b in live:
            self._proc.text = self.texts[b]
            out[b] = self._proc.mask().allowed
        return out

    def apply(self, logits: torch.Tensor) -> torch.Tensor:
        if logits.dim() != 2 or logits.shape[0] != len(self.texts):
            raise InvalidArgument(f"logits must be [batch = {len(self.texts)}, vocab], got {tuple(logits.shape)}")
        return logits.masked_fill(~self.masks().to(logits.device), float("-inf"))

    def advance(self, tokens) -> None:
        toks = tokens.tolist() if isinstance(tokens, torch.Tensor) else list(tokens)
        if len(toks) != len(self.texts):
            raise InvalidArgument("one token per sequence")
        for b, t in enumerate(toks):
            if self.finished[b]:
                continue
            if not 0 <= int(t) < len(self._proc.vocab):
                raise GrammarError.invalid_token_id(int(t))
            if int(t) == self.eos_id:
                self.finished[b] = True
            else:
                self.texts[b] += self._proc.vocab[int(t)]

    def is_complete(self, b: int) -> bool:
        return self._proc.grammar.is_complete(self.texts[b])


def apply_mask(logits: torch.Tensor, mask: TokenMask) -> torch.Tensor:
    """``logits[..., v] = -inf`` where the mask forbids token ``v``."""
    allowed = mask.allowed.to(logits.device)
    if logits.is_cuda and logits.dtype in (torch.float32, torch.bfloat16, torch.float16) and logits.is_contiguous():
        from ..ops import tensor_ops
        V = logits.shape[-1]
        pad = (-V) % 32
        bits = torch.nn.functional.pad(allowed.to(torch.int64), (0, pad)).view(-1, 32)
        words = (bits << torch.arange(32, device=bits.device)).sum(-1)                      # bit v%32 of word v//32 = token v allowed
        words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
        return tensor_ops.token_mask_(logits, words)
    return logits.masked_fill(~allowed, float("-inf"))


compute_mask_gpu = apply_mask
