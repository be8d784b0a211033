"""Loader variants, container inspection and graph export that sit on top of the format readers in this package.

* sharded SafeTensors: auto-detecting / memory-mapped / filtered loaders and a per-shard progress callback
  (ferrotorch-serialize/src/safetensors_io.rs:541-900);
* GGUF: typed metadata access, in-memory parsing, per-tensor dequantisation by name, whole-file state dicts
  (ferrotorch-serialize/src/gguf.rs:38-910);
* PyTorch checkpoints: a non-executing pickle reader that returns the opcode stream as a value tree, CRC validation of the zip container,
  memory-mapped loading (ferrotorch-serialize/src/pytorch_import.rs:35-141, 924; pytorch_export.rs:222, 474);
* ONNX from a traced IR graph or an exported program (ferrotorch-serialize/src/onnx_export.rs:743-1200).
"""
from __future__ import annotations

import enum
import io
import math
import mmap
import pickletools
import struct
import zipfile
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..errors import InvalidArgument
from . import formats as _F
from .safetensors_io import load_safetensors, load_safetensors_sharded


# ----------------------------------------------------------------------------------------------------------------------
# SafeTensors
# ----------------------------------------------------------------------------------------------------------------------
def load_safetensors_auto(path, **kw) -> Dict[str, torch.Tensor]:
    """A ``*.index.json`` path loads the shards it lists, anything else is one file (safetensors_io.rs:685)."""
    return load_safetensors_sharded(path, **kw) if str(path).endswith(".index.json") else load_safetensors(path, **kw)


@dataclass(frozen=True)
class ShardProgress:
    """What the progress callback sees before each shard is opened (safetensors_io.rs:703)."""
    shard_index: int
    shard_count: int
    shard_file: str
    tensors_in_shard: int
    tensors_loaded_so_far: int
    total_tensors: int


def _index(index_path) -> Tuple[Path, Dict[str, List[str]], int]:
    import json
    try:
        idx = json.loads(Path(index_path).read_text())
        wm = idx["weight_map"]
    except (OSError, ValueError, KeyError) as e:
        raise InvalidArgument(f"failed to read SafeTensors index {index_path}: {e}") from None
    by_file: Dict[str, List[str]] = {}
    for k in sorted(wm):                                      # shards in name order, tensors in name order: a deterministic walk
        by_file.setdefault(wm[k], []).append(k)
    return Path(index_path).parent, dict(sorted(by_file.items())), len(wm)


def load_safetensors_sharded_with_progress(index_path, progress: Callable[[ShardProgress], Any], dtype: Optional[torch.dtype] = None, device="cpu",
                                           filter_fn: Optional[Callable[[str], bool]] = None, mmap_shards: bool = False) -> Dict[str, torch.Tensor]:
    """Shard-by-shard load; ``progress`` is called once before each shard with the counts so far (its return value is ignored)."""
    base, by_file, total = _index(index_path)
    out: Dict[str, torch.Tensor] = {}
    for i, (fn, keys) in enumerate(by_file.items()):
        want = set(k for k in keys if filter_fn is None or filter_fn(k))
        progress(ShardProgress(i, len(by_file), fn, len(keys), len(out), total))
        if not want:
            continue
        if not (base / fn).exists():
            raise InvalidArgument(f"shard {fn} listed in {index_path} does not exist")
        got = load_safetensors(base / fn, dtype, device, lambda n: n in want, use_mmap=mmap_shards)
        missing = want - set(got)
        if missing:
            raise InvalidArgument(f"shard {fn} lacks tensors the index assigns to it: {sorted(missing)[:3]}")
        out.update(got)
    return out


def load_safetensors_sharded_mmap(index_path, **kw) -> Dict[str, torch.Tensor]:
    """Every shard is mapped instead of read, so peak host memory is one tensor, not one shard (safetensors_io.rs:820)."""
    return load_safetensors_sharded_with_progress(index_path, lambda p: None, mmap_shards=True, **kw)


def load_safetensors_sharded_filtered(index_path, predicate: Callable[[str], bool], **kw) -> Dict[str, torch.Tensor]:
    """Only the tensors ``predicate(name)`` accepts; shards without an accepted tensor are never opened (safetensors_io.rs:600)."""
    return load_safetensors_sharded_with_progress(index_path, lambda p: None, filter_fn=predicate, **kw)


# ----------------------------------------------------------------------------------------------------------------------
# GGUF
# ----------------------------------------------------------------------------------------------------------------------
class GgmlType(enum.IntEnum):
    """Tensor encodings of a GGUF file this reader dequantises (gguf.rs:38)."""
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q8_1 = 9
    BF16 = 30

    def block_size(self) -> int:
        return _F.GGML_TYPES[int(self)][1]

    def type_size(self) -> int:
        return _F.GGML_TYPES[int(self)][2]


_VALUE_KINDS = {0: "Uint8", 1: "Int8", 2: "Uint16", 3: "Int16", 4: "Uint32", 5: "Int32", 6: "Float32", 7: "Bool", 8: "String", 9: "Array", 10: "Uint64",
                11: "Int64", 12: "Float64"}


@dataclass(frozen=True)
class GgufValue:
    """One metadata value with its declared GGUF type (gguf.rs:141): ``kind`` is ``Uint8`` ... ``Float64``, ``Bool``, ``String`` or ``Array``."""
    kind: str
    value: Any

    def as_int(self) -> Optional[int]:
        return int(self.value) if self.kind.startswith(("Uint", "Int")) else None

    def as_float(self) -> Optional[float]:
        return float(self.value) if self.kind.startswith("Float") else None

    def as_str(self) -> Optional[str]:
        return self.value if self.kind == "String" else None


@dataclass
class GgufMetadata:
    """Key -> typed value (gguf.rs:159)."""
    entries: Dict[str, GgufValue] = field(default_factory=dict)

    def get(self, key: str) -> Optional[GgufValue]:
        return self.entries.get(key)

    def get_str(self, key: str) -> Optional[str]:
        v = self.entries.get(key)
        return v.as_str() if v else None

    def get_int(self, key: str) -> Optional[int]:
        v = self.entries.get(key)
        return v.as_int() if v else None

    def get_float(self, key: str) -> Optional[float]:
        v = self.entries.get(key)
        return v.as_float() if v else None

    def plain(self) -> Dict[str, Any]:
        return {k: v.value for k, v in self.entries.items()}


class _Reader:
    def __init__(self, data):
        self.d, self.p = memoryview(data), 0

    def take(self, n: int) -> bytes:
        if n < 0 or self.p + n > len(self.d):
            raise InvalidArgument(f"GGUF: unexpected end of data at offset {self.p} (need {n} bytes of {len(self.d)})")
        b = bytes(self.d[self.p: self.p + n])
        self.p += n
        return b

    def unpack(self, fmt: str):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def string(self) -> str:
        n = self.unpack("<Q")
        try:
            return self.take(n).decode("utf-8")
        except UnicodeDecodeError as e:
            raise InvalidArgument(f"GGUF: string is not valid UTF-8: {e}") from None

    def value(self, t: int, depth: int = 0) -> GgufValue:
        fmt = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 10: "<Q", 11: "<q", 12: "<d"}
        if t in fmt:
            return GgufValue(_VALUE_KINDS[t], self.unpack(fmt[t]))
        if t == 7:
            return GgufValue("Bool", self.unpack("<B") != 0)
        if t == 8:
            return GgufValue("String", self.string())
        if t == 9:
            if depth > 4:
                raise InvalidArgument("GGUF: arrays nested too deeply")
            et, n = self.unpack("<I"), self.unpack("<Q")
            if n > len(self.d):
                raise InvalidArgument(f"GGUF: array length {n} exceeds the file size")
            return GgufValue("Array", [self.value(et, depth + 1) for _ in range(n)])
        raise InvalidArgument(f"GGUF: unknown metadata value type {t}")


@dataclass
class GgufTensor:
    name: str
    dims: Tuple[int, ...]             # GGUF order: fastest-varying dimension first
    ggml_type: GgmlType
    offset: int


@dataclass
class GgufData:
    """A parsed GGUF file held in memory (or mapped): header version, typed metadata, tensor directory and the data region (gguf.rs:184)."""
    version: int
    metadata: GgufMetadata
    tensors: List[GgufTensor]
    data: Any                         # bytes-like: the region after the aligned tensor directory

    def tensor_names(self) -> List[str]:
        return [t.name for t in self.tensors]


def parse_gguf_bytes(data) -> GgufData:
    """Parse a whole GGUF image (versions 2 and 3) from a bytes-like object (gguf.rs:391)."""
    r = _Reader(data)
    magic = r.unpack("<I")
    if magic != 0x46554747:
        raise InvalidArgument(f"invalid GGUF magic: expected 0x46554747, got 0x{magic:08X}")
    version = r.unpack("<I")
    if version not in (2, 3):
        raise InvalidArgument(f"unsupported GGUF version {version} (2 and 3 are read)")
    n_tensors, n_kv = r.unpack("<Q"), r.unpack("<Q")
    if max(n_tensors, n_kv) > len(r.d):
        raise InvalidArgument("GGUF: tensor / metadata counts exceed the file size")
    meta = GgufMetadata()
    for _ in range(n_kv):
        k = r.string()
        meta.entries[k] = r.value(r.unpack("<I"))
    tensors = []
    for _ in range(n_tensors):
        name, nd = r.string(), r.unpack("<I")
        if nd > 8:
            raise InvalidArgument(f"GGUF: tensor {name!r} declares {nd} dimensions")
        dims = tuple(r.unpack("<Q") for _ in range(nd))
        gt, off = r.unpack("<I"), r.unpack("<Q")
        try:
            gt = GgmlType(gt)
        except ValueError:
            raise InvalidArgument(f"GGUF: tensor {name!r} has unsupported ggml type {gt}") from None
        tensors.append(GgufTensor(name, dims, gt, off))
    align = meta.get_int("general.alignment") or 32
    start = (r.p + align - 1) // align * align
    return GgufData(version, meta, tensors, r.d[min(start, len(r.d)):])


def load_gguf(path) -> GgufData:
    try:
        raw = Path(path).read_bytes()
    except OSError as e:
        raise InvalidArgument(f"failed to read GGUF file {path}: {e}") from None
    return parse_gguf_bytes(raw)


def load_gguf_mmap(path) -> GgufData:
    """As :func:`load_gguf` but over a read-only mapping: tensor bytes are paged in when a tensor is dequantised (gguf.rs:373)."""
    try:
        with open(path, "rb") as f:
            m = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    except (OSError, ValueError) as e:
        raise InvalidArgument(f"failed to open GGUF file {path}: {e}") from None
    return parse_gguf_bytes(m)


def dequantize_gguf_tensor(file: GgufData, tensor_name: str) -> torch.Tensor:
    """f32 tensor of ``tensor_name`` in row-major order (dims reversed from GGUF's fastest-first order) (gguf.rs:834)."""
    info = next((t for t in file.tensors if t.name == tensor_name), None)
    if info is None:
        raise InvalidArgument(f'tensor "{tensor_name}" not found in GGUF file')
    n = math.prod(info.dims) if info.dims else 1
    blk, bsz = info.ggml_type.block_size(), info.ggml_type.type_size()
    if n % blk:
        raise InvalidArgument(f'tensor "{tensor_name}": {n} elements is not a multiple of the {info.ggml_type.name} block size {blk}')
    nbytes = n // blk * bsz
    if info.offset + nbytes > len(file.data):
        raise InvalidArgument(f'tensor "{tensor_name}": data range {info.offset}..{info.offset + nbytes} exceeds the data region ({len(file.data)} bytes)')
    raw = bytes(file.data[info.offset: info.offset + nbytes])
    return _F.dequantize_gguf(raw, int(info.ggml_type), n).reshape(tuple(reversed(info.dims)))


def load_gguf_state_dict(path) -> Dict[str, torch.Tensor]:
    f = load_gguf(path)
    return {t.name: dequantize_gguf_tensor(f, t.name) for t in f.tensors}


def load_gguf_state_dict_mmap(path) -> Dict[str, torch.Tensor]:
    f = load_gguf_mmap(path)
    return {t.name: dequantize_gguf_tensor(f, t.name) for t in f.tensors}


# ----------------------------------------------------------------------------------------------------------------------
# pickle as data
# ----------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class PickleValue:
    """A pickle stream read as data, never executed (pytorch_import.rs:35). ``kind`` is one of None, Bool, Int, Float, Bytes, String, Tuple,
    List, Dict (``value`` = list of pairs), Global (``value`` = (module, name)), Reduce (``value`` = (callable, args)), Build
    (``value`` = (obj, state)), PersistentLoad."""
    kind: str
    value: Any = None

    def items(self) -> List[Tuple["PickleValue", "PickleValue"]]:
        if self.kind != "Dict":
            raise InvalidArgument(f"PickleValue.items on a {self.kind}")
        return list(self.value)

    def get(self, key: str) -> Optional["PickleValue"]:
        return next((v for k, v in self.items() if k.kind == "String" and k.value == key), None)


class _Mark:
    pass


def parse_pickle(data: bytes) -> PickleValue:
    """Decode protocol 0-5 opcodes into a :class:`PickleValue` tree. Globals stay names, ``REDUCE`` / ``BUILD`` / persistent ids stay nodes:
    nothing is imported or called (pytorch_import.rs:141)."""
    stack: List[Any] = []
    memo: Dict[int, PickleValue] = {}
    PV = PickleValue

    def pop_mark() -> List[PickleValue]:
        for i in range(len(stack) - 1, -1, -1):
            if isinstance(stack[i], _Mark):
                items = stack[i + 1:]
                del stack[i:]
                return items
        raise InvalidArgument("pickle: MARK not found")

    def pop() -> PickleValue:
        if not stack or isinstance(stack[-1], _Mark):
            raise InvalidArgument("pickle: stack underflow")
        return stack.pop()

    def mutate(f):
        top = pop()
        stack.append(f(top))

    try:
        ops = list(pickletools.genops(data))
    except Exception as e:
        raise InvalidArgument(f"pickle: malformed stream: {e}") from None
    for op, arg, _pos in ops:
        n = op.name
        if n in ("PROTO", "FRAME"):
            continue
        if n == "STOP":
            return pop()
        if n == "MARK":
            stack.append(_Mark())
        elif n == "NONE":
            stack.append(PV("None"))
        elif n in ("NEWTRUE", "NEWFALSE"):
            stack.append(PV("Bool", n == "NEWTRUE"))
        elif n in ("BININT", "BININT1", "BININT2", "LONG1", "LONG4", "INT", "LONG"):
            stack.append(PV("Bool", arg) if isinstance(arg, bool) else PV("Int", int(arg)))
        elif n in ("BINFLOAT", "FLOAT"):
            stack.append(PV("Float", float(arg)))
        elif n in ("BINUNICODE", "SHORT_BINUNICODE", "BINUNICODE8", "UNICODE"):
            stack.append(PV("String", arg))
        elif n in ("BINBYTES", "SHORT_BINBYTES", "BINBYTES8", "BYTEARRAY8"):
            stack.append(PV("Bytes", bytes(arg)))
        elif n in ("BINSTRING", "SHORT_BINSTRING", "STRING"):
            stack.append(PV("Bytes", arg.encode("latin-1") if isinstance(arg, str) else bytes(arg)))
        elif n == "EMPTY_DICT":
            stack.append(PV("Dict", []))
        elif n == "EMPTY_LIST":
            stack.append(PV("List", []))
        elif n == "EMPTY_TUPLE":
            stack.append(PV("Tuple", []))
        elif n == "TUPLE":
            stack.append(PV("Tuple", pop_mark()))
        elif n in ("TUPLE1", "TUPLE2", "TUPLE3"):
            k = int(n[-1])
            items = [pop() for _ in range(k)][::-1]
            stack.append(PV("Tuple", items))
        elif n == "LIST":
            stack.append(PV("List", pop_mark()))
        elif n == "DICT":
            it = pop_mark()
            stack.append(PV("Dict", list(zip(it[0::2], it[1::2]))))
        elif n in ("BINPUT", "LONG_BINPUT", "PUT"):
            memo[int(arg)] = stack[-1]
        elif n == "MEMOIZE":
            memo[len(memo)] = stack[-1]
        elif n in ("BINGET", "LONG_BINGET", "GET"):
            if int(arg) not in memo:
                raise InvalidArgument(f"pickle: memo key {arg} not found")
            stack.append(memo[int(arg)])
        elif n == "GLOBAL":
            module, _, name = arg.partition(" ")
            stack.append(PV("Global", (module, name)))
        elif n == "STACK_GLOBAL":
            name, module = pop(), pop()
            stack.append(PV("Global", (module.value, name.value)))
        elif n == "REDUCE":
            args, fn = pop(), pop()
            stack.append(PV("Reduce", (fn, args)))
        elif n in ("NEWOBJ", "NEWOBJ_EX"):
            kw = pop() if n == "NEWOBJ_EX" else None
            args, cls = pop(), pop()
            stack.append(PV("Reduce", (cls, args if kw is None else PV("Tuple", [args, kw]))))
        elif n == "BUILD":
            state, obj = pop(), pop()
            stack.append(PV("Build", (obj, state)))
        elif n == "BINPERSID":
            stack.append(PV("PersistentLoad", pop()))
        elif n == "PERSID":
            stack.append(PV("PersistentLoad", PV("String", arg)))
        elif n == "SETITEM":
            v, k = pop(), pop()
            mutate(lambda d: _dict_with(d, [(k, v)]))
        elif n == "SETITEMS":
            it = pop_mark()
            mutate(lambda d: _dict_with(d, list(zip(it[0::2], it[1::2]))))
        elif n == "APPEND":
            v = pop()
            mutate(lambda l: _list_with(l, [v]))
        elif n == "APPENDS":
            it = pop_mark()
            mutate(lambda l: _list_with(l, it))
        elif n == "POP":
            pop()
        elif n == "DUP":
            stack.append(stack[-1])
        else:
            raise InvalidArgument(f"pickle: unsupported opcode {n}")
    raise InvalidArgument("unexpected end of pickle data")


def _dict_with(d: PickleValue, pairs) -> PickleValue:
    if d.kind == "Dict":
        d.value.extend(pairs)                                # in place, so memoised references see the items (as a real unpickler's dict would)
        return d
    if d.kind in ("Reduce", "Build"):                        # e.g. an OrderedDict() call being filled: keep the items beside the constructor
        return PickleValue("Build", (d, PickleValue("Dict", list(pairs))))
    raise InvalidArgument(f"pickle: SETITEM on a {d.kind}")


def _list_with(l: PickleValue, items) -> PickleValue:
    if l.kind != "List":
        raise InvalidArgument(f"pickle: APPEND on a {l.kind}")
    l.value.extend(items)
    return l


# ----------------------------------------------------------------------------------------------------------------------
# PyTorch zip checkpoints
# ----------------------------------------------------------------------------------------------------------------------
def save_pytorch(state: Dict[str, torch.Tensor], path) -> None:
    """``torch.load``-readable zip checkpoint, keys written in sorted order (pytorch_export.rs:222)."""
    _F.save_pytorch_state_dict(dict(sorted(state.items())), path)


def validate_checkpoint(path) -> None:
    """Reads every entry of the zip container and checks it against its stored CRC-32 (pytorch_export.rs:474)."""
    try:
        z = zipfile.ZipFile(path)
    except OSError as e:
        raise InvalidArgument(f"failed to open checkpoint file {path}: {e}") from None
    except zipfile.BadZipFile as e:
        raise InvalidArgument(f"failed to read ZIP archive {path}: {e}") from None
    with z:
        for info in z.infolist():
            try:
                with z.open(info) as f:
                    crc = 0
                    while True:
                        chunk = f.read(1 << 20)
                        if not chunk:
                            break
                        crc = zipfile.crc32(chunk, crc)
            except (zipfile.BadZipFile, OSError, EOFError) as e:
                raise InvalidArgument(f'CRC32 integrity check failed for entry "{info.filename}": {e}') from None
            if crc & 0xFFFFFFFF != info.CRC:
                raise InvalidArgument(f'CRC32 mismatch for entry "{info.filename}": expected 0x{info.CRC:08X}, got 0x{crc & 0xFFFFFFFF:08X}')


def load_pytorch_state_dict_mmap(path, dtype: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
    """Tensors are views of a read-only mapping of the checkpoint (its storages are stored uncompressed and aligned), converted to ``dtype``
    only when one is given (pytorch_import.rs:924)."""
    try:
        sd = torch.load(str(path), map_location="cpu", mmap=True, weights_only=True)
    except Exception as e:
        raise InvalidArgument(f"failed to open pytorch file {path}: {e}") from None
    if not isinstance(sd, dict):
        raise InvalidArgument(f"{path}: expected a state dict, got {type(sd).__name__}")
    if isinstance(sd.get("state_dict"), dict):
        sd = sd["state_dict"]
    out = {k: v for k, v in sd.items() if torch.is_tensor(v)}
    return {k: (v.to(dtype) if dtype is not None and v.is_floating_point() else v) for k, v in out.items()}
