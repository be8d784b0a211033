"""Native state-dict container, training checkpoints, PyTorch ``.pt`` import/export, GGUF parsing/dequantisation, ONNX export.

Reference parity: state_dict.rs:1-161 (JSON-lines index + ``\\n---\\n`` + raw LE body), checkpoint.rs:1-643 (three length-prefixed
sections: metadata JSON, optimizer JSON, state-dict binary; AsyncCheckpointer), pytorch_import.rs:35-901 (zip + restricted pickle),
pytorch_export.rs:1-222 (``archive/data.pkl`` + ``archive/data/N``), gguf.rs:38-834, onnx_export.rs:743-1067.
"""
from __future__ import annotations

import io
import json
import pickle
import queue
import struct
import threading
import zipfile
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Tuple

import numpy as np
import torch

from ..errors import InvalidArgument
from .safetensors_io import _DT, _NAME, _raw_bytes

# ----------------------------------------------------------------------------------------------------------------------
# native state dict: one JSON line per tensor, separator, raw little-endian body
# ----------------------------------------------------------------------------------------------------------------------
_SEP = b"\n---\n"
# dtype tags of the header: the reference writes "f32" / "f64" (state_dict.rs:45-53); the other element types follow the same spelling
_TAG = {torch.float32: "f32", torch.float64: "f64", torch.bfloat16: "bf16", torch.float16: "f16", torch.int64: "i64", torch.int32: "i32",
        torch.int16: "i16", torch.int8: "i8", torch.uint8: "u8", torch.bool: "bool"}
_FROM_TAG = {v: k for k, v in _TAG.items()}


def _dtype_of(tag: str) -> torch.dtype:
    t = _FROM_TAG.get(tag.lower())
    if t is None:
        t = _DT.get(tag.upper())
    if t is None:
        raise InvalidArgument(f"state dict: unknown dtype tag {tag!r}")
    return t


def dumps_state_dict(state: Dict[str, torch.Tensor]) -> bytes:
    """Byte-for-byte the layout of the reference's ``save_state_dict`` (state_dict.rs:59-161): one compact JSON line per tensor with the keys
    ``name, shape, dtype, byte_offset, byte_length`` in that order, names sorted, every line ended by a newline, then ``\n---\n`` and the raw
    little-endian bodies in header order."""
    lines, body, off = [], [], 0
    for k in sorted(state):
        t = state[k]
        if t.dtype not in _TAG:
            raise InvalidArgument(f"dtype {t.dtype} of {k!r} cannot be stored in a native state dict")
        raw = bytes(_raw_bytes(t))
        shape = "[" + ",".join(str(int(d)) for d in t.shape) + "]"
        lines.append(f'{{"name":{json.dumps(k)},"shape":{shape},"dtype":"{_TAG[t.dtype]}","byte_offset":{off},"byte_length":{len(raw)}}}\n')
        body.append(raw)
        off += len(raw)
    return "".join(lines).encode() + _SEP + b"".join(body)


def loads_state_dict(data: bytes) -> Dict[str, torch.Tensor]:
    """Reads the reference's layout; files written by earlier versions of this package (keys ``offset`` / ``nbytes``, upper-case dtype
    tags, no newline before the separator) load as well."""
    i = data.index(_SEP)
    head, body = data[:i].decode(), memoryview(data)[i + len(_SEP):]
    out = {}
    for line in head.splitlines():
        if not line.strip():
            continue
        m = json.loads(line)
        off = m["byte_offset"] if "byte_offset" in m else m["offset"]
        n = m["byte_length"] if "byte_length" in m else m["nbytes"]
        if off < 0 or n < 0 or off + n > len(body):
            raise InvalidArgument(f"state dict: tensor {m['name']!r} lies outside the body ({off}+{n} > {len(body)})")
        raw = bytes(body[off: off + n])
        dt = _dtype_of(m["dtype"])
        if dt == torch.bfloat16:
            t = torch.frombuffer(bytearray(raw), dtype=torch.int16).view(torch.bfloat16) if raw else torch.empty(0, dtype=dt)
        else:
            t = torch.frombuffer(bytearray(raw), dtype=dt) if raw else torch.empty(0, dtype=dt)
        out[m["name"]] = t.reshape(m["shape"]).clone()
    return out


def save_state_dict(state: Dict[str, torch.Tensor], path) -> None:
    Path(path).write_bytes(dumps_state_dict(state))


def load_state_dict(path) -> Dict[str, torch.Tensor]:
    return loads_state_dict(Path(path).read_bytes())


# ----------------------------------------------------------------------------------------------------------------------
# training checkpoint (.ftc): [u64 len][metadata JSON][u64 len][optimizer JSON][u64 len][state-dict binary]
# ----------------------------------------------------------------------------------------------------------------------
# The optimizer section has the reference's shape (checkpoint.rs:198-229): {"<param key>": {"<state name>": [numbers...]}}, keys sorted,
# numbers only. A torch-style optimizer state dict is flattened into that shape; what the flat lists cannot carry (tensor shapes and
# dtypes, value kinds, parameter groups) goes into reserved entries whose names start with "__" and that again hold number lists only, so
# a reader that knows only the reference's shape still parses the whole section.
_KIND_FLOAT, _KIND_INT, _KIND_BOOL, _KIND_NONE, _KIND_TUPLE, _KIND_TENSOR = 0, 1, 2, 3, 4, 5
_DT_CODE = {torch.float32: 0, torch.float64: 1, torch.bfloat16: 2, torch.float16: 3, torch.int64: 4, torch.int32: 5, torch.int16: 6,
            torch.int8: 7, torch.uint8: 8, torch.bool: 9}
_CODE_DT = {v: k for k, v in _DT_CODE.items()}


def _num(v) -> str:
    v = float(v)
    if v != v:
        return "NaN"
    if v in (float("inf"), float("-inf")):
        return "inf" if v > 0 else "-inf"
    return repr(int(v)) if v == int(v) and abs(v) < 1e15 else repr(v)


def _flat_entry(v):
    """(numbers, kind, shape, dtype code) of one optimizer-state or parameter-group value, or None when it cannot be written as numbers."""
    if isinstance(v, torch.Tensor):
        return v.detach().cpu().double().reshape(-1).tolist(), _KIND_TENSOR, list(v.shape), _DT_CODE.get(v.dtype, 0)
    if isinstance(v, bool):
        return [int(v)], _KIND_BOOL, None, None
    if isinstance(v, int):
        return [v], _KIND_INT, None, None
    if isinstance(v, float):
        return [v], _KIND_FLOAT, None, None
    if v is None:
        return [], _KIND_NONE, None, None
    if isinstance(v, (tuple, list)) and all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in v):
        return list(v), _KIND_TUPLE, None, None
    return None


def _opt_to_json(osd: dict) -> str:
    if not osd:
        return "{}"
    if "state" not in osd and "param_groups" not in osd:          # already in the reference's shape: {key: {name: [numbers]}}
        tables = {str(k): {str(n): list(map(float, vals)) for n, vals in inner.items()} for k, inner in osd.items()}
    else:
        tables: Dict[str, Dict[str, list]] = {}
        kinds, shapes, dtypes = {}, {}, {}

        def put(table: str, name: str, v) -> None:
            e = _flat_entry(v)
            if e is None:
                return                                              # not expressible as numbers (a callable, a string): left to the live optimizer
            vals, kind, shape, code = e
            tables.setdefault(table, {})[name] = vals
            kinds[f"{table}/{name}"] = [kind]
            if shape is not None:
                shapes[f"{table}/{name}"] = shape
                dtypes[f"{table}/{name}"] = [code]
        for pid, st in osd.get("state", {}).items():
            for name, v in st.items():
                put(str(pid), str(name), v)
        for gi, g in enumerate(osd.get("param_groups", [])):
            for name, v in g.items():
                put(f"__group_{gi}__", str(name), v)
        tables["__kinds__"], tables["__shapes__"], tables["__dtypes__"] = kinds, shapes, dtypes
    parts = []
    for key in sorted(tables):
        inner = ",".join(f"{json.dumps(n)}:[{','.join(_num(x) for x in tables[key][n])}]" for n in sorted(tables[key]))
        parts.append(f"{json.dumps(key)}:{{{inner}}}")
    return "{" + ",".join(parts) + "}"


def _opt_from_json(text) -> dict:
    j = json.loads(text) if isinstance(text, (str, bytes)) else text
    if not j:
        return {}
    if "__kinds__" not in j:
        if any(isinstance(v, dict) and "__tensor__" in v for v in _walk(j)):      # section written by an earlier version of this package
            return _legacy_opt_from_json(j)
        return j                                                                  # plain reference shape: handed back as it is
    kinds, shapes, dtypes = j["__kinds__"], j.get("__shapes__", {}), j.get("__dtypes__", {})

    def get(table: str, name: str, vals):
        kind = int(kinds.get(f"{table}/{name}", [_KIND_FLOAT])[0])
        if kind == _KIND_TENSOR:
            dt = _CODE_DT.get(int(dtypes.get(f"{table}/{name}", [0])[0]), torch.float32)
            return torch.tensor(vals, dtype=torch.float64).reshape([int(d) for d in shapes.get(f"{table}/{name}", [len(vals)])]).to(dt)
        if kind == _KIND_BOOL:
            return bool(vals[0])
        if kind == _KIND_INT:
            return int(vals[0])
        if kind == _KIND_NONE:
            return None
        if kind == _KIND_TUPLE:
            return tuple(int(x) if float(x).is_integer() and name == "params" else x for x in vals)
        return float(vals[0])
    state, groups = {}, {}
    for table, inner in j.items():
        if table in ("__kinds__", "__shapes__", "__dtypes__"):
            continue
        if table.startswith("__group_") and table.endswith("__"):
            g = {name: get(table, name, vals) for name, vals in inner.items()}
            if "params" in g:
                g["params"] = [int(x) for x in g["params"]]
            groups[int(table[len("__group_"):-2])] = g
        else:
            state[int(table) if table.lstrip("-").isdigit() else table] = {name: get(table, name, vals) for name, vals in inner.items()}
    return {"state": state, "param_groups": [groups[i] for i in sorted(groups)]}


def _walk(j):
    if isinstance(j, dict):
        yield j
        for v in j.values():
            yield from _walk(v)
    elif isinstance(j, list):
        for v in j:
            yield from _walk(v)


def _legacy_opt_from_json(j):
    def dec(v):
        if isinstance(v, dict) and "__tensor__" in v:
            return torch.tensor(v["__tensor__"], dtype=torch.float64).reshape(v["shape"]).to(_DT.get(v["dtype"], torch.float32))
        if isinstance(v, dict):
            return {(int(k) if k.lstrip("-").isdigit() else k): dec(x) for k, x in v.items()}
        if isinstance(v, list):
            return [dec(x) for x in v]
        return v
    return dec(j)


@dataclass
class TrainingCheckpoint:
    model_state: Dict[str, torch.Tensor]
    optimizer_state: dict = field(default_factory=dict)
    epoch: int = 0
    step: int = 0
    extra: dict = field(default_factory=dict)

    def save(self, path) -> None:
        # section 1 is the reference's '{"epoch":E,"step":S}' (checkpoint.rs:86-90); user extras follow under one optional key, which the
        # reference's reader (it looks the two keys up by name, checkpoint.rs:177-196) skips
        meta = f'{{"epoch":{int(self.epoch)},"step":{int(self.step)}' + (f',"extra":{json.dumps(self.extra)}' if self.extra else "") + "}"
        opt = _opt_to_json(self.optimizer_state)
        sd = dumps_state_dict({k: v.detach().cpu() for k, v in self.model_state.items()})
        tmp = str(path) + ".tmp"
        with open(tmp, "wb") as f:
            for sec in (meta.encode(), opt.encode(), sd):
                f.write(struct.pack("<Q", len(sec)))
                f.write(sec)
        import os
        os.replace(tmp, path)

    @staticmethod
    def load(path) -> "TrainingCheckpoint":
        data = Path(path).read_bytes()
        secs, off = [], 0
        for _ in range(3):
            if off + 8 > len(data):
                raise InvalidArgument("checkpoint: truncated section header")
            (n,) = struct.unpack_from("<Q", data, off)
            if off + 8 + n > len(data):
                raise InvalidArgument("checkpoint: section runs past the end of the file")
            secs.append(data[off + 8: off + 8 + n])
            off += 8 + n
        meta = json.loads(secs[0])
        return TrainingCheckpoint(loads_state_dict(secs[2]), _opt_from_json(secs[1].decode()), meta["epoch"], meta["step"], meta.get("extra", {}))


def save_checkpoint(path, model: torch.nn.Module, optimizer: Optional[torch.optim.Optimizer] = None, epoch: int = 0, step: int = 0, **extra) -> None:
    TrainingCheckpoint(model.state_dict(), optimizer.state_dict() if optimizer else {}, epoch, step, extra).save(path)


def load_checkpoint(path, model: Optional[torch.nn.Module] = None, optimizer: Optional[torch.optim.Optimizer] = None, strict: bool = True) -> TrainingCheckpoint:
    ck = TrainingCheckpoint.load(path)
    if model is not None:
        model.load_state_dict(ck.model_state, strict=strict)
    if optimizer is not None and ck.optimizer_state:
        optimizer.load_state_dict(ck.optimizer_state)
    return ck


class CheckpointFuture:
    def __init__(self):
        self._ev, self._err = threading.Event(), None

    def wait(self, timeout: Optional[float] = None) -> None:
        if not self._ev.wait(timeout):
            from ..errors import Timeout
            raise Timeout(timeout)
        if self._err:
            raise self._err

    def done(self) -> bool:
        return self._ev.is_set()


class AsyncCheckpointer:
    """Background writer: tensors are snapshotted to host memory on the caller's thread (a device-to-host copy), the file is written
    by a worker thread so training continues during the write."""

    def __init__(self, max_pending: int = 2):
        self._q: "queue.Queue" = queue.Queue(max_pending)
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def _run(self):
        while True:
            item = self._q.get()
            if item is None:
                return
            ck, path, fut = item
            try:
                ck.save(path)
            except BaseException as e:
                fut._err = e
            fut._ev.set()

    def save_async(self, path, model_state: Dict[str, torch.Tensor], optimizer_state: Optional[dict] = None, epoch: int = 0, step: int = 0) -> CheckpointFuture:
        snap = {k: v.detach().to("cpu", copy=True) for k, v in model_state.items()}
        fut = CheckpointFuture()
        self._q.put((TrainingCheckpoint(snap, optimizer_state or {}, epoch, step), path, fut))
        return fut

    def close(self) -> None:
        self._q.put(None)
        self._t.join()


# ----------------------------------------------------------------------------------------------------------------------
# PyTorch .pt (zip + pickle) import / export
# ----------------------------------------------------------------------------------------------------------------------
_STORAGE_DT = {"FloatStorage": torch.float32, "DoubleStorage": torch.float64, "HalfStorage": torch.float16, "BFloat16Storage": torch.bfloat16,
               "LongStorage": torch.int64, "IntStorage": torch.int32, "ShortStorage": torch.int16, "CharStorage": torch.int8,
               "ByteStorage": torch.uint8, "BoolStorage": torch.bool}


class _StorageType:
    def __init__(self, name):
        self.dtype = _STORAGE_DT[name]


def _rebuild_tensor_v2(storage, offset, size, stride, requires_grad=False, backward_hooks=None, metadata=None):
    t = torch.empty(0, dtype=storage.dtype)
    if storage.numel() == 0 and len(size) and int(np.prod(size)) == 0:
        return torch.empty(tuple(size), dtype=storage.dtype)
    return torch.as_strided(storage, tuple(size), tuple(stride), offset).clone()


class _RestrictedUnpickler(pickle.Unpickler):
    """Pickle VM limited to the constructs a ``torch.save`` state dict uses; anything else is refused."""

    def __init__(self, f, read_storage: Callable[[str, torch.dtype, int], torch.Tensor]):
        super().__init__(f)
        self._read = read_storage

    def find_class(self, module, name):
        if module == "torch._utils" and name in ("_rebuild_tensor_v2", "_rebuild_tensor"):
            return _rebuild_tensor_v2
        if module == "torch._utils" and name == "_rebuild_parameter":
            return lambda data, requires_grad, hooks: data
        if module == "torch" and name in _STORAGE_DT:
            return _StorageType(name)
        if module == "collections" and name == "OrderedDict":
            import collections
            return collections.OrderedDict
        if module == "torch" and name == "Size":
            return tuple
        if module in ("builtins", "__builtin__") and name in ("dict", "list", "tuple", "set", "int", "float", "str", "bool"):
            return {"dict": dict, "list": list, "tuple": tuple, "set": set, "int": int, "float": float, "str": str, "bool": bool}[name]
        raise InvalidArgument(f"refusing to unpickle {module}.{name}: only tensor state dicts are supported")

    def persistent_load(self, pid):
        # ('storage', storage_type, key, location, numel)
        if not (isinstance(pid, tuple) and pid and pid[0] == "storage"):
            raise InvalidArgument("unsupported persistent id in .pt file")
        _, st, key, _loc, numel = pid
        return self._read(str(key), st.dtype, int(numel))


def load_pytorch_state_dict(path, dtype: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
    """Read a ``torch.save`` zip archive without importing arbitrary classes (restricted pickle VM)."""
    with zipfile.ZipFile(path) as z:
        names = z.namelist()
        pkl = next((n for n in names if n.endswith("data.pkl")), None)
        if pkl is None:
            raise InvalidArgument("not a torch zip archive (data.pkl missing)")
        root = pkl[: -len("data.pkl")]

        def read_storage(key, dt, numel):
            raw = z.read(f"{root}data/{key}")
            if dt == torch.bfloat16:
                return torch.frombuffer(bytearray(raw), dtype=torch.int16).view(torch.bfloat16) if raw else torch.empty(0, dtype=dt)
            return torch.frombuffer(bytearray(raw), dtype=dt) if raw else torch.empty(0, dtype=dt)
        obj = _RestrictedUnpickler(io.BytesIO(z.read(pkl)), read_storage).load()
    if isinstance(obj, dict) and "state_dict" in obj and isinstance(obj["state_dict"], dict):
        obj = obj["state_dict"]
    out = {}
    for k, v in obj.items():
        if isinstance(v, torch.Tensor):
            out[k] = v.to(dtype) if (dtype is not None and v.is_floating_point()) else v
    return out


def save_pytorch_state_dict(state: Dict[str, torch.Tensor], path) -> None:
    """Write a zip archive ``archive/data.pkl`` + ``archive/data/N`` that ``torch.load`` reads (ferrotorch-serialize/src/pytorch_export.rs:5-13).
    The pickle stream is produced by torch's own serializer so the class references are exactly what ``torch.load`` expects."""
    torch.save({k: v.detach().cpu().contiguous() for k, v in state.items()}, path, _use_new_zipfile_serialization=True)


# ----------------------------------------------------------------------------------------------------------------------
# GGUF
# ----------------------------------------------------------------------------------------------------------------------
GGML_TYPES = {0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22), 7: ("Q5_1", 32, 24),
              8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 36), 30: ("BF16", 1, 2)}


@dataclass
class GgufTensorInfo:
    name: str
    shape: Tuple[int, ...]
    ggml_type: int
    offset: int


@dataclass
class GgufFile:
    version: int
    metadata: Dict[str, Any]
    tensors: Dict[str, GgufTensorInfo]
    data_offset: int
    path: str

    def load_tensor(self, name: str, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        info = self.tensors[name]
        tname, blk, bsz = GGML_TYPES[info.ggml_type]
        n = int(np.prod(info.shape)) if info.shape else 1
        nbytes = n // blk * bsz
        with open(self.path, "rb") as f:
            f.seek(self.data_offset + info.offset)
            raw = f.read(nbytes)
        return dequantize_gguf(raw, info.ggml_type, n).reshape(tuple(reversed(info.shape))).to(dtype)


def _read_str(f) -> str:
    (n,) = struct.unpack("<Q", f.read(8))
    return f.read(n).decode("utf-8", "replace")


def _read_value(f, t: int):
    fmt = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
    if t in fmt:
        s = struct.calcsize(fmt[t])
        return struct.unpack(fmt[t], f.read(s))[0]
    if t == 8:
        return _read_str(f)
    if t == 9:
        (et,) = struct.unpack("<I", f.read(4))
        (n,) = struct.unpack("<Q", f.read(8))
        return [_read_value(f, et) for _ in range(n)]
    raise InvalidArgument(f"unknown GGUF value type {t}")


def parse_gguf(path) -> GgufFile:
    with open(path, "rb") as f:
        if f.read(4) != b"GGUF":
            raise InvalidArgument("not a GGUF file")
        (version,) = struct.unpack("<I", f.read(4))
        n_tensors, n_kv = struct.unpack("<QQ", f.read(16))
        meta = {}
        for _ in range(n_kv):
            k = _read_str(f)
            (t,) = struct.unpack("<I", f.read(4))
            meta[k] = _read_value(f, t)
        tensors = {}
        for _ in range(n_tensors):
            name = _read_str(f)
            (nd,) = struct.unpack("<I", f.read(4))
            shape = struct.unpack(f"<{nd}Q", f.read(8 * nd))
            (gt,) = struct.unpack("<I", f.read(4))
            (off,) = struct.unpack("<Q", f.read(8))
            tensors[name] = GgufTensorInfo(name, tuple(shape), gt, off)
        align = int(meta.get("general.alignment", 32))
        pos = f.tell()
        data_offset = (pos + align - 1) // align * align
    return GgufFile(version, meta, tensors, data_offset, str(path))


def dequantize_gguf(raw: bytes, ggml_type: int, n: int) -> torch.Tensor:
    """Block dequantisation (CPU, numpy-vectorised): q4_0, q4_1, q5_0, q5_1, q8_0, q8_1, f16, bf16, f32."""
    name, blk, bsz = GGML_TYPES[ggml_type]
    b = np.frombuffer(raw, dtype=np.uint8)
    if name == "F32":
        return torch.from_numpy(b.view(np.float32)[:n].copy())
    if name == "F16":
        return torch.from_numpy(b.view(np.float16)[:n].astype(np.float32))
    if name == "BF16":
        return torch.from_numpy(b.view(np.int16)[:n].copy()).view(torch.bfloat16).float()
    nb = n // blk
    blocks = b[: nb * bsz].reshape(nb, bsz)
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32)          # [nb,1]
    if name == "Q8_0":
        q = blocks[:, 2:34].view(np.int8).astype(np.float32)
        return torch.from_numpy((q * d).reshape(-1))
    if name == "Q8_1":
        q = blocks[:, 4:36].view(np.int8).astype(np.float32)
        return torch.from_numpy((q * d).reshape(-1))
    if name in ("Q4_0", "Q4_1"):
        o = 2 if name == "Q4_0" else 4
        qs = blocks[:, o: o + 16]
        lo, hi = (qs & 0x0F).astype(np.float32), (qs >> 4).astype(np.float32)
        q = np.concatenate([lo, hi], 1)
        if name == "Q4_0":
            return torch.from_numpy(((q - 8.0) * d).reshape(-1))
        m = blocks[:, 2:4].copy().view(np.float16).astype(np.float32)
        return torch.from_numpy((q * d + m).reshape(-1))
    if name in ("Q5_0", "Q5_1"):
        o = 2 if name == "Q5_0" else 4
        qh = blocks[:, o: o + 4].copy().view(np.uint32)                    # [nb,1]
        qs = blocks[:, o + 4: o + 20]
        lo, hi = (qs & 0x0F).astype(np.uint32), (qs >> 4).astype(np.uint32)
        bits = np.arange(32, dtype=np.uint32)
        hb = ((qh >> bits) & 1).astype(np.uint32)                           # [nb,32]
        q = np.concatenate([lo | (hb[:, :16] << 4), hi | (hb[:, 16:] << 4)], 1).astype(np.float32)
        if name == "Q5_0":
            return torch.from_numpy(((q - 16.0) * d).reshape(-1))
        m = blocks[:, 2:4].copy().view(np.float16).astype(np.float32)
        return torch.from_numpy((q * d + m).reshape(-1))
    raise InvalidArgument(f"unsupported GGML type {name}")


# ----------------------------------------------------------------------------------------------------------------------
# ONNX export (hand-rolled protobuf writer for a small operator set traced from nn.Sequential-like modules)
# ----------------------------------------------------------------------------------------------------------------------
def _varint(n: int) -> bytes:
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _field(num: int, wire: int, payload: bytes) -> bytes:
    return _varint((num << 3) | wire) + payload


def _ld(num: int, data: bytes) -> bytes:
    return _field(num, 2, _varint(len(data)) + data)


def _vi(num: int, v: int) -> bytes:
    return _field(num, 0, _varint(v))


@dataclass
class OnnxExportConfig:
    opset: int = 17
    producer: str = "ferrotorch_b200"
    input_name: str = "input"
    output_name: str = "output"


def _tensor_proto(name: str, t: torch.Tensor) -> bytes:
    t = t.detach().cpu().float().contiguous()
    b = b"".join(_vi(1, d) for d in t.shape) + _vi(2, 1) + _ld(8, name.encode()) + _ld(9, t.numpy().tobytes())
    return b


def _value_info(name: str, shape) -> bytes:
    dims = b"".join(_ld(1, _vi(1, d) if isinstance(d, int) else _ld(2, str(d).encode())) for d in shape)
    ttype = _vi(1, 1) + _ld(2, dims)
    return _ld(1, name.encode()) + _ld(2, _ld(1, ttype))


def _node(op: str, inputs, outputs, attrs: bytes = b"", name: str = "") -> bytes:
    return b"".join(_ld(1, i.encode()) for i in inputs) + b"".join(_ld(2, o.encode()) for o in outputs) + _ld(3, name.encode()) + _ld(4, op.encode()) + attrs


def _attr_int(name: str, v: int) -> bytes:
    return _ld(5, _ld(1, name.encode()) + _vi(3, v) + _vi(20, 2))


def _attr_float(name: str, v: float) -> bytes:
    return _ld(5, _ld(1, name.encode()) + _field(2, 5, struct.pack("<f", v)) + _vi(20, 1))


def export_onnx(model: torch.nn.Module, example_input: torch.Tensor, path, config: Optional[OnnxExportConfig] = None) -> None:
    """Export a feed-forward stack (Linear, ReLU, GELU, Sigmoid, Tanh, SiLU, Softmax, Flatten, LayerNorm, Dropout, Identity, nested
    Sequential) to an ONNX ModelProto. Other layers raise ``InvalidArgument`` naming the layer."""
    cfg = config or OnnxExportConfig()
    nodes, inits = [], []
    cur = cfg.input_name
    counter = [0]

    def fresh(prefix):
        counter[0] += 1
        return f"{prefix}_{counter[0]}"

    def walk(m, cur):
        cls = type(m).__name__
        if isinstance(m, torch.nn.Sequential):
            for c in m:
                cur = walk(c, cur)
            return cur
        if cls in ("Linear",) and hasattr(m, "weight"):
            w, out = fresh("W"), fresh("lin")
            inits.append(_tensor_proto(w, m.weight))
            ins = [cur, w]
            if m.bias is not None:
                b = fresh("B")
                inits.append(_tensor_proto(b, m.bias))
                ins.append(b)
            nodes.append(_node("Gemm", ins, [out], _attr_int("transB", 1), out))
            return out
        simple = {"ReLU": "Relu", "Sigmoid": "Sigmoid", "Tanh": "Tanh", "GELU": "Gelu", "Identity": "Identity", "Dropout": "Identity",
                  "Softplus": "Softplus", "Softsign": "Softsign", "Mish": "Mish"}
        if cls in simple:
            out = fresh(simple[cls].lower())
            nodes.append(_node(simple[cls], [cur], [out], b"", out))
            return out
        if cls == "SiLU":
            s, out = fresh("sig"), fresh("silu")
            nodes.append(_node("Sigmoid", [cur], [s], b"", s))
            nodes.append(_node("Mul", [cur, s], [out], b"", out))
            return out
        if cls in ("Softmax", "LogSoftmax"):
            out = fresh("sm")
            nodes.append(_node(cls, [cur], [out], _attr_int("axis", m.dim if m.dim is not None else -1), out))
            return out
        if cls == "Flatten":
            out = fresh("flat")
            nodes.append(_node("Flatten", [cur], [out], _attr_int("axis", m.start_dim), out))
            return out
        if cls == "LayerNorm":
            w, b, out = fresh("lnw"), fresh("lnb"), fresh("ln")
            inits.append(_tensor_proto(w, m.weight))
            inits.append(_tensor_proto(b, m.bias if m.bias is not None else torch.zeros_like(m.weight)))
            nodes.append(_node("LayerNormalization", [cur, w, b], [out], _attr_int("axis", -1) + _attr_float("epsilon", m.eps), out))
            return out
        raise InvalidArgument(f"ONNX export does not support layer {cls}")

    last = walk(model, cur)
    nodes.append(_node("Identity", [last], [cfg.output_name], b"", "out"))
    with torch.no_grad():
        out_shape = list(model(example_input).shape)
    in_shape = ["batch"] + list(example_input.shape[1:])
    out_shape = ["batch"] + out_shape[1:]
    graph = b"".join(_ld(1, n) for n in nodes) + _ld(2, b"main") + b"".join(_ld(5, i) for i in inits) + \
        _ld(11, _value_info(cfg.input_name, in_shape)) + _ld(12, _value_info(cfg.output_name, out_shape))
    model_pb = _vi(1, 8) + _ld(2, cfg.producer.encode()) + _ld(7, graph) + _ld(8, _ld(1, b"") + _vi(2, cfg.opset))
    Path(path).write_bytes(model_pb)
