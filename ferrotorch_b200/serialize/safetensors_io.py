"""SafeTensors reader/writer implemented from the format definition (8-byte LE header length, JSON header, raw LE tensor data):
single file, sharded (``model.safetensors.index.json``), memory-mapped and filtered loads.

Byte compatibility: files written here load with the reference and with the ``safetensors`` library and vice versa. F32/F64
tensors are written exactly as the reference writes them; BF16/F16/integer tensors are written natively (the reference's writer
rejects anything but F32/F64: ferrotorch-serialize/src/safetensors_io.rs:55-64) and F16/BF16 files are cast on load to the
requested dtype as the reference does (:172-175).

Reference parity: safetensors_io.rs:109 (save), :399 (load), :541 (load_sharded), :789 (mmap / filtered).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Optional

import numpy as np
import torch

from ..errors import InvalidArgument

_DT = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
       "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool}
_NAME = {v: k for k, v in _DT.items()}
_NP = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I64": np.int64, "I32": np.int32, "I16": np.int16,
       "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_}


def _raw_bytes(t: torch.Tensor) -> memoryview:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return memoryview(t.view(torch.int16).numpy()).cast("B")
    return memoryview(t.numpy()).cast("B") if t.numel() else memoryview(b"")


def save_safetensors(state: Dict[str, torch.Tensor], path, metadata: Optional[Dict[str, str]] = None) -> None:
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(state.keys())
    for k in order:
        t = state[k]
        if t.dtype not in _NAME:
            raise InvalidArgument(f"dtype {t.dtype} of {k!r} cannot be stored in SafeTensors")
        n = t.numel() * t.element_size()
        header[k] = {"dtype": _NAME[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    tmp = str(path) + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for k in order:
            f.write(_raw_bytes(state[k]))
    os.replace(tmp, path)


def _read_header(f) -> tuple:
    (n,) = struct.unpack("<Q", f.read(8))
    if n > 100 * 1024 * 1024:
        raise InvalidArgument("SafeTensors header too large")
    return json.loads(f.read(n)), 8 + n


def _tensor_from(buf, info: dict, base: int, dtype: Optional[torch.dtype], copy: bool) -> torch.Tensor:
    a, b = info["data_offsets"]
    name = info["dtype"]
    arr = np.frombuffer(buf, dtype=_NP[name], count=(b - a) // np.dtype(_NP[name]).itemsize, offset=base + a)
    t = torch.from_numpy(arr.copy() if copy else arr)
    if name == "BF16":
        t = t.view(torch.bfloat16)
    t = t.reshape(info["shape"])
    if dtype is not None and t.is_floating_point() and t.dtype != dtype:
        t = t.to(dtype)
    return t


def load_safetensors(path, dtype: Optional[torch.dtype] = None, device="cpu", filter_fn: Optional[Callable[[str], bool]] = None,
                     use_mmap: bool = True, parallel: Optional[bool] = None) -> Dict[str, torch.Tensor]:
    """Load a file. ``dtype`` casts floating tensors (F16/BF16 files load into any requested float type); ``filter_fn`` selects names;
    ``use_mmap`` maps the file instead of reading it; ``parallel`` reads tensors on a thread pool (default: on for files > 64 MiB,
    off when ``FERROTORCH_FORCE_SERIAL_LOAD`` is set)."""
    out: Dict[str, torch.Tensor] = {}
    with open(path, "rb") as f:
        header, base = _read_header(f)
        names = [k for k in header if k != "__metadata__" and (filter_fn is None or filter_fn(k))]
        size = os.fstat(f.fileno()).st_size
        if parallel is None:
            parallel = size > (64 << 20) and not os.environ.get("FERROTORCH_FORCE_SERIAL_LOAD")
        buf = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) if (use_mmap and size > 0) else f.read()
        base_off = base if use_mmap and size > 0 else 0
        if not (use_mmap and size > 0):
            base_off = 0
            buf = buf  # bytes after the header

        def one(k):
            t = _tensor_from(buf, header[k], base_off, dtype, copy=True)
            return k, (t.to(device) if str(device) != "cpu" else t)
        if parallel and len(names) > 1:
            with ThreadPoolExecutor(max_workers=min(8, len(names))) as ex:
                for k, t in ex.map(one, names):
                    out[k] = t
        else:
            for k in names:
                out[k] = one(k)[1]
        if use_mmap and size > 0:
            buf.close()
    return out


def load_safetensors_filtered(path, predicate: Callable[[str], bool], **kw):
    return load_safetensors(path, filter_fn=predicate, **kw)


def load_safetensors_mmap(path, **kw):
    return load_safetensors(path, use_mmap=True, **kw)


def safetensors_metadata(path) -> Dict[str, dict]:
    with open(path, "rb") as f:
        header, _ = _read_header(f)
    return header


def save_safetensors_sharded(state: Dict[str, torch.Tensor], directory, max_shard_bytes: int = 5 * 1024 ** 3, prefix: str = "model") -> Path:
    """Writes ``{prefix}-0000X-of-0000N.safetensors`` shards and ``{prefix}.safetensors.index.json``; returns the index path."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    shards: List[Dict[str, torch.Tensor]] = [{}]
    cur = 0
    for k in sorted(state):
        n = state[k].numel() * state[k].element_size()
        if shards[-1] and cur + n > max_shard_bytes:
            shards.append({})
            cur = 0
        shards[-1][k] = state[k]
        cur += n
    weight_map, total = {}, 0
    for i, sh in enumerate(shards):
        name = f"{prefix}-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_safetensors(sh, d / name)
        for k, t in sh.items():
            weight_map[k] = name
            total += t.numel() * t.element_size()
    idx = d / f"{prefix}.safetensors.index.json"
    idx.write_text(json.dumps({"metadata": {"total_size": total}, "weight_map": weight_map}, indent=2))
    return idx


def load_safetensors_sharded(index_path, dtype: Optional[torch.dtype] = None, device="cpu", filter_fn=None) -> Dict[str, torch.Tensor]:
    idx = json.loads(Path(index_path).read_text())
    base = Path(index_path).parent
    by_file: Dict[str, List[str]] = {}
    for k, fn in idx["weight_map"].items():
        if filter_fn is None or filter_fn(k):
            by_file.setdefault(fn, []).append(k)
    out: Dict[str, torch.Tensor] = {}
    for fn, keys in by_file.items():
        ks = set(keys)
        out.update(load_safetensors(base / fn, dtype, device, lambda n: n in ks))
    return out
