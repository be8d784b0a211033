"""Loader variants, GGUF typed access, the non-executing pickle reader, checkpoint validation and ONNX export of IR graphs."""
import io
import pickle
import struct
import zipfile
from collections import OrderedDict

import numpy as np
import pytest
import torch

from ferrotorch_b200 import jit, serialize as S
from ferrotorch_b200.errors import InvalidArgument


def test_sharded_safetensors_variants(tmp_path):
    sd = {f"layer{i}.w": torch.randn(8, 8) for i in range(6)}
    idx = S.save_safetensors_sharded(sd, tmp_path, max_shard_bytes=600)
    seen = []
    got = S.load_safetensors_sharded_with_progress(idx, seen.append)
    assert all(torch.equal(got[k], v) for k, v in sd.items()) and len(seen) >= 3
    assert [p.shard_index for p in seen] == list(range(len(seen))) and all(p.shard_count == len(seen) and p.total_tensors == 6 for p in seen)
    assert seen[0].tensors_loaded_so_far == 0 and seen[-1].tensors_loaded_so_far + seen[-1].tensors_in_shard == 6
    assert all(torch.equal(S.load_safetensors_sharded_mmap(idx)[k], v) for k, v in sd.items())
    part = S.load_safetensors_sharded_filtered(idx, lambda n: n in ("layer0.w", "layer5.w"))
    assert sorted(part) == ["layer0.w", "layer5.w"]
    assert sorted(S.load_safetensors_auto(idx)) == sorted(sd)
    S.save_safetensors(sd, str(tmp_path / "one.safetensors"))
    assert sorted(S.load_safetensors_auto(tmp_path / "one.safetensors")) == sorted(sd)
    (tmp_path / seen[1].shard_file).unlink()
    with pytest.raises(InvalidArgument):
        S.load_safetensors_sharded_with_progress(idx, lambda p: None)
    assert sorted(S.load_safetensors_sharded_filtered(idx, lambda n: n in seen_names(seen[0], idx))) != []      # untouched shards still load


def seen_names(p, idx):
    import json
    wm = json.loads(open(idx).read())["weight_map"]
    return [k for k, f in wm.items() if f == p.shard_file]


def _gguf_image(version=3):
    def s(x):
        b = x.encode()
        return struct.pack("<Q", len(b)) + b
    w = np.arange(64, dtype=np.float32).reshape(2, 32)
    q8_scale = np.float16(0.5)
    q8 = (np.arange(32, dtype=np.int8) - 16)
    kv = s("general.architecture") + struct.pack("<I", 8) + s("llama")
    kv += s("llama.block_count") + struct.pack("<I", 4) + struct.pack("<I", 2)
    kv += s("llama.rope.freq_base") + struct.pack("<I", 6) + struct.pack("<f", 10000.0)
    kv += s("general.alignment") + struct.pack("<I", 4) + struct.pack("<I", 64)
    kv += s("tokenizer.ggml.tokens") + struct.pack("<I", 9) + struct.pack("<I", 8) + struct.pack("<Q", 2) + s("a") + s("b")
    kv += s("flag") + struct.pack("<I", 7) + b"\x01"
    ti = s("w.f32") + struct.pack("<I", 2) + struct.pack("<QQ", 32, 2) + struct.pack("<I", 0) + struct.pack("<Q", 0)
    ti += s("w.q8") + struct.pack("<I", 1) + struct.pack("<Q", 32) + struct.pack("<I", 8) + struct.pack("<Q", 256)
    head = b"GGUF" + struct.pack("<I", version) + struct.pack("<QQ", 2, 6) + kv + ti
    head += b"\0" * (-len(head) % 64)
    return head + w.tobytes() + q8_scale.tobytes() + q8.tobytes(), w, (q8.astype(np.float32) * 0.5)


def test_gguf_typed_api(tmp_path):
    img, w, q = _gguf_image()
    f = S.parse_gguf_bytes(img)
    assert f.version == 3 and f.tensor_names() == ["w.f32", "w.q8"] and f.tensors[0].ggml_type is S.GgmlType.F32 and f.tensors[1].ggml_type.block_size() == 32
    m = f.metadata
    assert m.get_str("general.architecture") == "llama" and m.get_int("llama.block_count") == 2 and m.get_float("llama.rope.freq_base") == 10000.0
    assert m.get("flag") == S.GgufValue("Bool", True) and [v.value for v in m.get("tokenizer.ggml.tokens").value] == ["a", "b"]
    assert m.get_int("general.architecture") is None and m.get_str("nope") is None and m.plain()["llama.block_count"] == 2
    assert torch.equal(S.dequantize_gguf_tensor(f, "w.f32"), torch.from_numpy(w)) and S.dequantize_gguf_tensor(f, "w.f32").shape == (2, 32)
    assert torch.equal(S.dequantize_gguf_tensor(f, "w.q8"), torch.from_numpy(q))
    with pytest.raises(InvalidArgument):
        S.dequantize_gguf_tensor(f, "absent")
    p = tmp_path / "m.gguf"
    p.write_bytes(img)
    for loader in (S.load_gguf_state_dict, S.load_gguf_state_dict_mmap):
        sd = loader(p)
        assert torch.equal(sd["w.f32"], torch.from_numpy(w)) and torch.equal(sd["w.q8"], torch.from_numpy(q))
    old = S.parse_gguf(p)                                      # the path-based reader agrees
    assert torch.equal(old.load_tensor("w.q8"), torch.from_numpy(q))
    for bad in (b"GGML" + img[4:], img[:40], _gguf_image(version=9)[0], img[:-40]):
        with pytest.raises(InvalidArgument):
            g = S.parse_gguf_bytes(bad)
            S.dequantize_gguf_tensor(g, "w.q8")
    with pytest.raises(InvalidArgument):
        S.load_gguf(tmp_path / "missing.gguf")


class _Evil:
    def __reduce__(self):
        import os
        return (os.system, ("echo should-never-run > /dev/null",))


def test_pickle_is_read_as_data():
    v = S.parse_pickle(pickle.dumps({"a": 1, "b": [1.5, None, True, b"xy"], "c": ("t", -7)}, protocol=3))
    assert v.kind == "Dict" and v.get("a") == S.PickleValue("Int", 1) and v.get("c").value[1].value == -7
    assert [x.kind for x in v.get("b").value] == ["Float", "None", "Bool", "Bytes"]
    evil = S.parse_pickle(pickle.dumps(_Evil(), protocol=2))
    assert evil.kind == "Reduce" and evil.value[0].kind == "Global" and evil.value[0].value[1] == "system"       # named, not called
    # a real torch checkpoint: the state dict is an OrderedDict build whose tensors are _rebuild_tensor_v2 reductions over persistent ids
    buf = io.BytesIO()
    torch.save(OrderedDict(w=torch.arange(6.0).view(2, 3), b=torch.zeros(3)), buf)
    raw = zipfile.ZipFile(io.BytesIO(buf.getvalue()))
    data = raw.read([n for n in raw.namelist() if n.endswith("data.pkl")][0])
    tree = S.parse_pickle(data)

    def walk(t, acc):
        if isinstance(t, S.PickleValue):
            acc.append(t)
            walk(t.value, acc)
        elif isinstance(t, (list, tuple)):
            for x in t:
                walk(x, acc)
        return acc
    nodes = walk(tree, [])
    globs = {n.value for n in nodes if n.kind == "Global"}
    assert ("torch._utils", "_rebuild_tensor_v2") in globs and ("collections", "OrderedDict") in globs
    assert sum(n.kind == "PersistentLoad" for n in nodes) == 2 and {n.value for n in nodes if n.kind == "String"} >= {"w", "b", "storage"}
    for bad in (b"", b"\x80\x02}q\x00", b"\x80\x02h\x05."):
        with pytest.raises(InvalidArgument):
            S.parse_pickle(bad)


def test_checkpoint_validation_and_mmap_load(tmp_path):
    sd = {"b.weight": torch.randn(4, 4), "a.bias": torch.arange(4.0)}
    p = tmp_path / "m.pt"
    S.save_pytorch(sd, p)
    S.validate_checkpoint(p)
    back = torch.load(p, weights_only=True)
    assert list(back) == ["a.bias", "b.weight"] and all(torch.equal(back[k], v) for k, v in sd.items())
    mm = S.load_pytorch_state_dict_mmap(p)
    assert all(torch.equal(mm[k], v) for k, v in sd.items())
    raw = bytearray(p.read_bytes())
    needle = sd["b.weight"].numpy().tobytes()[:8]
    at = bytes(raw).find(needle)
    raw[at] ^= 0xFF                                            # flip one stored byte: the entry no longer matches its CRC
    (tmp_path / "bad.pt").write_bytes(bytes(raw))
    with pytest.raises(InvalidArgument):
        S.validate_checkpoint(tmp_path / "bad.pt")
    (tmp_path / "junk.pt").write_bytes(b"not a zip")
    for q in (tmp_path / "junk.pt", tmp_path / "absent.pt"):
        with pytest.raises(InvalidArgument):
            S.validate_checkpoint(q)


# ---- an independent reader + evaluator for the ONNX subset the exporter writes ------------------------------------------------------------------
def _pb(buf):
    i, out = 0, []
    while i < len(buf):
        key = sh = 0
        while True:
            b = buf[i]; i += 1; key |= (b & 0x7F) << sh; sh += 7          # noqa: E702
            if not b & 0x80:
                break
        num, wire = key >> 3, key & 7
        if wire == 0:
            v = sh = 0
            while True:
                b = buf[i]; i += 1; v |= (b & 0x7F) << sh; sh += 7      # noqa: E702
                if not b & 0x80:
                    break
            out.append((num, v))
        elif wire == 2:
            n = sh = 0
            while True:
                b = buf[i]; i += 1; n |= (b & 0x7F) << sh; sh += 7      # noqa: E702
                if not b & 0x80:
                    break
            out.append((num, bytes(buf[i: i + n]))); i += n             # noqa: E702
        elif wire == 5:
            out.append((num, struct.unpack("<f", buf[i: i + 4])[0])); i += 4   # noqa: E702
        else:
            raise AssertionError(wire)
    return out


def _s64(v):
    return v - (1 << 64) if v >= 1 << 63 else v


def _run_onnx(model: bytes, feeds):
    top = _pb(model)
    opset = dict(_pb([v for k, v in top if k == 8][0]))[2]
    g = _pb([v for k, v in top if k == 7][0])
    env = dict(feeds)
    for k, v in g:
        if k == 5:
            f = _pb(v)
            dims = [x for n, x in f if n == 1]
            et = [x for n, x in f if n == 2][0]
            nm = [x for n, x in f if n == 8][0].decode()
            raw = [x for n, x in f if n == 9][0]
            dt = {1: np.float32, 7: np.int64, 11: np.float64, 9: np.bool_}[et]
            env[nm] = torch.from_numpy(np.frombuffer(raw, dtype=dt).reshape(dims).copy())
    names = {"in": [_pb(v)[0][1].decode() for k, v in g if k == 11], "out": [_pb(v)[0][1].decode() for k, v in g if k == 12]}
    F = torch.nn.functional
    for k, v in g:
        if k != 1:
            continue
        f = _pb(v)
        ins, outs, op = [x.decode() for n, x in f if n == 1], [x.decode() for n, x in f if n == 2], [x for n, x in f if n == 4][0].decode()
        at = {}
        for n, x in f:
            if n == 5:
                a = _pb(x)
                an, ty = [y for m, y in a if m == 1][0].decode(), [y for m, y in a if m == 20][0]
                at[an] = {1: lambda: [y for m, y in a if m == 2][0], 2: lambda: _s64([y for m, y in a if m == 3][0]),
                          3: lambda: [y for m, y in a if m == 4][0].decode(), 7: lambda: [_s64(y) for m, y in a if m == 8]}[ty]()
        x = [env[i] for i in ins]
        simple = {"Add": torch.add, "Sub": torch.sub, "Mul": torch.mul, "Div": torch.div, "MatMul": torch.matmul, "Relu": torch.relu, "Sigmoid": torch.sigmoid,
                  "Tanh": torch.tanh, "Exp": torch.exp, "Sqrt": torch.sqrt, "Reciprocal": torch.reciprocal, "Neg": torch.neg, "Identity": lambda t: t,
                  "Erf": torch.erf, "Max": torch.maximum, "Pow": torch.pow, "Where": torch.where}
        if op in simple:
            r = simple[op](*x)
        elif op == "Gemm":
            r = x[0] @ (x[1].t() if at.get("transB") else x[1]) + (x[2] if len(x) > 2 else 0)
        elif op == "Gelu":
            r = F.gelu(x[0], approximate=at.get("approximate", "none"))
        elif op == "Softmax":
            r = torch.softmax(x[0], at["axis"])
        elif op == "Transpose":
            r = x[0].permute(at["perm"])
        elif op == "Reshape":
            r = x[0].reshape(x[1].tolist())
        elif op in ("ReduceSum", "ReduceMean"):
            axes = x[1].tolist() if len(x) > 1 else at["axes"]
            r = (torch.sum if op == "ReduceSum" else torch.mean)(x[0], axes, keepdim=bool(at["keepdims"]))
        elif op == "LayerNormalization":
            nd = -at["axis"]
            r = F.layer_norm(x[0], x[0].shape[-nd:], x[1], x[2] if len(x) > 2 else None, at["epsilon"])
        elif op == "Slice":
            idx = [slice(None)] * x[0].dim()
            idx[int(x[3])] = slice(int(x[1]), min(int(x[2]), x[0].shape[int(x[3])]), int(x[4]))
            r = x[0][tuple(idx)]
        elif op == "Concat":
            r = torch.cat(x, at["axis"])
        elif op == "Unsqueeze":
            r = x[0].unsqueeze(int(x[1][0]))
        elif op == "Expand":
            r = x[0].expand(torch.broadcast_shapes(tuple(x[0].shape), tuple(x[1].tolist())))
        elif op == "Clip":
            r = torch.clamp(x[0], x[1], x[2])
        else:
            raise AssertionError(f"evaluator: {op}")
        env[outs[0]] = r
    return [env[n] for n in names["out"]], names, opset


class _Block(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.ln, self.fc1, self.fc2 = torch.nn.LayerNorm(16), torch.nn.Linear(16, 32), torch.nn.Linear(32, 16)

    def forward(self, x):
        h = self.ln(x)
        a = torch.softmax(h @ h.transpose(-1, -2) / 4.0, -1) @ h
        y = self.fc2(torch.nn.functional.gelu(self.fc1(a))) * torch.sigmoid(a)
        return x + torch.cat([y[..., :8], y[..., 8:].clamp(-0.5, 0.5)], -1), y.pow(2).mean(-1, keepdim=True).rsqrt()


def test_onnx_from_ir_graph_runs_the_same_numbers(tmp_path):
    torch.manual_seed(0)
    m = _Block().eval()
    x = torch.randn(2, 5, 16)
    g = jit.trace(m, (x,))
    want = m(x)
    data = S.ir_graph_to_onnx(g)
    got, names, opset = _run_onnx(data, {"input": x})
    assert opset == 17 and names["in"] == ["input"] and names["out"] == ["output_0", "output_1"]
    for a, b in zip(got, want):
        assert torch.allclose(a, b, atol=1e-5), (a - b).abs().max()
    got64, _, _ = _run_onnx(S.ir_graph_to_onnx(g, S.OnnxExportConfig(opset=18), 11), {"input": x.double()})
    assert got64[0].dtype == torch.float64 and torch.allclose(got64[0].float(), want[0], atol=1e-5)
    S.export_ir_graph_to_onnx(g, tmp_path / "g.onnx")
    assert (tmp_path / "g.onnx").read_bytes() == data
    prog = jit.export(m, (x,))
    S.export_from_program(prog, tmp_path / "p.onnx")
    assert torch.allclose(_run_onnx((tmp_path / "p.onnx").read_bytes(), {"input": x})[0][0], want[0], atol=1e-5)
    with pytest.raises(InvalidArgument):
        S.ir_graph_to_onnx(g, S.OnnxExportConfig(opset=13))
    bad = jit.IrGraph()
    v = bad.add_input((4,), torch.float32)
    bad.set_outputs(bad.add_node("atan2", [v.id, v.id], [((4,), torch.float32)]).outputs)
    with pytest.raises(InvalidArgument, match="no ONNX mapping"):
        S.ir_graph_to_onnx(bad)
