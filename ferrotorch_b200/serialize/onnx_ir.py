"""ONNX export of a traced IR graph (``ferrotorch_b200.jit.IrGraph``) and of an exported program.

The writer emits ModelProto bytes directly (field numbers of onnx.proto3) with opset >= 17: one ONNX node per IR node for the operators that
have a direct counterpart, small fixed expansions for the rest (``silu`` = x * Sigmoid(x), ``rsqrt`` = Reciprocal(Sqrt(x)), ``square``,
``addcmul`` ...), constants as initializers, symbolic dimensions as ``dim_param``. An IR operator outside the table is an
:class:`InvalidArgument` naming it, never a silently wrong graph.

Reference parity: ferrotorch-serialize/src/onnx_export.rs:743 (ir_graph_to_onnx), :1107 (export_ir_graph_to_onnx), :1165 (export_from_program).
"""
from __future__ import annotations

import struct
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from ..errors import InvalidArgument
from .formats import OnnxExportConfig, _attr_float, _attr_int, _field, _ld, _node, _varint, _vi

# TensorProto.DataType
ELEM_FLOAT, ELEM_UINT8, ELEM_INT8, ELEM_INT16, ELEM_INT32, ELEM_INT64, ELEM_BOOL, ELEM_FLOAT16, ELEM_DOUBLE, ELEM_BFLOAT16 = 1, 2, 3, 5, 6, 7, 9, 10, 11, 16
_ELEM = {"f32": ELEM_FLOAT, "f64": ELEM_DOUBLE, "f16": ELEM_FLOAT16, "bf16": ELEM_BFLOAT16, "i64": ELEM_INT64, "i32": ELEM_INT32, "i16": ELEM_INT16,
         "i8": ELEM_INT8, "u8": ELEM_UINT8, "bool": ELEM_BOOL}
_NP = {ELEM_FLOAT: np.float32, ELEM_DOUBLE: np.float64, ELEM_FLOAT16: np.float16, ELEM_INT64: np.int64, ELEM_INT32: np.int32, ELEM_INT16: np.int16,
       ELEM_INT8: np.int8, ELEM_UINT8: np.uint8, ELEM_BOOL: np.bool_}

_UNARY = {"neg": "Neg", "abs": "Abs", "exp": "Exp", "log": "Log", "sqrt": "Sqrt", "reciprocal": "Reciprocal", "sin": "Sin", "cos": "Cos", "tanh": "Tanh",
          "sigmoid": "Sigmoid", "relu": "Relu", "erf": "Erf", "floor": "Floor", "ceil": "Ceil", "round": "Round", "sign": "Sign", "softplus": "Softplus",
          "mish": "Mish", "logical_not": "Not", "isnan": "IsNaN", "contiguous": "Identity", "dropout": "Identity"}
_BINARY = {"add": "Add", "sub": "Sub", "mul": "Mul", "div": "Div", "pow": "Pow", "maximum": "Max", "minimum": "Min", "eq": "Equal", "lt": "Less",
           "le": "LessOrEqual", "gt": "Greater", "ge": "GreaterOrEqual", "logical_and": "And", "logical_or": "Or", "matmul": "MatMul", "bmm": "MatMul"}
_REDUCE = {"sum": "ReduceSum", "mean": "ReduceMean", "amax": "ReduceMax", "amin": "ReduceMin", "prod": "ReduceProd", "logsumexp": "ReduceLogSumExp"}


def _attr_ints(name: str, vs: Sequence[int]) -> bytes:
    return _ld(5, _ld(1, name.encode()) + b"".join(_vi(8, v & 0xFFFFFFFFFFFFFFFF) for v in vs) + _vi(20, 7))


def _attr_str(name: str, v: str) -> bytes:
    return _ld(5, _ld(1, name.encode()) + _ld(4, v.encode()) + _vi(20, 3))


def _sint(v: int) -> int:
    return v & 0xFFFFFFFFFFFFFFFF                            # protobuf int64 varints are two's complement


def _tensor(name: str, t: torch.Tensor, elem: Optional[int] = None) -> bytes:
    t = t.detach().cpu().contiguous()
    if elem is None:
        elem = {torch.float32: ELEM_FLOAT, torch.float64: ELEM_DOUBLE, torch.float16: ELEM_FLOAT16, torch.bfloat16: ELEM_BFLOAT16, torch.int64: ELEM_INT64,
                torch.int32: ELEM_INT32, torch.int16: ELEM_INT16, torch.int8: ELEM_INT8, torch.uint8: ELEM_UINT8, torch.bool: ELEM_BOOL}[t.dtype]
    if elem == ELEM_BFLOAT16:
        raw = t.to(torch.bfloat16).view(torch.int16).numpy().tobytes()
    else:
        raw = t.numpy().astype(_NP[elem], copy=False).tobytes()
    return b"".join(_vi(1, d) for d in t.shape) + _vi(2, elem) + _ld(8, name.encode()) + _ld(9, raw)


def _value_info(name: str, shape, elem: int) -> bytes:
    dims = b"".join(_ld(1, _vi(1, d) if isinstance(d, int) else _ld(2, str(d).encode())) for d in shape)
    return _ld(1, name.encode()) + _ld(2, _ld(1, _vi(1, elem) + _ld(2, dims)))


def ir_graph_to_onnx(graph, config: Optional[OnnxExportConfig] = None, elem_type: int = ELEM_FLOAT) -> bytes:
    """ModelProto bytes for ``graph``. Floating constants and graph inputs / outputs are written as ``elem_type`` (``ELEM_FLOAT`` or
    ``ELEM_DOUBLE``, as in the reference); integer and boolean values keep their type."""
    cfg = config or OnnxExportConfig()
    if cfg.opset < 17:
        raise InvalidArgument(f"ONNX opset version must be >= 17, got {cfg.opset}")
    if elem_type not in (ELEM_FLOAT, ELEM_DOUBLE, ELEM_FLOAT16, ELEM_BFLOAT16):
        raise InvalidArgument(f"elem_type must be a floating TensorProto type, got {elem_type}")
    graph.validate()
    name: Dict[int, str] = {}
    for i, v in enumerate(graph.inputs):
        name[v] = cfg.input_name if len(graph.inputs) == 1 else f"{cfg.input_name}_{i}"
    nodes: List[bytes] = []
    inits: List[bytes] = []
    counter = [0]

    def elem_of(vid: int) -> int:
        dt = graph.values[vid].dtype
        return elem_type if dt in ("f32", "f64", "f16", "bf16") else _ELEM[dt]

    def fresh(prefix: str) -> str:
        counter[0] += 1
        return f"{prefix}_{counter[0]}"

    def const(t: torch.Tensor, prefix: str = "c") -> str:
        n = fresh(prefix)
        inits.append(_tensor(n, t, elem_type if t.is_floating_point() else None))
        return n

    def i64(vals: Sequence[int]) -> str:
        return const(torch.tensor(list(vals), dtype=torch.int64), "shape")

    def scalar_like(vid: int, x: float) -> str:
        return const(torch.tensor(x, dtype=torch.float64 if elem_of(vid) == ELEM_DOUBLE else torch.float32), "k")

    def emit(op: str, ins: Sequence[str], outs: Sequence[str], attrs: bytes = b"") -> None:
        nodes.append(_node(op, ins, outs, attrs, fresh(op.lower())))

    for vid, t in graph.constants.items():
        name[vid] = f"const_{vid}"
        inits.append(_tensor(name[vid], t, elem_type if t.is_floating_point() else None))

    for n in graph.topo_order():
        op, a = n.op, n.attrs
        if op in ("input", "constant", "output"):
            continue
        ins = [name[i] for i in n.inputs]
        outs = [f"v{o}" for o in n.outputs]
        for o, nm in zip(n.outputs, outs):
            name[o] = nm
        o0 = outs[0]
        rank = len(graph.values[n.inputs[0]].shape) if n.inputs else 0
        if op in _UNARY:
            emit(_UNARY[op], ins[:1], outs)
        elif op in _BINARY:
            emit(_BINARY[op], ins, outs)
        elif op == "ne":
            t = fresh("eq")
            emit("Equal", ins, [t])
            emit("Not", [t], outs)
        elif op == "gelu":
            emit("Gelu", ins, outs, _attr_str("approximate", "none"))
        elif op == "gelu_tanh":
            emit("Gelu", ins, outs, _attr_str("approximate", "tanh"))
        elif op == "silu":
            t = fresh("sig")
            emit("Sigmoid", ins, [t])
            emit("Mul", [ins[0], t], outs)
        elif op == "rsqrt":
            t = fresh("sqrt")
            emit("Sqrt", ins, [t])
            emit("Reciprocal", [t], outs)
        elif op == "square":
            emit("Mul", [ins[0], ins[0]], outs)
        elif op in ("exp2", "log2"):
            k = scalar_like(n.inputs[0], 0.6931471805599453)
            t = fresh("t")
            if op == "exp2":
                emit("Mul", [ins[0], k], [t])
                emit("Exp", [t], outs)
            else:
                emit("Log", ins, [t])
                emit("Div", [t, k], outs)
        elif op == "fmod":
            emit("Mod", ins, outs, _attr_int("fmod", 1))
        elif op == "cast":
            emit("Cast", ins, outs, _attr_int("to", elem_of(n.outputs[0])))
        elif op == "where":
            emit("Where", ins, outs)
        elif op == "clamp":
            emit("Clip", ins, outs)
        elif op in ("addcmul", "addcdiv"):
            t, u = fresh("t"), fresh("u")
            emit("Mul" if op == "addcmul" else "Div", ins[1:3], [t])
            emit("Mul", [t, scalar_like(n.inputs[0], float(a.get("value", 1)))], [u])
            emit("Add", [ins[0], u], outs)
        elif op == "lerp":
            t, u = fresh("t"), fresh("u")
            emit("Sub", [ins[1], ins[0]], [t])
            emit("Mul", [t, ins[2]], [u])
            emit("Add", [ins[0], u], outs)
        elif op in _REDUCE:
            dims, keep = [int(d) for d in a["dims"]], int(bool(a.get("keepdim", False)))
            if op == "sum" or cfg.opset >= 18:
                emit(_REDUCE[op], [ins[0], i64(dims)], outs, _attr_int("keepdims", keep))
            else:
                emit(_REDUCE[op], ins[:1], outs, _attr_ints("axes", dims) + _attr_int("keepdims", keep))
        elif op in ("argmax", "argmin"):
            emit("ArgMax" if op == "argmax" else "ArgMin", ins, outs, _attr_int("axis", _sint(int(a["dim"]))) + _attr_int("keepdims", int(bool(a.get("keepdim", False)))))
        elif op in ("reshape", "expand"):
            if op == "reshape":
                emit("Reshape", [ins[0], i64([int(s) if isinstance(s, int) else -1 for s in a["shape"]])], outs)
            else:                                            # Expand broadcasts both ways: 1 keeps a (symbolic) input dimension as it is
                emit("Expand", [ins[0], i64([int(s) if isinstance(s, int) else 1 for s in graph.values[n.outputs[0]].shape])], outs)
        elif op == "flatten":
            shp = [int(s) if isinstance(s, int) else -1 for s in graph.values[n.outputs[0]].shape]
            emit("Reshape", [ins[0], i64(shp)], outs)
        elif op == "permute":
            emit("Transpose", ins, outs, _attr_ints("perm", [int(d) % rank for d in a["dims"]]))
        elif op == "transpose":
            perm = list(range(rank))
            d0, d1 = int(a["d0"]) % rank, int(a["d1"]) % rank
            perm[d0], perm[d1] = perm[d1], perm[d0]
            emit("Transpose", ins, outs, _attr_ints("perm", perm))
        elif op in ("unsqueeze", "squeeze"):
            emit("Unsqueeze" if op == "unsqueeze" else "Squeeze", [ins[0], i64([int(a["dim"])])], outs)
        elif op == "slice":
            start = 0 if a.get("start") is None else int(a["start"])
            end = (1 << 62) if a.get("end") is None else int(a["end"])
            emit("Slice", [ins[0], i64([start]), i64([end]), i64([int(a["dim"])]), i64([int(a.get("step", 1))])], outs)
        elif op == "select":
            emit("Gather", [ins[0], const(torch.tensor(int(a["index"]), dtype=torch.int64), "idx")], outs, _attr_int("axis", _sint(int(a["dim"]))))
        elif op == "index_select":
            emit("Gather", ins, outs, _attr_int("axis", _sint(int(a["dim"]))))
        elif op == "gather":
            emit("GatherElements", ins, outs, _attr_int("axis", _sint(int(a["dim"]))))
        elif op == "embedding":
            emit("Gather", ins, outs, _attr_int("axis", 0))
        elif op == "cat":
            emit("Concat", ins, outs, _attr_int("axis", _sint(int(a["dim"]))))
        elif op == "stack":
            us = []
            for x in ins:
                u = fresh("u")
                emit("Unsqueeze", [x, i64([int(a["dim"])])], [u])
                us.append(u)
            emit("Concat", us, outs, _attr_int("axis", _sint(int(a["dim"]))))
        elif op == "linear":
            if rank == 2:
                emit("Gemm", ins, outs, _attr_int("transB", 1))
            else:
                wt, mm = fresh("wt"), (fresh("mm") if len(ins) > 2 else o0)
                emit("Transpose", [ins[1]], [wt], _attr_ints("perm", [1, 0]))
                emit("MatMul", [ins[0], wt], [mm])
                if len(ins) > 2:
                    emit("Add", [mm, ins[2]], outs)
        elif op == "addmm":
            emit("Gemm", [ins[1], ins[2], ins[0]], outs)
        elif op == "conv2d":
            pair = lambda v: [int(v), int(v)] if isinstance(v, int) else [int(x) for x in v]  # noqa: E731
            p = pair(a.get("padding", 0))
            emit("Conv", ins, outs, _attr_ints("strides", pair(a.get("stride", 1))) + _attr_ints("pads", p + p) + _attr_ints("dilations", pair(a.get("dilation", 1)))
                 + _attr_int("group", int(a.get("groups", 1))))
        elif op in ("softmax", "log_softmax"):
            emit("Softmax" if op == "softmax" else "LogSoftmax", ins, outs, _attr_int("axis", _sint(int(a["dim"]))))
        elif op == "layer_norm":
            norm = int(a["normalized"])
            shape = [int(s) for s in graph.values[n.inputs[0]].shape[rank - norm:]]
            w = ins[1] if a.get("has_w") else const(torch.ones(shape), "lnw")
            extra = [ins[1 + bool(a.get("has_w"))]] if a.get("has_b") else []
            emit("LayerNormalization", [ins[0], w] + extra, outs, _attr_int("axis", _sint(-norm)) + _attr_float("epsilon", float(a["eps"])))
        elif op == "rms_norm":
            sq, ms, ad, rs, y = (fresh(p) for p in ("sq", "ms", "ad", "rs", "y"))
            emit("Mul", [ins[0], ins[0]], [sq])
            if cfg.opset >= 18:
                emit("ReduceMean", [sq, i64([-1])], [ms], _attr_int("keepdims", 1))
            else:
                emit("ReduceMean", [sq], [ms], _attr_ints("axes", [-1]) + _attr_int("keepdims", 1))
            emit("Add", [ms, scalar_like(n.inputs[0], float(a["eps"]))], [ad])
            emit("Sqrt", [ad], [rs])
            emit("Div", [ins[0], rs], [y if len(ins) > 1 else o0])
            if len(ins) > 1:
                emit("Mul", [y, ins[1]], outs)
        else:
            raise InvalidArgument(f"ONNX export: IR operator '{op}' has no ONNX mapping (run the graph without fusion passes, or extend the table)")

    out_names = []
    for i, v in enumerate(graph.outputs):
        nm = cfg.output_name if len(graph.outputs) == 1 else f"{cfg.output_name}_{i}"
        emit("Identity", [name[v]], [nm])
        out_names.append(nm)
    g = b"".join(_ld(1, x) for x in nodes) + _ld(2, b"main") + b"".join(_ld(5, x) for x in inits)
    g += b"".join(_ld(11, _value_info(name[v], graph.values[v].shape, elem_of(v))) for v in graph.inputs)
    g += b"".join(_ld(12, _value_info(nm, graph.values[v].shape, elem_of(v))) for nm, v in zip(out_names, graph.outputs))
    return _vi(1, 8) + _ld(2, cfg.producer.encode()) + _ld(7, g) + _ld(8, _ld(1, b"") + _vi(2, cfg.opset))


def export_ir_graph_to_onnx(graph, path, config: Optional[OnnxExportConfig] = None, elem_type: int = ELEM_FLOAT) -> None:
    data = ir_graph_to_onnx(graph, config, elem_type)
    try:
        Path(path).write_bytes(data)
    except OSError as e:
        raise InvalidArgument(f"failed to write ONNX file {path}: {e}") from None


def export_from_program(program, path, config: Optional[OnnxExportConfig] = None) -> None:
    """An exported program's graph with its recorded input shapes; the element type follows the program's first floating input."""
    dts = [dt for _, dt in getattr(program, "input_specs", [])]
    elem = ELEM_DOUBLE if "f64" in dts and "f32" not in dts else ELEM_FLOAT
    export_ir_graph_to_onnx(program.graph, path, config, elem)
