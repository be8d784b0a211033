"""Reference interpreter: evaluates an :class:`IrGraph` node by node with eager tensor ops. It is the semantic oracle for the
optimisation passes and the code generators, and the fallback executor for graphs (or segments) that are not compiled.

Reference parity: ferrotorch-jit/src/interpreter.rs:71-154.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch
import torch.nn.functional as F
from torch.utils._pytree import tree_unflatten

from ..errors import InvalidArgument
from .ir import IrGraph, IrNode, dtype_of

_U = {"neg": torch.neg, "abs": torch.abs, "exp": torch.exp, "exp2": torch.exp2, "log": torch.log, "log2": torch.log2, "sqrt": torch.sqrt,
      "rsqrt": torch.rsqrt, "reciprocal": torch.reciprocal, "sin": torch.sin, "cos": torch.cos, "tanh": torch.tanh, "sigmoid": torch.sigmoid,
      "relu": torch.relu, "gelu": F.gelu, "gelu_tanh": lambda x: F.gelu(x, approximate="tanh"), "silu": F.silu, "erf": torch.erf,
      "floor": torch.floor, "ceil": torch.ceil, "round": torch.round, "sign": torch.sign, "square": torch.square, "softplus": F.softplus,
      "mish": F.mish, "logical_not": torch.logical_not, "isnan": torch.isnan}
_B = {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div, "pow": torch.pow, "maximum": torch.maximum, "minimum": torch.minimum,
      "eq": torch.eq, "ne": torch.ne, "lt": torch.lt, "le": torch.le, "gt": torch.gt, "ge": torch.ge, "logical_and": torch.logical_and,
      "logical_or": torch.logical_or, "fmod": torch.fmod, "atan2": torch.atan2}


def eval_node(n: IrNode, ins: List[torch.Tensor], g: IrGraph):
    op, a = n.op, n.attrs
    if op in _U:
        return _U[op](ins[0])
    if op in _B:
        return _B[op](ins[0], ins[1])
    if op == "cast":
        return ins[0].to(dtype_of(a["dtype"]))
    if op == "where":
        return torch.where(ins[0], ins[1], ins[2])
    if op == "clamp":
        return torch.clamp(ins[0], ins[1], ins[2])
    if op == "addcmul":
        return torch.addcmul(ins[0], ins[1], ins[2], value=a.get("value", 1))
    if op == "addcdiv":
        return torch.addcdiv(ins[0], ins[1], ins[2], value=a.get("value", 1))
    if op == "lerp":
        return torch.lerp(ins[0], ins[1], ins[2])
    if op in ("sum", "mean", "amax", "amin", "prod", "var", "logsumexp"):
        dims, keep = list(a["dims"]), a.get("keepdim", False)
        if op == "prod":
            out = ins[0]
            for d in sorted(dims, reverse=True):
                out = out.prod(d, keepdim=keep)
            return out
        return getattr(torch, op)(ins[0], dims, keepdim=keep)
    if op in ("argmax", "argmin"):
        return getattr(torch, op)(ins[0], a["dim"], a.get("keepdim", False))
    if op == "reshape":
        return ins[0].reshape(a["shape"])
    if op == "flatten":
        return ins[0].flatten(a.get("start", 0), a.get("end", -1))
    if op == "permute":
        return ins[0].permute(a["dims"])
    if op == "transpose":
        return ins[0].transpose(a["d0"], a["d1"])
    if op == "expand":
        return ins[0].expand(a["shape"])
    if op == "unsqueeze":
        return ins[0].unsqueeze(a["dim"])
    if op == "squeeze":
        return ins[0].squeeze(a["dim"])
    if op == "contiguous":
        return ins[0].contiguous()
    if op == "slice":
        idx = [slice(None)] * ins[0].dim()
        idx[a["dim"]] = slice(a.get("start"), a.get("end"), a.get("step", 1))
        return ins[0][tuple(idx)]
    if op == "select":
        return ins[0].select(a["dim"], a["index"])
    if op == "cat":
        return torch.cat(ins, a["dim"])
    if op == "stack":
        return torch.stack(ins, a["dim"])
    if op == "index_select":
        return ins[0].index_select(a["dim"], ins[1])
    if op == "gather":
        return ins[0].gather(a["dim"], ins[1])
    if op in ("matmul", "bmm"):
        return torch.matmul(ins[0], ins[1])
    if op == "addmm":
        return torch.addmm(ins[0], ins[1], ins[2])
    if op == "linear":
        return F.linear(ins[0], ins[1], ins[2] if len(ins) > 2 else None)
    if op == "conv2d":
        return F.conv2d(ins[0], ins[1], ins[2] if len(ins) > 2 else None, a.get("stride", 1), a.get("padding", 0), a.get("dilation", 1), a.get("groups", 1))
    if op == "embedding":
        return F.embedding(ins[1], ins[0])
    if op == "softmax":
        return torch.softmax(ins[0], a["dim"])
    if op == "log_softmax":
        return torch.log_softmax(ins[0], a["dim"])
    if op == "layer_norm":
        x = ins[0]
        w = ins[1] if a.get("has_w") else None
        b = ins[1 + bool(a.get("has_w"))] if a.get("has_b") else None
        return F.layer_norm(x, x.shape[x.dim() - a["normalized"]:], w, b, a["eps"])
    if op == "rms_norm":
        x = ins[0].float()
        y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + a["eps"])
        return (y * ins[1].float()).to(ins[0].dtype) if len(ins) > 1 else y.to(ins[0].dtype)
    if op == "dropout":
        return ins[0]                                   # traced graphs are inference graphs
    if op == "fused":
        return run_graph(a["body"], ins)
    if op == "fused_reduce":
        outs = run_graph(a["body"], ins)
        red = getattr(torch, a["red_op"])(outs[a["red_index"]], [-1], keepdim=a["keepdim"])
        return [red] + [o for i, o in enumerate(outs) if i != a["red_index"]]
    if op == "opaque":
        flat = list(a["skeleton"])
        for slot, t in zip(a["slots"], ins):
            flat[slot] = t
        args, kwargs = tree_unflatten(flat, a["spec"])
        return a["func"](*args, **kwargs)
    raise InvalidArgument(f"interpreter: unsupported op {op}")


def run_graph(g: IrGraph, inputs: Sequence[torch.Tensor]):
    if len(inputs) != len(g.inputs):
        raise InvalidArgument(f"graph takes {len(g.inputs)} inputs, got {len(inputs)}")
    env: Dict[int, torch.Tensor] = dict(g.constants)
    for vid, t in zip(g.inputs, inputs):
        env[vid] = t
    for n in g.topo_order():
        out = eval_node(n, [env[i] for i in n.inputs], g)
        outs = out if isinstance(out, (tuple, list)) else [out]
        for vid, t in zip(n.outputs, [o for o in outs if isinstance(o, torch.Tensor)]):
            env[vid] = t
    res = [env[o] for o in g.outputs]
    return res


class Interpreter:
    def __init__(self, graph: IrGraph):
        graph.validate()
        self.graph = graph

    def __call__(self, *inputs):
        out = run_graph(self.graph, inputs)
        return out[0] if getattr(self.graph, "single_output", len(out) == 1) else tuple(out)
