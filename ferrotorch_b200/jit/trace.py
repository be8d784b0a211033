"""Tracer: runs a function eagerly once under a dispatch recorder and builds an :class:`IrGraph` from the primitive ops it executed.

Every tensor the function touches that is neither an argument nor produced inside the trace (module parameters, closed-over
buffers) becomes a graph constant held by reference, so later in-place parameter updates are seen by the compiled graph.
Ops without an IR equivalent are kept as ``opaque`` nodes that re-run the recorded primitive.

Reference parity: ferrotorch-jit/src/trace.rs:1-7,223 (post-hoc walk of the autograd graph; here the recorder sits on the
dispatcher, which also sees ops that do not require grad).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
from torch.utils._python_dispatch import TorchDispatchMode
from torch.utils._pytree import tree_flatten, tree_map, tree_unflatten

from ..errors import InvalidArgument
from .ir import IrGraph, dtype_name

aten = torch.ops.aten

_UNARY = {aten.neg.default: "neg", aten.abs.default: "abs", aten.exp.default: "exp", aten.exp2.default: "exp2", aten.log.default: "log",
          aten.log2.default: "log2", aten.sqrt.default: "sqrt", aten.rsqrt.default: "rsqrt", aten.reciprocal.default: "reciprocal",
          aten.sin.default: "sin", aten.cos.default: "cos", aten.tanh.default: "tanh", aten.sigmoid.default: "sigmoid", aten.relu.default: "relu",
          aten.silu.default: "silu", aten.erf.default: "erf", aten.floor.default: "floor", aten.ceil.default: "ceil", aten.round.default: "round",
          aten.sign.default: "sign", aten.mish.default: "mish", aten.logical_not.default: "logical_not", aten.isnan.default: "isnan"}
_BINARY = {aten.add.Tensor: "add", aten.sub.Tensor: "sub", aten.mul.Tensor: "mul", aten.div.Tensor: "div", aten.pow.Tensor_Tensor: "pow",
           aten.pow.Tensor_Scalar: "pow", aten.maximum.default: "maximum", aten.minimum.default: "minimum", aten.eq.Tensor: "eq", aten.eq.Scalar: "eq",
           aten.ne.Tensor: "ne", aten.ne.Scalar: "ne", aten.lt.Tensor: "lt", aten.lt.Scalar: "lt", aten.le.Tensor: "le", aten.le.Scalar: "le",
           aten.gt.Tensor: "gt", aten.gt.Scalar: "gt", aten.ge.Tensor: "ge", aten.ge.Scalar: "ge", aten.logical_and.default: "logical_and",
           aten.logical_or.default: "logical_or", aten.add.Scalar: "add", aten.sub.Scalar: "sub", aten.mul.Scalar: "mul", aten.div.Scalar: "div",
           aten.fmod.Tensor: "fmod", aten.atan2.default: "atan2"}
_REDUCE = {aten.sum.dim_IntList: "sum", aten.mean.dim: "mean", aten.amax.default: "amax", aten.amin.default: "amin"}
_ALIAS = {aten.detach.default, aten.alias.default, aten.clone.default, aten.contiguous.default if hasattr(aten.contiguous, "default") else None,
          aten.lift_fresh.default, aten.lift_fresh_copy.default if hasattr(aten, "lift_fresh_copy") else None}


class _Recorder(TorchDispatchMode):
    def __init__(self, graph: IrGraph, env: Dict[int, int]):
        super().__init__()
        self.g, self.env = graph, env          # env: id(tensor) -> value id
        self.keep: List[torch.Tensor] = []     # keeps traced tensors alive so ids stay unique
        self.saved: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}      # id(tensor written in place) -> (tensor, its content before the first write)

    # -- helpers
    def vid(self, t: torch.Tensor) -> int:
        k = id(t)
        if k not in self.env:
            self.env[k] = self.g.add_constant(t).id
            self.keep.append(t)
        return self.env[k]

    def scalar(self, x, like: torch.Tensor) -> int:
        dt = like.dtype if like.dtype.is_floating_point or isinstance(x, (bool, int)) and not isinstance(x, float) else torch.get_default_dtype()
        if isinstance(x, float) and not like.dtype.is_floating_point:
            dt = torch.get_default_dtype()
        return self.g.add_constant(torch.tensor(x, dtype=dt, device=like.device)).id

    def bind(self, out, node) -> None:
        outs = out if isinstance(out, (tuple, list)) else [out]
        for t, v in zip([o for o in outs if isinstance(o, torch.Tensor)], node.outputs):
            self.env[id(t)] = v
            self.keep.append(t)

    def emit(self, op, ins, out, **attrs):
        outs = out if isinstance(out, (tuple, list)) else [out]
        specs = [(tuple(o.shape), o.dtype) for o in outs if isinstance(o, torch.Tensor)]
        n = self.g.add_node(op, ins, specs, **attrs)
        self.bind(out, n)
        return n

    # -- dispatch
    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        schema = getattr(func, "_schema", None)
        if schema is not None and (schema.is_mutable or any(a.alias_info is not None and a.alias_info.is_write for a in schema.arguments)) and not any(k in str(func) for k in ("bernoulli_", "uniform_", "normal_", "random_", "exponential_")):
            # An operation that writes into one of its arguments. The graph is a dataflow of values: a write through a view, into an input,
            # or between two reads of the same tensor has no faithful form in it, so the caller runs such a function eagerly.
            self.g.mutations.append(str(func))
            # Tracing must leave no trace: what is about to be overwritten (a module's running statistics, a captured buffer, an input) is
            # kept and put back when the trace ends.
            named = list(zip(args, schema.arguments)) + [(kwargs[spec.name], spec) for spec in schema.arguments if spec.name in kwargs]
            for a, spec in named:
                if isinstance(a, torch.Tensor) and spec.alias_info is not None and spec.alias_info.is_write:
                    base = a._base if a._base is not None else a
                    if id(base) not in self.saved:
                        self.saved[id(base)] = (base, base.clone())
        out = func(*args, **kwargs)
        try:
            self.record(func, args, kwargs, out)
        except _Unsupported:
            self.record_opaque(func, args, kwargs, out)
        return out

    def record_opaque(self, func, args, kwargs, out):
        flat, spec = tree_flatten((args, kwargs))
        ins, slots = [], []
        for i, a in enumerate(flat):
            if isinstance(a, torch.Tensor):
                slots.append(i)
                ins.append(self.vid(a))
        name = str(func)
        if not ins and isinstance(out, torch.Tensor) and not any(k in name for k in ("rand", "normal", "bernoulli", "empty", "multinomial")):
            self.env[id(out)] = self.g.add_constant(out).id       # deterministic factory call (ones, arange, full, ...): a constant
            self.keep.append(out)
            return
        skeleton = [None if isinstance(a, torch.Tensor) else a for a in flat]
        self.emit("opaque", ins, out, func=func, skeleton=skeleton, slots=slots, spec=spec, name=str(func))

    def record(self, func, args, kwargs, out):
        g = self.g
        if func in _ALIAS:
            self.env[id(out)] = self.vid(args[0])
            self.keep.append(out)
            return
        if func in _UNARY:
            self.emit(_UNARY[func], [self.vid(args[0])], out)
            return
        if func in _BINARY:
            a, b = args[0], args[1]
            ta = a if isinstance(a, torch.Tensor) else None
            tb = b if isinstance(b, torch.Tensor) else None
            like = ta if ta is not None else tb
            va = self.vid(a) if ta is not None else self.scalar(a, like)
            vb = self.vid(b) if tb is not None else self.scalar(b, like)
            alpha = kwargs.get("alpha", 1)
            if alpha != 1:
                sc = self.scalar(alpha, like)
                tmp = g.add_node("mul", [vb, sc], [(tuple(torch.broadcast_shapes(tb.shape if tb is not None else (), ())), out.dtype)])
                vb = tmp.outputs[0]
            if func in (aten.div.Tensor,) and kwargs.get("rounding_mode"):
                raise _Unsupported
            self.emit(_BINARY[func], [va, vb], out)
            return
        if func is aten.gelu.default:
            self.emit("gelu_tanh" if kwargs.get("approximate", "none") == "tanh" else "gelu", [self.vid(args[0])], out)
            return
        if func is aten.where.self:
            self.emit("where", [self.vid(args[0]), self.vid(args[1]), self.vid(args[2])], out)
            return
        if func in (aten.clamp.default, aten.hardtanh.default):
            lo = args[1] if len(args) > 1 else kwargs.get("min")
            hi = args[2] if len(args) > 2 else kwargs.get("max")
            x = args[0]
            lo = float("-inf") if lo is None else lo
            hi = float("inf") if hi is None else hi
            self.emit("clamp", [self.vid(x), self.scalar(float(lo), x), self.scalar(float(hi), x)], out)
            return
        if func is aten.addcmul.default:
            v = kwargs.get("value", 1)
            self.emit("addcmul", [self.vid(args[0]), self.vid(args[1]), self.vid(args[2])], out, value=v)
            return
        if func is aten._to_copy.default:
            if kwargs.get("dtype") is None or (kwargs.get("device") is not None and torch.device(kwargs["device"]) != args[0].device):
                raise _Unsupported
            self.emit("cast", [self.vid(args[0])], out, dtype=dtype_name(kwargs["dtype"]))
            return
        if func in _REDUCE:
            dims = args[1] if len(args) > 1 else kwargs.get("dim", [])
            keep = args[2] if len(args) > 2 else kwargs.get("keepdim", False)
            nd = args[0].dim()
            dims = sorted(d % nd for d in (dims if dims else range(nd)))
            self.emit(_REDUCE[func], [self.vid(args[0])], out, dims=tuple(dims), keepdim=bool(keep))
            return
        if func in (aten.sum.default, aten.mean.default):
            self.emit("sum" if func is aten.sum.default else "mean", [self.vid(args[0])], out, dims=tuple(range(args[0].dim())), keepdim=False)
            return
        if func in (aten.view.default, aten._unsafe_view.default, aten.reshape.default):
            self.emit("reshape", [self.vid(args[0])], out, shape=tuple(out.shape))
            return
        if func is aten.permute.default:
            self.emit("permute", [self.vid(args[0])], out, dims=tuple(args[1]))
            return
        if func is aten.transpose.int:
            self.emit("transpose", [self.vid(args[0])], out, d0=args[1], d1=args[2])
            return
        if func is aten.t.default:
            self.emit("transpose", [self.vid(args[0])], out, d0=0, d1=1 if args[0].dim() > 1 else 0)
            return
        if func is aten.expand.default:
            self.emit("expand", [self.vid(args[0])], out, shape=tuple(out.shape))
            return
        if func is aten.unsqueeze.default:
            self.emit("unsqueeze", [self.vid(args[0])], out, dim=args[1])
            return
        if func in (aten.squeeze.dim, aten.squeeze.default, aten.squeeze.dims):
            self.emit("reshape", [self.vid(args[0])], out, shape=tuple(out.shape))
            return
        if func is aten.slice.Tensor:
            dim = args[1] if len(args) > 1 else 0
            start = args[2] if len(args) > 2 else None
            end = args[3] if len(args) > 3 else None
            step = args[4] if len(args) > 4 else 1
            self.emit("slice", [self.vid(args[0])], out, dim=dim, start=start, end=end, step=step)
            return
        if func is aten.select.int:
            self.emit("select", [self.vid(args[0])], out, dim=args[1], index=args[2])
            return
        if func is aten.cat.default:
            self.emit("cat", [self.vid(t) for t in args[0]], out, dim=args[1] if len(args) > 1 else kwargs.get("dim", 0))
            return
        if func is aten.mm.default or func is aten.bmm.default:
            self.emit("matmul", [self.vid(args[0]), self.vid(args[1])], out)
            return
        if func is aten.addmm.default:
            if kwargs.get("beta", 1) != 1 or kwargs.get("alpha", 1) != 1:
                raise _Unsupported
            self.emit("addmm", [self.vid(args[0]), self.vid(args[1]), self.vid(args[2])], out)
            return
        if func is aten._softmax.default:
            self.emit("softmax", [self.vid(args[0])], out, dim=args[1] % args[0].dim())
            return
        if func is aten._log_softmax.default:
            self.emit("log_softmax", [self.vid(args[0])], out, dim=args[1] % args[0].dim())
            return
        if func is aten.embedding.default:
            self.emit("embedding", [self.vid(args[0]), self.vid(args[1])], out)
            return
        if func is aten.native_layer_norm.default:
            x, ns, w, b, eps = args
            ins = [self.vid(x)] + ([self.vid(w)] if w is not None else []) + ([self.vid(b)] if b is not None else [])
            n = self.g.add_node("layer_norm", ins, [(tuple(out[0].shape), out[0].dtype)], normalized=len(ns), eps=eps, has_w=w is not None, has_b=b is not None)
            self.env[id(out[0])] = n.outputs[0]
            self.keep.append(out[0])
            return
        raise _Unsupported


class _Unsupported(Exception):
    pass


def trace(fn: Callable, example_inputs: Sequence[torch.Tensor]) -> IrGraph:
    """Runs ``fn(*example_inputs)`` once and returns the recorded graph. Tensor outputs (a tensor, or a flat tuple/list of tensors)
    become graph outputs."""
    g = IrGraph()
    env: Dict[int, int] = {}
    for t in example_inputs:
        if not isinstance(t, torch.Tensor):
            raise InvalidArgument("trace inputs must be tensors")
        env[id(t)] = g.add_input(t.shape, t.dtype).id
    rec = _Recorder(g, env)
    # Some primitives update an argument without saying so in their signature (batch normalisation and its running statistics), so a
    # module's buffers are kept as a whole.
    buffers = [(b, b.clone()) for b in fn.buffers()] if isinstance(fn, torch.nn.Module) else []
    try:
        with torch.no_grad(), rec:
            out = fn(*example_inputs)
    finally:
        with torch.no_grad():
            for base, before in list(rec.saved.values()) + buffers:
                base.copy_(before)
    outs = [out] if isinstance(out, torch.Tensor) else list(out)
    ids = []
    for o in outs:
        if not isinstance(o, torch.Tensor):
            raise InvalidArgument("traced function must return tensors")
        ids.append(rec.vid(o))
    g.set_outputs(ids)
    g.single_output = isinstance(out, torch.Tensor)
    g.validate()
    return g
