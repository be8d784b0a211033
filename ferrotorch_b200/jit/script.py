"""Graph builder for scripted functions: ``@script`` runs a Python function over symbolic values whose operators append IR nodes,
producing an :class:`IrGraph` without executing any tensor math (the counterpart of the reference's ``#[script]`` macro).

Reference parity: ferrotorch-jit-script/src/lib.rs:1-14.
"""
from __future__ import annotations

from typing import Callable, List, Sequence, Tuple

import torch

from ..errors import InvalidArgument
from .ir import ELEMENTWISE_UNARY, IrGraph, dtype_name, dtype_of


class Value:
    def __init__(self, b: "GraphBuilder", vid: int):
        self.b, self.id = b, vid

    @property
    def shape(self):
        return self.b.g.values[self.id].shape

    @property
    def dtype(self):
        return dtype_of(self.b.g.values[self.id].dtype)

    def _bin(self, o, op, rev=False):
        o = o if isinstance(o, Value) else self.b.constant(o, self.dtype)
        a, c = (o, self) if rev else (self, o)
        return self.b.binary(op, a, c)

    __add__ = lambda s, o: s._bin(o, "add")             # noqa: E731
    __radd__ = lambda s, o: s._bin(o, "add", True)      # noqa: E731
    __sub__ = lambda s, o: s._bin(o, "sub")             # noqa: E731
    __rsub__ = lambda s, o: s._bin(o, "sub", True)      # noqa: E731
    __mul__ = lambda s, o: s._bin(o, "mul")             # noqa: E731
    __rmul__ = lambda s, o: s._bin(o, "mul", True)      # noqa: E731
    __truediv__ = lambda s, o: s._bin(o, "div")         # noqa: E731
    __rtruediv__ = lambda s, o: s._bin(o, "div", True)  # noqa: E731
    __pow__ = lambda s, o: s._bin(o, "pow")             # noqa: E731
    __gt__ = lambda s, o: s._bin(o, "gt")               # noqa: E731
    __lt__ = lambda s, o: s._bin(o, "lt")               # noqa: E731
    __ge__ = lambda s, o: s._bin(o, "ge")               # noqa: E731
    __le__ = lambda s, o: s._bin(o, "le")               # noqa: E731
    __neg__ = lambda s: s.b.unary("neg", s)             # noqa: E731
    __matmul__ = lambda s, o: s.b.matmul(s, o)          # noqa: E731

    def __getattr__(self, name):
        if name in ELEMENTWISE_UNARY and name != "cast":
            return lambda: self.b.unary(name, self)
        raise AttributeError(name)

    def sum(self, dim=None, keepdim=False):
        return self.b.reduce("sum", self, dim, keepdim)

    def mean(self, dim=None, keepdim=False):
        return self.b.reduce("mean", self, dim, keepdim)

    def reshape(self, *shape):
        shape = tuple(shape[0]) if len(shape) == 1 and isinstance(shape[0], (tuple, list)) else tuple(shape)
        n = 1
        for s in self.shape:
            n *= s
        if -1 in shape:
            known = 1
            for s in shape:
                known *= s if s != -1 else 1
            shape = tuple(n // known if s == -1 else s for s in shape)
        return Value(self.b, self.b.g.add_node("reshape", [self.id], [(shape, self.dtype)], shape=shape).outputs[0])

    def transpose(self, d0, d1):
        shp = list(self.shape)
        shp[d0], shp[d1] = shp[d1], shp[d0]
        return Value(self.b, self.b.g.add_node("transpose", [self.id], [(tuple(shp), self.dtype)], d0=d0, d1=d1).outputs[0])

    def softmax(self, dim=-1):
        return Value(self.b, self.b.g.add_node("softmax", [self.id], [(self.shape, self.dtype)], dim=dim % len(self.shape)).outputs[0])

    def to(self, dtype):
        return Value(self.b, self.b.g.add_node("cast", [self.id], [(self.shape, dtype)], dtype=dtype_name(dtype)).outputs[0])


class GraphBuilder:
    def __init__(self):
        self.g = IrGraph()

    def input(self, shape: Sequence[int], dtype=torch.float32) -> Value:
        return Value(self, self.g.add_input(tuple(shape), dtype).id)

    def constant(self, x, dtype=torch.float32) -> Value:
        t = x if isinstance(x, torch.Tensor) else torch.tensor(x, dtype=dtype)
        return Value(self, self.g.add_constant(t).id)

    def unary(self, op: str, a: Value) -> Value:
        return Value(self, self.g.add_node(op, [a.id], [(a.shape, a.dtype)]).outputs[0])

    def binary(self, op: str, a: Value, b: Value) -> Value:
        shape = tuple(torch.broadcast_shapes(tuple(a.shape), tuple(b.shape)))
        dt = torch.bool if op in ("eq", "ne", "lt", "le", "gt", "ge") else torch.promote_types(a.dtype, b.dtype)
        return Value(self, self.g.add_node(op, [a.id, b.id], [(shape, dt)]).outputs[0])

    def where(self, c: Value, a: Value, b: Value) -> Value:
        shape = tuple(torch.broadcast_shapes(tuple(c.shape), tuple(a.shape), tuple(b.shape)))
        return Value(self, self.g.add_node("where", [c.id, a.id, b.id], [(shape, a.dtype)]).outputs[0])

    def matmul(self, a: Value, b: Value) -> Value:
        if a.shape[-1] != b.shape[-2 if len(b.shape) > 1 else 0]:
            raise InvalidArgument(f"matmul shapes {a.shape} x {b.shape}")
        batch = tuple(torch.broadcast_shapes(tuple(a.shape[:-2]), tuple(b.shape[:-2])))
        return Value(self, self.g.add_node("matmul", [a.id, b.id], [(batch + (a.shape[-2], b.shape[-1]), a.dtype)]).outputs[0])

    def reduce(self, op: str, a: Value, dim, keepdim: bool) -> Value:
        nd = len(a.shape)
        dims = tuple(range(nd)) if dim is None else tuple(sorted(d % nd for d in ([dim] if isinstance(dim, int) else dim)))
        shape = tuple((1 if i in dims else s) for i, s in enumerate(a.shape) if keepdim or i not in dims)
        return Value(self, self.g.add_node(op, [a.id], [(shape, a.dtype)], dims=dims, keepdim=keepdim).outputs[0])

    def finish(self, outs) -> IrGraph:
        outs = [outs] if isinstance(outs, Value) else list(outs)
        self.g.set_outputs([o.id for o in outs])
        self.g.single_output = len(outs) == 1
        self.g.validate()
        return self.g


def script(*input_specs: Tuple[Sequence[int], torch.dtype]) -> Callable[[Callable], "ScriptedFunction"]:
    """``@script(((4, 8), torch.float32), ...)``: the decorated function receives one :class:`Value` per spec (plus the builder as the
    keyword ``builder`` if it declares it) and returns Values; the result is a callable backed by the built graph."""
    def deco(fn: Callable) -> "ScriptedFunction":
        b = GraphBuilder()
        vals = [b.input(s, dt) for s, dt in input_specs]
        import inspect
        kw = {"builder": b} if "builder" in inspect.signature(fn).parameters else {}
        return ScriptedFunction(b.finish(fn(*vals, **kw)), fn.__name__)
    return deco


class ScriptedFunction:
    def __init__(self, graph: IrGraph, name: str = "scripted"):
        self.graph, self.name = graph, name

    def __call__(self, *inputs):
        from .interpreter import Interpreter
        return Interpreter(self.graph)(*inputs)
