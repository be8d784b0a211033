"""Graph IR of the tracing JIT: typed values, op nodes, topological order, structural fingerprint and JSON serialisation.

Reference parity: ferrotorch-jit/src/{graph.rs:14-674 (IrOpKind, IrGraph, fingerprint, topo order), serialize.rs:431-491}.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ..errors import InvalidArgument

# op name -> (arity or None for variadic, kind)
ELEMENTWISE_UNARY = {"neg", "abs", "exp", "exp2", "log", "log2", "sqrt", "rsqrt", "reciprocal", "sin", "cos", "tanh", "sigmoid", "relu", "gelu",
                     "gelu_tanh", "silu", "erf", "floor", "ceil", "round", "sign", "square", "softplus", "mish", "logical_not", "isnan", "cast"}
ELEMENTWISE_BINARY = {"add", "sub", "mul", "div", "pow", "maximum", "minimum", "eq", "ne", "lt", "le", "gt", "ge", "logical_and", "logical_or",
                      "fmod", "atan2"}
ELEMENTWISE_TERNARY = {"where", "clamp", "addcmul", "addcdiv", "lerp"}
ELEMENTWISE = ELEMENTWISE_UNARY | ELEMENTWISE_BINARY | ELEMENTWISE_TERNARY
REDUCTIONS = {"sum", "mean", "amax", "amin", "prod", "argmax", "argmin", "var", "logsumexp"}
SHAPE_OPS = {"reshape", "permute", "transpose", "expand", "squeeze", "unsqueeze", "slice", "select", "cat", "stack", "contiguous", "flatten", "index_select",
             "gather", "split_item"}
CONTRACTIONS = {"matmul", "linear", "bmm", "addmm", "conv2d", "embedding"}
COMPOSITE = {"softmax", "log_softmax", "layer_norm", "rms_norm", "dropout", "cross_entropy", "attention", "fused", "fused_reduce"}
ALL_OPS = ELEMENTWISE | REDUCTIONS | SHAPE_OPS | CONTRACTIONS | COMPOSITE | {"input", "constant", "output", "opaque"}

_DT = {"f32": torch.float32, "f64": torch.float64, "bf16": torch.bfloat16, "f16": torch.float16, "i64": torch.int64, "i32": torch.int32, "bool": torch.bool,
       "u8": torch.uint8, "i8": torch.int8, "i16": torch.int16}
_DT_INV = {v: k for k, v in _DT.items()}


def dtype_name(dt: torch.dtype) -> str:
    return _DT_INV[dt]


def dtype_of(name: str) -> torch.dtype:
    return _DT[name]


@dataclass
class IrValue:
    id: int
    shape: Tuple[Any, ...]            # ints or symbolic dim names (str)
    dtype: str
    producer: Optional[int] = None    # node id

    def numel(self) -> int:
        n = 1
        for s in self.shape:
            if not isinstance(s, int):
                raise InvalidArgument("symbolic shape has no concrete numel")
            n *= s
        return n


@dataclass
class IrNode:
    id: int
    op: str
    inputs: List[int]                 # value ids
    outputs: List[int]                # value ids
    attrs: Dict[str, Any] = field(default_factory=dict)


class IrGraph:
    def __init__(self):
        self.mutations: List[str] = []          # in-place operations seen while tracing (names); a non-empty list sends the caller to eager execution
        self.values: Dict[int, IrValue] = {}
        self.nodes: Dict[int, IrNode] = {}
        self.inputs: List[int] = []
        self.outputs: List[int] = []
        self.constants: Dict[int, torch.Tensor] = {}
        self._next_v = 0
        self._next_n = 0

    # ---- construction
    def new_value(self, shape, dtype, producer=None) -> IrValue:
        dt = dtype if isinstance(dtype, str) else dtype_name(dtype)
        v = IrValue(self._next_v, tuple(shape), dt, producer)
        self.values[v.id] = v
        self._next_v += 1
        return v

    def add_input(self, shape, dtype) -> IrValue:
        v = self.new_value(shape, dtype)
        self.inputs.append(v.id)
        return v

    def add_constant(self, t: torch.Tensor) -> IrValue:
        v = self.new_value(t.shape, t.dtype)
        # A trainable leaf (a module's parameter) is kept as it is, so that a compiled module can be trained: gradients reach it through the
        # eagerly evaluated nodes and through the recompute backward of the generated kernels. Anything else is cut from its history.
        self.constants[v.id] = t if (t.requires_grad and t.is_leaf) else t.detach()
        return v

    def add_node(self, op: str, inputs: Sequence[int], out_specs: Sequence[Tuple[Sequence[int], Any]], **attrs) -> IrNode:
        if op not in ALL_OPS:
            raise InvalidArgument(f"unknown IR op {op}")
        n = IrNode(self._next_n, op, list(inputs), [], dict(attrs))
        self._next_n += 1
        for shape, dt in out_specs:
            n.outputs.append(self.new_value(shape, dt, n.id).id)
        self.nodes[n.id] = n
        return n

    def set_outputs(self, ids: Sequence[int]) -> None:
        self.outputs = list(ids)

    # ---- queries
    def users(self) -> Dict[int, List[int]]:
        u: Dict[int, List[int]] = {v: [] for v in self.values}
        for n in self.nodes.values():
            for i in n.inputs:
                u[i].append(n.id)
        return u

    def topo_order(self) -> List[IrNode]:
        """Kahn's algorithm over value dependencies; node ids break ties so the order is deterministic."""
        indeg = {nid: 0 for nid in self.nodes}
        prod = {v.id: v.producer for v in self.values.values()}
        succ: Dict[int, List[int]] = {nid: [] for nid in self.nodes}
        for n in self.nodes.values():
            for i in set(n.inputs):
                p = prod.get(i)
                if p is not None and p in self.nodes:
                    indeg[n.id] += 1
                    succ[p].append(n.id)
        import heapq
        ready = [nid for nid, d in indeg.items() if d == 0]
        heapq.heapify(ready)
        order = []
        while ready:
            nid = heapq.heappop(ready)
            order.append(self.nodes[nid])
            for s in succ[nid]:
                indeg[s] -= 1
                if indeg[s] == 0:
                    heapq.heappush(ready, s)
        if len(order) != len(self.nodes):
            raise InvalidArgument("IR graph has a cycle")
        return order

    def fingerprint(self) -> str:
        """Structural hash: op kinds, attributes, shapes, dtypes and wiring, independent of value numbering."""
        ren: Dict[int, int] = {}
        for i in self.inputs:
            ren[i] = len(ren)
        h = hashlib.sha256()
        for i in self.inputs:
            v = self.values[i]
            h.update(f"in:{v.shape}:{v.dtype};".encode())
        for n in self.topo_order():
            ins = []
            for i in n.inputs:
                if i in self.constants and i not in ren:
                    c = self.constants[i]
                    ren[i] = len(ren)
                    # small constants are part of the structure (literals); large ones (weights) are identified by shape and dtype only
                    data = hashlib.sha256(c.detach().contiguous().cpu().reshape(-1).view(torch.uint8).numpy().tobytes()).hexdigest()[:16] if c.numel() <= 4096 else "ref"
                    h.update(f"c:{tuple(c.shape)}:{c.dtype}:{data};".encode())
                ins.append(ren[i])
            for o in n.outputs:
                ren[o] = len(ren)
            outs = [(self.values[o].shape, self.values[o].dtype) for o in n.outputs]
            h.update(f"{n.op}:{ins}:{sorted((k, str(v)) for k, v in n.attrs.items() if k != 'body')}:{outs};".encode())
            if "body" in n.attrs:
                h.update(n.attrs["body"].fingerprint().encode())
        h.update(f"out:{[ren.get(o, -1) for o in self.outputs]}".encode())
        return h.hexdigest()

    def validate(self) -> None:
        defined = set(self.inputs) | set(self.constants)
        for n in self.topo_order():
            for i in n.inputs:
                if i not in defined:
                    raise InvalidArgument(f"node {n.id} ({n.op}) reads undefined value {i}")
            defined.update(n.outputs)
        for o in self.outputs:
            if o not in defined:
                raise InvalidArgument(f"graph output {o} is undefined")

    def node_count(self, op: Optional[str] = None) -> int:
        return sum(1 for n in self.nodes.values() if op is None or n.op == op)

    # ---- (de)serialisation
    def to_json(self) -> str:
        def enc_attr(v):
            if isinstance(v, IrGraph):
                return {"__graph__": json.loads(v.to_json())}
            if isinstance(v, torch.dtype):
                return {"__dtype__": dtype_name(v)}
            if isinstance(v, (tuple, list)):
                return [enc_attr(x) for x in v]
            return v
        d = {"version": 1, "inputs": self.inputs, "outputs": self.outputs,
             "values": [[v.id, list(v.shape), v.dtype, v.producer] for v in self.values.values()],
             "nodes": [[n.id, n.op, n.inputs, n.outputs, {k: enc_attr(v) for k, v in n.attrs.items()}] for n in self.nodes.values()],
             "constants": {str(k): {"shape": list(t.shape), "dtype": dtype_name(t.dtype), "data": t.contiguous().cpu().flatten().tolist()} for k, t in self.constants.items()}}
        return json.dumps(d)

    @classmethod
    def from_json(cls, s: str) -> "IrGraph":
        def dec_attr(v):
            if isinstance(v, dict) and "__graph__" in v:
                return cls.from_json(json.dumps(v["__graph__"]))
            if isinstance(v, dict) and "__dtype__" in v:
                return dtype_of(v["__dtype__"])
            if isinstance(v, list):
                return tuple(dec_attr(x) for x in v)
            return v
        d = json.loads(s)
        if d.get("version") != 1:
            raise InvalidArgument("unsupported IR version")
        g = cls()
        for vid, shape, dt, prod in d["values"]:
            g.values[vid] = IrValue(vid, tuple(shape), dt, prod)
        for nid, op, ins, outs, attrs in d["nodes"]:
            g.nodes[nid] = IrNode(nid, op, ins, outs, {k: dec_attr(v) for k, v in attrs.items()})
        g.inputs, g.outputs = d["inputs"], d["outputs"]
        for k, c in d["constants"].items():
            g.constants[int(k)] = torch.tensor(c["data"], dtype=dtype_of(c["dtype"])).reshape(c["shape"])
        g._next_v = max(g.values, default=-1) + 1
        g._next_n = max(g.nodes, default=-1) + 1
        return g

    def __repr__(self):
        lines = [f"graph({', '.join(f'%{i}:{self.values[i].dtype}{list(self.values[i].shape)}' for i in self.inputs)}):"]
        for n in self.topo_order():
            a = ", ".join(f"{k}={v}" for k, v in n.attrs.items() if k != "body")
            lines.append(f"  {', '.join('%' + str(o) for o in n.outputs)} = {n.op}({', '.join('%' + str(i) for i in n.inputs)}{', ' + a if a else ''})")
        lines.append(f"  return {', '.join('%' + str(o) for o in self.outputs)}")
        return "\n".join(lines)
