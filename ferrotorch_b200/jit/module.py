"""``compile``: trace -> optimise -> execute, with shape/dtype guards, per-signature graph cache, graph-break accounting,
AOT joint forward/backward capture, symbolic dimensions, export and kernel autotuning.

Reference parity: ferrotorch-jit/src/{module.rs:267 (compile), aot_autograd.rs:29,83,455, graph_break.rs:95-228, symbolic.rs:80-404,
export.rs:35-691, autotune.rs:77-372}.
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..errors import FerrotorchError, InvalidArgument
from . import passes
from .codegen import CudaFusedKernel, CudaFusedReduceKernel, HostFusedKernel, HostFusedReduceKernel
from .interpreter import eval_node
from .ir import IrGraph, dtype_name
from .trace import trace


# ----------------------------------------------------------------------------------------------------------------------
# symbolic shapes
# ----------------------------------------------------------------------------------------------------------------------
class SymbolicDim:
    """A named dimension with optional bounds; arithmetic builds expression strings evaluated against a binding."""

    def __init__(self, name: str, min: int = 1, max: Optional[int] = None, expr: Optional[str] = None):  # noqa: A002
        self.name, self.min, self.max, self.expr = name, min, max, expr or name

    def _bin(self, o, op):
        oe = o.expr if isinstance(o, SymbolicDim) else repr(int(o))
        return SymbolicDim(self.name, expr=f"({self.expr} {op} {oe})")

    __add__ = lambda s, o: s._bin(o, "+")      # noqa: E731
    __sub__ = lambda s, o: s._bin(o, "-")      # noqa: E731
    __mul__ = lambda s, o: s._bin(o, "*")      # noqa: E731
    __floordiv__ = lambda s, o: s._bin(o, "//")  # noqa: E731
    __radd__, __rmul__ = __add__, __mul__

    def evaluate(self, binding: Dict[str, int]) -> int:
        return int(eval(self.expr, {"__builtins__": {}}, dict(binding)))     # expression strings are built only by this class

    def __repr__(self):
        return f"Sym({self.expr})"


class ShapeEnv:
    """Binds symbolic dims to the sizes seen in example inputs and records guards (bounds, equalities) checked on later calls."""

    def __init__(self):
        self.binding: Dict[str, int] = {}
        self.guards: List[Tuple[str, Callable[[Dict[str, int]], bool]]] = []
        self.dims: Dict[str, SymbolicDim] = {}

    def bind(self, spec: Sequence[Any], shape: Sequence[int], binding: Optional[Dict[str, int]] = None) -> Dict[str, int]:
        b = self.binding if binding is None else binding
        if len(spec) != len(shape):
            raise InvalidArgument(f"rank mismatch: spec {spec} vs shape {tuple(shape)}")
        for s, n in zip(spec, shape):
            if isinstance(s, SymbolicDim):
                self.dims[s.name] = s
                if s.expr != s.name:
                    if s.evaluate(b) != n:
                        raise InvalidArgument(f"dimension {s} evaluates to {s.evaluate(b)}, got {n}")
                    continue
                if n < s.min or (s.max is not None and n > s.max):
                    raise InvalidArgument(f"dimension {s.name}={n} outside [{s.min}, {s.max}]")
                if b.setdefault(s.name, n) != n:
                    raise InvalidArgument(f"dimension {s.name} bound to {b[s.name]}, got {n}")
            elif s is not None and s != n:
                raise InvalidArgument(f"static dimension {s} != {n}")
        return b

    def check(self, specs, shapes) -> Optional[Dict[str, int]]:
        b: Dict[str, int] = {}
        try:
            for spec, shape in zip(specs, shapes):
                self.bind(spec, shape, b)
        except InvalidArgument:
            return None
        return b


# ----------------------------------------------------------------------------------------------------------------------
# compiled function
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class CompileStats:
    traces: int = 0
    cache_hits: int = 0
    fused_kernels: int = 0
    graph_breaks: int = 0
    kernel_launches: int = 0
    guard_failures: int = 0


@dataclass
class GraphSegment:
    nodes: List[int]
    compiled: bool


def split_at_breaks(g: IrGraph) -> List[GraphSegment]:
    """Maximal runs of IR-native nodes between ``opaque`` nodes (each opaque node is its own eager segment)."""
    segs: List[GraphSegment] = []
    cur: List[int] = []
    for n in g.topo_order():
        if n.op == "opaque":
            if cur:
                segs.append(GraphSegment(cur, True))
                cur = []
            segs.append(GraphSegment([n.id], False))
        else:
            cur.append(n.id)
    if cur:
        segs.append(GraphSegment(cur, True))
    return segs


class _FusedWithGrad(torch.autograd.Function):
    """A generated kernel inside a differentiated computation: the forward pass runs the kernel and keeps only its inputs; the backward pass
    evaluates the region's body again with the interpreter under autograd (the region's intermediates are recomputed, not stored) and
    differentiates that."""

    @staticmethod
    def forward(ctx, kernel, node, graph, *ins):
        ctx.node, ctx.graph = node, graph
        ctx.save_for_backward(*ins)
        out = kernel([t.detach() for t in ins])
        if isinstance(out, (tuple, list)):
            outs = tuple(out)
            ctx.mark_non_differentiable(*[o for o in outs if not (o.is_floating_point() or o.is_complex())])
            return outs
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, *grad_outputs):
        needs = ctx.needs_input_grad[3:]
        with torch.enable_grad():
            leaves = [t.detach().requires_grad_(bool(need) and (t.is_floating_point() or t.is_complex())) for t, need in zip(ctx.saved_tensors, needs)]
            out = eval_node(ctx.node, leaves, ctx.graph)
            outs = list(out) if isinstance(out, (tuple, list)) else [out]
            pairs = [(o, go) for o, go in zip(outs, grad_outputs) if go is not None and isinstance(o, torch.Tensor) and o.requires_grad]
            wanted = [leaf for leaf in leaves if leaf.requires_grad]
            grads = torch.autograd.grad([o for o, _ in pairs], wanted, [go for _, go in pairs], allow_unused=True) if pairs and wanted else ()
        it = iter(grads)
        return (None, None, None, *[next(it, None) if leaf.requires_grad else None for leaf in leaves])


class _EagerExecutable:
    """A function that writes into tensors in place (into an input, through a view, or between two reads of one tensor) is run as written:
    the value graph has no faithful form for such writes. The traced graph is kept for inspection."""

    def __init__(self, fn: Callable, g: IrGraph):
        self.fn, self.g = fn, g

    def run(self, inputs: Sequence[torch.Tensor]):
        out = self.fn(*inputs)
        return [out] if isinstance(out, torch.Tensor) else list(out)


class _Executable:
    """One optimised graph plus its compiled fused kernels."""

    def __init__(self, g: IrGraph, backend: str, stats: CompileStats):
        self.g, self.backend, self.stats = g, backend, stats
        self.order = g.topo_order()
        self.kernels: Dict[int, Any] = {}
        self.segments = split_at_breaks(g)
        stats.graph_breaks += sum(1 for s in self.segments if not s.compiled)
        if backend in ("cuda", "host"):
            for n in self.order:
                try:
                    if n.op == "fused":
                        self.kernels[n.id] = (CudaFusedKernel if backend == "cuda" else HostFusedKernel)(n.attrs["body"])
                        stats.fused_kernels += 1
                    elif n.op == "fused_reduce":
                        cls = CudaFusedReduceKernel if backend == "cuda" else HostFusedReduceKernel
                        self.kernels[n.id] = cls(n.attrs["body"], n.attrs["red_op"], n.attrs["red_index"], n.attrs["keepdim"])
                        stats.fused_kernels += 1
                except InvalidArgument:
                    pass                                           # ops without a code template stay on the interpreter
        users = g.users()
        self.last_use: Dict[int, int] = {}
        for i, n in enumerate(self.order):
            for v in n.inputs:
                self.last_use[v] = i

    def run(self, inputs: Sequence[torch.Tensor]):
        g = self.g
        env: Dict[int, torch.Tensor] = dict(g.constants)
        for vid, t in zip(g.inputs, inputs):
            env[vid] = t
        keep = set(g.outputs) | set(g.constants)
        for i, n in enumerate(self.order):
            ins = [env[v] for v in n.inputs]
            k = self.kernels.get(n.id)
            if k is not None and (self.backend == "host" or any(t.is_cuda for t in ins)):
                if torch.is_grad_enabled() and any(t.requires_grad for t in ins):
                    out = _FusedWithGrad.apply(k, n, g, *ins)
                else:
                    out = k([t.detach() for t in ins])
                self.stats.kernel_launches += 1
            else:
                out = eval_node(n, ins, g)
            outs = out if isinstance(out, (tuple, list)) else [out]
            for vid, t in zip(n.outputs, [o for o in outs if isinstance(o, torch.Tensor)]):
                env[vid] = t
            for v in n.inputs:                                     # free dead intermediates early (the liveness the memory plan models)
                if self.last_use.get(v) == i and v not in keep:
                    env.pop(v, None)
        return [env[o] for o in g.outputs]


class CompiledFunction:
    def __init__(self, fn: Callable, backend: str = "auto", dynamic_dims: Optional[Sequence[Optional[Sequence[Any]]]] = None, fuse: bool = True):
        if backend not in ("auto", "cuda", "host", "interpreter"):
            raise InvalidArgument(f"unknown backend {backend}")
        self.fn, self.backend, self.fuse = fn, backend, fuse
        self.cache: Dict[Tuple, _Executable] = {}
        self.stats = CompileStats()
        self.dynamic_dims = dynamic_dims
        self.shape_env = ShapeEnv() if dynamic_dims is not None else None

    def _sig(self, inputs) -> Tuple:
        for t in inputs:
            if not isinstance(t, torch.Tensor):
                raise InvalidArgument(f"compiled callables take tensors; got {type(t).__name__} (close over Python numbers, or pass them as 0-d tensors)")
        return tuple((tuple(t.shape), t.dtype, t.device.type) for t in inputs)

    def _backend_for(self, inputs) -> str:
        if self.backend != "auto":
            return self.backend
        return "cuda" if any(t.is_cuda for t in inputs) else "host"

    def graph_for(self, *inputs) -> IrGraph:
        return self._get(inputs).g

    def _get(self, inputs) -> _Executable:
        sig = self._sig(inputs)
        ex = self.cache.get(sig)
        if ex is not None:
            self.stats.cache_hits += 1
            return ex
        if self.shape_env is not None and self.cache:
            if self.shape_env.check(self.dynamic_dims, [t.shape for t in inputs]) is None:
                self.stats.guard_failures += 1
                raise InvalidArgument(f"input shapes {[tuple(t.shape) for t in inputs]} violate the declared symbolic dimensions")
        elif self.shape_env is not None:
            for spec, t in zip(self.dynamic_dims, inputs):
                self.shape_env.bind(spec, t.shape)
        owner = self.fn if isinstance(self.fn, torch.nn.Module) else getattr(self.fn, "__self__", None)
        kept = [(b, b.detach().clone()) for b in owner.buffers()] if isinstance(owner, torch.nn.Module) else []
        try:
            g = trace(self.fn, [t.clone() if isinstance(t, torch.Tensor) else t for t in inputs])    # copies: tracing runs the function once
        finally:
            with torch.no_grad():
                for b, before in kept:             # running statistics and other buffers as they were before the tracing run
                    b.copy_(before)
        self.stats.traces += 1
        if g.mutations:
            ex = _EagerExecutable(self.fn, g)
            self.stats.graph_breaks += 1
            self.cache[sig] = ex
            return ex
        passes.optimize(g, fuse=self.fuse)
        ex = _Executable(g, self._backend_for(inputs), self.stats)
        self.cache[sig] = ex
        return ex

    def __call__(self, *inputs):
        ex = self._get(inputs)
        out = ex.run(inputs)
        return out[0] if getattr(ex.g, "single_output", len(out) == 1) else tuple(out)


def compile(fn: Callable, example_inputs: Optional[Sequence[torch.Tensor]] = None, backend: str = "auto", dynamic_dims=None, fuse: bool = True) -> CompiledFunction:  # noqa: A001
    """Returns a callable that traces ``fn`` on first use of each input signature, optimises the graph (folding, CSE, DCE, elementwise
    fusion) and runs fused regions as generated kernels (``cuda``: NVRTC sm_100a; ``host``: C++), everything else eagerly."""
    cf = CompiledFunction(fn.forward if isinstance(fn, torch.nn.Module) else fn, backend, dynamic_dims, fuse)
    if example_inputs is not None:
        cf._get(tuple(example_inputs))
    return cf


# ----------------------------------------------------------------------------------------------------------------------
# AOT autograd
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class JointGraph:
    graph: IrGraph
    num_primals: int
    num_outputs: int

    def forward_backward(self, primals: Sequence[torch.Tensor], tangents: Sequence[torch.Tensor]):
        from .interpreter import run_graph
        res = run_graph(self.graph, list(primals) + list(tangents))
        return res[: self.num_outputs], res[self.num_outputs:]


def aot_trace_joint(fn: Callable, primals: Sequence[torch.Tensor]) -> JointGraph:
    """Captures forward and backward in one graph: inputs are (primals..., tangents...), outputs (outputs..., grads of primals...)."""
    from .trace import _Recorder
    g = IrGraph()
    env: Dict[int, int] = {}
    ps = [p.detach().clone().requires_grad_(True) for p in primals]
    for p in ps:
        env[id(p)] = g.add_input(p.shape, p.dtype).id
    rec = _Recorder(g, env)
    with torch.enable_grad(), rec:
        out = fn(*ps)
        outs = [out] if isinstance(out, torch.Tensor) else list(out)
    tangents = [torch.ones_like(o) for o in outs]
    for t in tangents:
        env[id(t)] = g.add_input(t.shape, t.dtype).id
    with torch.enable_grad(), rec:
        grads = torch.autograd.grad(outs, ps, tangents, allow_unused=True)
    grads = [gr if gr is not None else torch.zeros_like(p) for gr, p in zip(grads, ps)]
    g.set_outputs([rec.vid(o) for o in outs] + [rec.vid(gr) for gr in grads])
    g.single_output = False
    g.validate()
    return JointGraph(g, len(ps), len(outs))


class AotFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, joint: JointGraph, *primals):
        ctx.joint = joint
        ctx.save_for_backward(*primals)
        from .interpreter import run_graph
        zeros = [torch.zeros(joint.graph.values[v].shape, dtype=primals[0].dtype, device=primals[0].device) for v in joint.graph.inputs[joint.num_primals:]]
        res = run_graph(joint.graph, list(primals) + zeros)
        outs = res[: joint.num_outputs]
        return outs[0] if joint.num_outputs == 1 else tuple(outs)

    @staticmethod
    def backward(ctx, *tangents):
        _, grads = ctx.joint.forward_backward(ctx.saved_tensors, tangents)
        return (None, *grads)


def aot_function(fn: Callable, example_primals: Sequence[torch.Tensor]) -> Callable:
    joint = aot_trace_joint(fn, example_primals)
    passes.optimize(joint.graph, fuse=True)
    return lambda *primals: AotFunction.apply(joint, *primals)


# ----------------------------------------------------------------------------------------------------------------------
# export
# ----------------------------------------------------------------------------------------------------------------------
class ExportedProgram:
    """A traced graph with its weights, storable as ``<path>.json`` (structure) + ``<path>.safetensors`` (large constants)."""

    def __init__(self, graph: IrGraph, input_specs: List[Tuple[Tuple[int, ...], str]]):
        self.graph, self.input_specs = graph, input_specs

    def __call__(self, *inputs):
        from .interpreter import Interpreter
        for (shape, dt), t in zip(self.input_specs, inputs):
            if tuple(t.shape) != tuple(shape) or dtype_name(t.dtype) != dt:
                raise InvalidArgument(f"exported program expects {dt}{list(shape)}, got {dtype_name(t.dtype)}{list(t.shape)}")
        return Interpreter(self.graph)(*inputs)

    def save(self, path: str) -> None:
        from ..serialize import save_safetensors
        g = self.graph
        big = {f"c{k}": t.contiguous() for k, t in g.constants.items() if t.numel() > 64}
        small = IrGraph.from_json(g.to_json()) if not big else None
        if big:
            keep = dict(g.constants)
            g.constants = {k: t for k, t in keep.items() if t.numel() <= 64}
            try:
                js = g.to_json()
            finally:
                g.constants = keep
            save_safetensors(big, path + ".safetensors")
        else:
            js = g.to_json()
        with open(path + ".json", "w") as f:
            json.dump({"graph": json.loads(js), "inputs": [[list(s), d] for s, d in self.input_specs], "single_output": getattr(g, "single_output", True),
                       "external_constants": sorted(big)}, f)

    @classmethod
    def load(cls, path: str) -> "ExportedProgram":
        from ..serialize import load_safetensors
        d = json.load(open(path + ".json"))
        g = IrGraph.from_json(json.dumps(d["graph"]))
        if d["external_constants"]:
            for k, t in load_safetensors(path + ".safetensors").items():
                g.constants[int(k[1:])] = t
        g.single_output = d["single_output"]
        g.validate()
        return cls(g, [(tuple(s), dt) for s, dt in d["inputs"]])


def export(fn: Callable, example_inputs: Sequence[torch.Tensor], strict: bool = True) -> ExportedProgram:
    g = trace(fn.forward if isinstance(fn, torch.nn.Module) else fn, example_inputs)
    bad = sorted({n.attrs["name"] for n in g.nodes.values() if n.op == "opaque"})
    if bad and strict:
        raise FerrotorchError(f"export: the function uses ops without a portable IR form: {bad}")
    passes.optimize(g, fuse=False)
    return ExportedProgram(g, [(tuple(t.shape), dtype_name(t.dtype)) for t in example_inputs])


# ----------------------------------------------------------------------------------------------------------------------
# autotune
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class TuneResult:
    best: Any
    timings_ms: Dict[str, float]


class Autotuner:
    """Times candidate configurations of a callable factory and remembers the winner per key (in memory and in a JSON file)."""

    def __init__(self, cache_path: Optional[str] = None, warmup: int = 2, iters: int = 5):
        self.cache_path, self.warmup, self.iters = cache_path, warmup, iters
        self.cache: Dict[str, Any] = {}
        if cache_path and os.path.exists(cache_path):
            self.cache = json.load(open(cache_path))

    def _time(self, fn: Callable[[], Any]) -> float:
        cuda = torch.cuda.is_available()
        for _ in range(self.warmup):
            fn()
        if cuda:
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(self.iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / self.iters
        t = time.perf_counter()
        for _ in range(self.iters):
            fn()
        return (time.perf_counter() - t) * 1e3 / self.iters

    def tune(self, key: str, candidates: Sequence[Any], make: Callable[[Any], Callable[[], Any]]) -> TuneResult:
        if key in self.cache:
            return TuneResult(self.cache[key], {})
        timings = {}
        for c in candidates:
            try:
                timings[json.dumps(c)] = self._time(make(c))
            except Exception:                                      # a candidate that cannot run is skipped, not fatal
                continue
        if not timings:
            raise FerrotorchError(f"autotune: no candidate ran for {key}")
        best = json.loads(min(timings, key=timings.get))
        self.cache[key] = best
        if self.cache_path:
            with open(self.cache_path, "w") as f:
                json.dump(self.cache, f)
        return TuneResult(best, timings)
