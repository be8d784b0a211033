"""The object-level JIT API: traced modules, compile / optimisation configs, graph-break segmentation, symbolic-shape guards, export specs,
code-generation backends, the loop IR with its C++ / CUDA emitters, fused unary chains, reduction kernels and graph autotuning.

Everything here is built on the tracer (``trace.py``), the passes (``passes.py``), the interpreter and the fused-kernel generators
(``codegen.py``); this module gives those pieces the shapes a user of the reference reaches for.

Reference parity (ferrotorch-jit/src): module.rs:29-430 (CompileConfig, TracedModule, compile_with_config, AotCompiledModule), optimize.rs:21-60,
graph_break.rs:95-300, symbolic.rs:80-460, export.rs:35-720, aot_autograd.rs:29-520, codegen.rs:41-1000 (Codegen, CompiledGraph, backends),
codegen_ir.rs:25-420 (Expr, LoopIR, lower_to_loops), codegen_cpu.rs:36, codegen_gpu.rs:75-561, codegen_jit.rs:91-300, fusion.rs:54-1300,
interpreter.rs:71-200, autotune.rs:77-380, error.rs (JitError).
"""
from __future__ import annotations

import contextlib
import ctypes
import enum
import hashlib
import json
import os
import re
import subprocess
import threading
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

import torch

from ..errors import FerrotorchError, InvalidArgument, ShapeMismatch
from . import codegen as _cg
from . import passes
from .interpreter import eval_node, run_graph
from .ir import IrGraph, dtype_name
from .module import Autotuner as _BaseAutotuner
from .module import ExportedProgram, JointGraph, _Executable, CompileStats, aot_trace_joint, split_at_breaks
from .passes import MemoryPlan
from .trace import trace


class JitError(FerrotorchError):
    """Failure inside the JIT (trace, pass, code generation, kernel build)."""


# ----------------------------------------------------------------------------------------------------------------------
# interpretation
# ----------------------------------------------------------------------------------------------------------------------
def interpret_multi(graph: IrGraph, inputs: Sequence[torch.Tensor]) -> List[torch.Tensor]:
    if len(inputs) != len(graph.inputs):
        raise InvalidArgument(f"interpret: graph takes {len(graph.inputs)} inputs, got {len(inputs)}")
    return list(run_graph(graph, list(inputs)))


def interpret(graph: IrGraph, inputs: Sequence[torch.Tensor]) -> torch.Tensor:
    """Single-output form (interpreter.rs:71): a graph with no or several outputs is refused and points at :func:`interpret_multi`."""
    if len(graph.outputs) != 1:
        raise InvalidArgument("interpret: graph has no outputs" if not graph.outputs else
                              f"interpret: graph has {len(graph.outputs)} outputs; use interpret_multi")
    return interpret_multi(graph, inputs)[0]


def interpret_multi_with_captures(graph: IrGraph, inputs: Sequence[torch.Tensor], capture_topo_indices: Sequence[int]):
    """Outputs plus the values produced by the nodes at the given positions of the topological order (what a backward graph saves from
    the forward pass) (interpreter.rs:154)."""
    order = graph.topo_order()
    bad = [i for i in capture_topo_indices if not 0 <= i < len(order)]
    if bad:
        raise InvalidArgument(f"interpret_multi_with_captures: topological index {bad[0]} out of range for {len(order)} nodes")
    env: Dict[int, torch.Tensor] = dict(graph.constants)
    env.update(zip(graph.inputs, inputs))
    for n in order:
        if n.op in ("input", "constant", "output"):
            continue
        out = eval_node(n, [env[v] for v in n.inputs], graph)
        for vid, t in zip(n.outputs, out if isinstance(out, (list, tuple)) else [out]):
            env[vid] = t
    return [env[o] for o in graph.outputs], [env[order[i].outputs[0]] for i in capture_topo_indices]


# ----------------------------------------------------------------------------------------------------------------------
# configs, traced module, compile_with_config
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class OptimizationConfig:
    constant_folding: bool = True
    dead_code_elimination: bool = True
    operator_fusion: bool = True
    memory_planning: bool = True


def optimize_with_config(graph: IrGraph, config: Optional[OptimizationConfig] = None) -> Optional[MemoryPlan]:
    """Runs the enabled passes in the reference's order (fold, eliminate, fuse) and returns the memory plan when one was asked for
    (optimize.rs:48)."""
    c = config or OptimizationConfig()
    if c.constant_folding:
        passes.constant_folding(graph)
        passes.algebraic_simplification(graph)
        passes.common_subexpression_elimination(graph)
    if c.dead_code_elimination:
        passes.dead_code_elimination(graph)
    if c.operator_fusion:
        passes.fuse_elementwise(graph)
        passes.fuse_reductions(graph)
    graph.validate()
    return passes.plan_memory(graph) if c.memory_planning else None


@dataclass
class CompileConfig:
    optimization: OptimizationConfig = field(default_factory=OptimizationConfig)
    fullgraph: bool = False              # refuse graph breaks instead of falling back to eager segments
    cache_size: int = 8                  # compiled specialisations kept per function

    @classmethod
    def from_optimization(cls, config: OptimizationConfig) -> "CompileConfig":
        return cls(optimization=config)


class TracedModule:
    """An optimised graph that runs like the function it was traced from (module.rs:75). Fused regions run as generated host / sm_100a
    kernels, the rest on the interpreter."""

    def __init__(self, graph: IrGraph, backend: str = "auto", memory_plan: Optional[MemoryPlan] = None):
        graph.validate()
        self._graph, self._backend, self.memory_plan = graph, backend, memory_plan
        self._exe: Dict[str, _Executable] = {}
        self.stats = CompileStats()

    def graph(self) -> IrGraph:
        return self._graph

    def input_count(self) -> int:
        return len(self._graph.inputs)

    def output_shape(self) -> Tuple[int, ...]:
        return tuple(self._graph.values[self._graph.outputs[0]].shape)

    def forward_multi(self, inputs: Sequence[torch.Tensor]):
        if len(inputs) != self.input_count():
            raise InvalidArgument(f"TracedModule: expected {self.input_count()} inputs, got {len(inputs)}")
        for i, (vid, t) in enumerate(zip(self._graph.inputs, inputs)):
            want = self._graph.values[vid].shape
            if all(isinstance(d, int) for d in want) and tuple(t.shape) != tuple(want):
                raise ShapeMismatch(f"TracedModule: input {i} has shape {list(t.shape)}, the graph was traced with {list(want)}")
        be = self._backend if self._backend != "auto" else ("cuda" if any(t.is_cuda for t in inputs) else "host")
        if be not in self._exe:
            self._exe[be] = _Executable(self._graph, be, self.stats)
        out = self._exe[be].run(list(inputs))
        return out[0] if len(out) == 1 else tuple(out)

    def forward(self, x: torch.Tensor):
        return self.forward_multi([x])

    def __call__(self, *inputs):
        return self.forward_multi(inputs)

    # -- persistence: structure as JSON, constants inline (base85), one blob --------------------------------------------
    def to_bytes(self) -> bytes:
        return b"FTJM1\n" + self._graph.to_json().encode("utf-8")

    @classmethod
    def from_bytes(cls, data: bytes) -> "TracedModule":
        if not data.startswith(b"FTJM1\n"):
            raise InvalidArgument("TracedModule.from_bytes: not a traced-module blob")
        try:
            return cls(IrGraph.from_json(data[6:].decode("utf-8")))
        except (ValueError, KeyError, TypeError) as e:
            raise InvalidArgument(f"TracedModule.from_bytes: malformed graph: {e}") from None

    def save(self, path) -> None:
        try:
            Path(path).write_bytes(self.to_bytes())
        except OSError as e:
            raise InvalidArgument(f"TracedModule.save: {path}: {e}") from None

    @classmethod
    def load(cls, path) -> "TracedModule":
        try:
            return cls.from_bytes(Path(path).read_bytes())
        except OSError as e:
            raise InvalidArgument(f"TracedModule.load: {path}: {e}") from None


def _fn_of(f):
    return f.forward if isinstance(f, torch.nn.Module) else f


def compile_with_config(f: Callable, example_inputs: Sequence[torch.Tensor], config: Optional[CompileConfig] = None, backend: str = "auto") -> TracedModule:
    """Trace once on ``example_inputs``, optimise under ``config`` and return the :class:`TracedModule` (module.rs:287). ``fullgraph`` turns a
    graph break (an operation the tracer can only keep as an opaque call) into an error."""
    cfg = config or CompileConfig()
    g = trace(_fn_of(f), tuple(example_inputs))
    if cfg.fullgraph and any(n.op == "opaque" for n in g.nodes.values()):
        ops = sorted({str(n.attrs.get("name", "opaque")) for n in g.nodes.values() if n.op == "opaque"})
        raise JitError(f"compile(fullgraph=True): the function has graph breaks at {ops}")
    plan = optimize_with_config(g, cfg.optimization)
    return TracedModule(g, backend, plan)


# ----------------------------------------------------------------------------------------------------------------------
# graph breaks
# ----------------------------------------------------------------------------------------------------------------------
class Segment:
    """One piece of a function split at graph breaks: ``Compiled`` holds a :class:`TracedModule`, ``Eager`` a plain callable
    (graph_break.rs:95). Both map the running list of live values to the values the next segment needs."""

    def __init__(self, kind: str, payload, in_ids: List[int], out_ids: List[int]):
        self.kind, self.payload, self.in_ids, self.out_ids = kind, payload, in_ids, out_ids

    def is_compiled(self) -> bool:
        return self.kind == "compiled"

    def __repr__(self):
        return f"Compiled(TracedModule({self.payload.graph().node_count()} nodes))" if self.is_compiled() else "Eager(<closure>)"


class SegmentedModule:
    def __init__(self, segments: List[Segment], inputs: List[int], outputs: List[int], constants: Dict[int, torch.Tensor]):
        self._segments, self._inputs, self._outputs, self._constants = segments, inputs, outputs, constants

    def segments(self) -> List[Segment]:
        return list(self._segments)

    def segment_count(self) -> int:
        return len(self._segments)

    def is_fully_compiled(self) -> bool:
        return all(s.is_compiled() for s in self._segments)

    def forward_multi(self, inputs: Sequence[torch.Tensor]):
        env: Dict[int, torch.Tensor] = dict(self._constants)
        env.update(zip(self._inputs, inputs))
        for s in self._segments:
            res = s.payload.forward_multi([env[v] for v in s.in_ids]) if s.is_compiled() else s.payload(*[env[v] for v in s.in_ids])
            res = list(res) if isinstance(res, (tuple, list)) else [res]
            env.update(zip(s.out_ids, res))
        out = [env[o] for o in self._outputs]
        return out[0] if len(out) == 1 else tuple(out)

    def forward(self, x):
        return self.forward_multi([x])

    __call__ = lambda self, *a: self.forward_multi(a)  # noqa: E731


class TraceResult:
    """``Unbroken(graph)`` or ``Segmented(module)`` (graph_break.rs:195)."""

    def __init__(self, graph: Optional[IrGraph] = None, segmented: Optional[SegmentedModule] = None):
        self.graph, self.segmented = graph, segmented

    def is_unbroken(self) -> bool:
        return self.graph is not None


def _subgraph(g: IrGraph, node_ids: List[int], needed_after: set) -> Tuple[IrGraph, List[int], List[int]]:
    """Nodes ``node_ids`` of ``g`` as a graph of their own: inputs are the values they read but do not produce (constants are copied in),
    outputs the values they produce that someone outside still needs."""
    sub = IrGraph()
    produced = {o for nid in node_ids for o in g.nodes[nid].outputs}
    remap: Dict[int, int] = {}
    in_ids: List[int] = []
    for nid in node_ids:
        for v in g.nodes[nid].inputs:
            if v in produced or v in remap:
                continue
            if v in g.constants:
                remap[v] = sub.add_constant(g.constants[v]).id
            else:
                remap[v] = sub.add_input(g.values[v].shape, g.values[v].dtype).id
                in_ids.append(v)
    for nid in node_ids:
        n = g.nodes[nid]
        m = sub.add_node(n.op, [remap[v] for v in n.inputs], [(g.values[o].shape, g.values[o].dtype) for o in n.outputs], **n.attrs)
        remap.update(zip(n.outputs, m.outputs))
    out_ids = [o for nid in node_ids for o in g.nodes[nid].outputs if o in needed_after]
    sub.set_outputs([remap[o] for o in out_ids])
    return sub, in_ids, out_ids


def trace_with_breaks(f: Callable, example_inputs: Sequence[torch.Tensor], config: Optional[CompileConfig] = None) -> TraceResult:
    """Trace ``f``; without graph breaks the result is the optimised graph, otherwise a :class:`SegmentedModule` whose compiled runs are
    optimised one by one and whose breaks call the original operation eagerly (graph_break.rs:228)."""
    cfg = config or CompileConfig()
    g = trace(_fn_of(f), tuple(example_inputs))
    segs = split_at_breaks(g)
    if all(s.compiled for s in segs):
        optimize_with_config(g, cfg.optimization)
        return TraceResult(graph=g)
    if cfg.fullgraph:
        raise JitError("trace_with_breaks(fullgraph=True): the function has graph breaks")
    users_after: List[set] = []
    need = set(g.outputs)
    for s in reversed(segs):
        users_after.append(set(need))
        for nid in s.nodes:
            need |= set(g.nodes[nid].inputs)
    users_after.reverse()
    out: List[Segment] = []
    for s, needed in zip(segs, users_after):
        real = [nid for nid in s.nodes if g.nodes[nid].op not in ("input", "constant", "output")]
        if not real:
            continue
        sub, in_ids, out_ids = _subgraph(g, real, needed)
        if not out_ids:
            continue
        if s.compiled:
            optimize_with_config(sub, cfg.optimization)
            out.append(Segment("compiled", TracedModule(sub), in_ids, out_ids))
        else:
            out.append(Segment("eager", (lambda sg: lambda *xs: run_graph(sg, list(xs)))(sub), in_ids, out_ids))
    return TraceResult(segmented=SegmentedModule(out, list(g.inputs), list(g.outputs), dict(g.constants)))


# ----------------------------------------------------------------------------------------------------------------------
# symbolic shapes
# ----------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class SymbolicDimSpec:
    """Dimension ``dim_index`` of one input may vary within ``[min, max]`` (symbolic.rs:89)."""
    dim_index: int
    min: Optional[int] = None
    max: Optional[int] = None


class ShapeSignature:
    """Which dimensions of which inputs are symbolic (symbolic.rs:80)."""

    def __init__(self):
        self.entries: List[List[SymbolicDimSpec]] = []

    def _slot(self, i: int) -> List[SymbolicDimSpec]:
        while len(self.entries) <= i:
            self.entries.append([])
        return self.entries[i]

    def symbolic_dim(self, input_index: int, dim: int) -> "ShapeSignature":
        return self.symbolic_dim_with_range(input_index, dim, None, None)

    def symbolic_dim_with_range(self, input_index: int, dim: int, lo: Optional[int], hi: Optional[int]) -> "ShapeSignature":
        if lo is not None and hi is not None and lo > hi:
            raise InvalidArgument(f"ShapeSignature: empty range [{lo}, {hi}]")
        slot = self._slot(input_index)
        slot[:] = [s for s in slot if s.dim_index != dim] + [SymbolicDimSpec(dim, lo, hi)]
        return self

    def symbolic_dims_for(self, input_index: int) -> List[SymbolicDimSpec]:
        return list(self.entries[input_index]) if input_index < len(self.entries) else []

    def is_symbolic(self, input_index: int, dim: int) -> bool:
        return any(s.dim_index == dim for s in self.symbolic_dims_for(input_index))


class Guard:
    """Checks runtime shapes against the traced ones: static dimensions must match exactly, symbolic ones must be non-zero and inside
    their range (symbolic.rs:171-270)."""

    def __init__(self, trace_shapes: Sequence[Sequence[int]], signature: ShapeSignature):
        self.trace_shapes, self.signature = [tuple(s) for s in trace_shapes], signature

    def check(self, inputs: Sequence[Sequence[int]]) -> None:
        who = "SymbolicTracedModule guard"
        if len(inputs) != len(self.trace_shapes):
            raise InvalidArgument(f"{who}: expected {len(self.trace_shapes)} inputs, got {len(inputs)}")
        for i, (got, want) in enumerate(zip(inputs, self.trace_shapes)):
            if len(got) != len(want):
                raise InvalidArgument(f"{who}: input {i} rank mismatch: expected {len(want)}, got {len(got)} (shape {list(got)} vs signature {list(want)})")
            for d, (a, e) in enumerate(zip(got, want)):
                sym = next((s for s in self.signature.symbolic_dims_for(i) if s.dim_index == d), None)
                if sym is None:
                    if a != e:
                        raise InvalidArgument(f"{who}: input {i} dim {d} is static ({e}) but runtime value is {a}")
                elif a == 0:
                    raise InvalidArgument(f"{who}: input {i} dim {d} is symbolic but runtime value is 0")
                elif (sym.min is not None and a < sym.min) or (sym.max is not None and a > sym.max):
                    raise InvalidArgument(f"{who}: input {i} dim {d} = {a} outside [{sym.min}, {sym.max}]")


def patch_reshape_for_symbolic_dims(graph: IrGraph, trace_shapes: Sequence[Sequence[int]], signature: ShapeSignature) -> int:
    """Rewrites reshape targets that baked in a traced symbolic extent: when exactly one target dimension equals the traced size of a
    symbolic input dimension (and no other target dimension is already ``-1``) it becomes ``-1``, so the reshape follows the runtime size
    (symbolic.rs:329). Returns the number of rewritten nodes."""
    sym_sizes = {trace_shapes[i][s.dim_index] for i in range(len(trace_shapes)) for s in signature.symbolic_dims_for(i)}
    n_patched = 0
    for n in graph.nodes.values():
        if n.op != "reshape" or -1 in n.attrs["shape"]:
            continue
        hits = [k for k, d in enumerate(n.attrs["shape"]) if d in sym_sizes]
        if len(hits) == 1:
            shp = list(n.attrs["shape"])
            shp[hits[0]] = -1
            n.attrs["shape"] = shp
            n_patched += 1
    return n_patched


class SymbolicTracedModule:
    """A traced module that accepts any shapes its guard allows. A new combination of symbolic extents is re-traced once and cached
    (at most ``cache_size`` specialisations), so every run executes a graph whose shapes are exact (symbolic.rs:281)."""

    def __init__(self, f: Callable, inner: TracedModule, guard: Guard, config: CompileConfig):
        self._f, self._inner, self._guard, self._cfg = f, inner, guard, config
        self._cache: Dict[Tuple, TracedModule] = {tuple(guard.trace_shapes): inner}

    def inner(self) -> TracedModule:
        return self._inner

    def guard(self) -> Guard:
        return self._guard

    def specializations(self) -> int:
        return len(self._cache)

    def forward_symbolic(self, inputs: Sequence[torch.Tensor]):
        shapes = tuple(tuple(t.shape) for t in inputs)
        self._guard.check(shapes)
        m = self._cache.get(shapes)
        if m is None:
            m = compile_with_config(self._f, inputs, self._cfg)
            if len(self._cache) >= max(self._cfg.cache_size, 1):
                self._cache.pop(next(k for k in self._cache if k != tuple(self._guard.trace_shapes)), None)
            self._cache[shapes] = m
        return m.forward_multi(inputs)

    __call__ = lambda self, *a: self.forward_symbolic(a)  # noqa: E731


def compile_symbolic(f: Callable, example_inputs: Sequence[torch.Tensor], signature: ShapeSignature, config: Optional[CompileConfig] = None) -> SymbolicTracedModule:
    cfg = config or CompileConfig()
    shapes = [tuple(t.shape) for t in example_inputs]
    guard = Guard(shapes, signature)
    guard.check(shapes)
    return SymbolicTracedModule(_fn_of(f), compile_with_config(f, example_inputs, cfg), guard, cfg)


# ----------------------------------------------------------------------------------------------------------------------
# export specs
# ----------------------------------------------------------------------------------------------------------------------
class DimSpec:
    """``DimSpec.Static(n)`` or ``DimSpec.dynamic(name)`` / ``dynamic_range(name, min, max)`` (export.rs:35)."""

    def __init__(self, size: Optional[int] = None, name: Optional[str] = None, min: Optional[int] = None, max: Optional[int] = None):  # noqa: A002
        self.size, self.name, self.min, self.max = size, name, min, max

    @classmethod
    def Static(cls, n: int) -> "DimSpec":  # noqa: N802
        return cls(size=int(n))

    @classmethod
    def dynamic(cls, name: str) -> "DimSpec":
        return cls(name=name)

    @classmethod
    def dynamic_range(cls, name: str, lo: int, hi: int) -> "DimSpec":
        if lo > hi:
            raise InvalidArgument(f"DimSpec: empty range [{lo}, {hi}] for {name}")
        return cls(name=name, min=lo, max=hi)

    def is_dynamic(self) -> bool:
        return self.name is not None

    def __eq__(self, o):
        return isinstance(o, DimSpec) and (self.size, self.name, self.min, self.max) == (o.size, o.name, o.min, o.max)

    def __repr__(self):
        return f"Static({self.size})" if not self.is_dynamic() else f"Dynamic({self.name!r}, min={self.min}, max={self.max})"


@dataclass
class InputSpec:
    shape: List[DimSpec]

    @classmethod
    def all_static(cls, shape: Sequence[int]) -> "InputSpec":
        return cls([DimSpec.Static(d) for d in shape])

    def has_dynamic_dims(self) -> bool:
        return any(d.is_dynamic() for d in self.shape)

    def rank(self) -> int:
        return len(self.shape)


@dataclass
class ExportedProgramMetadata:
    num_graph_nodes: int
    input_shapes: List[List[int]]
    output_shape: List[int]
    state_dict_keys: List[str]

    def to_json(self) -> str:
        return json.dumps(self.__dict__)

    @classmethod
    def parse(cls, s: str) -> "ExportedProgramMetadata":
        try:
            d = json.loads(s)
            return cls(int(d["num_graph_nodes"]), [list(x) for x in d["input_shapes"]], list(d["output_shape"]), list(d["state_dict_keys"]))
        except (ValueError, KeyError, TypeError) as e:
            raise InvalidArgument(f"ExportedProgram metadata: {e}") from None


def program_metadata(program: ExportedProgram, state_dict_keys: Sequence[str] = ()) -> ExportedProgramMetadata:
    g = program.graph
    return ExportedProgramMetadata(len(g.nodes), [list(s) for s, _ in program.input_specs], list(g.values[g.outputs[0]].shape), sorted(state_dict_keys))


class DynamicExportedProgram:
    """An exported function with dynamic dimensions: inputs are checked against the :class:`InputSpec` list (rank, static extents, ranges, and
    equal runtime values for dimensions that share a name) and each distinct shape runs a graph traced for it (export.rs:130-260, 691)."""

    def __init__(self, f: Callable, example_inputs: Sequence[torch.Tensor], specs: Sequence[InputSpec]):
        if len(specs) != len(example_inputs):
            raise InvalidArgument(f"export_with_dynamic_shapes: {len(example_inputs)} inputs but {len(specs)} specs")
        self._f, self.input_specs = _fn_of(f), list(specs)
        self._programs: Dict[Tuple, ExportedProgram] = {}
        self.check_inputs(example_inputs)
        self.run(example_inputs)

    def check_inputs(self, inputs: Sequence[torch.Tensor]) -> None:
        if len(inputs) != len(self.input_specs):
            raise InvalidArgument(f"ExportedProgram: expected {len(self.input_specs)} inputs, got {len(inputs)}")
        bound: Dict[str, int] = {}
        for i, (t, spec) in enumerate(zip(inputs, self.input_specs)):
            if t.dim() != spec.rank():
                raise ShapeMismatch(f"ExportedProgram: input {i} has rank {t.dim()}, the spec has rank {spec.rank()}")
            for d, (n, ds) in enumerate(zip(t.shape, spec.shape)):
                if not ds.is_dynamic():
                    if n != ds.size:
                        raise ShapeMismatch(f"ExportedProgram: input {i} dim {d} must be {ds.size}, got {n}")
                    continue
                if (ds.min is not None and n < ds.min) or (ds.max is not None and n > ds.max):
                    raise ShapeMismatch(f"ExportedProgram: input {i} dim {d} ('{ds.name}') = {n} outside [{ds.min}, {ds.max}]")
                if bound.setdefault(ds.name, n) != n:
                    raise ShapeMismatch(f"ExportedProgram: dimension '{ds.name}' is {bound[ds.name]} in one place and {n} in another")

    def run(self, inputs: Sequence[torch.Tensor]):
        from .module import export
        key = tuple(tuple(t.shape) for t in inputs)
        if key not in self._programs:
            self._programs[key] = export(self._f, tuple(inputs))
        return self._programs[key](*inputs)

    def run_with_guards(self, inputs: Sequence[torch.Tensor]):
        self.check_inputs(inputs)
        return self.run(inputs)

    __call__ = lambda self, *a: self.run_with_guards(a)  # noqa: E731


def export_with_dynamic_shapes(f: Callable, example_inputs: Sequence[torch.Tensor], specs: Sequence[InputSpec]) -> DynamicExportedProgram:
    return DynamicExportedProgram(f, example_inputs, specs)


# ----------------------------------------------------------------------------------------------------------------------
# AOT autograd
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class AotGraphPair:
    """Forward and backward as separate graphs (aot_autograd.rs:29). ``forward`` returns the outputs followed by the saved values;
    ``backward`` takes (saved..., output gradients...) and returns one gradient per primal."""
    forward: IrGraph
    backward: IrGraph
    num_outputs: int
    num_saved: int
    saved_tensor_indices: List[int]      # positions, in the forward graph's topological order, of the nodes whose values are saved


def decompose_forward_backward(joint: Union[JointGraph, Callable], primals: Optional[Sequence[torch.Tensor]] = None) -> AotGraphPair:
    """Split a joint graph (inputs: primals + tangents; outputs: outputs + gradients) at the values the gradient half reads from the forward
    half. Nodes that depend on a tangent go to the backward graph, everything else to the forward graph (aot_autograd.rs:83)."""
    if not isinstance(joint, JointGraph):
        joint = aot_trace_joint(_fn_of(joint), primals)
    g, P, O = joint.graph, joint.num_primals, joint.num_outputs
    order = [n for n in g.topo_order() if n.op not in ("input", "constant", "output")]
    tainted = set(g.inputs[P:])
    bwd_nodes, fwd_nodes = [], []
    for n in order:
        if any(v in tainted for v in n.inputs):
            tainted |= set(n.outputs)
            bwd_nodes.append(n.id)
        else:
            fwd_nodes.append(n.id)
    fwd_produced = {o for nid in fwd_nodes for o in g.nodes[nid].outputs} | set(g.inputs[:P])
    saved = []
    for nid in bwd_nodes:
        for v in g.nodes[nid].inputs:
            if v in fwd_produced and v not in saved and v not in g.constants:
                saved.append(v)
    for o in g.outputs[O:]:                                   # a gradient that is itself a forward value (e.g. d(x*c)/dx = c broadcast)
        if o in fwd_produced and o not in saved and o not in g.constants:
            saved.append(o)
    fwd, _, fwd_out = _subgraph_io(g, fwd_nodes, list(g.inputs[:P]), list(g.outputs[:O]) + saved)
    bwd, _, _ = _subgraph_io(g, bwd_nodes, saved + list(g.inputs[P:]), list(g.outputs[O:]))
    pos = {n.id: i for i, n in enumerate(fwd.topo_order())}
    idx = []
    for v in fwd.outputs[O:]:
        p = fwd.values[v].producer
        idx.append(pos.get(p, -1) if p is not None else -1)
    return AotGraphPair(fwd, bwd, O, len(saved), idx)


def _subgraph_io(g: IrGraph, node_ids: List[int], inputs: List[int], outputs: List[int]):
    sub = IrGraph()
    remap: Dict[int, int] = {}
    for v in inputs:
        remap[v] = sub.add_input(g.values[v].shape, g.values[v].dtype).id
    for nid in node_ids:
        n = g.nodes[nid]
        for v in n.inputs:
            if v not in remap:
                if v not in g.constants:
                    raise JitError(f"decompose: value {v} is read before it is defined in this half")
                remap[v] = sub.add_constant(g.constants[v]).id
        m = sub.add_node(n.op, [remap[v] for v in n.inputs], [(g.values[o].shape, g.values[o].dtype) for o in n.outputs], **n.attrs)
        remap.update(zip(n.outputs, m.outputs))
    for v in outputs:
        if v not in remap:
            if v not in g.constants:
                raise JitError(f"decompose: output value {v} is not produced by this half")
            remap[v] = sub.add_constant(g.constants[v]).id
    sub.set_outputs([remap[v] for v in outputs])
    sub.single_output = False
    sub.validate()
    return sub, inputs, outputs


class AotCompiledModule:
    """Forward / backward pair compiled ahead of time (module.rs:315): ``forward_with_ctx`` runs the forward graph and keeps the saved
    values, ``backward`` turns an output gradient into input gradients without re-running the forward pass."""

    def __init__(self, pair: AotGraphPair):
        self.pair = pair
        self._fwd, self._bwd = TracedModule(pair.forward), TracedModule(pair.backward)
        self._saved: List[torch.Tensor] = []

    def forward_graph(self) -> IrGraph:
        return self.pair.forward

    def backward_graph(self) -> IrGraph:
        return self.pair.backward

    def saved_tensor_indices(self) -> List[int]:
        return list(self.pair.saved_tensor_indices)

    def saved_tensors(self) -> List[torch.Tensor]:
        return list(self._saved)

    def forward_with_ctx(self, inputs: Sequence[torch.Tensor]):
        res = self._fwd.forward_multi([t.detach() for t in inputs])
        res = list(res) if isinstance(res, tuple) else [res]
        self._saved = res[self.pair.num_outputs:]
        outs = res[: self.pair.num_outputs]
        return outs[0] if len(outs) == 1 else tuple(outs)

    def backward(self, *grad_outputs: torch.Tensor):
        if len(grad_outputs) != self.pair.num_outputs:
            raise InvalidArgument(f"AotCompiledModule.backward: {self.pair.num_outputs} output gradients expected, got {len(grad_outputs)}")
        if len(self._saved) != self.pair.num_saved:
            raise JitError("AotCompiledModule.backward called before forward_with_ctx")
        res = self._bwd.forward_multi(list(self._saved) + list(grad_outputs))
        return res


def compile_aot(f: Callable, example_inputs: Sequence[torch.Tensor], config: Optional[CompileConfig] = None) -> AotCompiledModule:
    pair = decompose_forward_backward(f, example_inputs)
    cfg = config or CompileConfig()
    for g in (pair.forward, pair.backward):
        optimize_with_config(g, OptimizationConfig(cfg.optimization.constant_folding, cfg.optimization.dead_code_elimination, cfg.optimization.operator_fusion, False))
    pos = {n.id: i for i, n in enumerate(pair.forward.topo_order())}      # positions in the optimised forward graph
    pair.saved_tensor_indices = [pos.get(pair.forward.values[v].producer, -1) for v in pair.forward.outputs[pair.num_outputs:]]
    return AotCompiledModule(pair)


# ----------------------------------------------------------------------------------------------------------------------
# code-generation backends
# ----------------------------------------------------------------------------------------------------------------------
class CompiledGraph:
    """A graph turned into something executable by a :class:`Codegen` backend (codegen.rs:41)."""

    def __init__(self, execute: Callable[[Sequence[torch.Tensor]], List[torch.Tensor]], num_inputs: int, output_shape: Tuple[int, ...], backend: str):
        self._execute, self._num_inputs, self._output_shape, self.backend = execute, num_inputs, tuple(output_shape), backend

    def num_inputs(self) -> int:
        return self._num_inputs

    def output_shape(self) -> Tuple[int, ...]:
        return self._output_shape

    def execute(self, inputs: Sequence[torch.Tensor]):
        if len(inputs) != self._num_inputs:
            raise InvalidArgument(f"CompiledGraph: expected {self._num_inputs} inputs, got {len(inputs)}")
        out = self._execute(list(inputs))
        return out[0] if len(out) == 1 else tuple(out)

    __call__ = lambda self, *a: self.execute(a)  # noqa: E731


class Codegen:
    """Backend interface: ``compile(graph) -> CompiledGraph`` and a ``name`` (codegen.rs:98)."""

    def name(self) -> str:
        raise NotImplementedError

    def compile(self, graph: IrGraph) -> CompiledGraph:  # noqa: A003
        raise NotImplementedError

    @staticmethod
    def _shape(graph: IrGraph) -> Tuple[int, ...]:
        return tuple(graph.values[graph.outputs[0]].shape) if graph.outputs else ()


class InterpreterBackend(Codegen):
    """Node-by-node evaluation; always available, the fallback of the others."""

    def name(self) -> str:
        return "interpreter"

    def compile(self, graph: IrGraph) -> CompiledGraph:  # noqa: A003
        graph.validate()
        return CompiledGraph(lambda xs: list(run_graph(graph, xs)), len(graph.inputs), self._shape(graph), self.name())


def _clone_graph(g: IrGraph) -> IrGraph:
    c = IrGraph.from_json(g.to_json())
    if hasattr(g, "single_output"):
        c.single_output = g.single_output
    return c


class NativeBackend(Codegen):
    """Fuses elementwise regions and reductions and runs them as compiled host kernels (C++ built with the system compiler, cached by source
    hash); other nodes run on the interpreter."""

    def name(self) -> str:
        return "native"

    def compile(self, graph: IrGraph) -> CompiledGraph:  # noqa: A003
        g = _clone_graph(graph)
        passes.optimize(g, fuse=True)
        exe = _Executable(g, "host", CompileStats())
        cg = CompiledGraph(lambda xs: exe.run(xs), len(g.inputs), self._shape(g), self.name())
        cg.fused_kernels = exe.stats.fused_kernels
        return cg


class InductorTarget(enum.Enum):
    """Where generated code runs (codegen.rs:756). The reference's ``CpuRust`` target emits Rust; the host target here emits C++."""
    CpuCpp = "cpu_cpp"
    GpuCuda = "gpu_cuda"
    GpuPtx = "gpu_ptx"


InductorTarget.CpuRust = InductorTarget.CpuCpp                # the reference's spelling of the host target


class InductorCompileStatus:
    """``Compiled(graph)`` when code generation produced kernels, ``FellBackToInterpreter(graph)`` when it could not (codegen.rs:978)."""

    def __init__(self, compiled: CompiledGraph, fell_back: bool, reason: str = ""):
        self.compiled, self.fell_back, self.reason = compiled, fell_back, reason

    def is_compiled(self) -> bool:
        return not self.fell_back

    def into_compiled(self) -> CompiledGraph:
        return self.compiled


class InductorBackend(Codegen):
    """Fusing code generator with a selectable target. ``GpuCuda`` / ``GpuPtx`` build sm_100a kernels with NVRTC and need CUDA inputs at
    run time; when kernels cannot be built the graph still runs, on the interpreter, and the status says so."""

    def __init__(self, target: InductorTarget = InductorTarget.CpuCpp):
        self.target = target

    def name(self) -> str:
        return f"inductor-{self.target.value}"

    def compile_with_status(self, graph: IrGraph) -> InductorCompileStatus:
        g = _clone_graph(graph)
        passes.optimize(g, fuse=True)
        backend = "host" if self.target is InductorTarget.CpuCpp else "cuda"
        try:
            if backend == "cuda" and not torch.cuda.is_available():
                raise JitError("no CUDA device: sm_100a kernels can be generated but not loaded")
            exe = _Executable(g, backend, CompileStats())
            return InductorCompileStatus(CompiledGraph(lambda xs: exe.run(xs), len(g.inputs), self._shape(g), self.name()), False)
        except FerrotorchError as e:
            return InductorCompileStatus(InterpreterBackend().compile(graph), True, str(e))

    def compile(self, graph: IrGraph) -> CompiledGraph:  # noqa: A003
        return self.compile_with_status(graph).into_compiled()


# ----------------------------------------------------------------------------------------------------------------------
# loop IR and its emitters
# ----------------------------------------------------------------------------------------------------------------------
class BinOpKind(enum.Enum):
    Add = "+"
    Sub = "-"
    Mul = "*"
    Div = "/"
    Mod = "%"

    def __str__(self):
        return self.value


class UnaryOpKind(enum.Enum):
    Neg = "neg"
    Exp = "exp"
    Log = "log"
    Sqrt = "sqrt"
    Abs = "abs"
    Sigmoid = "sigmoid"
    Tanh = "tanh"
    Relu = "relu"
    Gelu = "gelu"
    Silu = "silu"

    def __str__(self):
        return self.value


class Expr:
    """Scalar expression tree of the loop IR (codegen_ir.rs:25): ``Var``, ``Const``, ``IntConst``, ``BinOp``, ``UnaryOp``, ``FnCall``, ``Index``
    (``buffer[index]``), ``Cast``. Built with the class methods; ``kind`` names the variant."""

    def __init__(self, kind: str, **kw):
        self.kind = kind
        self.__dict__.update(kw)

    @classmethod
    def Var(cls, name: str): return cls("Var", name=name)                                                # noqa: E704,N802
    @classmethod
    def Const(cls, v: float): return cls("Const", value=float(v))                                        # noqa: E704,N802
    @classmethod
    def IntConst(cls, v: int): return cls("IntConst", value=int(v))                                      # noqa: E704,N802
    @classmethod
    def BinOp(cls, op: BinOpKind, lhs: "Expr", rhs: "Expr"): return cls("BinOp", op=op, lhs=lhs, rhs=rhs)    # noqa: E704,N802
    @classmethod
    def UnaryOp(cls, op: UnaryOpKind, operand: "Expr"): return cls("UnaryOp", op=op, operand=operand)        # noqa: E704,N802
    @classmethod
    def FnCall(cls, name: str, args: Sequence["Expr"]): return cls("FnCall", name=name, args=list(args))     # noqa: E704,N802
    @classmethod
    def Index(cls, buffer: str, index: "Expr"): return cls("Index", buffer=buffer, index=index)              # noqa: E704,N802
    @classmethod
    def Cast(cls, target_type: str, operand: "Expr"): return cls("Cast", target_type=target_type, operand=operand)   # noqa: E704,N802

    def __eq__(self, o):
        return isinstance(o, Expr) and self.__dict__ == o.__dict__

    def __repr__(self):
        return f"Expr.{self.kind}({', '.join(f'{k}={v!r}' for k, v in self.__dict__.items() if k != 'kind')})"


class LoopIR:
    """Statement of the loop IR (codegen_ir.rs:120): ``Loop`` (var, start, end, body), ``Store`` (buffer[index] = value), ``Let``, ``Assign``,
    ``Accumulate`` (var += value), ``If``, ``Comment``."""

    def __init__(self, kind: str, **kw):
        self.kind = kind
        self.__dict__.update(kw)

    @classmethod
    def Loop(cls, var: str, start: Expr, end: Expr, body: Sequence["LoopIR"]): return cls("Loop", var=var, start=start, end=end, body=list(body))   # noqa: E704,N802
    @classmethod
    def Store(cls, buffer: str, index: Expr, value: Expr): return cls("Store", buffer=buffer, index=index, value=value)    # noqa: E704,N802
    @classmethod
    def Let(cls, var: str, value: Expr): return cls("Let", var=var, value=value)                          # noqa: E704,N802
    @classmethod
    def Assign(cls, var: str, value: Expr): return cls("Assign", var=var, value=value)                    # noqa: E704,N802
    @classmethod
    def Accumulate(cls, var: str, value: Expr): return cls("Accumulate", var=var, value=value)            # noqa: E704,N802
    @classmethod
    def If(cls, condition: Expr, then_body: Sequence["LoopIR"], else_body: Sequence["LoopIR"] = ()):      # noqa: N802
        return cls("If", condition=condition, then_body=list(then_body), else_body=list(else_body))
    @classmethod
    def Comment(cls, text: str): return cls("Comment", text=text)                                         # noqa: E704,N802

    def __eq__(self, o):
        return isinstance(o, LoopIR) and self.__dict__ == o.__dict__

    def __repr__(self):
        return f"LoopIR.{self.kind}"


_IDENT = re.compile(r"^[A-Za-z_][A-Za-z0-9_]*$")
_FN_OK = {"exp", "log", "sqrt", "fabs", "tanh", "sin", "cos", "pow", "fmax", "fmin", "floor", "ceil", "erf", "fma", "expm1", "log1p"}


def _ident(s: str, what: str) -> str:
    if not _IDENT.match(s):
        raise InvalidArgument(f"{what} {s!r} is not a valid identifier")
    return s


def _buf(name: str) -> str:
    """Buffer names of a kernel: ``in<k>`` is input ``k``, ``out`` the output."""
    if name == "out":
        return "out"
    m = re.fullmatch(r"in(\d+)", name)
    if not m:
        raise InvalidArgument(f"loop IR buffer {name!r}: buffers are named in0, in1, ... and out")
    return f"in[{int(m.group(1))}]"


def _emit_expr(e: Expr) -> str:
    k = e.kind
    if k == "Var":
        return _ident(e.name, "variable")
    if k == "Const":
        return repr(float(e.value)) if e.value == e.value and abs(e.value) != float("inf") else ("NAN" if e.value != e.value else ("INFINITY" if e.value > 0 else "-INFINITY"))
    if k == "IntConst":
        return f"{int(e.value)}LL"
    if k == "BinOp":
        a, b = _emit_expr(e.lhs), _emit_expr(e.rhs)
        if e.op is BinOpKind.Mod:
            return f"ft_mod({a}, {b})"
        return f"({a} {e.op.value} {b})"
    if k == "UnaryOp":
        x = _emit_expr(e.operand)
        return {UnaryOpKind.Neg: f"(-{x})", UnaryOpKind.Exp: f"exp({x})", UnaryOpKind.Log: f"log({x})", UnaryOpKind.Sqrt: f"sqrt({x})",
                UnaryOpKind.Abs: f"fabs({x})", UnaryOpKind.Sigmoid: f"(1.0 / (1.0 + exp(-({x}))))", UnaryOpKind.Tanh: f"tanh({x})",
                UnaryOpKind.Relu: f"fmax({x}, 0.0)", UnaryOpKind.Gelu: f"(0.5 * ({x}) * (1.0 + erf(({x}) * 0.7071067811865476)))",
                UnaryOpKind.Silu: f"(({x}) / (1.0 + exp(-({x}))))"}[e.op]
    if k == "FnCall":
        if e.name not in _FN_OK:
            raise InvalidArgument(f"loop IR: unknown function {e.name!r} (known: {sorted(_FN_OK)})")
        return f"{e.name}({', '.join(_emit_expr(a) for a in e.args)})"
    if k == "Index":
        return f"{_buf(e.buffer)}[{_emit_expr(e.index)}]"
    if k == "Cast":
        t = {"f64": "double", "f32": "float", "i64": "long long", "i32": "int", "usize": "long long"}.get(e.target_type)
        if t is None:
            raise InvalidArgument(f"loop IR: unknown cast target {e.target_type!r}")
        return f"(({t})({_emit_expr(e.operand)}))"
    raise InvalidArgument(f"loop IR: unknown expression kind {k}")


def _emit_stmt(s: LoopIR, out: List[str], depth: int, declared: set) -> None:
    pad = "    " * depth
    k = s.kind
    if k == "Comment":
        out.append(f"{pad}// {s.text}".replace("\n", " "))
    elif k == "Loop":
        v = _ident(s.var, "loop variable")
        out.append(f"{pad}for (long long {v} = {_emit_expr(s.start)}; {v} < {_emit_expr(s.end)}; ++{v}) {{")
        inner = set(declared) | {v}
        for b in s.body:
            _emit_stmt(b, out, depth + 1, inner)
        out.append(f"{pad}}}")
    elif k == "Store":
        out.append(f"{pad}{_buf(s.buffer)}[{_emit_expr(s.index)}] = {_emit_expr(s.value)};")
    elif k == "Let":
        v = _ident(s.var, "variable")
        out.append(f"{pad}double {v} = {_emit_expr(s.value)};")
        declared.add(v)
    elif k == "Assign":
        out.append(f"{pad}{_ident(s.var, 'variable')} = {_emit_expr(s.value)};")
    elif k == "Accumulate":
        out.append(f"{pad}{_ident(s.var, 'variable')} += {_emit_expr(s.value)};")
    elif k == "If":
        out.append(f"{pad}if ({_emit_expr(s.condition)}) {{")
        for b in s.then_body:
            _emit_stmt(b, out, depth + 1, set(declared))
        if s.else_body:
            out.append(f"{pad}}} else {{")
            for b in s.else_body:
                _emit_stmt(b, out, depth + 1, set(declared))
        out.append(f"{pad}}}")
    else:
        raise InvalidArgument(f"loop IR: unknown statement kind {k}")


_LOOP_PRELUDE = "#include <cmath>\nstatic inline double ft_mod(double a, double b) { return std::fmod(a, b); }\nstatic inline long long ft_mod(long long a, long long b) { return a % b; }\nusing namespace std;\n"


class CpuCodegen:
    """Loop IR -> C++ source of ``extern "C" void <fn>(const double* const* in, double* out, int n)`` (codegen_cpu.rs:36; the reference
    emits Rust with the same buffer convention)."""

    @staticmethod
    def generate_cpp_source(loops: Sequence[LoopIR], fn_name: str) -> str:
        _ident(fn_name, "function name")
        lines = [_LOOP_PRELUDE, f'extern "C" void {fn_name}(const double* const* in, double* out, int n) {{', "    (void)n;"]
        declared: set = set()
        for s in loops:
            _emit_stmt(s, lines, 1, declared)
        lines.append("}")
        return "\n".join(lines) + "\n"

    generate_source = generate_cpp_source
    generate_rust_source = generate_cpp_source                # the reference's method name; the language here is C++


class GpuCodegen:
    """Loop IR -> CUDA C++ (codegen_gpu.rs:75): the outermost loop becomes the grid-stride loop of a kernel, inner statements are emitted as
    they are; :meth:`generate_ptx_source` compiles that source for sm_100a with NVRTC."""

    @staticmethod
    def generate_cuda_source(loops: Sequence[LoopIR], kernel_name: str, block_size: int = 256) -> str:
        _ident(kernel_name, "kernel name")
        lines = ["__device__ inline double ft_mod(double a, double b) { return fmod(a, b); }", "__device__ inline long long ft_mod(long long a, long long b) { return a % b; }",
                 f'extern "C" __global__ void __launch_bounds__({int(block_size)}) {kernel_name}(const double* const* in, double* out, int n) {{']
        declared: set = set()
        for s in loops:
            if s.kind == "Loop":
                v = _ident(s.var, "loop variable")
                lines.append(f"    for (long long {v} = {_emit_expr(s.start)} + blockIdx.x * (long long)blockDim.x + threadIdx.x; {v} < {_emit_expr(s.end)}; "
                             f"{v} += (long long)gridDim.x * blockDim.x) {{")
                for b in s.body:
                    _emit_stmt(b, lines, 2, set(declared) | {v})
                lines.append("    }")
            else:
                _emit_stmt(s, lines, 1, declared)
        lines.append("}")
        return "\n".join(lines) + "\n"

    @staticmethod
    def generate_ptx_source(loops: Sequence[LoopIR], kernel_name: str, block_size: int = 256) -> bytes:
        return _cg.compile_cuda(GpuCodegen.generate_cuda_source(loops, kernel_name, block_size))


class JitCompiledKernel:
    """A loop-IR kernel compiled for the host: ``execute(inputs)`` takes f64 tensors (or lists) and returns the f64 output of ``output_len``
    elements (codegen_jit.rs:91)."""

    def __init__(self, fn, lib, num_inputs: int, output_len: int, source: str):
        self._fn, self._lib, self._num_inputs, self._output_len, self.source = fn, lib, num_inputs, output_len, source

    def num_inputs(self) -> int:
        return self._num_inputs

    def output_len(self) -> int:
        return self._output_len

    def execute(self, inputs: Sequence) -> torch.Tensor:
        if len(inputs) != self._num_inputs:
            raise InvalidArgument(f"JitCompiledKernel: expected {self._num_inputs} inputs, got {len(inputs)}")
        ts = [torch.as_tensor(x, dtype=torch.float64).contiguous() for x in inputs]
        out = torch.zeros(self._output_len, dtype=torch.float64)
        ptrs = (ctypes.c_void_p * max(len(ts), 1))(*[t.data_ptr() for t in ts])
        self._fn(ptrs, ctypes.c_void_p(out.data_ptr()), ctypes.c_int(self._output_len))
        return out


def compile_loop_ir_kernel(loops: Sequence[LoopIR], num_inputs: int, output_len: int) -> JitCompiledKernel:
    """Build a host kernel from loop IR with the system C++ compiler (the reference JITs through Cranelift; codegen_jit.rs:261). Shared
    objects are cached by source hash beside the other generated kernels."""
    used = set()

    def scan_e(e: Expr):
        if e.kind == "Index":
            used.add(e.buffer)
        for v in e.__dict__.values():
            if isinstance(v, Expr):
                scan_e(v)
            elif isinstance(v, list):
                [scan_e(x) for x in v if isinstance(x, Expr)]

    def scan_s(s: LoopIR):
        if s.kind == "Store":
            used.add(s.buffer)
        for v in s.__dict__.values():
            if isinstance(v, Expr):
                scan_e(v)
            elif isinstance(v, list):
                for x in v:
                    scan_s(x) if isinstance(x, LoopIR) else (scan_e(x) if isinstance(x, Expr) else None)
    [scan_s(s) for s in loops]
    for b in used:
        m = re.fullmatch(r"in(\d+)", b)
        if m and int(m.group(1)) >= num_inputs:
            raise InvalidArgument(f"loop IR reads {b} but the kernel has {num_inputs} inputs")
    src = CpuCodegen.generate_cpp_source(loops, "ft_loop_kernel")
    key = hashlib.sha256((_cg._HOST_FLAGS_TAG + src).encode()).hexdigest()
    d = _cg._cache_dir
    d.mkdir(parents=True, exist_ok=True)
    so = d / f"loop_{key}.so"
    if not so.exists():
        cpp = d / f"loop_{key}.cpp"
        cpp.write_text(src)
        tmp = d / f"loop_{key}.{os.getpid()}.tmp.so"
        r = subprocess.run([os.environ.get("CXX", "g++"), "-O3", "-march=native", "-fno-math-errno", "-shared", "-fPIC", "-std=c++17", str(cpp), "-o", str(tmp)],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise JitError("loop-IR kernel compilation failed:\n" + r.stderr + "\n--- source ---\n" + src)
        os.replace(tmp, so)
    lib = ctypes.CDLL(str(so))
    fn = lib.ft_loop_kernel
    fn.restype = None
    return JitCompiledKernel(fn, lib, num_inputs, output_len, src)


def lower_to_loops(graph: IrGraph) -> List[LoopIR]:
    """Loop IR of a graph made of elementwise operations over equally-shaped inputs (and an optional final full reduction ``sum`` / ``mean`` /
    ``prod`` to a scalar): one loop, one ``Let`` per node (codegen_ir.rs:378). Other graphs are refused."""
    un = {"neg": UnaryOpKind.Neg, "exp": UnaryOpKind.Exp, "log": UnaryOpKind.Log, "sqrt": UnaryOpKind.Sqrt, "abs": UnaryOpKind.Abs, "sigmoid": UnaryOpKind.Sigmoid,
          "tanh": UnaryOpKind.Tanh, "relu": UnaryOpKind.Relu, "gelu": UnaryOpKind.Gelu, "silu": UnaryOpKind.Silu}
    bi = {"add": BinOpKind.Add, "sub": BinOpKind.Sub, "mul": BinOpKind.Mul, "div": BinOpKind.Div, "fmod": BinOpKind.Mod}
    order = [n for n in graph.topo_order() if n.op not in ("input", "constant", "output")]
    if len(graph.outputs) != 1 or not order:
        raise InvalidArgument("lower_to_loops: one output and at least one operation expected")
    shape = tuple(graph.values[graph.inputs[0]].shape) if graph.inputs else ()
    numel = 1
    for d in shape:
        numel *= d
    i = Expr.Var("i")
    name: Dict[int, Expr] = {v: Expr.Index(f"in{k}", i) for k, v in enumerate(graph.inputs)}
    for v, t in graph.constants.items():
        if t.numel() != 1:
            raise InvalidArgument("lower_to_loops: only scalar constants are supported")
        name[v] = Expr.Const(float(t))
    body: List[LoopIR] = []
    red = None
    for n in order:
        if n.op in un and tuple(graph.values[n.outputs[0]].shape) == shape:
            e = Expr.UnaryOp(un[n.op], name[n.inputs[0]])
        elif n.op in bi and tuple(graph.values[n.outputs[0]].shape) == shape:
            e = Expr.BinOp(bi[n.op], name[n.inputs[0]], name[n.inputs[1]])
        elif n.op in ("sum", "mean", "prod") and n is order[-1] and graph.values[n.outputs[0]].numel() == 1:
            red = (n.op, name[n.inputs[0]])
            break
        else:
            raise InvalidArgument(f"lower_to_loops: operation '{n.op}' is outside the elementwise / full-reduction subset")
        var = f"t{n.outputs[0]}"
        body.append(LoopIR.Let(var, e))
        name[n.outputs[0]] = Expr.Var(var)
    if red is None:
        body.append(LoopIR.Store("out", i, name[graph.outputs[0]]))
        return [LoopIR.Loop("i", Expr.IntConst(0), Expr.IntConst(numel), body)]
    op, val = red
    acc = [LoopIR.Let("acc", Expr.Const(1.0 if op == "prod" else 0.0))]
    body.append(LoopIR.Assign("acc", Expr.BinOp(BinOpKind.Mul, Expr.Var("acc"), val)) if op == "prod" else LoopIR.Accumulate("acc", val))
    fin = Expr.BinOp(BinOpKind.Div, Expr.Var("acc"), Expr.Const(float(max(numel, 1)))) if op == "mean" else Expr.Var("acc")
    return acc + [LoopIR.Loop("i", Expr.IntConst(0), Expr.IntConst(numel), body), LoopIR.Store("out", Expr.IntConst(0), fin)]


# ----------------------------------------------------------------------------------------------------------------------
# fused unary chains and reduction kernels (fusion.rs)
# ----------------------------------------------------------------------------------------------------------------------
class FusionGroupKind(enum.Enum):
    """What a fusion group of the DAG pass contains (dag_fusion.rs): pure elementwise work, or elementwise work feeding a reduction."""
    Elementwise = "elementwise"
    Reduction = "reduction"
    Opaque = "opaque"


class ReductionKind(enum.Enum):
    Sum = "sum"
    Prod = "prod"
    Mean = "mean"


class FusedOp:
    """One step of a :class:`FusedChain` (fusion.rs:88): unary ``Neg Relu Sigmoid Tanh Gelu Silu Sqrt Abs Exp Log``, parameterised
    ``Pow(p) ScalarMul(c) ScalarAdd(c)``, and the binary markers ``Add Sub Mul Div`` (applied with the chain's second operand)."""

    def __init__(self, name: str, param: Optional[float] = None):
        self.name, self.param = name, param

    def __eq__(self, o):
        return isinstance(o, FusedOp) and (self.name, self.param) == (o.name, o.param)

    def __hash__(self):
        return hash((self.name, self.param))

    def __repr__(self):
        return f"FusedOp.{self.name}" + (f"({self.param})" if self.param is not None else "")

    @classmethod
    def Pow(cls, p: float): return cls("Pow", float(p))                   # noqa: E704,N802
    @classmethod
    def ScalarMul(cls, c: float): return cls("ScalarMul", float(c))       # noqa: E704,N802
    @classmethod
    def ScalarAdd(cls, c: float): return cls("ScalarAdd", float(c))       # noqa: E704,N802


for _n in ("Add", "Sub", "Mul", "Div", "Neg", "Relu", "Sigmoid", "Tanh", "Gelu", "Silu", "Sqrt", "Abs", "Exp", "Log"):
    setattr(FusedOp, _n, FusedOp(_n))

_CHAIN_IR = {"Neg": "neg", "Relu": "relu", "Sigmoid": "sigmoid", "Tanh": "tanh", "Gelu": "gelu", "Silu": "silu", "Sqrt": "sqrt", "Abs": "abs", "Exp": "exp",
             "Log": "log", "Add": "add", "Sub": "sub", "Mul": "mul", "Div": "div"}


class FusedChain:
    """A sequence of elementwise steps applied in one pass over the data (fusion.rs:201)."""

    def __init__(self, ops: Sequence[FusedOp] = ()):
        self._ops = list(ops)

    def push(self, op: FusedOp) -> "FusedChain":
        self._ops.append(op)
        return self

    def ops(self) -> List[FusedOp]:
        return list(self._ops)

    def __len__(self):
        return len(self._ops)

    def is_empty(self) -> bool:
        return not self._ops

    def needs_second_operand(self) -> bool:
        return any(o.name in ("Add", "Sub", "Mul", "Div") for o in self._ops)

    def to_graph(self, shape: Sequence[int], dtype: torch.dtype) -> IrGraph:
        g = IrGraph()
        cur = g.add_input(shape, dtype).id
        other = g.add_input(shape, dtype).id if self.needs_second_operand() else None
        spec = [(tuple(shape), dtype)]
        for o in self._ops:
            if o.name in ("Pow", "ScalarMul", "ScalarAdd"):
                c = g.add_constant(torch.tensor(o.param, dtype=dtype)).id
                cur = g.add_node({"Pow": "pow", "ScalarMul": "mul", "ScalarAdd": "add"}[o.name], [cur, c], spec).outputs[0]
            elif o.name in ("Add", "Sub", "Mul", "Div"):
                cur = g.add_node(_CHAIN_IR[o.name], [cur, other], spec).outputs[0]
            else:
                cur = g.add_node(_CHAIN_IR[o.name], [cur], spec).outputs[0]
        g.set_outputs([cur])
        return g


_fusion_state = threading.local()
_chain_kernels: Dict[Tuple, Any] = {}


def is_fusion_enabled() -> bool:
    return getattr(_fusion_state, "on", False)


@contextlib.contextmanager
def _fusion_scope():
    prev = is_fusion_enabled()
    _fusion_state.on = True
    try:
        yield
    finally:
        _fusion_state.on = prev


def with_fusion(f: Optional[Callable] = None):
    """``with_fusion(fn)`` runs ``fn`` with chain fusion switched on for this thread and restores the previous setting afterwards, also when
    ``fn`` raises (fusion.rs:62); without an argument it is the same thing as a context manager."""
    if f is None:
        return _fusion_scope()
    with _fusion_scope():
        return f()


def apply_fused(x: torch.Tensor, chain: FusedChain, other: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All steps of ``chain`` in one generated kernel over ``x`` (host C++ for CPU tensors, NVRTC sm_100a for CUDA tensors), on the device of
    the input (fusion.rs:1251). An empty chain returns ``x`` unchanged."""
    if chain.is_empty():
        return x
    if chain.needs_second_operand():
        if other is None or other.shape != x.shape:
            raise InvalidArgument("apply_fused: the chain has a binary step and needs a second operand of the same shape")
    if x.dtype not in (torch.float32, torch.float64, torch.bfloat16, torch.float16):
        raise InvalidArgument(f"apply_fused: floating tensors only, got {x.dtype}")
    key = (tuple(chain.ops()), tuple(x.shape), x.dtype, x.device.type)
    k = _chain_kernels.get(key)
    if k is None:
        body = chain.to_graph(tuple(x.shape), x.dtype)
        k = (_cg.CudaFusedKernel if x.is_cuda else _cg.HostFusedKernel)(body)
        _chain_kernels[key] = k
    ins = [x.contiguous()] + ([other.contiguous()] if chain.needs_second_operand() else [])
    return k(ins)[0]


def estimate_numel_for_inputs(shapes: Sequence[Sequence[int]]) -> int:
    best = 0
    for s in shapes:
        n = 1
        for d in s:
            n *= d
        best = max(best, n)
    return best


def estimate_matmul_dims(lhs_shape: Sequence[int], rhs_shape: Sequence[int]) -> Tuple[int, int, int]:
    """``(M, K, N)`` of a 2-D product, checking that the inner dimensions agree (fusion.rs:1162)."""
    if len(lhs_shape) != 2 or len(rhs_shape) != 2:
        raise InvalidArgument(f"estimate_matmul_dims: 2-D shapes expected, got {list(lhs_shape)} and {list(rhs_shape)}")
    if lhs_shape[1] != rhs_shape[0]:
        raise InvalidArgument(f"estimate_matmul_dims: inner dimensions differ ({lhs_shape[1]} vs {rhs_shape[0]})")
    return lhs_shape[0], lhs_shape[1], rhs_shape[1]


def generate_reduction_c(kind: ReductionKind, fn_name: str) -> str:
    """C source of ``float <fn>(const float* x, long n)``: a SIMD-annotated full reduction (fusion.rs:753)."""
    _ident(fn_name, "function name")
    ident, clause, step = {ReductionKind.Sum: ("0.0f", "+", "acc += x[i];"), ReductionKind.Mean: ("0.0f", "+", "acc += x[i];"),
                           ReductionKind.Prod: ("1.0f", "*", "acc *= x[i];")}[kind]
    fin = "return n > 0 ? acc / (float)n : 0.0f / 0.0f;" if kind is ReductionKind.Mean else "return acc;"
    return (f"float {fn_name}(const float* x, long n) {{\n    float acc = {ident};\n    #pragma omp simd reduction({clause}:acc)\n"
            f"    for (long i = 0; i < n; ++i) {{ {step} }}\n    {fin}\n}}\n")


def generate_reduction_cuda(kind: ReductionKind, kernel_name: str) -> str:
    """CUDA source of a block-parallel full reduction: warp shuffles, one shared-memory stage, one atomic per block into ``out[0]`` (which
    the caller sets to the identity; ``Mean`` divides by ``n`` inside the last step of each block's contribution)."""
    _ident(kernel_name, "kernel name")
    op = "*" if kind is ReductionKind.Prod else "+"
    ident = "1.0f" if kind is ReductionKind.Prod else "0.0f"
    scale = " / (float)n" if kind is ReductionKind.Mean else ""
    merge = ("unsigned int* a = (unsigned int*)out; unsigned int old = *a, assumed; do { assumed = old; old = atomicCAS(a, assumed, __float_as_uint(__uint_as_float(assumed) * v)); } "
             "while (assumed != old);") if kind is ReductionKind.Prod else "atomicAdd(out, v);"
    return (f'extern "C" __global__ void {kernel_name}(const float* x, float* out, long n) {{\n'
            f"    __shared__ float warp_acc[32];\n    float v = {ident};\n"
            f"    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) v = v {op} x[i];\n"
            f"    for (int o = 16; o > 0; o >>= 1) v = v {op} __shfl_down_sync(0xffffffffu, v, o);\n"
            f"    if ((threadIdx.x & 31) == 0) warp_acc[threadIdx.x >> 5] = v;\n    __syncthreads();\n"
            f"    if (threadIdx.x < 32) {{\n        v = threadIdx.x < (blockDim.x + 31) / 32 ? warp_acc[threadIdx.x] : {ident};\n"
            f"        for (int o = 16; o > 0; o >>= 1) v = v {op} __shfl_down_sync(0xffffffffu, v, o);\n"
            f"        if (threadIdx.x == 0) {{ v = v{scale}; {merge} }}\n    }}\n}}\n")


def generate_reduction_ptx(kind: ReductionKind, kernel_name: str) -> bytes:
    """The reduction kernel compiled for sm_100a with NVRTC (fusion.rs:816 writes the PTX text by hand; here the compiler does)."""
    return _cg.compile_cuda(generate_reduction_cuda(kind, kernel_name))


# ----------------------------------------------------------------------------------------------------------------------
# graph autotuning (autotune.rs)
# ----------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class AutotuneKey:
    """Structure of the graph plus the input shapes (autotune.rs:77)."""
    graph_fingerprint: str
    input_shapes: Tuple[Tuple[int, ...], ...]

    @classmethod
    def from_graph(cls, graph: IrGraph, input_shapes: Sequence[Sequence[int]]) -> "AutotuneKey":
        return cls(graph.fingerprint(), tuple(tuple(s) for s in input_shapes))


@dataclass
class AutotuneCandidate:
    _name: str
    backend: Codegen

    def name(self) -> str:
        return self._name


@dataclass
class AutotuneResult:
    _winner: str
    _time_s: float
    _compiled: CompiledGraph
    _timings: List[Tuple[str, float]]

    def winner_name(self) -> str:
        return self._winner

    def winner_time(self) -> float:
        return self._time_s

    def winner_compiled(self) -> CompiledGraph:
        return self._compiled

    def all_timings(self) -> List[Tuple[str, float]]:
        return list(self._timings)


class Autotuner(_BaseAutotuner):
    """Two uses. ``Autotuner().with_candidate(name, backend)...tune(graph, inputs)`` compiles the graph with every candidate backend, times
    them (warm-up, then the mean of ``iterations`` runs; CUDA inputs are timed with events) and caches the winner per
    :class:`AutotuneKey` (autotune.rs:172). ``tune(key, candidates, make)`` is the configuration sweep of the base class."""

    def __init__(self, cache_path: Optional[str] = None, warmup: int = 2, iters: int = 5):
        super().__init__(cache_path, warmup, iters)
        self._candidates: List[AutotuneCandidate] = []
        self._graph_cache: Dict[AutotuneKey, Tuple[str, float]] = {}
        self._lock = threading.Lock()

    def with_candidate(self, name: str, backend: Codegen) -> "Autotuner":
        self._candidates.append(AutotuneCandidate(name, backend))
        return self

    def with_iterations(self, iterations: int) -> "Autotuner":
        self.iters = max(int(iterations), 1)
        return self

    def with_warmup(self, warmup: int) -> "Autotuner":
        self.warmup = max(int(warmup), 0)
        return self

    def iterations(self) -> int:
        return self.iters

    def candidate_count(self) -> int:
        return len(self._candidates)

    def cached(self, key: AutotuneKey) -> Optional[Tuple[str, float]]:
        with self._lock:
            return self._graph_cache.get(key)

    def clear_cache(self) -> None:
        with self._lock:
            self._graph_cache.clear()

    def cache_size(self) -> int:
        with self._lock:
            return len(self._graph_cache)

    def tune(self, graph, inputs, make=None):  # noqa: D401
        if not isinstance(graph, IrGraph):
            return super().tune(graph, inputs, make)
        if not self._candidates:
            raise InvalidArgument("Autotuner.tune: no candidates registered")
        ins = [torch.as_tensor(x) for x in inputs]
        key = AutotuneKey.from_graph(graph, [tuple(t.shape) for t in ins])
        timings, compiled = [], {}
        for c in self._candidates:
            try:
                cg = c.backend.compile(graph)
                t = self._time(lambda: cg.execute(ins)) * 1e-3
            except FerrotorchError:
                continue
            timings.append((c.name(), t))
            compiled[c.name()] = cg
        if not timings:
            raise JitError("Autotuner.tune: every candidate failed to compile or run")
        winner, best = min(timings, key=lambda p: p[1])
        with self._lock:
            self._graph_cache[key] = (winner, best)
        return AutotuneResult(winner, best, compiled[winner], timings)
