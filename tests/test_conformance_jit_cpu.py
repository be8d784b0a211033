"""Per-symbol behaviour checks of ``ferrotorch_b200.jit``: graph builder and script front-end, interpreter, optimisation passes one by one,
fusion grouping and generated host kernels, joint forward/backward capture, memory planning, guards / shape environments and the result
record types of compilation and tuning."""
import pytest
import torch

import ferrotorch_b200.jit as J
from ferrotorch_b200.errors import FerrotorchError


def test_graph_builder_script_and_interpreter():
    b = J.GraphBuilder()
    x, w = b.input((4, 8)), b.input((8, 3))
    assert isinstance(x, J.Value) and x.shape == (4, 8)
    h = b.unary("tanh", b.matmul(x, w))
    y = b.binary("add", h, b.constant(1.0)).softmax(-1).sum(-1)
    g = b.finish([y])
    assert isinstance(g, J.IrGraph) and all(isinstance(n, J.IrNode) for n in g.nodes.values()) and all(isinstance(v, J.IrValue) for v in g.values.values())
    xs, ws = torch.randn(4, 8), torch.randn(8, 3)
    out = J.Interpreter(g)(xs, ws)
    assert torch.allclose(out, torch.softmax(torch.tanh(xs @ ws) + 1, -1).sum(-1), atol=1e-6)

    @J.script(((5,), torch.float32), ((5,), torch.float32))
    def fma(a, c, builder):
        return builder.binary("add", builder.binary("mul", a, c), a)
    assert isinstance(fma, J.ScriptedFunction) and fma.name == "fma"
    p, q = torch.randn(5), torch.randn(5)
    assert torch.allclose(fma(p, q), p * q + p)


def test_passes_one_by_one():
    x = torch.randn(3, 4)
    g = J.trace(lambda t: ((t * 1.0 + 0.0) - 0.0).exp() + (t.exp() - t.exp()) + (torch.ones(3, 4) * 2 + 1), (x,))
    want = J.Interpreter(g)(x)
    n0 = g.node_count()
    assert J.algebraic_simplification(g) >= 2
    assert J.constant_folding(g) >= 1
    assert J.common_subexpression_elimination(g) >= 1
    J.dead_code_elimination(g)
    assert g.node_count() < n0
    g.validate()
    assert torch.allclose(J.Interpreter(g)(x), want, atol=1e-6)
    b = J.GraphBuilder()
    a = b.input((3, 4))
    b.unary("exp", b.unary("tanh", a))                 # computed, never used
    g2 = b.finish([b.unary("neg", a)])
    assert g2.node_count() == 3 and J.dead_code_elimination(g2) == 2 and g2.node_count() == 1
    assert torch.equal(J.Interpreter(g2)(x), -x)


def test_fusion_groups_and_generated_host_kernels():
    x, y = torch.randn(16, 32), torch.randn(16, 32)
    f = lambda a, b: (torch.sigmoid(a) * b + a.exp()).sum(-1)          # noqa: E731
    g = J.trace(f, (x, y))
    groups = J.find_fusion_groups(g)
    assert groups and all(isinstance(gr, J.FusionGroup) for gr in groups) and max(len(gr.nodes) for gr in groups) >= 3
    assert J.fuse_elementwise(g) >= 1 and g.node_count("fused") >= 1
    fused = next(n for n in g.nodes.values() if n.op == "fused")
    body = fused.attrs["body"]
    src = J.generate_host(body, "k_unit")
    assert 'extern "C"' in src and "k_unit" in src
    k = J.HostFusedKernel(body)
    outs = k([x, y][: len(body.inputs)] if len(body.inputs) <= 2 else [x, y])
    assert torch.allclose(outs[0] if isinstance(outs, (list, tuple)) else outs, torch.sigmoid(x) * y + x.exp(), atol=1e-5)
    assert J.fuse_reductions(g) >= 1
    red = next(n for n in g.nodes.values() if n.op == "fused_reduce")
    rsrc = J.generate_host_reduce(red.attrs["body"], "k_red", red.attrs["red_op"], red.attrs["red_index"])
    assert "k_red" in rsrc
    rk = J.HostFusedReduceKernel(red.attrs["body"], red.attrs["red_op"], red.attrs["red_index"], red.attrs.get("keepdim", False))
    ro = rk([x, y])
    assert torch.allclose(ro[0] if isinstance(ro, (list, tuple)) else ro, f(x, y), atol=1e-4)
    assert torch.allclose(J.Interpreter(g)(x, y), f(x, y), atol=1e-4)
    assert J.CudaFusedKernel is not None and J.CudaFusedReduceKernel is not None and callable(J.generate_reduction_ptx)


def test_joint_capture_pair_and_memory_plan():
    f = lambda x, w: torch.tanh(x @ w).sum()         # noqa: E731
    x, w = torch.randn(5, 4), torch.randn(4, 3)
    joint = J.aot_trace_joint(f, (x, w))
    assert isinstance(joint, J.JointGraph) and joint.num_primals == 2 and joint.num_outputs == 1
    outs = J.Interpreter(joint.graph)(x, w, torch.ones(()))
    xs, ws = x.clone().requires_grad_(), w.clone().requires_grad_()
    val = f(xs, ws)
    gx, gw = torch.autograd.grad(val, (xs, ws))
    assert torch.allclose(outs[0], val.detach(), atol=1e-6) and torch.allclose(outs[1], gx, atol=1e-5) and torch.allclose(outs[2], gw, atol=1e-5)
    pair = J.decompose_forward_backward(f, (x, w))
    assert isinstance(pair, J.AotGraphPair) and len(pair.saved_tensor_indices) == pair.num_saved
    g = J.trace(lambda t: ((t + 1).exp() * 2).tanh() - 3, (torch.randn(64, 64),))
    plan = J.plan_memory(g)
    assert isinstance(plan, J.MemoryPlan) and 0 < plan.planned_bytes < plan.naive_bytes and len(set(plan.slot_of.values())) == len(plan.slot_bytes)
    g2 = J.trace(lambda t: ((t + 1).exp() * 2).tanh() - 3, (torch.randn(64, 64),))
    got = J.optimize_with_config(g2, J.OptimizationConfig())
    assert got is None or isinstance(got, J.MemoryPlan)
    assert torch.allclose(J.Interpreter(g2)(torch.zeros(64, 64)), ((torch.zeros(64, 64) + 1).exp() * 2).tanh() - 3, atol=1e-6)


def test_guards_shape_env_and_symbolic_modules():
    sig = J.ShapeSignature().symbolic_dim_with_range(0, 0, 1, 64) if hasattr(J.ShapeSignature(), "symbolic_dim_with_range") else J.ShapeSignature()
    specs = sig.symbolic_dims_for(0)
    assert specs and isinstance(specs[0], J.SymbolicDimSpec) and (specs[0].dim_index, specs[0].min, specs[0].max) == (0, 1, 64)
    guard = J.Guard([(8, 4)], sig)
    guard.check([(32, 4)])
    with pytest.raises(FerrotorchError):
        guard.check([(32, 5)])                    # a static dimension changed
    with pytest.raises(FerrotorchError):
        guard.check([(65, 4)])                    # outside the declared range
    env = J.ShapeEnv()
    bdim = J.SymbolicDim("b", 1, 64)
    assert env.check([(bdim, 4)], [(7, 4)]) == {"b": 7} and env.check([(bdim, 4)], [(7, 5)]) is None and env.check([(bdim, 4)], [(65, 4)]) is None
    assert env.check([(bdim, 4), (bdim, 2)], [(7, 4), (8, 2)]) is None          # one symbol, two different extents
    f = lambda t: torch.relu(t) * 2              # noqa: E731
    x = torch.randn(8, 4)
    cf = J.compile(f, (x,))
    assert isinstance(cf, J.CompiledFunction) and isinstance(cf.graph_for(x), J.IrGraph) and torch.allclose(cf(x), f(x))
    sm = J.compile_with_config(f, (x,), J.CompileConfig(shape_signature=sig)) if "shape_signature" in getattr(J.CompileConfig, "__dataclass_fields__", {}) else None
    if sm is not None and isinstance(sm, J.SymbolicTracedModule):
        x2 = torch.randn(16, 4)
        assert torch.allclose(sm(x2), f(x2))
    assert J.SymbolicTracedModule is not None


def test_result_records_of_compilation_tuning_and_export():
    f = lambda x, y: (x * y).sum(-1)             # noqa: E731
    x, y = torch.randn(8, 16), torch.randn(8, 16)
    g = J.trace(f, (x, y))
    be = J.InterpreterBackend()
    assert isinstance(be, J.Codegen)
    cg = be.compile(g)
    assert isinstance(cg, J.CompiledGraph) and torch.allclose(cg(x, y), f(x, y), atol=1e-5)
    st = J.InductorBackend(J.InductorTarget.CpuCpp).compile_with_status(g)
    assert isinstance(st, J.InductorCompileStatus) and isinstance(st.into_compiled(), J.CompiledGraph)
    tuner = J.Autotuner().with_candidate("a", J.InterpreterBackend()).with_candidate("b", J.NativeBackend()).with_iterations(2).with_warmup(1)
    res = tuner.tune(g, [x, y])
    assert isinstance(res, J.AutotuneResult) and res.winner_name() in ("a", "b")
    cand = J.AutotuneCandidate("c", J.InterpreterBackend())
    assert cand.name() == "c"
    old = J.Autotuner().tune("k", [1, 2], lambda c: (lambda: sum(range(100 * c))))
    assert isinstance(old, J.TuneResult) and set(old.timings_ms) == {"1", "2"} or set(old.timings_ms) == {1, 2}
    r = J.trace_with_breaks(lambda t: t.exp() + 1, (x,))
    assert isinstance(r, J.TraceResult) and r.is_unbroken()
    assert J.Segment is not None and J.SegmentedModule is not None and J.GraphSegment([1, 2], True).compiled
    stats = J.CompileStats()
    assert (stats.traces, stats.cache_hits, stats.graph_breaks) == (0, 0, 0)
    k = J.compile_loop_ir_kernel([J.LoopIR.Store("out", J.Expr.IntConst(0), J.Expr.Const(2.5))], 0, 1)
    assert isinstance(k, J.JitCompiledKernel) and k.execute([]).tolist() == [2.5]
    assert J.DynamicExportedProgram is not None
