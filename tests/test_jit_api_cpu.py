"""Object-level JIT API: traced modules, configs, graph breaks, symbolic guards, export specs, AOT pairs, backends, loop IR, fused chains."""
import math

import pytest
import torch

from ferrotorch_b200 import jit as J
from ferrotorch_b200.errors import FerrotorchError, InvalidArgument


def f_mlp(x, w):
    return torch.relu(x @ w + 1.0).tanh() * 2.0


def test_traced_module_config_and_persistence(tmp_path):
    x, w = torch.randn(4, 8), torch.randn(8, 3)
    m = J.compile_with_config(f_mlp, (x, w), J.CompileConfig())
    assert torch.allclose(m(x, w), f_mlp(x, w), atol=1e-6) and m.input_count() == 2 and m.output_shape() == (4, 3) and m.memory_plan is not None
    assert torch.allclose(m.forward_multi([x * 2, w]), f_mlp(x * 2, w), atol=1e-6)
    plain = J.compile_with_config(f_mlp, (x, w), J.CompileConfig.from_optimization(J.OptimizationConfig(operator_fusion=False, memory_planning=False)))
    assert plain.memory_plan is None and plain.graph().node_count("fused") == 0 and m.graph().node_count("fused") >= 1
    with pytest.raises(FerrotorchError):
        m(x[:2], w)
    with pytest.raises(InvalidArgument):
        m(x)
    m.save(tmp_path / "m.ftj")
    back = J.TracedModule.load(tmp_path / "m.ftj")
    assert torch.allclose(back(x, w), f_mlp(x, w), atol=1e-6) and J.TracedModule.from_bytes(m.to_bytes()).input_count() == 2
    with pytest.raises(InvalidArgument):
        J.TracedModule.from_bytes(b"junk")
    g = J.trace(f_mlp, (x, w))
    assert torch.allclose(J.interpret(g, [x, w]), f_mlp(x, w), atol=1e-6) and len(J.interpret_multi(g, [x, w])) == 1
    outs, caps = J.interpret_multi_with_captures(g, [x, w], [0])
    first = [n for n in g.topo_order() if n.op not in ("input", "constant", "output")][0] if g.topo_order()[0].op in ("input", "constant") else g.topo_order()[0]
    assert torch.allclose(outs[0], f_mlp(x, w), atol=1e-6) and len(caps) == 1
    with pytest.raises(InvalidArgument):
        J.interpret(g, [x])
    with pytest.raises(InvalidArgument):
        J.interpret_multi_with_captures(g, [x, w], [999])


def f_break(x):
    y = torch.relu(x) * 2.0
    z = torch.unique_consecutive(y.flatten()).sum()          # not an IR operation: the tracer keeps it as an opaque call
    return y + z


def test_graph_breaks_segment_and_fullgraph_refuses():
    x = torch.tensor([[1.0, -2.0, 3.0], [3.0, 0.5, -1.0]])
    g = J.trace(f_break, (x,))
    if not any(n.op == "opaque" for n in g.nodes.values()):
        pytest.skip("the tracer lowered every operation of this function")
    r = J.trace_with_breaks(f_break, (x,))
    assert not r.is_unbroken() and r.segmented.segment_count() >= 3 and not r.segmented.is_fully_compiled()
    kinds = [s.is_compiled() for s in r.segmented.segments()]
    assert kinds[0] and not all(kinds) and "Eager" in repr(r.segmented.segments()[kinds.index(False)])
    assert torch.allclose(r.segmented(x), f_break(x)) and torch.allclose(r.segmented.forward(x + 1), f_break(x + 1))
    with pytest.raises(J.JitError):
        J.trace_with_breaks(f_break, (x,), J.CompileConfig(fullgraph=True))
    with pytest.raises(J.JitError):
        J.compile_with_config(f_break, (x,), J.CompileConfig(fullgraph=True))
    whole = J.trace_with_breaks(lambda t: t.exp() + 1, (x,))
    assert whole.is_unbroken() and whole.graph.node_count() >= 1


def test_symbolic_guard_and_specialisation():
    f = lambda x, w: (x @ w).reshape(x.shape[0], -1).sum(-1)     # noqa: E731
    x, w = torch.randn(4, 8), torch.randn(8, 3)
    sig = J.ShapeSignature().symbolic_dim_with_range(0, 0, 1, 16)
    assert sig.is_symbolic(0, 0) and not sig.is_symbolic(0, 1) and not sig.is_symbolic(1, 0) and sig.symbolic_dims_for(0)[0].max == 16
    m = J.compile_symbolic(f, (x, w), sig, J.CompileConfig(cache_size=2))
    for b in (4, 7, 16, 7):
        xb = torch.randn(b, 8)
        assert torch.allclose(m(xb, w), f(xb, w), atol=1e-5)
    assert m.specializations() == 2 and m.inner().input_count() == 2
    for bad, msg in ((torch.randn(17, 8), "outside"), (torch.randn(4, 9), "static"), (torch.randn(0, 8), "0"), (torch.randn(4, 8, 1), "rank")):
        with pytest.raises(InvalidArgument, match=msg):
            m(bad, w)
    with pytest.raises(InvalidArgument, match="expected 2 inputs"):
        m.guard().check([(4, 8)])
    g = J.IrGraph()
    v = g.add_input((4, 6), torch.float32)
    g.set_outputs(g.add_node("reshape", [v.id], [((4, 2, 3), torch.float32)], shape=[4, 2, 3]).outputs)
    assert J.patch_reshape_for_symbolic_dims(g, [(4, 6)], J.ShapeSignature().symbolic_dim(0, 0)) == 1
    assert [n.attrs["shape"] for n in g.nodes.values() if n.op == "reshape"] == [[-1, 2, 3]]
    assert J.interpret(g, [torch.zeros(10, 6)]).shape == (10, 2, 3)
    with pytest.raises(InvalidArgument):
        J.ShapeSignature().symbolic_dim_with_range(0, 0, 5, 2)


def test_export_with_dynamic_shapes_checks_specs():
    f = lambda a, b: torch.softmax(a @ b.transpose(-1, -2), -1)  # noqa: E731
    a, b = torch.randn(2, 5, 4), torch.randn(2, 7, 4)
    specs = [J.InputSpec([J.DimSpec.dynamic_range("batch", 1, 8), J.DimSpec.dynamic("q"), J.DimSpec.Static(4)]),
             J.InputSpec([J.DimSpec.dynamic_range("batch", 1, 8), J.DimSpec.dynamic("k"), J.DimSpec.Static(4)])]
    assert specs[0].has_dynamic_dims() and specs[0].rank() == 3 and not J.InputSpec.all_static([2, 3]).has_dynamic_dims() and J.DimSpec.Static(4) == J.DimSpec.Static(4)
    p = J.export_with_dynamic_shapes(f, (a, b), specs)
    a2, b2 = torch.randn(3, 6, 4), torch.randn(3, 2, 4)
    assert torch.allclose(p(a2, b2), f(a2, b2), atol=1e-6) and torch.allclose(p.run_with_guards([a, b]), f(a, b), atol=1e-6)
    for xa, xb in ((torch.randn(3, 6, 4), torch.randn(4, 2, 4)), (torch.randn(9, 6, 4), torch.randn(9, 2, 4)), (torch.randn(3, 6, 5), torch.randn(3, 2, 5)),
                   (torch.randn(3, 6), torch.randn(3, 2, 4))):
        with pytest.raises(FerrotorchError):
            p(xa, xb)
    with pytest.raises(InvalidArgument):
        J.export_with_dynamic_shapes(f, (a, b), specs[:1])
    prog = J.export(f, (a, b))
    meta = J.program_metadata(prog, ["w"])
    again = J.ExportedProgramMetadata.parse(meta.to_json())
    assert again == meta and meta.input_shapes == [[2, 5, 4], [2, 7, 4]] and meta.output_shape == [2, 5, 7] and meta.num_graph_nodes > 0
    with pytest.raises(InvalidArgument):
        J.ExportedProgramMetadata.parse("{}")


def test_aot_pair_matches_autograd():
    f = lambda x, w: (torch.tanh(x @ w) * x.sum(-1, keepdim=True)).sum()   # noqa: E731
    x, w = torch.randn(5, 4), torch.randn(4, 4)
    pair = J.decompose_forward_backward(f, (x, w))
    assert pair.num_outputs == 1 and pair.num_saved >= 1 and len(pair.forward.inputs) == 2 and len(pair.backward.inputs) == pair.num_saved + 1
    m = J.compile_aot(f, (x, w))
    xs, ws = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    want = f(xs, ws)
    gx, gw = torch.autograd.grad(want, (xs, ws))
    out = m.forward_with_ctx([x, w])
    assert torch.allclose(out, want.detach(), atol=1e-5) and len(m.saved_tensors()) == pair.num_saved == len(m.saved_tensor_indices())
    dx, dw = m.backward(torch.ones(()))
    assert torch.allclose(dx, gx, atol=1e-5) and torch.allclose(dw, gw, atol=1e-5)
    dx2, _ = m.backward(torch.tensor(3.0))                     # the saved values serve any number of backward calls
    assert torch.allclose(dx2, 3 * gx, atol=1e-5)
    with pytest.raises(InvalidArgument):
        m.backward()
    with pytest.raises(J.JitError):
        J.AotCompiledModule(pair).backward(torch.ones(()))


def test_codegen_backends_and_autotuner():
    f = lambda x, y: (torch.sigmoid(x) * y + x.exp()).sum(-1)    # noqa: E731
    x, y = torch.randn(64, 33), torch.randn(64, 33)
    g = J.trace(f, (x, y))
    want = f(x, y)
    for be in (J.InterpreterBackend(), J.NativeBackend(), J.InductorBackend(J.InductorTarget.CpuCpp)):
        cg = be.compile(g)
        assert torch.allclose(cg.execute([x, y]), want, atol=1e-4), be.name()
        assert cg.num_inputs() == 2 and cg.output_shape() == (64,) and cg.backend == be.name()
    assert J.NativeBackend().compile(g).fused_kernels >= 1 and g.node_count("fused") == 0        # the caller's graph is left as traced
    st = J.InductorBackend(J.InductorTarget.GpuCuda).compile_with_status(g)
    if not torch.cuda.is_available():
        assert not st.is_compiled() and "CUDA" in st.reason and torch.allclose(st.into_compiled()(x, y), want, atol=1e-4)
    assert J.InductorTarget.CpuRust is J.InductorTarget.CpuCpp
    with pytest.raises(InvalidArgument):
        J.InterpreterBackend().compile(g).execute([x])
    t = J.Autotuner().with_candidate("interp", J.InterpreterBackend()).with_candidate("native", J.NativeBackend()).with_iterations(3).with_warmup(1)
    assert t.candidate_count() == 2 and t.iterations() == 3
    r = t.tune(g, [x, y])
    assert r.winner_name() in ("interp", "native") and len(r.all_timings()) == 2 and r.winner_time() == min(s for _, s in r.all_timings())
    assert torch.allclose(r.winner_compiled()(x, y), want, atol=1e-4)
    key = J.AutotuneKey.from_graph(g, [(64, 33), (64, 33)])
    assert t.cached(key) == (r.winner_name(), r.winner_time()) and t.cache_size() == 1 and t.cached(J.AutotuneKey.from_graph(g, [(1, 1), (1, 1)])) is None
    t.clear_cache()
    assert t.cache_size() == 0
    with pytest.raises(InvalidArgument):
        J.Autotuner().tune(g, [x, y])
    old = J.Autotuner().tune("k", [1, 2], lambda c: (lambda: sum(range(1000 * c))))             # the configuration sweep still works
    assert old.best in (1, 2)


def test_loop_ir_emitters_and_kernel():
    E, L = J.Expr, J.LoopIR
    i = E.Var("i")
    body = [L.Let("a", E.Index("in0", i)), L.Let("b", E.Index("in1", i)),
            L.Let("t", E.BinOp(J.BinOpKind.Add, E.UnaryOp(J.UnaryOpKind.Sigmoid, E.Var("a")), E.BinOp(J.BinOpKind.Mul, E.Var("b"), E.Const(0.5)))),
            L.If(E.BinOp(J.BinOpKind.Sub, E.Var("t"), E.Const(1.0)), [L.Assign("t", E.FnCall("fmax", [E.Var("t"), E.Const(0.0)]))], []),
            L.Store("out", i, E.BinOp(J.BinOpKind.Mod, E.Var("t"), E.Const(3.0)))]
    loops = [L.Comment("sigmoid(a) + b / 2, clamped, mod 3"), L.Loop("i", E.IntConst(0), E.IntConst(10), body)]
    k = J.compile_loop_ir_kernel(loops, 2, 10)
    a, b = torch.linspace(-3, 3, 10, dtype=torch.float64), torch.linspace(0, 9, 10, dtype=torch.float64)
    want = torch.fmod(torch.clamp_min(torch.sigmoid(a) + 0.5 * b, 0.0), 3.0)
    assert torch.allclose(k.execute([a, b]), want, atol=1e-12) and (k.num_inputs(), k.output_len()) == (2, 10)
    src = J.CpuCodegen.generate_cpp_source(loops, "kern")
    assert 'extern "C" void kern(' in src and "for (long long i = 0LL; i < 10LL; ++i)" in src and J.CpuCodegen.generate_rust_source(loops, "kern") == src
    cu = J.GpuCodegen.generate_cuda_source(loops, "kern_gpu")
    assert "__global__" in cu and "blockIdx.x" in cu and "gridDim.x" in cu
    acc = [L.Let("acc", E.Const(0.0)), L.Loop("i", E.IntConst(0), E.IntConst(10), [L.Accumulate("acc", E.Index("in0", i))]), L.Store("out", E.IntConst(0), E.Var("acc"))]
    assert torch.allclose(J.compile_loop_ir_kernel(acc, 1, 1).execute([a]), a.sum().reshape(1))
    for bad in ([L.Store("weights", i, E.Const(1.0))], [L.Store("out", E.IntConst(0), E.Index("in3", E.IntConst(0)))],
                [L.Store("out", E.IntConst(0), E.FnCall("system", []))], [L.Let("a b", E.Const(1.0))]):
        with pytest.raises(InvalidArgument):
            J.compile_loop_ir_kernel(bad, 1, 1)
    g = J.trace(lambda p, q: (torch.tanh(p) * q - p).abs(), (a, b))
    lowered = J.lower_to_loops(g)
    assert torch.allclose(J.compile_loop_ir_kernel(lowered, 2, 10).execute([a, b]), (torch.tanh(a) * b - a).abs(), atol=1e-12)
    gm = J.trace(lambda p: p.exp().mean(), (a,))
    assert torch.allclose(J.compile_loop_ir_kernel(J.lower_to_loops(gm), 1, 1).execute([a])[0], a.exp().mean(), atol=1e-12)
    with pytest.raises(InvalidArgument):
        J.lower_to_loops(J.trace(lambda p, q: p.view(2, 5) @ q.view(5, 2), (a, b)))


def test_fused_chain_and_reductions(tmp_path):
    F = J.FusedOp
    chain = J.FusedChain().push(F.ScalarMul(2.0)).push(F.Tanh).push(F.ScalarAdd(1.0)).push(F.Pow(2.0)).push(F.Sqrt).push(F.Neg)
    x = torch.randn(1000)
    assert len(chain) == 6 and not chain.is_empty() and not chain.needs_second_operand()
    assert torch.allclose(J.apply_fused(x, chain), -torch.sqrt((torch.tanh(2 * x) + 1) ** 2), atol=1e-6)
    xb = torch.randn(64, 8).to(torch.bfloat16)
    assert J.apply_fused(xb, J.FusedChain([F.Silu, F.Abs])).dtype == torch.bfloat16
    both = J.FusedChain([F.Relu, F.Mul, F.Exp])
    y = torch.randn(1000)
    assert both.needs_second_operand() and torch.allclose(J.apply_fused(x, both, y), torch.exp(torch.relu(x) * y), atol=1e-5)
    with pytest.raises(InvalidArgument):
        J.apply_fused(x, both)
    with pytest.raises(InvalidArgument):
        J.apply_fused(torch.arange(4), J.FusedChain([F.Neg]))
    assert J.apply_fused(x, J.FusedChain()) is x and F.Pow(2.0) == F.Pow(2.0) != F.Pow(3.0)
    assert not J.is_fusion_enabled() and J.with_fusion(J.is_fusion_enabled) and not J.is_fusion_enabled()
    with pytest.raises(ZeroDivisionError):
        J.with_fusion(lambda: 1 / 0)
    assert not J.is_fusion_enabled()
    with J.with_fusion():
        assert J.is_fusion_enabled()
    assert J.estimate_numel_for_inputs([[2, 3], [4, 5, 6], []]) == 120 and J.estimate_numel_for_inputs([]) == 0 and J.estimate_matmul_dims([4, 8], [8, 3]) == (4, 8, 3)
    for bad in (([4, 8], [7, 3]), ([4], [4, 3])):
        with pytest.raises(InvalidArgument):
            J.estimate_matmul_dims(*bad)
    # the generated C reductions compile and give the right numbers
    import ctypes
    import subprocess
    src = "".join(J.generate_reduction_c(k, f"red_{k.value}") for k in J.ReductionKind)
    (tmp_path / "r.c").write_text(src)
    subprocess.run(["gcc", "-O2", "-fopenmp-simd", "-shared", "-fPIC", str(tmp_path / "r.c"), "-o", str(tmp_path / "r.so")], check=True)
    lib = ctypes.CDLL(str(tmp_path / "r.so"))
    v = torch.rand(37) + 0.5
    for k, want in ((J.ReductionKind.Sum, v.sum()), (J.ReductionKind.Mean, v.mean()), (J.ReductionKind.Prod, v.prod())):
        fn = getattr(lib, f"red_{k.value}")
        fn.restype = ctypes.c_float
        assert math.isclose(fn(ctypes.c_void_p(v.data_ptr()), ctypes.c_long(37)), float(want), rel_tol=1e-4)
    cu = J.generate_reduction_cuda(J.ReductionKind.Mean, "mean_k")
    assert "__shfl_down_sync" in cu and "atomicAdd" in cu and "/ (float)n" in cu and "atomicCAS" in J.generate_reduction_cuda(J.ReductionKind.Prod, "p")
    with pytest.raises(InvalidArgument):
        J.generate_reduction_c(J.ReductionKind.Sum, "bad name")
    assert J.FusionGroupKind.Elementwise is not J.FusionGroupKind.Reduction
