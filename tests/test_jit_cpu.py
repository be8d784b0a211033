"""Tracing JIT: IR, tracer, passes, interpreter, host code generation, NVRTC compilation (no GPU needed), AOT, export, script, guards."""
import os
import tempfile

import pytest
import torch
import torch.nn.functional as F

from ferrotorch_b200 import jit


def _f(x, y, b):
    h = F.gelu(x * y + b) * torch.sigmoid(x) - 0.5
    return torch.where(h > 0, h, h * 0.1).sum(-1), torch.tanh(h)


def _inputs():
    g = torch.Generator().manual_seed(0)
    return torch.randn(4, 64, generator=g), torch.randn(4, 64, generator=g), torch.randn(64, generator=g)


def test_trace_interpret_and_serialise():
    x, y, b = _inputs()
    g = jit.trace(_f, (x, y, b))
    assert g.node_count("gelu") == 1 and g.node_count("opaque") == 0
    for a, r in zip(jit.run_graph(g, (x, y, b)), _f(x, y, b)):
        assert torch.equal(a, r)
    g2 = jit.IrGraph.from_json(g.to_json())
    assert g2.fingerprint() == g.fingerprint()
    for a, r in zip(jit.run_graph(g2, (x, y, b)), _f(x, y, b)):
        assert torch.allclose(a, r)
    assert jit.trace(_f, (x, y, b)).fingerprint() == g.fingerprint()
    assert jit.trace(lambda x, y, b: _f(x, y, b)[1], (x, y, b)).fingerprint() != g.fingerprint()


def test_passes_fold_cse_dce_simplify_fuse():
    x = torch.randn(8, 16)

    def fn(t):
        c = torch.ones(16) * 2.0 + 1.0              # constant subgraph -> folded
        a = torch.exp(t) * c
        b = torch.exp(t) * c                        # duplicate -> CSE
        dead = torch.sin(t)                         # noqa: F841  unused -> DCE
        return (a + b) * 1.0 + 0.0                  # identities -> simplified
    g = jit.trace(fn, (x,))
    n0 = len(g.nodes)
    stats = jit.optimize(g)
    assert stats["folded"] >= 2 and stats["cse"] >= 2 and stats["dce"] >= 1 and stats["simplified"] >= 2 and stats["fused_groups"] == 1
    assert len(g.nodes) == 1 and len(g.nodes) < n0
    assert torch.allclose(jit.run_graph(g, (x,))[0], fn(x))


def test_fusion_never_creates_a_cycle():
    x = torch.randn(4, 8)

    def fn(t):
        a = torch.exp(t)
        s = a.sum(-1, keepdim=True)                 # reduction between two elementwise regions that share `a`
        return a / s + torch.tanh(a)
    g = jit.trace(fn, (x,))
    jit.optimize(g)
    g.validate()                                    # topo_order raises on a cycle
    assert torch.allclose(jit.run_graph(g, (x,))[0], fn(x), atol=1e-6)


def test_host_codegen_matches_eager_with_broadcast_and_bf16():
    x, y, b = _inputs()
    cf = jit.compile(_f, backend="host")
    for a, r in zip(cf(x, y, b), _f(x, y, b)):
        assert torch.allclose(a, r, atol=1e-5)
    assert cf.stats.fused_kernels == 1 and cf.stats.kernel_launches == 1
    cf(x, y, b)
    assert cf.stats.traces == 1 and cf.stats.cache_hits == 1
    xt = x.t().contiguous().t()                     # non-contiguous input goes through the strided path
    for a, r in zip(cf(xt, y, b), _f(xt, y, b)):
        assert torch.allclose(a, r, atol=1e-5)
    xb = x.bfloat16()
    fb = lambda t: torch.tanh(t) * t + 1            # noqa: E731
    assert torch.equal(jit.compile(fb, backend="host")(xb), fb(xb))


def test_cuda_codegen_compiles_for_sm100a_without_a_gpu():
    x, y, b = _inputs()
    g = jit.trace(_f, (x.bfloat16(), y.bfloat16(), b.bfloat16()))
    jit.optimize(g)
    body = next(n for n in g.nodes.values() if n.op in ("fused", "fused_reduce")).attrs["body"]
    for vec in (True, False):
        src = jit.generate_cuda(body, "k", vec)
        assert "__nv_bfloat16" in src and ("uint4" in src) == vec
        img = jit.compile_cuda(src)
        assert len(img) > 1000 and img[:4] == b"\x7fELF"


def test_module_compile_aot_export_script_and_guards():
    x = _inputs()[0]
    m = torch.nn.Sequential(torch.nn.Linear(64, 32), torch.nn.LayerNorm(32), torch.nn.GELU(), torch.nn.Linear(32, 8), torch.nn.Softmax(-1))
    cm = jit.compile(m, backend="host")
    assert torch.allclose(cm(x), m(x), atol=1e-6)
    with torch.no_grad():
        m[0].weight.mul_(0.5)                       # weights are referenced, not copied
    assert torch.allclose(cm(x), m(x), atol=1e-6)

    def g(a, w):
        return torch.tanh(a @ w).sum()
    a, w = torch.randn(3, 4), torch.randn(4, 5)
    a1, w1, a2, w2 = (t.clone().requires_grad_() for t in (a, w, a, w))
    jit.aot_function(g, (a, w))(a1, w1).backward()
    g(a2, w2).backward()
    assert torch.allclose(a1.grad, a2.grad) and torch.allclose(w1.grad, w2.grad)

    d = tempfile.mkdtemp()
    jit.export(m, (x,)).save(os.path.join(d, "m"))
    assert torch.allclose(jit.ExportedProgram.load(os.path.join(d, "m"))(x), m(x), atol=1e-6)
    with pytest.raises(Exception):
        jit.export(lambda t: torch.cumsum(t, 0), (x,))        # no portable IR form -> strict export refuses

    @jit.script(((4, 8), torch.float32), ((8,), torch.float32))
    def sf(p, q):
        return ((p * q + 1.0).tanh()).sum(-1)
    p, q = torch.randn(4, 8), torch.randn(8)
    assert torch.allclose(sf(p, q), torch.tanh(p * q + 1).sum(-1))

    B = jit.SymbolicDim("B", 1, 64)
    cd = jit.compile(lambda t: torch.relu(t) * 2 + 1, backend="host", dynamic_dims=[(B, 16)])
    assert cd(torch.randn(4, 16)).shape == (4, 16) and cd(torch.randn(7, 16)).shape == (7, 16)
    with pytest.raises(Exception):
        cd(torch.randn(7, 17))
    with pytest.raises(Exception):
        cd(torch.randn(128, 16))


def test_graph_breaks_memory_plan_autotune():
    x = torch.randn(4, 8)

    def fn(t):
        return torch.cumsum(torch.exp(t) + 1, 0) * 2 - 1
    cf = jit.compile(fn, backend="host")
    assert torch.allclose(cf(x), fn(x), atol=1e-6) and cf.stats.graph_breaks == 1
    segs = jit.split_at_breaks(cf.graph_for(x))
    assert [s.compiled for s in segs] == [True, False, True]
    mp = jit.plan_memory(jit.trace(_f, _inputs()))
    assert mp.planned_bytes < mp.naive_bytes
    d = tempfile.mkdtemp()
    at = jit.Autotuner(os.path.join(d, "tune.json"), warmup=1, iters=2)
    import time
    r = at.tune("k", [{"sleep": 0.002}, {"sleep": 0.0}], lambda c: (lambda: time.sleep(c["sleep"])))
    assert r.best == {"sleep": 0.0} and jit.Autotuner(os.path.join(d, "tune.json")).tune("k", [], None).best == {"sleep": 0.0}


def test_fused_elementwise_plus_row_reduction():
    def f(x, b):
        e = torch.exp(x - 1.0) * b
        return e.sum(-1, keepdim=True), torch.tanh(e)
    x, b = torch.randn(6, 33), torch.randn(33)
    g = jit.trace(f, (x, b))
    stats = jit.optimize(g)
    assert stats["fused_reductions"] == 1 and [n.op for n in g.nodes.values()] == ["fused_reduce"]
    for a, r in zip(jit.run_graph(g, (x, b)), f(x, b)):
        assert torch.allclose(a, r, atol=1e-5)
    cf = jit.compile(f, backend="host")
    for a, r in zip(cf(x, b), f(x, b)):
        assert torch.allclose(a, r, atol=1e-5)
    assert cf.stats.fused_kernels == 1 and cf.stats.kernel_launches == 1
    for op in ("mean", "amax", "amin"):
        fn = lambda t: getattr(torch, op)(torch.sigmoid(t) * t, -1)       # noqa: E731,B023
        assert torch.allclose(jit.compile(fn, backend="host")(x), fn(x), atol=1e-6)
    n = next(n for n in g.nodes.values() if n.op == "fused_reduce")
    img = jit.compile_cuda(jit.generate_cuda_reduce(n.attrs["body"], "k", "sum", n.attrs["red_index"]))
    assert img[:4] == b"\x7fELF"


def test_host_dense_loop_special_values_and_accuracy():
    """The dense host loop uses its own vectorisable expf / tanhf: infinities, NaN, exp(-inf) == 0 and accuracy against eager execution."""
    import torch
    from ferrotorch_b200 import jit
    x = torch.cat([torch.linspace(-110, 95, 200001), torch.tensor([float("inf"), -float("inf"), float("nan"), 0.0, -0.0, 88.7228, 88.723, -87.3,
                                                                    -103.9, -104.1, 1e-30, -1e-30]), torch.randn(70000) * 3]).contiguous()
    for f, tol in ((lambda a: torch.exp(a) * 0.5 + 0.25, 3e-7), (lambda a: torch.tanh(a) * 0.5 + 0.25, 2e-7), (lambda a: torch.sigmoid(a) * 0.5 + 0.25, 3e-7)):
        cf = jit.compile(f, example_inputs=[x], backend="auto")
        got, ref = cf(x), f(x)
        assert cf.stats.fused_kernels == 1
        assert torch.equal(torch.isnan(got), torch.isnan(ref)) and torch.equal(torch.isinf(got), torch.isinf(ref))
        fin = torch.isfinite(ref)
        assert ((got[fin] - ref[fin]).abs() <= tol * ref[fin].abs() + 1e-7).all()
    xl = torch.cat([torch.logspace(-44, 38, 100001), torch.linspace(0.5, 2.0, 50001), torch.tensor([0.0, -0.0, -1.0, float("inf"), float("nan"), 1.0])]).contiguous()
    xe = torch.cat([torch.linspace(-5, 5, 100001), torch.tensor([0.0, -0.0, float("inf"), -float("inf"), float("nan"), 1e-20, -1e-30, 30.0])]).contiguous()
    for f, x in ((lambda a: torch.log(a) * 1.5, xl), (lambda a: torch.erf(a) * 1.5, xe)):
        cf = jit.compile(f, example_inputs=[x], backend="auto")
        got, ref = cf(x), f(x)
        assert cf.stats.fused_kernels == 1
        assert torch.equal(torch.isnan(got), torch.isnan(ref)) and torch.equal(got[torch.isinf(ref)], ref[torch.isinf(ref)])
        fin = torch.isfinite(ref)
        assert ((got[fin] - ref[fin]).abs() <= 6e-7 * ref[fin].abs() + 1e-37).all()
