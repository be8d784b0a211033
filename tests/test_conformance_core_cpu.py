"""Per-symbol behaviour checks of ``ferrotorch_b200.core`` against PyTorch / closed forms: sparse and complex containers, quantisation,
masked and nested tensors, forward-mode duals, vmap variants, differentiable FFT / einsum, indexing helpers, error types and enums."""
import math

import pytest
import torch

import ferrotorch_b200.core as C
from ferrotorch_b200.errors import FerrotorchError


def _close(a, b, tol=1e-5):
    assert a.shape == b.shape and torch.allclose(a, b, atol=tol, rtol=tol), (a.shape, b.shape)


def test_sorting_and_indexing_helpers():
    torch.manual_seed(0)
    x = torch.randn(4, 7)
    assert torch.equal(C.argsort(x, 1, True), torch.argsort(x, 1, True))
    v, i = C.topk(x, 3, 1, False)
    tv, ti = torch.topk(x, 3, 1, False)
    assert torch.equal(v, tv) and torch.equal(i, ti)
    b = torch.tensor([-1.0, 0.0, 0.5, 2.0])
    assert torch.equal(C.bucketize(x, b, True), torch.bucketize(x, b, right=True))
    _close(C.histc(x, 5, -2.0, 2.0), torch.histc(x, 5, -2.0, 2.0))
    _close(C.select(x, 1, 2), x.select(1, 2))
    base = torch.arange(12.0)
    assert torch.equal(C.as_strided(base, (3, 2), (4, 1), 1), base.as_strided((3, 2), (4, 1), 1))
    cp = C.as_strided_copy(base, (3, 2), (4, 1), 1)
    assert torch.equal(cp, base.as_strided((3, 2), (4, 1), 1)) and cp.data_ptr() != base.data_ptr()
    sc = C.as_strided_scatter(base, torch.full((3, 2), -1.0), (3, 2), (4, 1), 1)
    assert torch.equal(sc, torch.as_strided_scatter(base, torch.full((3, 2), -1.0), (3, 2), (4, 1), 1)) and base[1] == 1.0
    t = C.from_slice([1, 2, 3, 4, 5, 6], (2, 3))
    assert t.shape == (2, 3) and t.dtype == torch.float32 and t[1, 0] == 4
    assert C.is_float(t) and not C.is_float(torch.zeros(1, dtype=torch.long))
    _close(C.rearrange_with(torch.arange(24.0).view(2, 12), "b (h w) -> b h w", h=3), torch.arange(24.0).view(2, 3, 4))
    zm, om = C.zeros_meta(3, 4), C.ones_meta(2, dtype=torch.bfloat16)
    assert zm.device.type == "meta" and zm.shape == (3, 4) and om.dtype == torch.bfloat16
    p = C.to_pinned(torch.arange(4.0))
    assert torch.equal(p, torch.arange(4.0))
    assert isinstance(C.gpu_backend_available(), bool)
    s = C.display(torch.arange(2000.0))
    assert s.startswith("tensor(") and "..." in s and "shape=" in s and len(s) < 600


def test_sparse_containers_match_dense_algebra():
    torch.manual_seed(1)
    d = torch.randn(5, 6) * (torch.rand(5, 6) > 0.6)
    rhs = torch.randn(6, 3)
    coo = C.SparseTensor.from_dense(d)
    assert coo.nnz() == int((d != 0).sum()) and torch.equal(coo.to_dense(), d)
    _close(coo.matmul(rhs), d @ rhs)
    csr = coo.to_csr()
    assert isinstance(csr, C.CsrTensor) and torch.equal(csr.to_dense(), d)
    ref = d.to_sparse_csr()
    assert torch.equal(csr.crow_indices(), ref.crow_indices()) and torch.equal(csr.col_indices(), ref.col_indices())
    _close(csr.values(), ref.values())
    _close(csr.matmul(rhs), d @ rhs)
    csc = csr.to_csc()
    assert isinstance(csc, C.CscTensor) and torch.equal(csc.to_dense(), d)
    _close(C.CscTensor.from_dense(d).matmul(rhs), d @ rhs)
    g = C.SparseGrad(torch.tensor([2, 0, 2]), torch.ones(3, 4), 5)
    dense = g.to_dense()
    assert dense.shape == (5, 4) and dense[2, 0] == 2 and dense[0, 0] == 1 and dense[1].abs().sum() == 0
    co = g.coalesce()
    assert sorted(co.indices.tolist()) == [0, 2] and torch.equal(co.to_dense(), dense)
    w = torch.randn(8, 16)
    s24 = C.SemiStructuredSparseTensor(w)
    kept = s24.to_dense()
    assert ((kept.view(8, 4, 4) != 0).sum(-1) <= 2).all()
    top2 = w.view(8, 4, 4).abs().topk(2, -1).indices
    assert torch.equal(kept.view(8, 4, 4).gather(-1, top2), w.view(8, 4, 4).gather(-1, top2))
    _close(C.sparse_matmul_24(s24, rhs := torch.randn(16, 5)), kept @ rhs)


def test_complex_tensor_on_split_parts():
    torch.manual_seed(2)
    z, w = torch.randn(3, 4, dtype=torch.complex64), torch.randn(4, 2, dtype=torch.complex64)
    a, b = C.ComplexTensor.from_torch(z), C.ComplexTensor.from_torch(w)
    assert torch.allclose(a.to_torch(), z)
    assert torch.allclose(a.conj().to_torch(), z.conj())
    _close(a.abs(), z.abs())
    assert torch.allclose(a.matmul(b).to_torch(), z @ w, atol=1e-5)


def test_quantisation_round_trips_and_observers():
    torch.manual_seed(3)
    w = torch.randn(16, 32)
    for scheme in C.QuantScheme:
        q = C.quantize(w, scheme, C.QuantDtype.Int8)
        assert isinstance(q, C.QuantizedTensor) and isinstance(q.params, C.QParams)
        step = q.params.scale.max().item()
        assert (C.dequantize(q) - w).abs().max() <= step * 0.51 + 1e-6 and torch.equal(q.dequantize(), C.dequantize(q))
    q4 = C.quantize(w, C.QuantScheme.PerTensorSymmetric, C.QuantDtype.Int4)
    assert (q4.params.qmin, q4.params.qmax) == (-7, 7) and int(q4.data.abs().max()) <= 7
    a, b = torch.randn(8, 16), torch.randn(16, 4)
    qa, qb = C.quantize(a), C.quantize(b)
    ref = C.dequantize(qa) @ C.dequantize(qb)
    _close(C.quantized_matmul(qa, qb), ref, 1e-3)
    named = C.quantize_named_tensors({"w": w, "b": torch.randn(16)})
    assert set(named) == {"w", "b"} and named["w"].params.scale.numel() == 16
    ho = C.HistogramObserver(bins=256, coverage=0.99)
    ho.observe(torch.cat([torch.randn(10000), torch.tensor([50.0])]))
    qp = ho.qparams()
    assert float(qp.scale) * 127 < 10.0                # the outlier is clipped away
    po = C.PerChannelMinMaxObserver(axis=0)
    po.observe(torch.tensor([[1.0, -2.0], [10.0, 5.0]]))
    assert po.qparams().scale.numel() == 2 and po.qparams().scale[1] > po.qparams().scale[0]


def test_masked_tensors():
    t = torch.tensor([[1.0, float("nan"), 3.0], [4.0, 5.0, float("inf")]])
    m = C.masked_invalid(t)
    assert m.mask.tolist() == [[True, False, True], [True, True, False]]
    assert C.masked_count(m).item() == 4 and C.masked_count(m, 1).tolist() == [2, 2]
    assert C.masked_max(m).item() == 5 and C.masked_min(m).item() == 1
    assert C.masked_max(m, 1).tolist() == [3.0, 5.0] and C.masked_min(m, 0).tolist() == [1.0, 5.0, 3.0]
    e = C.masked_equal(torch.tensor([1, 2, 1, 3]), 1)
    assert e.mask.tolist() == [False, True, False, True]
    w = C.masked_where(torch.tensor([True, False, True]), torch.tensor([1.0, 2.0, 3.0]))
    assert w.mask.tolist() == [False, True, False] and w.filled(-1.0).tolist() == [-1.0, 2.0, -1.0]


def test_nested_tensors_and_packed_form():
    torch.manual_seed(4)
    seqs = [torch.randn(n, 2, 8) for n in (3, 5, 1)]
    nt = C.NestedTensor(seqs)
    packed = nt.pack()
    assert isinstance(packed, C.PackedNestedTensor) and packed.data.shape[0] == 9 and packed.offsets.tolist() == [0, 3, 8, 9]
    back = packed.unpack()
    assert all(torch.equal(a, b) for a, b in zip(back.tensors, seqs))
    out = C.nested_scaled_dot_product_attention(nt, nt, nt, causal=True)
    for o, s in zip(out.tensors, seqs):
        q = s.transpose(0, 1).unsqueeze(0)
        ref = torch.nn.functional.scaled_dot_product_attention(q, q, q, is_causal=True)[0].transpose(0, 1)
        _close(o, ref)


def test_dual_numbers_give_directional_derivatives():
    torch.manual_seed(5)
    x, v = torch.randn(6), torch.randn(6)
    for dual_fn, fn in ((C.dual_cos, torch.cos), (C.dual_log, lambda t: torch.log(t.abs() + 1)), (C.dual_relu, torch.relu),
                        (C.dual_sigmoid, torch.sigmoid), (C.dual_tanh, torch.tanh)):
        xi = x.abs() + 1 if dual_fn is C.dual_log else x
        fi = torch.log if dual_fn is C.dual_log else fn
        d = dual_fn(C.DualTensor(xi, v))
        _, jv = torch.autograd.functional.jvp(fi, xi, v)
        _close(d.primal, fi(xi))
        _close(d.tangent, jv)
    s = C.dual_sum(C.DualTensor(x.view(2, 3), v.view(2, 3)), 1)
    _close(s.primal, x.view(2, 3).sum(1))
    _close(s.tangent, v.view(2, 3).sum(1))


def test_vmap_variants():
    torch.manual_seed(6)
    a, b, c = torch.randn(4, 3), torch.randn(4, 3), torch.randn(4, 3)
    _close(C.vmap2(torch.dot)(a, b), (a * b).sum(1))
    _close(C.vmap2(torch.dot, in_dims=(0, 1))(a, b.t()), (a * b).sum(1))
    _close(C.vmap3(lambda x, y, z: (x * y + z).sum())(a, b, c), (a * b + c).sum(1))
    _close(C.vmap_many(lambda x, y: x @ y, (0, None))(a, b[0]), a @ b[0])
    mn, mx = C.vmap_multi_output(lambda r: (r.min(), r.max()))(a)
    _close(mn, a.min(1).values)
    _close(mx, a.max(1).values)


def test_differentiable_fft_and_einsum():
    torch.manual_seed(7)
    x = torch.randn(3, 8, requires_grad=True)
    xc = torch.stack([x, torch.zeros_like(x)], -1)              # complex values travel as a trailing (re, im) pair
    y = C.fft_differentiable(xc)
    _close(y, torch.view_as_real(torch.fft.fft(x.detach())), 1e-5)
    _close(C.fft_differentiable(xc, 16), torch.view_as_real(torch.fft.fft(x.detach(), 16)), 1e-5)
    z = C.ifft_differentiable(y)
    _close(z[..., 0], x.detach(), 1e-5)
    z[..., 0].sum().backward()
    _close(x.grad, torch.ones_like(x), 1e-5)
    r = torch.view_as_real(torch.fft.rfft(x.detach()))
    _close(C.irfft_differentiable(r, 8), x.detach(), 1e-5)
    with pytest.raises(FerrotorchError):
        C.fft_differentiable(torch.randn(3, 8))
    a, b = torch.randn(2, 3, 4, requires_grad=True), torch.randn(2, 4, 5, requires_grad=True)
    out = C.einsum_differentiable("bij,bjk->bik", a, b)
    _close(out, torch.bmm(a, b))
    out.sum().backward()
    _close(a.grad, torch.ones(2, 3, 5) @ b.detach().transpose(1, 2))


def test_backward_entry_points_and_gradient_tools():
    x = torch.tensor([1.0, 2.0], requires_grad=True)
    with pytest.raises(C.BackwardNonScalar):
        C.backward_with_gradient(x * 2)
    with pytest.raises(C.NoGradFn):
        C.backward_with_gradient(torch.tensor(1.0))
    C.backward_with_gradient(x * 2, torch.tensor([1.0, 3.0]))
    assert x.grad.tolist() == [2.0, 6.0]
    assert issubclass(C.BackwardNonScalar, FerrotorchError) and issubclass(C.NotImplementedOnCuda, FerrotorchError)
    assert "cholesky" in str(C.NotImplementedOnCuda("cholesky"))
    a, b = torch.tensor(2.0, requires_grad=True), torch.tensor(3.0, requires_grad=True)
    C.backward_parallel([a * a, a * b], None)
    assert a.grad.item() == 7.0 and b.grad.item() == 2.0
    w = torch.tensor([3.0, 4.0], requires_grad=True)
    n = C.grad_norm((w * w).sum(), [w])
    assert abs(n.item() - 10.0) < 1e-5
    n.backward()                                       # differentiable: d||2w||/dw = 2 w/||w||
    _close(w.grad, torch.tensor([1.2, 1.6]))
    xs = torch.randn(5, 3, requires_grad=True)
    gp = C.gradient_penalty(lambda t: (t * 2).sum(1), xs, target=1.0)
    assert abs(gp.item() - (math.sqrt(12) - 1) ** 2) < 1e-4


def test_autocast_policy_dispatcher_profiler_rng_pool_enums():
    assert C.autocast_category("matmul") == C.AutocastCategory.Reduced and C.autocast_category("softmax") == C.AutocastCategory.Full
    a, b = torch.randn(2, 2), torch.randn(2, 2)
    ca, cb = C.autocast_cast("matmul", a, b)
    assert ca.dtype == torch.bfloat16 and cb.dtype == torch.bfloat16
    (cs,) = C.autocast_cast("softmax", a.bfloat16())
    assert cs.dtype == torch.float32
    d = C.Dispatcher()
    d.register("neg", C.DispatchKey.Cpu, lambda t, **kw: -t)
    assert torch.equal(d.call("neg", a), -a) and C.DispatchKey.Cpu in C.Dispatcher.keys_of(a)

    class Rec(C.OpProfiler):
        def __init__(self):
            self.ops = []

        def on_op(self, name, category, shapes, seconds):
            self.ops.append(name)

    rec = Rec()
    C.set_current_profiler(rec)
    assert C.current_profiler() is rec
    assert C.profile_op_scope("my_op", "test", [(2, 2)], lambda: 41 + 1) == 42
    C.set_current_profiler(None)
    assert C.current_profiler() is None and rec.ops == ["my_op"]
    assert C.cuda_rng() is C.cuda_rng()
    t = C.cpu_pool.take(1000)
    assert t.numel() >= 1000
    before = C.cpu_pool.stats()["hits"]
    C.cpu_pool.give(t)
    C.cpu_pool.take(1000)
    assert C.cpu_pool.stats()["hits"] == before + 1
    assert C.DType.BF16 in C.DType and len(list(C.DType)) == 8
    assert [m.name for m in C.MemoryFormat] == ["Contiguous", "ChannelsLast", "ChannelsLast3d"]
