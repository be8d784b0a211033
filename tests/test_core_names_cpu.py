"""Functional names of the core package: argument checks, FFT layout, cumulative / indexing results, dual arithmetic, anomaly mode, key sets."""
import pytest
import torch

from ferrotorch_b200 import core as C
from ferrotorch_b200.errors import FerrotorchError, InvalidArgument, ShapeMismatch


def test_shape_and_indexing_functions_check_like_the_reference():
    assert C.normalize_axis(-1, 3) == 2 and C.normalize_axis(0, 3) == 0
    for bad in (3, -4):
        with pytest.raises(InvalidArgument, match="out of bounds"):
            C.normalize_axis(bad, 3)
    assert C.broadcast_shapes([3, 1], [1, 4]) == (3, 4)
    with pytest.raises(ShapeMismatch):
        C.broadcast_shapes([3], [4])
    x = torch.arange(12.0).view(3, 4)
    assert torch.equal(C.sum_dim(x, -1), x.sum(1)) and C.mean_dim(x, 0, True).shape == (1, 4)
    assert torch.equal(C.cat([x, x], -1), torch.cat([x, x], 1))
    with pytest.raises(ShapeMismatch):
        C.cat([x, torch.zeros(2, 5)], 0)
    with pytest.raises(InvalidArgument):
        C.cat([])
    assert C.view_t(x, [2, -1]).shape == (2, 6) and C.view_t(x, [2, -1]).data_ptr() == x.data_ptr()
    with pytest.raises(ShapeMismatch):
        C.view_t(x.t(), [12])
    with pytest.raises(InvalidArgument):
        C.view_t(x, [-1, -1])
    assert C.permute_t(x, [1, 0]).shape == (4, 3) and C.contiguous_t(x.t()).is_contiguous()
    with pytest.raises(InvalidArgument):
        C.permute_t(x, [0, 0])
    assert [t.shape[1] for t in C.chunk_t(x, 3, 1)] == [2, 2] and [t.shape[0] for t in C.split_t(x, [1, 2], 0)] == [1, 2]
    with pytest.raises(InvalidArgument):
        C.split_t(x, [1, 1], 0)
    with pytest.raises(ShapeMismatch):
        C.expand(x, [2, 3, 5])
    assert torch.equal(C.roll(x, 1, -1), torch.roll(x, 1, 1)) and torch.equal(C.tril(x), torch.tril(x)) and torch.equal(C.triu(x, 1), torch.triu(x, 1))
    with pytest.raises(InvalidArgument):
        C.tril(torch.zeros(3))
    with pytest.raises(InvalidArgument):
        C.diag(torch.zeros(2, 2, 2))
    assert C.diagflat(torch.tensor([1.0, 2.0])).shape == (2, 2) and C.meshgrid([]) == []
    a, b = C.meshgrid([torch.arange(2), torch.arange(3)])
    assert a.shape == (2, 3) and b[0].tolist() == [0, 1, 2]
    with pytest.raises(InvalidArgument):
        C.meshgrid([torch.zeros(2, 2)])
    assert torch.allclose(C.cdist(x, x[:2]), torch.cdist(x, x[:2]))
    with pytest.raises(ShapeMismatch):
        C.cdist(x, torch.zeros(2, 5))
    assert torch.equal(C.clamp(x, 2.0, 5.0), x.clamp(2, 5))
    for bad in ((None, None), (3.0, 1.0)):
        with pytest.raises(InvalidArgument):
            C.clamp(x, *bad)
    w = C.where_cond([True, False, True, False], torch.ones(2, 2), torch.zeros(2, 2))
    assert w.tolist() == [[1, 0], [1, 0]]
    with pytest.raises(ShapeMismatch):
        C.where_cond([True], torch.ones(2, 2), torch.zeros(2, 2))
    assert torch.equal(C.gather(x, 1, [[0], [1], [3]]), x.gather(1, torch.tensor([[0], [1], [3]])))
    with pytest.raises(InvalidArgument):
        C.gather(x, 1, [[4], [0], [0]])
    assert C.scatter_add(torch.zeros(3, 4), 0, torch.zeros(3, 4, dtype=torch.long), x)[0].tolist() == x.sum(0).tolist()
    assert C.scatter(torch.zeros(3, 4), 1, [[1], [1], [1]], torch.ones(3, 1))[:, 1].tolist() == [1, 1, 1]
    src = torch.arange(8.0).view(4, 2).requires_grad_(True)
    seg = C.scatter_add_segments(src, [2, 0, 2, 1], 3)
    assert seg.tolist() == [[2, 3], [6, 7], [4, 6]]
    seg.sum().backward()
    assert torch.equal(src.grad, torch.ones(4, 2))
    for bad in ([0, 1, 2], [0, 1, 2, 3]):
        with pytest.raises(FerrotorchError):
            C.scatter_add_segments(src.detach(), bad, 3)
    vals, inv, counts = C.unique_consecutive(torch.tensor([1.0, 1.0, 2.0, 2.0, 2.0, 1.0]))
    assert vals.tolist() == [1, 2, 1] and inv == [0, 0, 1, 1, 1, 2] and counts == [2, 3, 1]
    r = C.cummax(torch.tensor([[1.0, 3.0, 2.0, 5.0]]), -1)
    assert isinstance(r, C.CumExtremeResult) and r.values.tolist() == [[1, 3, 3, 5]] and r.indices.tolist() == [[0, 1, 1, 3]]
    assert C.cummin(torch.tensor([3.0, 1.0, 2.0]), 0).indices.tolist() == [0, 1, 1] and C.cumprod(torch.tensor([1.0, 2.0, 3.0]), 0).tolist() == [1, 2, 6]
    z = torch.randn(5)
    assert torch.allclose(C.logcumsumexp(z, 0), torch.log(torch.cumsum(z.exp(), 0)), atol=1e-6)
    assert torch.allclose(C.xlogy(torch.tensor([0.0, 2.0]), torch.tensor([0.0, 3.0])), torch.tensor([0.0, 2 * 1.0986123])) and float(C.sinc(torch.tensor(0.0))) == 1.0
    C.validate_cond_branches([x], [x.clone()])
    for t, f in (([x], []), ([x], [x[:2]]), ([x], [x.long()])):
        with pytest.raises(FerrotorchError):
            C.validate_cond_branches(t, f)


def test_fft_family_uses_trailing_re_im_pairs():
    x = torch.randn(3, 8)
    c = torch.randn(3, 8, dtype=torch.complex64)
    cr = torch.view_as_real(c)
    assert torch.allclose(C.rfft(x), torch.view_as_real(torch.fft.rfft(x)), atol=1e-5) and C.rfft(x).shape == (3, 5, 2)
    assert torch.allclose(C.irfft(C.rfft(x), 8), x, atol=1e-5)
    assert torch.allclose(C.fft(cr), torch.view_as_real(torch.fft.fft(c)), atol=1e-5) and torch.allclose(C.ifft(C.fft(cr)), cr, atol=1e-5)
    assert torch.allclose(C.fft2(cr), torch.view_as_real(torch.fft.fft2(c)), atol=1e-4) and torch.allclose(C.ifft2(C.fft2(cr)), cr, atol=1e-5)
    assert torch.allclose(C.fftn(cr, [0]), torch.view_as_real(torch.fft.fftn(c, dim=[0])), atol=1e-5) and torch.allclose(C.ifftn(C.fftn(cr)), cr, atol=1e-5)
    assert torch.allclose(C.irfftn(C.rfftn(x), s=[3, 8]), x, atol=1e-5) and torch.allclose(C.hfft(C.ihfft(x), 8), x, atol=1e-5)
    assert torch.equal(C.fftshift(torch.arange(4)), torch.tensor([2, 3, 0, 1])) and torch.equal(C.ifftshift(C.fftshift(torch.arange(5))), torch.arange(5))
    assert C.fftfreq(4).tolist() == [0.0, 0.25, -0.5, -0.25] and C.rfftfreq(4, 0.5).tolist() == [0.0, 0.5, 1.0]
    with pytest.raises(ShapeMismatch):
        C.fft(x)                                              # last dimension is 8, not (re, im)
    with pytest.raises(InvalidArgument):
        C.fftfreq(0)
    assert torch.allclose(C.fft.fft2(c), torch.fft.fft2(c))   # the namespace keeps torch's complex forms
    xr = x.clone().requires_grad_(True)
    C.rfft_differentiable(xr).pow(2).sum().backward()
    assert xr.grad is not None and torch.isfinite(xr.grad).all()


def test_dual_arithmetic_matches_jvp():
    a, da, b, db = torch.randn(3, 3), torch.randn(3, 3), torch.rand(3, 3) + 1, torch.randn(3, 3)
    A, B = C.DualTensor(a, da), C.DualTensor(b, db)
    f = lambda p, q: ((p @ q) * p - q) / q + (-p)            # noqa: E731
    d = C.dual_add(C.dual_div(C.dual_sub(C.dual_mul(C.dual_matmul(A, B), A), B), B), C.dual_neg(A))
    want, tang = torch.func.jvp(f, (a, b), (da, db))
    assert torch.allclose(d.primal, want, atol=1e-5) and torch.allclose(d.tangent, tang, atol=1e-4)


def test_backward_seed_anomaly_autocast_debug():
    x = torch.randn(3, requires_grad=True)
    C.backward_with_grad(x * 2, torch.ones(3))
    assert x.grad.tolist() == [2, 2, 2]
    with pytest.raises(ShapeMismatch):
        C.backward_with_grad(x * 2, torch.ones(2))
    with pytest.raises(FerrotorchError):
        C.backward_with_grad(x * 2)
    with pytest.raises(FerrotorchError):
        C.backward_with_grad(torch.zeros(()))
    bad = torch.tensor([1.0, float("nan"), float("inf")])
    assert not C.AnomalyMode.is_enabled() and C.ForwardBacktrace.capture_if_enabled() is None
    C.check_gradient_anomaly(bad, "mul")                      # off: nothing happens
    with C.AnomalyMode.guard():
        bt = C.ForwardBacktrace.capture_if_enabled()
        assert C.AnomalyMode.is_enabled() and "test_backward_seed" in str(bt)
        with pytest.raises(InvalidArgument, match="NaN and Inf in gradient of mul"):
            C.check_gradient_anomaly(bad, "mul", bt)
        with pytest.raises(InvalidArgument, match="no forward backtrace"):
            C.check_gradient_anomaly(torch.tensor([float("inf")]), "div")
        C.check_gradient_anomaly(torch.ones(2), "add")
    assert not C.AnomalyMode.is_enabled()
    assert C.autocast_guard("matmul") is None and C.autocast_dtype() is C.AutocastDtype.BF16 and C.AutocastDtype.F16.torch_dtype() == torch.float16
    n0 = len(C.autocast_events())
    with C.autocast(torch.float16, device_type="cpu"):
        assert C.autocast_guard("matmul") is C.AutocastCategory.Reduced and C.autocast_dtype() is C.AutocastDtype.F16 and len(C.autocast_events()) == n0
        C.set_autocast_debug(True)
        assert C.is_autocast_debug() and C.autocast_guard("softmax") is C.AutocastCategory.Full and C.autocast_events()[-1] == ("softmax", "full")
        C.set_autocast_debug(False)


def test_key_sets_ids_storage_and_nn_names():
    K = C.DispatchKey
    s = C.DispatchKeySet.from_keys([K.Cpu, K.Autograd, K.Cpu])
    assert len(s) == 2 and s.contains(K.Autograd) and not s.contains(K.Cuda) and s.highest() is K.Vmap or s.highest() is K.Autograd
    assert s.insert(K.Cuda).contains(K.Cuda) and not s.contains(K.Cuda) and s.remove(K.Cpu) == C.DispatchKeySet.from_keys([K.Autograd])
    assert s.union(C.DispatchKeySet.from_keys([K.Meta])).keys() == [K.Autograd, K.Meta, K.Cpu] and s.intersection(C.DispatchKeySet.all()) == s
    assert C.DispatchKeySet.empty().is_empty() and C.DispatchKeySet.empty().highest() is None and len(C.DispatchKeySet.all()) == len(list(K))
    with pytest.raises(AttributeError):
        s.bits = 3
    t = torch.zeros(4, 4)
    assert C.TensorId.of(t) == C.TensorId.of(t) and C.TensorId.of(torch.zeros(1)) > C.TensorId.of(t) and C.TensorId.next() < C.TensorId.next()
    st, view = C.TensorStorage(t), C.TensorStorage(t[1:])
    assert st.is_cpu() and st.buffer() is C.StorageBuffer.Cpu and st.len() == 16 and st.nbytes() == 64 and st.shares_with(view) and not st.shares_with(C.TensorStorage(t.clone()))
    assert C.TensorStorage.cpu([1.0, 2.0]).len() == 2 and C.StorageBuffer.of(torch.empty(1, device="meta")) is C.StorageBuffer.Meta
    assert isinstance((torch.ones(1, requires_grad=True) * 2).grad_fn, C.GradFn) and torch.float32 in C.Float and torch.int64 in C.IntElement and torch.bool in C.Element
    assert issubclass(C.MinMaxObserver, C.Observer) and not issubclass(int, C.Observer) and C.EinopsReduction.Mean.value == "mean"
    from ferrotorch_b200 import nn
    assert C.FakeQuantize is nn.FakeQuantize and C.QatLayer is nn.FakeQuantize and C.QatModel is nn.QuantizedModel and C.prepare_qat is nn.prepare_qat
    assert C.gelu is nn.gelu and C.GeluApproximate is nn.GeluApproximate and C.flex_attention is nn.flex_attention
    x = torch.tensor([-10.0, -0.26, 0.24, 10.0], requires_grad=True)
    y = C.fake_quantize_differentiable(x, 0.5, 0, -4, 4)
    assert y.tolist() == [-2.0, -0.5, 0.0, 2.0]
    y.sum().backward()
    assert x.grad.tolist() == [0.0, 1.0, 1.0, 0.0]
    base = torch.arange(6.0, requires_grad=True)
    win = C.AsStridedBackward.apply(base, (4, 3), (1, 1))      # overlapping windows of length 3
    assert win[1].tolist() == [1, 2, 3]
    win.sum().backward()
    assert base.grad.tolist() == [1, 2, 3, 3, 2, 1]
    with pytest.raises(AttributeError):
        C.no_such_name


def test_meta_rules_and_parameterised_functionals():
    from ferrotorch_b200.nn import functional as Fn
    from ferrotorch_b200.errors import DeviceMismatch
    m = C.full_meta([4, 1, 6], 3.0)
    assert m.is_meta and m.shape == (4, 1, 6) and C.meta_like(torch.zeros(2, 3)).shape == (2, 3)
    mp = C.meta_propagate
    assert mp.unary_same_shape(m).shape == (4, 1, 6) and mp.unary_same_shape(torch.zeros(2)) is None
    assert mp.binary_broadcast(m, C.full_meta([5, 1])).shape == (4, 5, 6) and mp.binary_broadcast(torch.zeros(2), torch.zeros(2)) is None
    with pytest.raises(DeviceMismatch):
        mp.binary_broadcast(m, torch.zeros(6))
    with pytest.raises(ShapeMismatch):
        mp.binary_broadcast(m, C.full_meta([7]))
    assert mp.reduce_dim(m, -1).shape == (4, 1) and mp.reduce_dim(m, 0, True).shape == (1, 1, 6) and mp.reduce_all(m).shape == () and mp.reduce_all(torch.zeros(1)) is None
    for sa, sb, want in (([3], [3], ()), ([2, 3], [3], (2,)), ([3], [3, 4], (4,)), ([2, 3], [3, 4], (2, 4)), ([5, 1, 2, 3], [7, 3, 4], (5, 7, 2, 4))):
        assert mp.matmul(C.full_meta(sa), C.full_meta(sb)).shape == want == tuple(torch.matmul(torch.zeros(sa), torch.zeros(sb)).shape)
    with pytest.raises(ShapeMismatch):
        mp.matmul(C.full_meta([2, 3]), C.full_meta([4, 5]))
    with pytest.raises(InvalidArgument):
        mp.matmul(C.full_meta([]), C.full_meta([3]))
    assert mp(lambda a, b: a @ b, ((2, 3), torch.float32), ((3, 4), torch.float32)) == [((2, 4), torch.float32)]        # the whole-function form still works
    x = torch.linspace(-3, 3, 13)
    assert float(Fn.sum(x)) == pytest.approx(0.0, abs=1e-6) and float(Fn.mean(x)) == pytest.approx(0.0, abs=1e-6)
    assert torch.equal(Fn.hardtanh_with(x, -0.5, 2.0), x.clamp(-0.5, 2.0)) and torch.allclose(Fn.log_sigmoid(x), torch.log(torch.sigmoid(x)), atol=1e-6)
    assert torch.allclose(Fn.softplus_with(x, 2.0, 20.0), torch.log1p(torch.exp(2 * x)) / 2, atol=1e-6) and torch.allclose(Fn.elu_with(x, 0.5), torch.where(x > 0, x, 0.5 * (x.exp() - 1)))
    img = torch.randn(2, 3, 4)
    assert torch.allclose(Fn.prelu(img, [0.1, 0.2, 0.3]), torch.where(img > 0, img, img * torch.tensor([0.1, 0.2, 0.3]).view(1, 3, 1)))
    assert torch.allclose(Fn.prelu(img, 0.25), torch.where(img > 0, img, 0.25 * img)) and torch.allclose(Fn.gelu_with(x, "sigmoid"), x * torch.sigmoid(1.702 * x))
    for bad in (lambda: Fn.hardtanh_with(x, 1.0, 0.0), lambda: Fn.softplus_with(x, 0.0), lambda: Fn.prelu(img, [0.1, 0.2])):
        with pytest.raises(FerrotorchError):
            bad()
