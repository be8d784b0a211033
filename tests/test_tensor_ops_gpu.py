"""Generic device kernels (elementwise, strided, reductions, scans, indexing, Philox, unscale, GGUF dequant, token mask) against torch in f32."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _t(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2), (torch.float16, 2e-3), (torch.float64, 1e-12)])
def test_unary_forward_and_backward(dtype, tol):
    from ferrotorch_b200.ops import tensor_ops as T
    x = _t(333, 1001, dtype=dtype)
    ref_in = x.double() if dtype == torch.float64 else x.float()
    cases = {"neg": torch.neg, "abs": torch.abs, "exp": torch.exp, "tanh": torch.tanh, "sigmoid": torch.sigmoid, "relu": torch.relu, "gelu": F.gelu,
             "gelu_tanh": lambda t: F.gelu(t, approximate="tanh"), "silu": F.silu, "mish": F.mish, "erf": torch.erf, "sin": torch.sin, "cos": torch.cos,
             "floor": torch.floor, "sign": torch.sign, "square": torch.square, "hardswish": F.hardswish, "expm1": torch.expm1}
    for name, fn in cases.items():
        if name == "hardswish" and dtype == torch.float64:
            continue                                 # torch evaluates its double hardswish with single-precision constants
        got, ref = T.unary(name, x), fn(ref_in)
        err = ((got.to(ref.dtype) - ref).abs() / (1 + ref.abs())).max().item()
        assert err < tol * 4, (name, err)
    assert torch.allclose(T.unary("elu", x, 0.7).to(ref_in.dtype), F.elu(ref_in, 0.7), atol=tol * 4, rtol=tol * 4)
    assert torch.allclose(T.unary("clamp", x, -0.5, 0.25).to(ref_in.dtype), ref_in.clamp(-0.5, 0.25), atol=tol, rtol=tol)
    assert torch.allclose(T.unary("scale", x, 2.0, 1.0).to(ref_in.dtype), ref_in * 2 + 1, atol=tol * 4, rtol=tol * 4)
    pos = x.abs() + 0.5
    assert torch.allclose(T.unary("log", pos).to(ref_in.dtype), pos.to(ref_in.dtype).log(), atol=tol * 4, rtol=tol * 4)
    assert torch.allclose(T.unary("rsqrt", pos).to(ref_in.dtype), pos.to(ref_in.dtype).rsqrt(), atol=tol * 4, rtol=tol * 4)
    if dtype in (torch.float32, torch.float64):
        g = _t(333, 1001, dtype=dtype, seed=1)
        for name, fn, saved_is_out in [("relu", torch.relu, False), ("gelu", F.gelu, False), ("gelu_tanh", lambda t: F.gelu(t, approximate="tanh"), False),
                                       ("silu", F.silu, False), ("mish", F.mish, False), ("tanh_y", torch.tanh, True), ("sigmoid_y", torch.sigmoid, True),
                                       ("hardswish", F.hardswish, False)]:
            xr = x.clone().requires_grad_()
            y = fn(xr)
            y.backward(g)
            got = T.unary_backward(name, g, y.detach() if saved_is_out else x)
            assert torch.allclose(got, xr.grad, atol=1e-5, rtol=1e-4), name


def test_binary_broadcast_where_cast_strided():
    from ferrotorch_b200.ops import tensor_ops as T
    a, b = _t(64, 1, 33), _t(1, 17, 33, seed=1)
    for name, fn in [("add", torch.add), ("sub", torch.sub), ("mul", torch.mul), ("div", torch.div), ("maximum", torch.maximum), ("minimum", torch.minimum)]:
        assert torch.allclose(T.binary(name, a, b), fn(a, b), atol=1e-6), name
    x, y = _t(100, 257), _t(100, 257, seed=2)
    assert torch.equal(T.binary("add", x, y), x + y) and torch.equal(T.binary("lt", x, y), (x < y).float())
    xb, yb = x.bfloat16(), y.bfloat16()
    assert torch.equal(T.binary("mul", xb, yb), xb * yb)
    assert torch.equal(T.where(x > 0, x, y), torch.where(x > 0, x, y))
    assert torch.equal(T.where((a > 0), a, b), torch.where(a > 0, a, b))
    assert torch.equal(T.cast(x, torch.bfloat16), x.bfloat16()) and torch.equal(T.cast(xb, torch.float32), xb.float())
    assert torch.equal(T.cast(x, torch.float16), x.half()) and torch.equal(T.cast(x, torch.float64), x.double())
    xt = _t(8, 16, 32).permute(2, 0, 1)
    assert torch.equal(T.contiguous(xt), xt.contiguous()) and T.contiguous(xt).is_contiguous()
    assert torch.equal(T.unary("relu", xt), torch.relu(xt))
    assert torch.equal(T.cat([x, y, x[:3]], 0), torch.cat([x, y, x[:3]], 0)) and torch.equal(T.cat([x, y], 1), torch.cat([x, y], 1))
    z = torch.empty_like(x)
    assert float(T.fill_(z, 2.5).sum()) == 2.5 * z.numel()
    m = x > 1
    assert torch.equal(T.masked_fill_(x.clone(), m, -7.0), x.masked_fill(m, -7.0))


def test_reductions_and_scans():
    from ferrotorch_b200.ops import tensor_ops as T
    x = _t(37, 129, 65)
    for dim in (0, 1, 2):
        assert torch.allclose(T.reduce("sum", x, dim), x.sum(dim), atol=1e-4)
        assert torch.allclose(T.reduce("mean", x, dim, True), x.mean(dim, True), atol=1e-5)
        assert torch.equal(T.reduce("max", x, dim), x.amax(dim)) and torch.equal(T.reduce("min", x, dim), x.amin(dim))
        assert torch.allclose(T.reduce("logsumexp", x, dim), x.logsumexp(dim), atol=1e-4)
        assert torch.allclose(T.scan("cumsum", x, dim), x.cumsum(dim), atol=1e-4)
        assert torch.equal(T.scan("cummax", x, dim), x.cummax(dim).values)
        assert torch.allclose(T.scan("logcumsumexp", x, dim), x.logcumsumexp(dim), atol=1e-4)
        assert torch.allclose(T.scan("cumsum", x, dim, reverse=True), x.flip(dim).cumsum(dim).flip(dim), atol=1e-4)
    small = _t(5, 9, scale=0.5)
    assert torch.allclose(T.reduce("prod", small, 1), small.prod(1), atol=1e-6) and torch.allclose(T.scan("cumprod", small, 1), small.cumprod(1), atol=1e-6)
    big = _t(3_000_017)
    assert abs(float(T.reduce("sum", big)) - float(big.double().sum())) < 0.05
    assert torch.allclose(T.reduce("sumsq", big), (big.double() ** 2).sum().float(), rtol=1e-5)
    assert float(T.reduce("absmax", big)) == float(big.abs().max()) and float(T.reduce("max", big)) == float(big.max())
    xb = x.bfloat16()
    assert torch.allclose(T.reduce("sum", xb, 1).float(), xb.float().sum(1), atol=0.15, rtol=2e-2)


def test_indexing():
    from ferrotorch_b200 import _lib
    from ferrotorch_b200.ops import tensor_ops as T
    x = _t(50, 40, 24)
    idx = torch.randint(0, 40, (77,), device="cuda")
    assert torch.equal(T.index_select(x, 1, idx), x.index_select(1, idx))
    assert torch.equal(T.index_select(x.bfloat16(), 0, idx % 50), x.bfloat16().index_select(0, idx % 50))
    src = _t(50, 77, 24, seed=3)
    assert torch.allclose(T.index_add_(torch.zeros_like(x), 1, idx, src), torch.zeros_like(x).index_add_(1, idx, src), atol=1e-5)
    gi = torch.randint(0, 40, (50, 13, 24), device="cuda")
    assert torch.equal(T.gather(x, 1, gi), x.gather(1, gi))
    s2 = _t(50, 13, 24, seed=4)
    assert torch.allclose(T.scatter_add_(torch.zeros_like(x), 1, gi, s2), torch.zeros_like(x).scatter_add_(1, gi, s2), atol=1e-5)
    assert _lib.read_status() == 0
    bad = idx.clone()
    bad[5] = 1000                                    # out of range: reported through the status word, no fault, row zeroed
    out = T.index_select(x, 1, bad)
    st = _lib.read_status()
    assert st >> 24 == 0x21 and float(out[:, 5].abs().sum()) == 0.0 and _lib.read_status() == 0


def test_philox_stream_dropout_and_unscale():
    from ferrotorch_b200.ops import tensor_ops as T
    g = T.PhiloxGenerator(seed=1234567890123, offset=5)
    u = g.uniform_(torch.empty(1003, device="cuda"))
    assert torch.allclose(u.cpu(), T.philox_reference(1234567890123, 5, 1003), atol=1e-7) and g.offset == 5 + 251
    st = g.state()
    a = g.normal_(torch.empty(200_000, device="cuda"))
    g.set_state(st)
    assert torch.equal(a, g.normal_(torch.empty(200_000, device="cuda")))
    assert abs(float(a.mean())) < 0.01 and abs(float(a.std()) - 1) < 0.01
    x = torch.ones(1_000_000, device="cuda")
    y, m = g.dropout(x, 0.3, return_mask=True)
    assert abs(float(m.float().mean()) - 0.7) < 0.003 and torch.equal(y, m.float() / 0.7)
    grads = [_t(n, seed=i) * 1024 for i, n in enumerate([5, 1000, 70_001])]
    ref = [t / 1024 for t in grads]
    found, sq = torch.zeros((), device="cuda"), torch.zeros((), device="cuda")
    T.multi_unscale_(grads, 1 / 1024, found, sq)
    assert float(found) == 0 and all(torch.allclose(a, b) for a, b in zip(grads, ref))
    assert torch.allclose(sq, sum((t.double() ** 2).sum() for t in ref).float(), rtol=1e-4)
    grads[1][7] = float("inf")
    T.multi_unscale_(grads, 1.0, found, None)
    assert float(found) == 1


def test_gguf_dequant_and_token_mask():
    from ferrotorch_b200.ops import tensor_ops as T
    g = torch.Generator().manual_seed(0)
    for qt, nbytes in T.GGUF_BLOCK_BYTES.items():
        blocks = torch.randint(0, 256, (64, nbytes), dtype=torch.uint8, generator=g)
        blocks[:, :2] = torch.tensor([0.0123], dtype=torch.float16).view(torch.uint8)          # finite scale
        if qt in ("q4_1", "q5_1", "q8_1"):
            blocks[:, 2:4] = torch.tensor([-0.5], dtype=torch.float16).view(torch.uint8)
        ref = T._gguf_host(blocks.reshape(-1), qt, 64 * 32)
        got = T.gguf_dequantize(blocks.reshape(-1).cuda(), qt, 64 * 32)
        assert torch.allclose(got.cpu(), ref, atol=1e-6), qt
    V = 1000
    logits = _t(4, V)
    allow = torch.rand(V, generator=g) > 0.5
    words = torch.zeros((V + 31) // 32, dtype=torch.int64)
    for v in torch.nonzero(allow).flatten().tolist():
        words[v // 32] |= 1 << (v % 32)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32).cuda()
    ref = logits.masked_fill(~allow.cuda(), float("-inf"))
    assert torch.equal(T.token_mask_(logits.clone(), words), ref)
    assert torch.equal(T.token_mask_(logits.bfloat16(), words), ref.bfloat16())


def test_nms_kernels_match_host_sweep():
    from ferrotorch_b200.vision import ops as V
    g = torch.Generator().manual_seed(0)
    for n in (1, 63, 64, 65, 1000, 5000):
        b = torch.rand(n, 4, generator=g) * 100
        b[:, 2:] = b[:, :2] + torch.rand(n, 2, generator=g) * 30 + 1
        s = torch.rand(n, generator=g)
        assert torch.equal(V.nms(b.cuda(), s.cuda(), 0.5).cpu(), V.nms(b, s, 0.5)), n
    idx = torch.randint(0, 7, (5000,), generator=g)
    assert torch.equal(V.batched_nms(b.cuda(), s.cuda(), idx.cuda(), 0.4).cpu(), V.batched_nms(b, s, idx, 0.4))
