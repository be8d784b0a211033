"""The wider operation set of the native C++ tensor / autograd core (element-wise family, division, reshape, reductions along a dimension,
softmax, conv2d, max-pool) and its Adam / AdamW: values and gradients against PyTorch, then a small convolutional network trained by the
native core step for step beside the same network in PyTorch."""
import numpy as np
import pytest
import torch

from ferrotorch_b200 import native as N


def _t(a, grad=True):
    return N.Tensor(np.asarray(a, np.float32), requires_grad=grad)


def _check(native_fn, torch_fn, *arrays, tol=2e-5):
    nts = [_t(a) for a in arrays]
    tts = [torch.tensor(np.asarray(a, np.float32), requires_grad=True) for a in arrays]
    yn, yt = native_fn(*nts), torch_fn(*tts)
    assert tuple(yn.shape) == tuple(yt.shape), (yn.shape, yt.shape)
    assert np.allclose(yn.numpy(), yt.detach().numpy(), atol=tol, rtol=tol)
    w = np.random.default_rng(1).standard_normal(yt.shape).astype(np.float32)
    (yn * _t(w, False)).sum().backward()
    (yt * torch.tensor(w)).sum().backward()
    for a, b in zip(nts, tts):
        assert np.allclose(a.grad.numpy(), b.grad.numpy(), atol=tol * 5, rtol=tol * 5)


def test_elementwise_family_matches_pytorch():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 7)).astype(np.float32)
    pos = np.abs(x) + 0.5
    for name, tf, arg in (("exp", torch.exp, x), ("log", torch.log, pos), ("sqrt", torch.sqrt, pos), ("gelu", torch.nn.functional.gelu, x),
                          ("silu", torch.nn.functional.silu, x), ("abs", torch.abs, x), ("square", torch.square, x), ("reciprocal", torch.reciprocal, pos)):
        _check(lambda t, n=name: getattr(t, n)(), tf, arg)
    _check(lambda t: t.leaky_relu(0.2), lambda t: torch.nn.functional.leaky_relu(t, 0.2), x)
    _check(lambda t: t.pow(2.5), lambda t: t.pow(2.5), pos)
    _check(lambda t: t ** 3.0, lambda t: t ** 3.0, x)
    y = rng.standard_normal((5, 7)).astype(np.float32) + 3.0
    _check(lambda a, b: a / b, lambda a, b: a / b, x, y)
    _check(lambda a, b: a / b, lambda a, b: a / b, x, y[0])                        # a row vector broadcasts over the rows
    _check(lambda a: a / 4.0, lambda a: a / 4.0, x)
    with pytest.raises(Exception):
        _t(x) / _t(np.ones((3,), np.float32))


def test_reshape_reductions_and_softmax_match_pytorch():
    rng = np.random.default_rng(2)
    x = rng.standard_normal((2, 3, 4)).astype(np.float32)
    _check(lambda t: t.reshape(6, 4).t().reshape(2, -1), lambda t: t.reshape(6, 4).t().reshape(2, -1), x)        # a view of a transposed view
    _check(lambda t: t.flatten(1), lambda t: t.flatten(1), x)
    for dim in (0, 1, 2, -1):
        for keep in (False, True):
            _check(lambda t, d=dim, k=keep: t.sum(d, k), lambda t, d=dim, k=keep: t.sum(d, k), x)
            _check(lambda t, d=dim, k=keep: t.mean(d, k), lambda t, d=dim, k=keep: t.mean(d, k), x)
    _check(lambda t: t.softmax(), lambda t: torch.softmax(t, -1), x)
    _check(lambda t: t.log_softmax(), lambda t: torch.log_softmax(t, -1), x)
    _check(lambda a, b: N.mse_loss(a, b), torch.nn.functional.mse_loss, x, x[::-1].copy())
    for bad in (lambda: _t(x).reshape(5, 5), lambda: _t(x).reshape(-1, -1), lambda: _t(x).sum(3)):
        with pytest.raises(Exception):
            bad()


@pytest.mark.parametrize("stride,padding,bias", [(1, 0, True), (1, 1, True), (2, 1, False), ((2, 1), (0, 2), True)])
def test_conv2d_and_max_pool_match_pytorch(stride, padding, bias):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 3, 9, 8)).astype(np.float32)
    w = rng.standard_normal((4, 3, 3, 3)).astype(np.float32) * 0.3
    b = rng.standard_normal((4,)).astype(np.float32)
    if bias:
        _check(lambda a, c, d: N.conv2d(a, c, d, stride, padding), lambda a, c, d: torch.nn.functional.conv2d(a, c, d, stride, padding), x, w, b, tol=1e-4)
    else:
        _check(lambda a, c: N.conv2d(a, c, None, stride, padding), lambda a, c: torch.nn.functional.conv2d(a, c, None, stride, padding), x, w, tol=1e-4)
    _check(lambda a: N.max_pool2d(a, 2), lambda a: torch.nn.functional.max_pool2d(a, 2), x)
    _check(lambda a: N.max_pool2d(a, 3, 2), lambda a: torch.nn.functional.max_pool2d(a, 3, 2), x)
    with pytest.raises(Exception):
        N.conv2d(_t(x), _t(rng.standard_normal((4, 2, 3, 3))))


@pytest.mark.parametrize("decoupled", [False, True])
def test_adam_and_adamw_follow_pytorch(decoupled):
    rng = np.random.default_rng(4)
    w0, x, y = rng.standard_normal((6, 5)).astype(np.float32), rng.standard_normal((8, 5)).astype(np.float32), rng.standard_normal((8, 6)).astype(np.float32)
    wn, wt = _t(w0), torch.tensor(w0, requires_grad=True)
    on = (N.AdamW([wn], lr=0.05, weight_decay=0.1) if decoupled else N.Adam([wn], lr=0.05, weight_decay=0.1))
    ot = (torch.optim.AdamW([wt], lr=0.05, weight_decay=0.1) if decoupled else torch.optim.Adam([wt], lr=0.05, weight_decay=0.1))
    for _ in range(6):
        on.zero_grad()
        N.mse_loss(N.linear(_t(x, False), wn), _t(y, False)).backward()
        on.step()
        ot.zero_grad()
        torch.nn.functional.mse_loss(torch.tensor(x) @ wt.t(), torch.tensor(y)).backward()
        ot.step()
    assert np.allclose(wn.numpy(), wt.detach().numpy(), atol=2e-5)


def test_small_convolutional_network_trains_like_pytorch():
    """Conv - ReLU - MaxPool - Conv - GELU - Flatten - Linear with cross-entropy, Adam, 8 steps: losses and final weights track PyTorch."""
    rng = np.random.default_rng(5)
    net = N.Sequential(N.Conv2d(1, 4, 3, padding=1, rng=rng), N.ReLU(), N.MaxPool2d(2), N.Conv2d(4, 6, 3, stride=2, rng=rng), N.GELU(), N.Flatten(),
                       N.Linear(6 * 3 * 3, 5, rng=rng))
    ref = torch.nn.Sequential(torch.nn.Conv2d(1, 4, 3, padding=1), torch.nn.ReLU(), torch.nn.MaxPool2d(2), torch.nn.Conv2d(4, 6, 3, stride=2), torch.nn.GELU(),
                              torch.nn.Flatten(), torch.nn.Linear(54, 5))
    with torch.no_grad():
        for mine, theirs in zip([net.mods[0], net.mods[3], net.mods[6]], [ref[0], ref[3], ref[6]]):
            theirs.weight.copy_(torch.tensor(mine.weight.numpy()))
            theirs.bias.copy_(torch.tensor(mine.bias.numpy()))
    assert len(net.parameters()) == 6
    x = rng.standard_normal((16, 1, 14, 14)).astype(np.float32)
    y = rng.integers(0, 5, 16)
    on, ot = N.Adam(net.parameters(), lr=0.01), torch.optim.Adam(ref.parameters(), lr=0.01)
    losses = []
    for _ in range(8):
        on.zero_grad()
        ln = N.cross_entropy(net(_t(x, False)), y)
        ln.backward(threads=2)
        on.step()
        ot.zero_grad()
        lt = torch.nn.functional.cross_entropy(ref(torch.tensor(x)), torch.tensor(y))
        lt.backward()
        ot.step()
        losses.append((ln.item(), lt.item()))
    assert all(abs(a - b) < 2e-3 for a, b in losses) and losses[-1][0] < losses[0][0]
    assert np.allclose(net.mods[0].weight.numpy(), ref[0].weight.detach().numpy(), atol=2e-3)
    assert np.allclose(net.mods[6].weight.numpy(), ref[6].weight.detach().numpy(), atol=2e-3)


def test_permute_batched_matmul_layer_norm_embedding_and_suffix_broadcast_match_pytorch():
    rng = np.random.default_rng(6)
    x = rng.standard_normal((2, 3, 4, 5)).astype(np.float32)
    _check(lambda t: t.permute(0, 2, 1, 3).reshape(2, 4, 15), lambda t: t.permute(0, 2, 1, 3).reshape(2, 4, 15), x)
    _check(lambda t: t.transpose(1, 3), lambda t: t.transpose(1, 3).contiguous(), x)
    a, b = rng.standard_normal((2, 3, 4, 5)).astype(np.float32), rng.standard_normal((2, 3, 5, 6)).astype(np.float32)
    _check(lambda p, q: p @ q, lambda p, q: p @ q, a, b, tol=1e-4)
    _check(lambda p, q: p @ q.transpose(2, 3), lambda p, q: p @ q.transpose(2, 3), a, rng.standard_normal((2, 3, 7, 5)).astype(np.float32), tol=1e-4)
    w, bias = rng.standard_normal(5).astype(np.float32), rng.standard_normal(5).astype(np.float32)
    _check(lambda t, u, v: N.layer_norm(t, u, v), lambda t, u, v: torch.nn.functional.layer_norm(t, (5,), u, v), x, w, bias, tol=1e-4)
    _check(lambda t: N.layer_norm(t), lambda t: torch.nn.functional.layer_norm(t, (5,)), x, tol=1e-4)
    _check(lambda t, u: N.layer_norm(t, u), lambda t, u: torch.nn.functional.layer_norm(t, (5,), u), x, w, tol=1e-4)
    _check(lambda t: t.narrow(2, 1, 2).reshape(2, 3, 10) * 2.0, lambda t: t.narrow(2, 1, 2).reshape(2, 3, 10) * 2.0, x)
    _check(lambda t: t[1] + t[0] + t[-1], lambda t: t[1] + t[0] + t[-1], x)
    _check(lambda t: t.permute(1, 0, 2, 3)[1:3], lambda t: t.permute(1, 0, 2, 3)[1:3], x)
    mask = np.triu(np.full((4, 4), -1e4, np.float32), 1)
    s = rng.standard_normal((2, 3, 4, 4)).astype(np.float32)
    _check(lambda t, m: (t + m).softmax(), lambda t, m: torch.softmax(t + m, -1), s, mask)                          # a [S, S] mask under [B, H, S, S]
    _check(lambda t, m: t * m, lambda t, m: t * m, x, rng.standard_normal((4, 5)).astype(np.float32))
    ids = rng.integers(0, 9, (3, 6))
    table = rng.standard_normal((9, 4)).astype(np.float32)
    tn, tt = _t(table), torch.tensor(table, requires_grad=True)
    en, et = N.embedding(ids, tn), torch.nn.functional.embedding(torch.tensor(ids), tt)
    assert en.shape == (3, 6, 4) and np.allclose(en.numpy(), et.detach().numpy())
    en.square().sum().backward()
    et.square().sum().backward()
    assert np.allclose(tn.grad.numpy(), tt.grad.numpy(), atol=1e-5)
    for bad in (lambda: _t(x).narrow(1, 2, 5), lambda: _t(x)[::2], lambda: _t(x).permute(0, 1, 1, 2), lambda: _t(a) @ _t(a), lambda: N.embedding([[9]], tn), lambda: N.layer_norm(_t(x), _t(np.ones(4))),
                lambda: _t(x) + _t(np.ones((3, 5), np.float32))):
        with pytest.raises(Exception):
            bad()


def test_transformer_block_forward_and_backward_match_pytorch():
    """Pre-norm block with causal multi-head attention and a GELU MLP written on the native core against the same arithmetic in PyTorch."""
    rng = np.random.default_rng(7)
    B, S, D, H = 2, 6, 16, 4
    names = ["wq", "wk", "wv", "wo", "w1", "w2"]
    shapes = {"wq": (D, D), "wk": (D, D), "wv": (D, D), "wo": (D, D), "w1": (4 * D, D), "w2": (D, 4 * D)}
    P = {n: (rng.standard_normal(shapes[n]) / np.sqrt(shapes[n][1])).astype(np.float32) for n in names}
    x = rng.standard_normal((B, S, D)).astype(np.float32)
    mask = np.triu(np.full((S, S), -1e4, np.float32), 1)

    def block_native(xt, p):
        def heads(t):
            return t.reshape(B, S, H, D // H).permute(0, 2, 1, 3)
        h = N.layer_norm(xt)
        q, k, v = (heads(N.linear(h.reshape(B * S, D), p[n]).reshape(B, S, D)) for n in ("wq", "wk", "wv"))
        att = ((q @ k.transpose(2, 3)) * (1.0 / np.sqrt(D // H)) + N.Tensor(mask)).softmax()
        o = (att @ v).permute(0, 2, 1, 3).reshape(B * S, D)
        xt = xt + N.linear(o, p["wo"]).reshape(B, S, D)
        m = N.linear(N.linear(N.layer_norm(xt).reshape(B * S, D), p["w1"]).gelu(), p["w2"]).reshape(B, S, D)
        return xt + m

    def block_torch(xt, p):
        F = torch.nn.functional
        def heads(t):
            return t.reshape(B, S, H, D // H).permute(0, 2, 1, 3)
        h = F.layer_norm(xt, (D,))
        q, k, v = (heads(h @ p[n].t()) for n in ("wq", "wk", "wv"))
        att = torch.softmax((q @ k.transpose(2, 3)) / np.sqrt(D // H) + torch.tensor(mask), -1)
        o = (att @ v).permute(0, 2, 1, 3).reshape(B, S, D)
        xt = xt + o @ p["wo"].t()
        return xt + F.gelu(F.layer_norm(xt, (D,)) @ p["w1"].t()) @ p["w2"].t()
    pn = {n: _t(P[n]) for n in names}
    pt = {n: torch.tensor(P[n], requires_grad=True) for n in names}
    xn, xt = _t(x), torch.tensor(x, requires_grad=True)
    yn, yt = block_native(xn, pn), block_torch(xt, pt)
    assert np.allclose(yn.numpy(), yt.detach().numpy(), atol=2e-4)
    yn.square().mean().backward(threads=2)
    yt.square().mean().backward()
    assert np.allclose(xn.grad.numpy(), xt.grad.numpy(), atol=2e-4)
    for n in names:
        assert np.allclose(pn[n].grad.numpy(), pt[n].grad.numpy(), atol=2e-4), n


def test_smaller_first_operand_and_reflected_operators_match_torch():
    a = torch.rand(4, 3) + 0.5
    b = torch.rand(3) + 0.5
    for op in (lambda x, y: y + x, lambda x, y: y - x, lambda x, y: y * x, lambda x, y: y / x,
               lambda x, y: 2.0 - x, lambda x, y: 2.0 / x, lambda x, y: 1.5 + x):
        ta, tb = a.clone().requires_grad_(True), b.clone().requires_grad_(True)
        na, nb = N.Tensor(a.numpy().copy(), requires_grad=True), N.Tensor(b.numpy().copy(), requires_grad=True)
        to, no = op(ta, tb), op(na, nb)
        assert tuple(no.shape) == tuple(to.shape)
        np.testing.assert_allclose(no.numpy(), to.detach().numpy(), rtol=1e-5, atol=1e-6)
        to.sum().backward(); no.sum().backward()
        np.testing.assert_allclose(na.grad.numpy(), ta.grad.numpy(), rtol=1e-4, atol=1e-5)
        if tb.grad is not None:
            np.testing.assert_allclose(nb.grad.numpy(), tb.grad.numpy(), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dim", [0, 1, -1, -3])
def test_softmax_over_any_dimension(dim):
    x = torch.randn(3, 4, 5)
    for name in ("softmax", "log_softmax"):
        tx = x.clone().requires_grad_(True)
        nx = N.Tensor(x.numpy().copy(), requires_grad=True)
        to, no = getattr(tx, name)(dim), getattr(nx, name)(dim)
        np.testing.assert_allclose(no.numpy(), to.detach().numpy(), rtol=1e-5, atol=1e-6)
        w = torch.randn(3, 4, 5)
        (to * w).sum().backward(); (no * N.Tensor(w.numpy().copy())).sum().backward()
        np.testing.assert_allclose(nx.grad.numpy(), tx.grad.numpy(), rtol=1e-4, atol=1e-5)
