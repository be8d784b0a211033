"""The native C++ tensor / autograd core (csrc/runtime/core.cpp through ferrotorch_b200.native) against torch.autograd and torch.optim.SGD."""
import numpy as np
import pytest
import torch

from ferrotorch_b200 import errors, native as N


def _mlp_pair(seed=0):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((16, 12)).astype(np.float32)
    w1, b1 = rng.standard_normal((9, 12)).astype(np.float32) * 0.3, rng.standard_normal(9).astype(np.float32)
    w2, b2 = rng.standard_normal((4, 9)).astype(np.float32) * 0.3, rng.standard_normal(4).astype(np.float32)
    y = rng.integers(0, 4, 16)
    return x, (w1, b1, w2, b2), y


def test_forward_backward_match_torch_on_a_graph_with_shared_nodes():
    x, (w1, b1, w2, b2), y = _mlp_pair()
    P = [N.Tensor(a, requires_grad=True) for a in (w1, b1, w2, b2)]
    h = N.linear(N.Tensor(x), P[0], P[1]).tanh()
    h2 = h * h + h - h.sigmoid() * 0.5                    # h feeds four consumers: contributions must be summed once each
    loss = N.cross_entropy(N.linear(h2, P[2], P[3]), y) + (P[0] * P[0]).mean() * 0.1
    assert loss.grad_fn == "binary" and not loss.is_leaf and P[0].is_leaf
    loss.backward()
    T = [torch.tensor(a, requires_grad=True) for a in (w1, b1, w2, b2)]
    th = torch.tanh(torch.tensor(x) @ T[0].t() + T[1])
    th2 = th * th + th - torch.sigmoid(th) * 0.5
    tl = torch.nn.functional.cross_entropy(th2 @ T[2].t() + T[3], torch.tensor(y)) + (T[0] * T[0]).mean() * 0.1
    tl.backward()
    assert abs(loss.item() - tl.item()) < 1e-5
    for p, t in zip(P, T):
        assert np.allclose(p.grad.numpy(), t.grad.numpy(), atol=2e-6), np.abs(p.grad.numpy() - t.grad.numpy()).max()


def test_parallel_sweep_gives_the_same_bits_as_the_serial_one():
    x, (w1, b1, w2, b2), y = _mlp_pair(1)
    grads = []
    for threads in (1, 2, 8):
        P = [N.Tensor(a, requires_grad=True) for a in (w1, b1, w2, b2)]
        h = N.linear(N.Tensor(x), P[0], P[1]).relu()
        branches = h * h + h.tanh() + h.sigmoid() + h * P[1]             # independent branches the workers can take in any order
        N.cross_entropy(N.linear(branches, P[2], P[3]), y).backward(threads=threads)
        grads.append([p.grad.numpy().copy() for p in P])
    for g in grads[1:]:
        assert all(np.array_equal(a, b) for a, b in zip(grads[0], g))


def test_hooks_no_grad_accumulation_and_errors():
    w = N.Tensor(np.ones((3, 3), np.float32), requires_grad=True)
    x = N.Tensor(np.arange(9, dtype=np.float32).reshape(3, 3))
    seen, done = [], []
    w.register_hook(lambda g: g * 2.0)                                   # doubles every gradient that reaches w
    w.register_post_accumulate_grad_hook(lambda t: done.append(t.id))
    h = x @ w
    h.register_hook(lambda g: seen.append(g.copy()))                     # observes, does not change
    h.sum().backward()
    assert len(seen) == 1 and np.array_equal(seen[0], np.ones(9, np.float32)) and done == [w.id]
    expect = 2.0 * (x.numpy().T @ np.ones((3, 3), np.float32))
    assert np.allclose(w.grad.numpy(), expect)
    (x @ w).sum().backward()                                              # gradients accumulate until zero_grad
    assert np.allclose(w.grad.numpy(), 2 * expect) and len(done) == 2
    w.zero_grad()
    assert w.grad is None
    with N.no_grad():
        assert not (x @ w).requires_grad
    assert (x @ w).requires_grad and not (x @ w).detach().requires_grad
    with pytest.raises(errors.InvalidArgument):
        (x @ w).backward()                                                # non-scalar root without a gradient
    with pytest.raises(errors.InvalidArgument):
        x @ N.Tensor(np.ones((4, 2), np.float32))                         # inner dimensions differ
    with pytest.raises(errors.InvalidArgument):
        N.cross_entropy(x, [0, 1, 7])                                     # target out of range
    v = w.numpy()
    v[0, 0] = 5.0                                                          # numpy() of a contiguous tensor is a view of the native storage
    assert w.numpy()[0, 0] == 5.0 and x.t().numpy()[0, 1] == x.numpy()[1, 0]


@pytest.mark.parametrize("kw", [dict(momentum=0.0), dict(momentum=0.9), dict(momentum=0.9, nesterov=True, weight_decay=1e-2), dict(momentum=0.8, dampening=0.3)])
def test_native_sgd_matches_torch_sgd(kw):
    x, (w1, b1, w2, b2), y = _mlp_pair(2)
    P = [N.Tensor(a.copy(), requires_grad=True) for a in (w1, b1, w2, b2)]
    T = [torch.tensor(a.copy(), requires_grad=True) for a in (w1, b1, w2, b2)]
    on, ot = N.Sgd(P, lr=0.05, **kw), torch.optim.SGD(T, lr=0.05, **kw)
    for _ in range(12):
        on.zero_grad()
        N.cross_entropy(N.linear(N.linear(N.Tensor(x), P[0], P[1]).relu(), P[2], P[3]), y).backward()
        on.step()
        ot.zero_grad()
        torch.nn.functional.cross_entropy(torch.relu(torch.tensor(x) @ T[0].t() + T[1]) @ T[2].t() + T[3], torch.tensor(y)).backward()
        ot.step()
    for p, t in zip(P, T):
        assert np.allclose(p.numpy(), t.detach().numpy(), atol=2e-5)


def test_native_data_parallel_over_the_simulated_fabric_matches_one_process():
    import threading
    from ferrotorch_b200.distributed import SimulatedBackend
    from ferrotorch_b200.distributed.ddp import NativeDDP
    rng = np.random.default_rng(3)
    X, Y = rng.standard_normal((6, 32, 20)).astype(np.float32), rng.integers(0, 5, (6, 32))

    def build():
        r = np.random.default_rng(7)
        return N.Sequential(N.Linear(20, 16, rng=r), N.ReLU(), N.Linear(16, 5, rng=r))
    one = build()
    opt = N.Sgd(one.parameters(), lr=0.1, momentum=0.9)
    for s in range(6):
        opt.zero_grad()
        N.cross_entropy(one(N.Tensor(X[s])), Y[s]).backward()
        opt.step()
    out = {}

    def rank(r, backend):
        m = build()
        ddp = NativeDDP(m, backend, bucket_size_bytes=512)
        assert len(ddp.buckets) > 1
        ddp.broadcast_parameters(0)
        o = N.Sgd(m.parameters(), lr=0.1, momentum=0.9)
        for s in range(6):
            o.zero_grad()
            N.cross_entropy(ddp(N.Tensor(X[s, r * 16:(r + 1) * 16])), Y[s, r * 16:(r + 1) * 16]).backward()
            ddp.sync_gradients()
            o.step()
        out[r] = [p.numpy().copy() for p in m.parameters()]
    bs = SimulatedBackend.create_group(2)
    ts = [threading.Thread(target=rank, args=(r, bs[r])) for r in range(2)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    assert all(np.array_equal(a, b) for a, b in zip(out[0], out[1]))
    assert all(np.allclose(a, p.numpy(), atol=1e-5) for a, p in zip(out[0], one.parameters()))
