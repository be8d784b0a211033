"""The optimizers implemented in optim/elementwise.py against torch.optim trajectories (CPU tensor-operation forms)."""
import pytest
import torch

from ferrotorch_b200 import optim as O

CASES = [
    (O.Adagrad, torch.optim.Adagrad, dict(lr=0.05, lr_decay=0.01, weight_decay=0.01, initial_accumulator_value=0.1)),
    (O.Adagrad, torch.optim.Adagrad, dict(lr=0.05, maximize=True)),
    (O.Rmsprop, torch.optim.RMSprop, dict(lr=0.01, momentum=0.5, centered=True, weight_decay=0.01)),
    (O.Rmsprop, torch.optim.RMSprop, dict(lr=0.01)),
    (O.Adadelta, torch.optim.Adadelta, dict(lr=1.0, weight_decay=0.01)),
    (O.Adamax, torch.optim.Adamax, dict(lr=0.01, weight_decay=0.01)),
    (O.NAdam, torch.optim.NAdam, dict(lr=0.01, weight_decay=0.01)),
    (O.NAdam, torch.optim.NAdam, dict(lr=0.01, weight_decay=0.01, decoupled_weight_decay=True)),
    (O.RAdam, torch.optim.RAdam, dict(lr=0.01, weight_decay=0.01)),
    (O.RAdam, torch.optim.RAdam, dict(lr=0.01, weight_decay=0.01, decoupled_weight_decay=True)),
    (O.Rprop, torch.optim.Rprop, dict(lr=0.01)),
    (O.Asgd, torch.optim.ASGD, dict(lr=0.01, t0=5, weight_decay=0.01)),
]


def _run(cls, kw, steps=15, device="cpu"):
    g = torch.Generator().manual_seed(0)
    w = torch.randn(7, 5, generator=g).to(device).requires_grad_()
    b = torch.zeros(5, device=device, requires_grad=True)
    x = torch.randn(9, 7, generator=g).to(device)
    o = cls([w, b], **kw)
    for _ in range(steps):
        o.zero_grad()
        ((x @ w + b).tanh().pow(2).sum() + (w ** 2).sum() * 0.01).backward()
        o.step()
    return torch.cat([w.detach().reshape(-1), b.detach()]).cpu(), o


@pytest.mark.parametrize("ours,theirs,kw", CASES)
def test_trajectory_matches_torch(ours, theirs, kw):
    assert not issubclass(ours, theirs)                      # an implementation of its own, not the torch class under another name
    a, o = _run(ours, kw)
    b, _ = _run(theirs, kw)
    assert (a - b).abs().max().item() < 1e-6
    assert isinstance(o, O.Optimizer) and o.lr() == kw["lr"]


def test_config_objects_and_unknown_arguments():
    from ferrotorch_b200.optim.optimizers import AdamaxConfig
    w = torch.zeros(3, requires_grad=True)
    o = O.Adamax([w], AdamaxConfig(lr=0.5, betas=(0.8, 0.9)))
    assert o.param_groups[0]["lr"] == 0.5 and o.param_groups[0]["betas"] == (0.8, 0.9)
    with pytest.raises(TypeError):
        O.Adamax([w], lr=0.1, momentum=0.9)


def test_sparse_adam_touches_only_the_rows_in_the_gradient():
    torch.manual_seed(0)
    res = []
    for cls in (O.SparseAdam, torch.optim.SparseAdam):
        emb = torch.nn.Embedding(20, 4, sparse=True)
        with torch.no_grad():
            emb.weight.copy_(torch.arange(80.0).view(20, 4) / 10)
        o = cls(list(emb.parameters()), lr=0.1)
        for ids in ([1, 3, 3], [3, 7], [1, 19]):
            o.zero_grad()
            emb(torch.tensor(ids)).pow(2).sum().backward()
            o.step()
        res.append(emb.weight.detach().clone())
    assert torch.allclose(res[0], res[1], atol=1e-6)
    assert torch.equal(res[0][0], torch.arange(4.0) / 10)    # a row that never appeared is untouched
    with pytest.raises(RuntimeError):
        w = torch.zeros(3, requires_grad=True)
        w.grad = torch.ones(3)
        O.SparseAdam([w]).step()


@pytest.mark.parametrize("ls", [None, "strong_wolfe"])
def test_lbfgs_converges_like_torch(ls):
    out = []
    for cls in (O.Lbfgs, torch.optim.LBFGS):
        torch.manual_seed(0)
        w = torch.randn(6, requires_grad=True)
        A = torch.randn(6, 6)
        A = A @ A.t() + torch.eye(6)
        o = cls([w], lr=0.5 if ls is None else 1.0, max_iter=10, history_size=5, line_search_fn=ls)

        def closure():
            o.zero_grad()
            l = 0.5 * w @ A @ w - w.sum() + (w ** 4).sum() * 0.1
            l.backward()
            return l
        for _ in range(3):
            o.step(closure)
        out.append((float(closure().detach()), w.detach().clone()))
    assert abs(out[0][0] - out[1][0]) < 1e-5 and (out[0][1] - out[1][1]).abs().max().item() < 2e-3
