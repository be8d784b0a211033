"""Per-symbol behaviour checks of ``ferrotorch_b200.optim``: configuration records, scheduler enums and bases, the SWA rate schedule against
PyTorch's, the differentiable SGD steps and the scalar helpers."""
import math

import pytest
import torch

import ferrotorch_b200.optim as O
from ferrotorch_b200.distributions import Distribution, Normal, kl_divergence, register_kl


def test_config_records_feed_their_optimizers():
    w = torch.nn.Parameter(torch.tensor([1.0, -2.0]))
    cfg = O.SgdConfig(lr=0.5, momentum=0.9, nesterov=True)
    assert (cfg.lr, cfg.momentum, cfg.nesterov, cfg.weight_decay) == (0.5, 0.9, True, 0.0)
    a = O.AdamConfig(lr=1e-2, betas=(0.8, 0.9), amsgrad=True)
    assert a.betas == (0.8, 0.9) and a.amsgrad and a.eps == 1e-8
    m = O.MuonConfig()
    assert m.ns_steps == 5 and m.nesterov and m.momentum == 0.95
    s = O.SparseAdamConfig(lr=0.1)
    assert s.lr == 0.1 and s.betas == (0.9, 0.999)
    g = O.GradScalerConfig(init_scale=8.0, growth_interval=2)
    assert g.init_scale == 8.0 and g.backoff_factor == 0.5 and g.enabled
    st = O.GradScalerState(scale=8.0, growth_tracker=1)
    assert st.scale == 8.0 and st.growth_tracker == 1 and st.found_inf is False
    opt = O.Sgd([w], lr=cfg.lr, momentum=cfg.momentum, nesterov=cfg.nesterov)
    assert opt.param_groups[0]["momentum"] == 0.9


def test_scheduler_enums_and_bases():
    assert {e.value for e in O.AnnealStrategy} >= {"cos", "linear"}
    assert len(list(O.CyclicMode)) == 3 and len(list(O.PlateauMode)) == 2
    w = torch.nn.Parameter(torch.zeros(1))
    opt = O.Sgd([w], lr=1.0)

    class Halve(O.LrScheduler):
        def get_lr(self):
            return [g["lr"] * (0.5 if self.last_epoch else 1.0) for g in self.optimizer.param_groups]

    s = Halve(opt)
    s.step()
    s.step()
    assert s.get_last_lr() == [0.25] and s.last_epoch == 2
    opt2 = O.Sgd([w], lr=1.0)
    ms = O.MetricScheduler(opt2, mode="min", factor=0.1, patience=1)
    for metric in (1.0, 1.0, 1.0):
        ms.step(metric)
    assert abs(opt2.param_groups[0]["lr"] - 0.1) < 1e-12


@pytest.mark.parametrize("strategy", ["cos", "linear"])
def test_swa_rate_schedule_matches_torch(strategy):
    w = torch.nn.Parameter(torch.zeros(1))
    a, b = O.Sgd([w], lr=1.0), torch.optim.SGD([w], lr=1.0)
    sa, sb = O.Swalr(a, 0.05, anneal_epochs=4, anneal_strategy=strategy), torch.optim.swa_utils.SWALR(b, 0.05, anneal_epochs=4, anneal_strategy=strategy)
    for _ in range(7):
        assert abs(a.param_groups[0]["lr"] - b.param_groups[0]["lr"]) < 1e-12
        sa.step()
        sb.step()
    assert abs(a.param_groups[0]["lr"] - 0.05) < 1e-12
    with pytest.raises(ValueError):
        O.Swalr(a, 0.05, anneal_strategy="exp")
    assert O.Swalr(a, 0.05, anneal_strategy=O.AnnealStrategy("cos")).anneal_strategy == "cos"


def test_differentiable_sgd_steps_and_scalar_helpers():
    p = torch.tensor([1.0, 2.0], requires_grad=True)
    lr = torch.tensor(0.1, requires_grad=True)
    g = 2 * p
    (new,) = O.diff_sgd_step([p], [g], lr)
    assert torch.allclose(new, torch.tensor([0.8, 1.6]))
    new.sum().backward()
    assert abs(lr.grad.item() + 6.0) < 1e-6          # d(sum(p - lr * 2p))/d lr = -2 * sum(p)
    buf = torch.tensor([0.5, 0.5])
    out = O.diff_sgd_momentum_step([p.detach()], [g.detach()], [buf], 0.1, 0.9)
    new_p, new_b = out[0][0], out[1][0]
    assert torch.allclose(new_b, 0.9 * buf + g.detach()) and torch.allclose(new_p, p.detach() - 0.1 * new_b)
    assert torch.equal(O.elemwise_max(torch.tensor([1.0, 5.0]), torch.tensor([3.0, 2.0])), torch.tensor([3.0, 5.0]))
    s = O.scalar_on(2.5, torch.zeros(3, dtype=torch.float64))
    assert s.dtype == torch.float64 and s.dim() == 0 and s.item() == 2.5


def test_distribution_base_and_kl_registration():
    assert issubclass(Normal, Distribution)

    class Point(Distribution):
        def __init__(self, x):
            super().__init__()
            self.x = x

    with pytest.raises(NotImplementedError):
        kl_divergence(Point(torch.tensor(0.0)), Normal(torch.tensor(0.0), torch.tensor(1.0)))

    @register_kl(Point, Normal)
    def _kl_point_normal(p, q):
        return -q.log_prob(p.x)

    got = kl_divergence(Point(torch.tensor(0.5)), Normal(torch.tensor(0.0), torch.tensor(1.0)))
    assert abs(got.item() - (0.5 * 0.25 + 0.5 * math.log(2 * math.pi))) < 1e-6


def test_pytorch_spellings_name_the_same_classes():
    from ferrotorch_b200 import optim as O
    assert O.SGD is O.Sgd and O.RMSprop is O.Rmsprop and O.ASGD is O.Asgd and O.LBFGS is O.Lbfgs
    assert O.SWALR is O.Swalr and O.SequentialLR is O.SequentialLr
