"""The learning-rate schedulers of optim/scheduler.py (own implementations) step for step against torch.optim.lr_scheduler."""
import warnings

import pytest
import torch
from torch.optim import lr_scheduler as T

from ferrotorch_b200.optim import scheduler as S


def _opt():
    return torch.optim.SGD([torch.zeros(2, requires_grad=True)], lr=0.1, momentum=0.9)


def _run(make, steps, metric=None):
    o = _opt()
    s = make(o)
    out = []
    for i in range(steps):
        o.step()
        s.step(metric[i]) if metric is not None else s.step()
        out.append((o.param_groups[0]["lr"], o.param_groups[0]["momentum"]))
    return out, s


CASES = {
    "step": (lambda o: S.StepLR(o, 3, 0.5), lambda o: T.StepLR(o, 3, 0.5)),
    "multistep": (lambda o: S.MultiStepLR(o, [2, 5, 5, 9], 0.5), lambda o: T.MultiStepLR(o, [2, 5, 5, 9], 0.5)),
    "constant": (lambda o: S.ConstantLR(o, 0.25, 4), lambda o: T.ConstantLR(o, 0.25, 4)),
    "linear": (lambda o: S.LinearLR(o, 0.2, 0.9, 6), lambda o: T.LinearLR(o, 0.2, 0.9, 6)),
    "exponential": (lambda o: S.ExponentialLR(o, 0.9), lambda o: T.ExponentialLR(o, 0.9)),
    "polynomial": (lambda o: S.PolynomialLR(o, 10, 2.0), lambda o: T.PolynomialLR(o, 10, 2.0)),
    "cosine": (lambda o: S.CosineAnnealingLR(o, 7, 0.01), lambda o: T.CosineAnnealingLR(o, 7, 0.01)),
    "lambda": (lambda o: S.LambdaLR(o, lambda e: 0.95 ** e), lambda o: T.LambdaLR(o, lambda e: 0.95 ** e)),
    "multiplicative": (lambda o: S.MultiplicativeLR(o, lambda e: 0.9), lambda o: T.MultiplicativeLR(o, lambda e: 0.9)),
    "warm_restarts": (lambda o: S.CosineAnnealingWarmRestarts(o, 4, 2, 0.001), lambda o: T.CosineAnnealingWarmRestarts(o, 4, 2, 0.001)),
    "cyclic_triangular2": (lambda o: S.CyclicLR(o, 0.01, 0.1, 4, 6, mode="triangular2"), lambda o: T.CyclicLR(o, 0.01, 0.1, 4, 6, mode="triangular2")),
    "cyclic_exp_range": (lambda o: S.CyclicLR(o, 0.01, 0.1, 3, mode="exp_range", gamma=0.9), lambda o: T.CyclicLR(o, 0.01, 0.1, 3, mode="exp_range", gamma=0.9)),
    "one_cycle": (lambda o: S.OneCycleLR(o, 0.5, total_steps=25), lambda o: T.OneCycleLR(o, 0.5, total_steps=25)),
    "one_cycle_three_phase": (lambda o: S.OneCycleLR(o, 0.5, total_steps=25, three_phase=True, anneal_strategy="linear"),
                              lambda o: T.OneCycleLR(o, 0.5, total_steps=25, three_phase=True, anneal_strategy="linear")),
    "chained": (lambda o: S.ChainedScheduler([S.ConstantLR(o, 0.5, 3), S.ExponentialLR(o, 0.9)]),
                lambda o: T.ChainedScheduler([T.ConstantLR(o, 0.5, 3), T.ExponentialLR(o, 0.9)])),
    "sequential": (lambda o: S.SequentialLr(o, [S.LinearLR(o, 0.1, 1.0, 4), S.CosineAnnealingLR(o, 10)], [5]),
                   lambda o: T.SequentialLR(o, [T.LinearLR(o, 0.1, 1.0, 4), T.CosineAnnealingLR(o, 10)], [5])),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_scheduler_matches_torch_step_for_step(name):
    ours, theirs = CASES[name]
    steps = 24 if name.startswith("one_cycle") else 25
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        a, s = _run(ours, steps)
        b, _ = _run(theirs, steps)
    assert not isinstance(s, T.LRScheduler)                       # implemented here, not a torch class under another name
    assert max(max(abs(x[0] - y[0]), abs(x[1] - y[1])) for x, y in zip(a, b)) < 1e-12
    assert s.get_last_lr() == [a[-1][0]]


def test_reduce_on_plateau_and_state_dict_round_trip():
    m = [1.0, 0.9, 0.9, 0.9, 0.9, 0.95, 0.95, 0.95, 0.95] + [0.5] * 16
    a, s = _run(lambda o: S.ReduceLROnPlateau(o, factor=0.5, patience=2, cooldown=1), 25, m)
    b, _ = _run(lambda o: T.ReduceLROnPlateau(o, factor=0.5, patience=2, cooldown=1), 25, m)
    assert [x[0] for x in a] == [y[0] for y in b]
    o = _opt()
    s1 = S.StepLR(o, 3, 0.5)
    for _ in range(7):
        o.step()
        s1.step()
    sd = s1.state_dict()
    o2 = _opt()
    s2 = S.StepLR(o2, 3, 0.5)
    s2.load_state_dict(sd)
    assert s2.last_epoch == 7 and s2.get_last_lr() == s1.get_last_lr()
    with pytest.raises(ValueError):
        S.OneCycleLR(_opt(), 0.5)                                 # neither total_steps nor epochs x steps_per_epoch
    with pytest.raises(ValueError):
        S.ReduceLROnPlateau(_opt(), factor=1.5)
