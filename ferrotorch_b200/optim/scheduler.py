"""Learning-rate schedulers (ferrotorch-optim/src/scheduler/*.rs): the sixteen schedulers under the reference's names."""
from __future__ import annotations

import enum
import math
from typing import Callable, List, Sequence

import torch


class LrScheduler:
    """Base of the schedulers: ``step()`` advances ``last_epoch`` and writes the new rates into the optimizer's parameter groups.
    Subclasses implement ``get_lr()`` in the *chainable* form (next rate from the current one), as PyTorch does, so that several
    schedulers can act on one optimizer (``ChainedScheduler``); ``state_dict`` / ``load_state_dict`` carry everything but the optimizer.
    (ferrotorch-optim/src/scheduler/mod.rs:81 ``LrScheduler`` trait.)"""

    def __init__(self, optimizer, last_epoch: int = -1):
        self.optimizer = optimizer
        if last_epoch == -1:
            for g in optimizer.param_groups:
                g.setdefault("initial_lr", g["lr"])
        else:
            for i, g in enumerate(optimizer.param_groups):
                if "initial_lr" not in g:
                    raise KeyError(f"param 'initial_lr' is not specified in param_groups[{i}] when resuming an optimizer")
        self.base_lrs = [g["initial_lr"] for g in optimizer.param_groups]
        self.last_epoch = last_epoch
        self._initial_step()

    def _initial_step(self):
        self.last_epoch += 1
        self._apply(self.get_lr())

    def _apply(self, lrs):
        for g, lr in zip(self.optimizer.param_groups, lrs):
            g["lr"] = lr
        self._last_lr = [g["lr"] for g in self.optimizer.param_groups]

    def get_lr(self) -> List[float]:
        raise NotImplementedError

    def get_last_lr(self) -> List[float]:
        return self._last_lr

    def step(self, epoch=None) -> None:
        if epoch is None:
            self.last_epoch += 1
            self._apply(self.get_lr())
        else:
            self.last_epoch = epoch
            self._apply(self._closed_form() if hasattr(self, "_closed_form") else self.get_lr())

    def _cur(self):
        return [g["lr"] for g in self.optimizer.param_groups]

    def state_dict(self) -> dict:
        return {k: v for k, v in self.__dict__.items() if k != "optimizer" and not callable(v)}

    def load_state_dict(self, sd: dict) -> None:
        self.__dict__.update(sd)


class StepLR(LrScheduler):
    def __init__(self, optimizer, step_size: int, gamma: float = 0.1, last_epoch: int = -1):
        self.step_size, self.gamma = step_size, gamma
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        if self.last_epoch == 0 or self.last_epoch % self.step_size:
            return self._cur()
        return [lr * self.gamma for lr in self._cur()]

    def _closed_form(self):
        return [b * self.gamma ** (self.last_epoch // self.step_size) for b in self.base_lrs]


class MultiStepLR(LrScheduler):
    def __init__(self, optimizer, milestones: Sequence[int], gamma: float = 0.1, last_epoch: int = -1):
        from collections import Counter
        self.milestones, self.gamma = Counter(milestones), gamma
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        if self.last_epoch not in self.milestones:
            return self._cur()
        return [lr * self.gamma ** self.milestones[self.last_epoch] for lr in self._cur()]


class ConstantLR(LrScheduler):
    def __init__(self, optimizer, factor: float = 1.0 / 3, total_iters: int = 5, last_epoch: int = -1):
        if factor > 1.0 or factor < 0:
            raise ValueError("Constant multiplicative factor expected to be between 0 and 1.")
        self.factor, self.total_iters = factor, total_iters
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        if self.last_epoch == 0:
            return [lr * self.factor for lr in self._cur()]
        if self.last_epoch != self.total_iters:
            return self._cur()
        return [lr * (1.0 / self.factor) for lr in self._cur()]


class LinearLR(LrScheduler):
    def __init__(self, optimizer, start_factor: float = 1.0 / 3, end_factor: float = 1.0, total_iters: int = 5, last_epoch: int = -1):
        if start_factor > 1.0 or start_factor <= 0:
            raise ValueError("Starting multiplicative factor expected to be greater than 0 and less or equal to 1.")
        if end_factor > 1.0 or end_factor < 0:
            raise ValueError("Ending multiplicative factor expected to be between 0 and 1.")
        self.start_factor, self.end_factor, self.total_iters = start_factor, end_factor, total_iters
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        if self.last_epoch == 0:
            return [lr * self.start_factor for lr in self._cur()]
        if self.last_epoch > self.total_iters:
            return self._cur()
        d = self.end_factor - self.start_factor
        return [lr * (1.0 + d / (self.total_iters * self.start_factor + (self.last_epoch - 1) * d)) for lr in self._cur()]


class ExponentialLR(LrScheduler):
    def __init__(self, optimizer, gamma: float, last_epoch: int = -1):
        self.gamma = gamma
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        return self._cur() if self.last_epoch == 0 else [lr * self.gamma for lr in self._cur()]


class PolynomialLR(LrScheduler):
    def __init__(self, optimizer, total_iters: int = 5, power: float = 1.0, last_epoch: int = -1):
        self.total_iters, self.power = total_iters, power
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        if self.last_epoch == 0 or self.last_epoch > self.total_iters:
            return self._cur()
        f = ((1.0 - self.last_epoch / self.total_iters) / (1.0 - (self.last_epoch - 1) / self.total_iters)) ** self.power
        return [lr * f for lr in self._cur()]


class CosineAnnealingLR(LrScheduler):
    def __init__(self, optimizer, T_max: int, eta_min: float = 0.0, last_epoch: int = -1):
        self.T_max, self.eta_min = T_max, eta_min
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        t, T, m = self.last_epoch, self.T_max, self.eta_min
        if t == 0:
            return self._cur()
        if (t - 1 - T) % (2 * T) == 0:
            return [lr + (b - m) * (1 - math.cos(math.pi / T)) / 2 for b, lr in zip(self.base_lrs, self._cur())]
        return [(1 + math.cos(math.pi * t / T)) / (1 + math.cos(math.pi * (t - 1) / T)) * (lr - m) + m for lr in self._cur()]


class LambdaLR(LrScheduler):
    def __init__(self, optimizer, lr_lambda, last_epoch: int = -1):
        n = len(optimizer.param_groups)
        self.lr_lambdas = list(lr_lambda) if isinstance(lr_lambda, (list, tuple)) else [lr_lambda] * n
        if len(self.lr_lambdas) != n:
            raise ValueError(f"Expected {n} lr_lambdas, but got {len(self.lr_lambdas)}")
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        return [b * f(self.last_epoch) for f, b in zip(self.lr_lambdas, self.base_lrs)]

    def state_dict(self):
        return {k: v for k, v in self.__dict__.items() if k not in ("optimizer", "lr_lambdas")}


class MultiplicativeLR(LambdaLR):
    def get_lr(self):
        if self.last_epoch > 0:
            return [lr * f(self.last_epoch) for f, lr in zip(self.lr_lambdas, self._cur())]
        return self._cur()


class CosineAnnealingWarmRestarts(LrScheduler):
    def __init__(self, optimizer, T_0: int, T_mult: int = 1, eta_min: float = 0.0, last_epoch: int = -1):
        if T_0 <= 0 or not isinstance(T_0, int):
            raise ValueError(f"Expected positive integer T_0, but got {T_0}")
        if T_mult < 1 or not isinstance(T_mult, int):
            raise ValueError(f"Expected integer T_mult >= 1, but got {T_mult}")
        self.T_0, self.T_i, self.T_mult, self.eta_min, self.T_cur = T_0, T_0, T_mult, eta_min, last_epoch
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        return [self.eta_min + (b - self.eta_min) * (1 + math.cos(math.pi * self.T_cur / self.T_i)) / 2 for b in self.base_lrs]

    def _initial_step(self):
        self.last_epoch += 1
        self.T_cur = max(self.T_cur, 0) if self.last_epoch == 0 else self.T_cur
        self.T_cur = 0 if self.last_epoch == 0 else self.T_cur
        self._apply(self.get_lr())

    def step(self, epoch=None):
        if epoch is None:
            epoch = self.last_epoch + 1
            self.T_cur += 1
            if self.T_cur >= self.T_i:
                self.T_cur -= self.T_i
                self.T_i *= self.T_mult
        else:
            if epoch < 0:
                raise ValueError(f"Expected non-negative epoch, but got {epoch}")
            if epoch >= self.T_0:
                if self.T_mult == 1:
                    self.T_cur = epoch % self.T_0
                else:
                    n = int(math.log(epoch / self.T_0 * (self.T_mult - 1) + 1, self.T_mult))
                    self.T_cur = epoch - self.T_0 * (self.T_mult ** n - 1) / (self.T_mult - 1)
                    self.T_i = self.T_0 * self.T_mult ** n
            else:
                self.T_i, self.T_cur = self.T_0, epoch
        self.last_epoch = math.floor(epoch)
        self._apply(self.get_lr())


class CyclicLR(LrScheduler):
    def __init__(self, optimizer, base_lr, max_lr, step_size_up: int = 2000, step_size_down=None, mode: str = "triangular", gamma: float = 1.0,
                 scale_fn=None, scale_mode: str = "cycle", cycle_momentum: bool = True, base_momentum=0.8, max_momentum=0.9, last_epoch: int = -1):
        n = len(optimizer.param_groups)
        as_list = lambda v: list(v) if isinstance(v, (list, tuple)) else [v] * n          # noqa: E731
        base = as_list(base_lr)
        if last_epoch == -1:
            for g, lr in zip(optimizer.param_groups, base):
                g["lr"] = lr
        self.max_lrs = as_list(max_lr)
        up, down = float(step_size_up), float(step_size_down) if step_size_down is not None else float(step_size_up)
        self.total_size, self.step_ratio = up + down, up / (up + down)
        if mode not in ("triangular", "triangular2", "exp_range") and scale_fn is None:
            raise ValueError("mode is invalid and scale_fn is None")
        self.mode, self.gamma, self._scale_fn_custom = mode, gamma, scale_fn
        self.scale_mode = scale_mode if scale_fn is not None else ("iterations" if mode == "exp_range" else "cycle")
        self.cycle_momentum = cycle_momentum
        if cycle_momentum:
            key = "betas" if "betas" in optimizer.defaults else "momentum"
            if key not in optimizer.defaults:
                raise ValueError("optimizer must support momentum or beta1 with `cycle_momentum` option enabled")
            self._mkey = key
            self.base_momentums, self.max_momentums = as_list(base_momentum), as_list(max_momentum)
            if last_epoch == -1:
                for g, m in zip(optimizer.param_groups, self.max_momentums):
                    g[key] = (m, *g[key][1:]) if key == "betas" else m
        super().__init__(optimizer, last_epoch)
        self.base_lrs = base

    def scale_fn(self, x):
        if self._scale_fn_custom is not None:
            return self._scale_fn_custom(x)
        return 1.0 if self.mode == "triangular" else (1 / (2.0 ** (x - 1)) if self.mode == "triangular2" else self.gamma ** x)

    def get_lr(self):
        cycle = math.floor(1 + self.last_epoch / self.total_size)
        x = 1.0 + self.last_epoch / self.total_size - cycle
        sf = x / self.step_ratio if x <= self.step_ratio else (x - 1) / (self.step_ratio - 1)
        arg = cycle if self.scale_mode == "cycle" else self.last_epoch
        lrs = [b + (m - b) * sf * self.scale_fn(arg) for b, m in zip(self.base_lrs, self.max_lrs)]
        if self.cycle_momentum:
            for g, bm, mm in zip(self.optimizer.param_groups, self.base_momentums, self.max_momentums):
                mom = mm - (mm - bm) * sf * self.scale_fn(arg)
                g[self._mkey] = (mom, *g[self._mkey][1:]) if self._mkey == "betas" else mom
        return lrs

    def state_dict(self):
        return {k: v for k, v in self.__dict__.items() if k not in ("optimizer", "_scale_fn_custom")}


class OneCycleLR(LrScheduler):
    def __init__(self, optimizer, max_lr, total_steps=None, epochs=None, steps_per_epoch=None, pct_start: float = 0.3, anneal_strategy: str = "cos",
                 cycle_momentum: bool = True, base_momentum=0.85, max_momentum=0.95, div_factor: float = 25.0, final_div_factor: float = 1e4,
                 three_phase: bool = False, last_epoch: int = -1):
        if total_steps is None:
            if epochs is None or steps_per_epoch is None:
                raise ValueError("You must define either total_steps OR (epochs AND steps_per_epoch)")
            total_steps = epochs * steps_per_epoch
        if total_steps <= 0 or not 0 <= pct_start <= 1:
            raise ValueError("OneCycleLR: total_steps must be positive and pct_start in [0, 1]")
        if anneal_strategy not in ("cos", "linear"):
            raise ValueError(f"anneal_strategy must be one of 'cos' or 'linear', instead got {anneal_strategy}")
        self.total_steps, self._cos = total_steps, anneal_strategy == "cos"
        n = len(optimizer.param_groups)
        as_list = lambda v: list(v) if isinstance(v, (list, tuple)) else [v] * n          # noqa: E731
        max_lrs = as_list(max_lr)
        if three_phase:
            self._phases = [(float(pct_start * total_steps) - 1, "initial_lr", "max_lr", "max_momentum", "base_momentum"),
                            (float(2 * pct_start * total_steps) - 2, "max_lr", "initial_lr", "base_momentum", "max_momentum"),
                            (total_steps - 1, "initial_lr", "min_lr", "max_momentum", "max_momentum")]
        else:
            self._phases = [(float(pct_start * total_steps) - 1, "initial_lr", "max_lr", "max_momentum", "base_momentum"),
                            (total_steps - 1, "max_lr", "min_lr", "base_momentum", "max_momentum")]
        if last_epoch == -1:
            for g, m in zip(optimizer.param_groups, max_lrs):
                g["initial_lr"] = m / div_factor
                g["max_lr"] = m
                g["min_lr"] = g["initial_lr"] / final_div_factor
        self.cycle_momentum = cycle_momentum
        if cycle_momentum:
            key = "betas" if "betas" in optimizer.defaults else "momentum"
            if key not in optimizer.defaults:
                raise ValueError("optimizer must support momentum or beta1 with `cycle_momentum` option enabled")
            self._mkey = key
            if last_epoch == -1:
                for g, bm, mm in zip(optimizer.param_groups, as_list(base_momentum), as_list(max_momentum)):
                    g[key] = (mm, *g[key][1:]) if key == "betas" else mm
                    g["max_momentum"], g["base_momentum"] = mm, bm
        super().__init__(optimizer, last_epoch)

    def _anneal(self, a, b, pct):
        return b + (a - b) / 2.0 * (math.cos(math.pi * pct) + 1) if self._cos else (b - a) * pct + a

    def get_lr(self):
        t = self.last_epoch
        if t > self.total_steps:
            raise ValueError(f"Tried to step {t} times. The specified number of total steps is {self.total_steps}")
        lrs = []
        for g in self.optimizer.param_groups:
            start, lr, mom = 0.0, None, None
            for i, (end, a, b, ma, mb) in enumerate(self._phases):
                if t <= end or i == len(self._phases) - 1:
                    pct = (t - start) / (end - start)
                    lr = self._anneal(g[a], g[b], pct)
                    if self.cycle_momentum:
                        mom = self._anneal(g[ma], g[mb], pct)
                    break
                start = end
            lrs.append(lr)
            if self.cycle_momentum:
                g[self._mkey] = (mom, *g[self._mkey][1:]) if self._mkey == "betas" else mom
        return lrs


class ReduceLROnPlateau:
    """Cuts the rate by ``factor`` when a metric has not improved for ``patience`` epochs (``step(metric)``)."""

    def __init__(self, optimizer, mode: str = "min", factor: float = 0.1, patience: int = 10, threshold: float = 1e-4, threshold_mode: str = "rel",
                 cooldown: int = 0, min_lr=0.0, eps: float = 1e-8):
        if factor >= 1.0:
            raise ValueError("Factor should be < 1.0.")
        if mode not in ("min", "max") or threshold_mode not in ("rel", "abs"):
            raise ValueError("mode must be min|max and threshold_mode rel|abs")
        self.optimizer, self.mode, self.factor, self.patience = optimizer, mode, factor, patience
        self.threshold, self.threshold_mode, self.cooldown, self.eps = threshold, threshold_mode, cooldown, eps
        n = len(optimizer.param_groups)
        self.min_lrs = list(min_lr) if isinstance(min_lr, (list, tuple)) else [min_lr] * n
        self.best = math.inf if mode == "min" else -math.inf
        self.num_bad_epochs, self.cooldown_counter, self.last_epoch = 0, 0, 0
        self._last_lr = [g["lr"] for g in optimizer.param_groups]

    def _better(self, a):
        if self.mode == "min":
            return a < (self.best * (1 - self.threshold) if self.threshold_mode == "rel" else self.best - self.threshold)
        return a > (self.best * (1 + self.threshold) if self.threshold_mode == "rel" else self.best + self.threshold)

    def step(self, metrics, epoch=None):
        cur = float(metrics)
        self.last_epoch = self.last_epoch + 1 if epoch is None else epoch
        if self._better(cur):
            self.best, self.num_bad_epochs = cur, 0
        else:
            self.num_bad_epochs += 1
        if self.cooldown_counter > 0:
            self.cooldown_counter -= 1
            self.num_bad_epochs = 0
        if self.num_bad_epochs > self.patience:
            for g, m in zip(self.optimizer.param_groups, self.min_lrs):
                new = max(g["lr"] * self.factor, m)
                if g["lr"] - new > self.eps:
                    g["lr"] = new
            self.cooldown_counter, self.num_bad_epochs = self.cooldown, 0
        self._last_lr = [g["lr"] for g in self.optimizer.param_groups]

    def get_last_lr(self):
        return self._last_lr

    def state_dict(self):
        return {k: v for k, v in self.__dict__.items() if k != "optimizer"}

    def load_state_dict(self, sd):
        self.__dict__.update(sd)


class ChainedScheduler(LrScheduler):
    """Applies several chainable schedulers one after the other on every step."""

    def __init__(self, schedulers, optimizer=None):
        self._schedulers = list(schedulers)
        self.optimizer = optimizer or self._schedulers[0].optimizer
        if any(s.optimizer is not self.optimizer for s in self._schedulers):
            raise ValueError("ChainedScheduler expects all schedulers to belong to the same optimizer")
        self._last_lr = [g["lr"] for g in self.optimizer.param_groups]
        self.last_epoch = 0

    def step(self):
        for s in self._schedulers:
            s.step()
        self.last_epoch += 1
        self._last_lr = [g["lr"] for g in self.optimizer.param_groups]

    def state_dict(self):
        return {"schedulers": [s.state_dict() for s in self._schedulers], "last_epoch": self.last_epoch, "_last_lr": self._last_lr}

    def load_state_dict(self, sd):
        for s, d in zip(self._schedulers, sd["schedulers"]):
            s.load_state_dict(d)
        self.last_epoch, self._last_lr = sd["last_epoch"], sd["_last_lr"]


class SequentialLr(LrScheduler):
    """Runs ``schedulers[i]`` until ``milestones[i]``, then hands over to the next one (which starts from its own epoch 0)."""

    def __init__(self, optimizer, schedulers, milestones: Sequence[int], last_epoch: int = -1):
        if len(milestones) != len(schedulers) - 1:
            raise ValueError("Sequential Schedulers expects number of schedulers provided to be one more than the number of milestone points")
        self._schedulers, self._milestones, self.optimizer = list(schedulers), list(milestones), optimizer
        self.last_epoch = last_epoch + 1
        for g in optimizer.param_groups:
            g["lr"] = g["initial_lr"]
        for s in self._schedulers:                                   # undo the initial steps the constructors of the later ones took
            s.last_epoch -= 1
        self._schedulers[0]._initial_step()
        self._last_lr = self._schedulers[0].get_last_lr()

    def step(self):
        import bisect
        self.last_epoch += 1
        idx = bisect.bisect_right(self._milestones, self.last_epoch)
        s = self._schedulers[idx]
        if idx > 0 and self._milestones[idx - 1] == self.last_epoch:
            s.step(0)
        else:
            s.step()
        self._last_lr = s.get_last_lr()

    def state_dict(self):
        return {"schedulers": [s.state_dict() for s in self._schedulers], "last_epoch": self.last_epoch, "_last_lr": self._last_lr,
                "_milestones": self._milestones}

    def load_state_dict(self, sd):
        for s, d in zip(self._schedulers, sd["schedulers"]):
            s.load_state_dict(d)
        self.last_epoch, self._last_lr = sd["last_epoch"], sd["_last_lr"]


MetricScheduler = ReduceLROnPlateau
_s = None  # this module no longer rides torch.optim.lr_scheduler


class CyclicMode(enum.Enum):
    Triangular = "triangular"
    Triangular2 = "triangular2"
    ExpRange = "exp_range"


class AnnealStrategy(enum.Enum):
    Cos = "cos"
    Linear = "linear"


class PlateauMode(enum.Enum):
    Min = "min"
    Max = "max"


class LinearWarmup(LambdaLR):
    """Linear ramp from ``start_factor`` to 1 over ``warmup_steps``, then constant."""

    def __init__(self, optimizer, warmup_steps: int, start_factor: float = 0.0, last_epoch: int = -1):
        self.warmup_steps, self.start_factor = max(1, warmup_steps), start_factor
        super().__init__(optimizer, lambda s: min(1.0, start_factor + (1 - start_factor) * s / self.warmup_steps), last_epoch)


def cosine_warmup_scheduler(optimizer, warmup_steps: int, total_steps: int, min_lr_ratio: float = 0.0) -> LambdaLR:
    """Linear warm-up followed by cosine decay to ``min_lr_ratio`` of the base rate (ferrotorch-optim/src/scheduler/mod.rs:180)."""
    def f(step):
        if step < warmup_steps:
            return step / max(1, warmup_steps)
        prog = min(1.0, (step - warmup_steps) / max(1, total_steps - warmup_steps))
        return min_lr_ratio + (1 - min_lr_ratio) * 0.5 * (1 + math.cos(math.pi * prog))
    return LambdaLR(optimizer, f)
