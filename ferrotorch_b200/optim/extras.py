"""GradScaler, gradient accumulation, EMA / SWA weight averaging.

Reference parity: ferrotorch-optim/src/grad_scaler.rs:27-354, grad_accumulator.rs:28, ema.rs:45, swa.rs:81-405.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass, asdict
from typing import Dict, Iterable, List, Optional

import torch

from .. import ops
from ..errors import InvalidArgument
from .scheduler import LrScheduler


@dataclass
class GradScalerConfig:
    init_scale: float = 65536.0
    growth_factor: float = 2.0
    backoff_factor: float = 0.5
    growth_interval: int = 2000
    enabled: bool = True


@dataclass
class GradScalerState:
    scale: float
    growth_tracker: int
    found_inf: bool = False


class GradScaler:
    """Dynamic loss scaling. ``unscale_`` runs one multi-buffer kernel sequence over all gradients that multiplies by 1/scale and
    raises a device flag on any non-finite value; the flag is read once per step (the reference syncs per parameter:
    ferrotorch-optim/src/grad_scaler.rs:200-240)."""

    def __init__(self, config: Optional[GradScalerConfig] = None, **kw):
        self.cfg = config or GradScalerConfig(**kw)
        self._scale = self.cfg.init_scale
        self._growth = 0
        self._found_inf = False
        self._unscaled = False

    def scale(self, loss: torch.Tensor) -> torch.Tensor:
        return loss * self._scale if self.cfg.enabled else loss

    def get_scale(self) -> float:
        return self._scale

    def unscale_(self, optimizer: torch.optim.Optimizer) -> None:
        if not self.cfg.enabled or self._unscaled:
            return
        grads = [p.grad for g in optimizer.param_groups for p in g["params"] if p.grad is not None]
        inv = 1.0 / self._scale
        found = False
        cuda = [g for g in grads if g.is_cuda and g.is_contiguous() and g.dtype in (torch.float32, torch.bfloat16)]
        rest = [g for g in grads if not any(g is c for c in cuda)]
        if cuda:
            flag = torch.zeros(1, device=cuda[0].device, dtype=torch.int32)
            ops.grad_norm_([g.reshape(-1) for g in cuda], 0.0, found_inf=flag)
            for g in cuda:
                ops.scale_(g, inv)
            found = bool(flag.item())
        for g in rest:
            g.mul_(inv)
            found = found or not bool(torch.isfinite(g).all())
        self._found_inf = found
        self._unscaled = True

    def step(self, optimizer: torch.optim.Optimizer, *a, **k):
        if not self.cfg.enabled:
            return optimizer.step(*a, **k)
        self.unscale_(optimizer)
        if self._found_inf:
            return None                   # skip the update on overflow
        return optimizer.step(*a, **k)

    def update(self, new_scale: Optional[float] = None) -> None:
        if not self.cfg.enabled:
            return
        if new_scale is not None:
            self._scale = float(new_scale)
        elif self._found_inf:
            self._scale *= self.cfg.backoff_factor
            self._growth = 0
        else:
            self._growth += 1
            if self._growth >= self.cfg.growth_interval:
                self._scale *= self.cfg.growth_factor
                self._growth = 0
        self._found_inf, self._unscaled = False, False

    def state_dict(self) -> dict:
        return asdict(GradScalerState(self._scale, self._growth, self._found_inf))

    def load_state_dict(self, sd: dict) -> None:
        self._scale, self._growth, self._found_inf = float(sd["scale"]), int(sd["growth_tracker"]), bool(sd.get("found_inf", False))


class GradientAccumulator:
    """Counts micro-steps; ``should_step()`` is true every ``steps`` calls; ``scale_loss`` divides by ``steps``."""

    def __init__(self, steps: int):
        self.steps, self.count = max(1, steps), 0

    def scale_loss(self, loss: torch.Tensor) -> torch.Tensor:
        return loss / self.steps

    def accumulate(self) -> bool:
        self.count += 1
        return self.should_step()

    def should_step(self) -> bool:
        return self.count % self.steps == 0

    def reset(self) -> None:
        self.count = 0


class ExponentialMovingAverage:
    """Shadow copy ``s = decay*s + (1-decay)*p`` of a parameter list, with bias-corrected warm-up and swap-in/restore."""

    def __init__(self, params: Iterable[torch.Tensor], decay: float = 0.999, use_num_updates: bool = True):
        self.params = list(params)
        self.decay, self.num_updates = decay, 0 if use_num_updates else None
        self.shadow = [p.detach().clone() for p in self.params]
        self._backup: Optional[List[torch.Tensor]] = None

    @torch.no_grad()
    def update(self) -> None:
        d = self.decay
        if self.num_updates is not None:
            self.num_updates += 1
            d = min(d, (1 + self.num_updates) / (10 + self.num_updates))
        torch._foreach_lerp_(self.shadow, [p.detach() for p in self.params], 1 - d)

    @torch.no_grad()
    def copy_to(self) -> None:
        for s, p in zip(self.shadow, self.params):
            p.copy_(s)

    @torch.no_grad()
    def store(self) -> None:
        self._backup = [p.detach().clone() for p in self.params]

    @torch.no_grad()
    def restore(self) -> None:
        for b, p in zip(self._backup or [], self.params):
            p.copy_(b)
        self._backup = None

    def state_dict(self):
        return {"decay": self.decay, "num_updates": self.num_updates, "shadow": self.shadow}

    def load_state_dict(self, sd):
        self.decay, self.num_updates = sd["decay"], sd["num_updates"]
        for s, n in zip(self.shadow, sd["shadow"]):
            s.copy_(n)


class AveragingStrategy:
    """How :class:`AveragedModel` folds a new snapshot in (ferrotorch-optim/src/swa.rs:42): ``Swa`` is the equal-weight running mean,
    ``Ema(decay)`` is ``decay * avg + (1 - decay) * new``."""

    def __init__(self, kind: str, decay: float = 0.0):
        self.kind, self.decay = kind, float(decay)

    @classmethod
    def Ema(cls, decay: float) -> "AveragingStrategy":  # noqa: N802
        if not 0.0 <= decay <= 1.0:
            raise InvalidArgument(f"EMA decay must be in [0, 1], got {decay}")
        return cls("ema", decay)

    def avg_fn(self):
        if self.kind == "swa":
            return None
        d = self.decay
        return lambda avg, new, n: d * avg + (1.0 - d) * new

    def __eq__(self, other):
        return isinstance(other, AveragingStrategy) and (self.kind, self.decay) == (other.kind, other.decay)

    def __hash__(self):
        return hash((self.kind, self.decay))

    def __repr__(self):
        return "AveragingStrategy.Swa" if self.kind == "swa" else f"AveragingStrategy.Ema({self.decay})"


AveragingStrategy.Swa = AveragingStrategy("swa")


class AveragedModel(torch.nn.Module):
    """Stochastic weight averaging: running equal (or custom ``avg_fn``) average of a model's parameters; ``avg_fn`` may be an
    :class:`AveragingStrategy`."""

    def __init__(self, model: torch.nn.Module, avg_fn=None, use_buffers: bool = False):
        super().__init__()
        if isinstance(avg_fn, AveragingStrategy):
            self.strategy, avg_fn = avg_fn, avg_fn.avg_fn()
        else:
            self.strategy = None
        self.module = copy.deepcopy(model)
        self.avg_fn, self.use_buffers = avg_fn, use_buffers
        self.register_buffer("n_averaged", torch.tensor(0, dtype=torch.long))

    def forward(self, *a, **k):
        return self.module(*a, **k)

    @torch.no_grad()
    def update_parameters(self, model: torch.nn.Module) -> None:
        mine = list(self.module.parameters()) + (list(self.module.buffers()) if self.use_buffers else [])
        theirs = list(model.parameters()) + (list(model.buffers()) if self.use_buffers else [])
        n = int(self.n_averaged)
        for a, b in zip(mine, theirs):
            if n == 0:
                a.copy_(b)
            elif self.avg_fn is not None:
                a.copy_(self.avg_fn(a, b, n))
            elif a.is_floating_point():
                a.add_((b - a) / (n + 1))
        self.n_averaged += 1


class Swalr(LrScheduler):
    """Anneals every group's learning rate from its current value to a constant ``swa_lr`` over ``anneal_epochs`` steps (cosine or linear
    interpolation) and holds it there (ferrotorch-optim/src/swa.rs; PyTorch's ``SWALR``). Chainable: each step recovers the rate the
    annealing started from out of the current one."""

    def __init__(self, optimizer, swa_lr, anneal_epochs: int = 10, anneal_strategy: str = "cos", last_epoch: int = -1):
        strategy = getattr(anneal_strategy, "value", anneal_strategy)
        if strategy not in ("cos", "linear"):
            raise ValueError(f"anneal_strategy must be 'cos' or 'linear', got {anneal_strategy!r}")
        if not isinstance(anneal_epochs, int) or anneal_epochs < 0:
            raise ValueError(f"anneal_epochs must be a non-negative integer, got {anneal_epochs}")
        swa = list(swa_lr) if isinstance(swa_lr, (list, tuple)) else [swa_lr] * len(optimizer.param_groups)
        if len(swa) != len(optimizer.param_groups):
            raise ValueError("one swa_lr per parameter group")
        for g, v in zip(optimizer.param_groups, swa):
            g["swa_lr"] = float(v)
        self.anneal_epochs, self.anneal_strategy = anneal_epochs, strategy
        super().__init__(optimizer, last_epoch)

    def _alpha(self, t: float) -> float:
        t = max(0.0, min(1.0, t))
        return (1.0 - math.cos(math.pi * t)) / 2.0 if self.anneal_strategy == "cos" else t

    def get_lr(self):
        step = self.last_epoch
        if self.anneal_epochs == 0:
            step = max(1, step)
        n = max(1, self.anneal_epochs)
        prev, cur = self._alpha((step - 1) / n), self._alpha(step / n)
        out = []
        for g in self.optimizer.param_groups:
            start = g["swa_lr"] if prev == 1.0 else (g["lr"] - prev * g["swa_lr"]) / (1.0 - prev)
            out.append(g["swa_lr"] * cur + start * (1.0 - cur))
        return out
