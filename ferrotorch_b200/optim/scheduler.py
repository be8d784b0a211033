"""Learning-rate schedulers (ferrotorch-optim/src/scheduler/*.rs): the sixteen schedulers under the reference's names."""
from __future__ import annotations

import enum
import math
from typing import Callable, List, Sequence

import torch
from torch.optim import lr_scheduler as _s

LrScheduler = _s.LRScheduler
StepLR = _s.StepLR
MultiStepLR = _s.MultiStepLR
ExponentialLR = _s.ExponentialLR
CosineAnnealingLR = _s.CosineAnnealingLR
CosineAnnealingWarmRestarts = _s.CosineAnnealingWarmRestarts
CyclicLR = _s.CyclicLR
OneCycleLR = _s.OneCycleLR
LinearLR = _s.LinearLR
ConstantLR = _s.ConstantLR
LambdaLR = _s.LambdaLR
MultiplicativeLR = _s.MultiplicativeLR
PolynomialLR = _s.PolynomialLR
ReduceLROnPlateau = _s.ReduceLROnPlateau
ChainedScheduler = _s.ChainedScheduler
SequentialLr = _s.SequentialLR
MetricScheduler = _s.ReduceLROnPlateau


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


class LinearWarmup(_s.LambdaLR):
    """Linear ramp from ``start_factor`` to 1 over ``warmup_steps``, then constant."""

    def __init__(self, optimizer, warmup_steps: int, start_factor: float = 0.0, last_epoch: int = -1):
        self.warmup_steps, self.start_factor = max(1, warmup_steps), start_factor
        super().__init__(optimizer, lambda s: min(1.0, start_factor + (1 - start_factor) * s / self.warmup_steps), last_epoch)


def cosine_warmup_scheduler(optimizer, warmup_steps: int, total_steps: int, min_lr_ratio: float = 0.0) -> _s.LambdaLR:
    """Linear warm-up followed by cosine decay to ``min_lr_ratio`` of the base rate (ferrotorch-optim/src/scheduler/mod.rs:180)."""
    def f(step):
        if step < warmup_steps:
            return step / max(1, warmup_steps)
        prog = min(1.0, (step - warmup_steps) / max(1, total_steps - warmup_steps))
        return min_lr_ratio + (1 - min_lr_ratio) * 0.5 * (1 + math.cos(math.pi * prog))
    return _s.LambdaLR(optimizer, f)
