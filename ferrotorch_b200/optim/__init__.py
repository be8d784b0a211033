"""Optimizers, schedulers, loss scaling and weight averaging (API names follow ferrotorch-optim)."""
from .optimizers import (Optimizer, ParamGroup, SgdConfig, AdamConfig, AdamWConfig, MuonConfig, Sgd, Adam, AdamW, Adamax, NAdam, RAdam,
                         Adagrad, Adadelta, Adafactor, Rmsprop, Rprop, Asgd, SparseAdam, Lbfgs, LineSearchFn, Muon, Kfac,
                         newton_schulz_cubic, diff_sgd_step, diff_sgd_momentum_step, elemwise_max, scalar_on, AdadeltaConfig, AdagradConfig, AdamaxConfig,
                         AsgdConfig, NAdamConfig, RAdamConfig, RmspropConfig, RpropConfig, SparseAdamConfig, LbfgsConfig, AdafactorConfig, KfacConfig,
                         ParamKey, OptimizerState)
from .extras import (GradScaler, GradScalerConfig, GradScalerState, GradientAccumulator, ExponentialMovingAverage, AveragedModel, AveragingStrategy, Swalr)
from . import scheduler
from .scheduler import *  # noqa: F401,F403

# PyTorch's spellings of the same classes, so that code written against torch.optim runs unchanged.
SGD, RMSprop, ASGD, LBFGS, SWALR = Sgd, Rmsprop, Asgd, Lbfgs, Swalr
SequentialLR = SequentialLr  # noqa: F405
