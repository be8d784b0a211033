"""``from ferrotorch_b200.prelude import *``: the core names plus the layers, losses and optimisers most programs start from
(ferrotorch/src/lib.rs:44-52)."""
from .core import *  # noqa: F401,F403
from .core import Tensor, Device, DType, zeros, ones, rand, randn, arange, no_grad, enable_grad, backward  # noqa: F401
from .nn import (BatchNorm2d, Dropout, LayerNorm, Conv2d, Linear, Module, Parameter, Sequential, CrossEntropyLoss, MSELoss, GELU, ReLU, SiLU, Sigmoid,  # noqa: F401
                 Softmax, Tanh, GRU, LSTM)
from .optim import Adam, AdamW, Optimizer, Sgd  # noqa: F401
