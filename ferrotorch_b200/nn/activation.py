"""Activation layers (ferrotorch-nn/src/activation.rs:63-1401).

Every class here states its own math. CUDA float tensors go through the element-wise kernels of this package (one launch forward,
one backward, the derivative computed from the saved input or output); CPU tensors and the few forms without a kernel code are
composed from tensor primitives, so autograd differentiates them as written."""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..errors import InvalidArgument
from ..ops import tensor_ops as _t
from .module import Module, Parameter

_SELU_ALPHA = 1.6732632423543772848170429916717
_SELU_SCALE = 1.0507009873554804934193349852946


def _flat(x: torch.Tensor) -> torch.Tensor:
    """The ``numel`` elements of a dense tensor in memory order (channels-last and other permuted layouts keep their layout)."""
    return x.as_strided((x.numel(),), (1,), x.storage_offset())


def _dense(x: torch.Tensor) -> bool:
    if x.is_contiguous():
        return True
    if x.dim() == 4 and x.is_contiguous(memory_format=torch.channels_last):
        return True
    return x.dim() == 5 and x.is_contiguous(memory_format=torch.channels_last_3d)


def _run(op, x, a, b):
    if not _dense(x):
        x = x.contiguous()
    y = torch.empty_like(x)                         # same strides as x
    _t.unary(op, _flat(x), a, b, out=_flat(y))
    return x, y


class _Ew(torch.autograd.Function):
    """One unary kernel forward, its derivative kernel backward. ``saved`` says whether the derivative reads the input or the output."""

    @staticmethod
    def forward(ctx, x, op, bwd_op, a, b, saved):
        x, y = _run(op, x, a, b)
        ctx.save_for_backward(y if saved == "y" else x)
        ctx.meta = (bwd_op, a, b)
        return y

    @staticmethod
    def backward(ctx, g):
        (s,) = ctx.saved_tensors
        bwd_op, a, b = ctx.meta
        if g.stride() != s.stride() or g.dtype != s.dtype:
            g = torch.empty_like(s).copy_(g)
        out_flat = _t.unary_backward(bwd_op, _flat(g), _flat(s), a, b)      # fresh, in the memory order of ``s``
        return out_flat.as_strided(s.size(), s.stride()), None, None, None, None, None


def _kernel_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in (torch.float32, torch.bfloat16, torch.float16) and x.numel() > 0


def _ew(x, op, bwd_op, a=0.0, b=0.0, saved="x"):
    if torch.is_grad_enabled() and x.requires_grad:
        return _Ew.apply(x, op, bwd_op, a, b, saved)
    return _run(op, x, a, b)[1]


# -- functional forms (used by the classes below and by nn.functional) ---------------------------------------------------------------
def relu(x):
    return _ew(x, "relu", "relu") if _kernel_ok(x) else torch.where(x > 0, x, torch.zeros_like(x))        # no gradient at the origin


def relu6(x):
    return hardtanh(x, 0.0, 6.0)


def hardtanh(x, min_val: float = -1.0, max_val: float = 1.0):
    if min_val > max_val:
        raise InvalidArgument(f"hardtanh: min_val {min_val} > max_val {max_val}")
    if _kernel_ok(x):
        return _ew(x, "clamp", "hardtanh", min_val, max_val)          # derivative on the open interval, as for the host form below
    return torch.where(x <= min_val, torch.full_like(x, min_val), torch.where(x >= max_val, torch.full_like(x, max_val), x))


def leaky_relu(x, negative_slope: float = 0.01):
    return _ew(x, "leaky_relu", "leaky_relu", negative_slope) if _kernel_ok(x) else torch.where(x > 0, x, x * negative_slope)


def elu(x, alpha: float = 1.0):
    return _ew(x, "elu", "elu", alpha) if _kernel_ok(x) else torch.where(x > 0, x, alpha * torch.expm1(torch.clamp_max(x, 0)))


def celu(x, alpha: float = 1.0):
    if alpha == 0:
        raise InvalidArgument("celu: alpha must be non-zero")
    return torch.clamp_min(x, 0) + torch.clamp_max(alpha * torch.expm1(torch.clamp_max(x, 0) / alpha), 0)


def selu(x):
    return _SELU_SCALE * torch.where(x > 0, x, _SELU_ALPHA * torch.expm1(torch.clamp_max(x, 0)))


def sigmoid(x):
    return _ew(x, "sigmoid", "sigmoid_y", saved="y") if _kernel_ok(x) else 1.0 / (1.0 + torch.exp(-x))


def tanh(x):
    return _ew(x, "tanh", "tanh_y", saved="y") if _kernel_ok(x) else torch.tanh(x)


def silu(x):
    return _ew(x, "silu", "silu") if _kernel_ok(x) else x * sigmoid(x)


def softplus(x, beta: float = 1.0, threshold: float = 20.0):
    if beta <= 0:
        raise InvalidArgument(f"softplus: beta must be > 0, got {beta}")
    if _kernel_ok(x):
        return _ew(x, "softplus", "softplus", beta, threshold)
    bx = x * beta
    return torch.where(bx > threshold, x, torch.log1p(torch.exp(torch.clamp_max(bx, threshold))) / beta)


def mish(x):
    return _ew(x, "mish", "mish") if _kernel_ok(x) else x * torch.tanh(softplus(x))


def hardsigmoid(x):
    # written piecewise so that the derivative at the kinks x = -3, 3 is that of the flat outer pieces
    return torch.where(x <= -3, torch.zeros_like(x), torch.where(x >= 3, torch.ones_like(x), x / 6.0 + 0.5))


def hardswish(x):
    if _kernel_ok(x):
        return _ew(x, "hardswish", "hardswish")
    return torch.where(x <= -3, torch.zeros_like(x), torch.where(x >= 3, x, x * (x + 3) / 6.0))


def logsigmoid(x):
    # -softplus(-x), in the form that does not overflow for large |x|
    return torch.clamp_max(x, 0) - torch.log1p(torch.exp(-torch.abs(x)))


def softmax(x, dim: int = -1):
    z = x - x.amax(dim, keepdim=True).detach()
    e = torch.exp(z)
    return e / e.sum(dim, keepdim=True)


def log_softmax(x, dim: int = -1):
    z = x - x.amax(dim, keepdim=True).detach()
    return z - torch.log(torch.exp(z).sum(dim, keepdim=True))


def softmin(x, dim: int = -1):
    return softmax(-x, dim)


def glu(x, dim: int = -1):
    if x.shape[dim] % 2:
        raise InvalidArgument(f"glu: dimension {dim} has odd size {x.shape[dim]}")
    a, b = x.chunk(2, dim)
    return a * sigmoid(b)


def threshold(x, threshold_: float, value: float):
    return torch.where(x > threshold_, x, torch.full_like(x, value))


def softshrink(x, lambd: float = 0.5):
    if lambd < 0:
        raise InvalidArgument("softshrink: lambd must be >= 0")
    return torch.where(x > lambd, x - lambd, torch.where(x < -lambd, x + lambd, torch.zeros_like(x)))


def hardshrink(x, lambd: float = 0.5):
    return torch.where(torch.abs(x) > lambd, x, torch.zeros_like(x))


def tanhshrink(x):
    return x - tanh(x)


def softsign(x):
    return x / (1.0 + torch.abs(x))


def prelu(x, weight):
    w = weight
    if w.numel() != 1:
        if x.dim() < 2 or w.numel() != x.shape[1]:
            raise InvalidArgument(f"prelu: {w.numel()} slopes for input shape {list(x.shape)}")
        w = w.view(1, -1, *([1] * (x.dim() - 2)))
    return torch.clamp_min(x, 0) + w * torch.clamp_max(x, 0)


def rrelu(x, lower: float = 1.0 / 8, upper: float = 1.0 / 3, training: bool = False, generator: Optional[torch.Generator] = None):
    if not training:
        return leaky_relu(x, (lower + upper) / 2)
    slope = torch.empty_like(x).uniform_(lower, upper, generator=generator)
    return torch.where(x >= 0, x, x * slope)


# -- modules -----------------------------------------------------------------------------------------------------------------------------
class _Stateless(Module):
    def __init__(self, inplace: bool = False):
        super().__init__()
        self.inplace = inplace


def _simple(name: str, fn, doc: str):
    def forward(self, x):
        y = fn(x)
        if self.inplace and not (torch.is_grad_enabled() and x.requires_grad):
            return x.copy_(y)          # under autograd the result is a fresh tensor: the graph keeps the input
        return y
    return type(name, (_Stateless,), {"forward": forward, "__doc__": doc, "__module__": __name__})


ReLU = _simple("ReLU", relu, "``max(x, 0)``.")
ReLU6 = _simple("ReLU6", relu6, "``min(max(x, 0), 6)``.")
SELU = _simple("SELU", selu, "``scale * (max(0, x) + min(0, alpha * (exp(x) - 1)))`` with the self-normalising constants.")
SiLU = _simple("SiLU", silu, "``x * sigmoid(x)``.")
Mish = _simple("Mish", mish, "``x * tanh(softplus(x))``.")
Sigmoid = _simple("Sigmoid", sigmoid, "``1 / (1 + exp(-x))``.")
Tanh = _simple("Tanh", tanh, "Hyperbolic tangent.")
HardSigmoid = _simple("HardSigmoid", hardsigmoid, "``clamp(x / 6 + 1/2, 0, 1)``.")
HardSwish = _simple("HardSwish", hardswish, "``x * hardsigmoid(x)``.")
LogSigmoid = _simple("LogSigmoid", logsigmoid, "``log(sigmoid(x))`` evaluated without overflow.")
Tanhshrink = _simple("Tanhshrink", tanhshrink, "``x - tanh(x)``.")
Softsign = _simple("Softsign", softsign, "``x / (1 + |x|)``.")


class LeakyReLU(Module):
    def __init__(self, negative_slope: float = 0.01, inplace: bool = False):
        super().__init__()
        self.negative_slope, self.inplace = negative_slope, inplace

    def forward(self, x):
        return leaky_relu(x, self.negative_slope)

    def extra_repr(self):
        return f"negative_slope={self.negative_slope}"


class ELU(Module):
    def __init__(self, alpha: float = 1.0, inplace: bool = False):
        super().__init__()
        self.alpha, self.inplace = alpha, inplace

    def forward(self, x):
        return elu(x, self.alpha)


class CELU(Module):
    def __init__(self, alpha: float = 1.0, inplace: bool = False):
        super().__init__()
        if alpha == 0:
            raise InvalidArgument("CELU: alpha must be non-zero")
        self.alpha, self.inplace = alpha, inplace

    def forward(self, x):
        return celu(x, self.alpha)


class Hardtanh(Module):
    def __init__(self, min_val: float = -1.0, max_val: float = 1.0, inplace: bool = False):
        super().__init__()
        if min_val > max_val:
            raise InvalidArgument(f"Hardtanh: min_val {min_val} > max_val {max_val}")
        self.min_val, self.max_val, self.inplace = min_val, max_val, inplace

    def forward(self, x):
        return hardtanh(x, self.min_val, self.max_val)


class Softplus(Module):
    def __init__(self, beta: float = 1.0, threshold: float = 20.0):
        super().__init__()
        if beta <= 0:
            raise InvalidArgument(f"Softplus: beta must be > 0, got {beta}")
        self.beta, self.threshold = beta, threshold

    def forward(self, x):
        return softplus(x, self.beta, self.threshold)


class _DimModule(Module):
    _fn = None

    def __init__(self, dim: Optional[int] = None):
        super().__init__()
        self.dim = dim

    def _axis(self, x) -> int:
        if self.dim is not None:
            return self.dim
        return 0 if x.dim() in (0, 1, 3) else 1       # the legacy implicit choice

    def forward(self, x):
        return type(self)._fn(x, self._axis(x))


class Softmax(_DimModule):
    _fn = staticmethod(softmax)


class LogSoftmax(_DimModule):
    _fn = staticmethod(log_softmax)


class Softmin(_DimModule):
    _fn = staticmethod(softmin)


class Softmax2d(Module):
    """Softmax over the channel dimension of ``[N, C, H, W]`` or ``[C, H, W]``."""

    def forward(self, x):
        if x.dim() not in (3, 4):
            raise InvalidArgument(f"Softmax2d expects a 3-D or 4-D input, got {x.dim()}-D")
        return softmax(x, -3)


class GLU(Module):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, x):
        return glu(x, self.dim)


class Threshold(Module):
    def __init__(self, threshold: float, value: float, inplace: bool = False):
        super().__init__()
        self.threshold, self.value, self.inplace = threshold, value, inplace

    def forward(self, x):
        return threshold(x, self.threshold, self.value)


class Softshrink(Module):
    def __init__(self, lambd: float = 0.5):
        super().__init__()
        if lambd < 0:
            raise InvalidArgument("Softshrink: lambd must be >= 0")
        self.lambd = lambd

    def forward(self, x):
        return softshrink(x, self.lambd)


class Hardshrink(Module):
    def __init__(self, lambd: float = 0.5):
        super().__init__()
        self.lambd = lambd

    def forward(self, x):
        return hardshrink(x, self.lambd)


class PReLU(Module):
    """``max(0, x) + a * min(0, x)`` with one learnable slope, or one per channel (dimension 1)."""

    def __init__(self, num_parameters: int = 1, init: float = 0.25, device=None, dtype=None):
        super().__init__()
        self.num_parameters = num_parameters
        self.weight = Parameter(torch.full((num_parameters,), float(init), device=device, dtype=dtype))

    def forward(self, x):
        return prelu(x, self.weight)


class RReLU(Module):
    """Leaky ReLU whose negative slope is drawn from ``U(lower, upper)`` per element while training and fixed at the mean otherwise."""

    def __init__(self, lower: float = 1.0 / 8, upper: float = 1.0 / 3, inplace: bool = False):
        super().__init__()
        if not lower <= upper:
            raise InvalidArgument("RReLU: lower must be <= upper")
        self.lower, self.upper, self.inplace = lower, upper, inplace

    def forward(self, x):
        return rrelu(x, self.lower, self.upper, self.training)


__all__ = ["ReLU", "ReLU6", "SELU", "SiLU", "Mish", "Sigmoid", "Tanh", "HardSigmoid", "HardSwish", "LogSigmoid", "Tanhshrink", "Softsign",
           "LeakyReLU", "ELU", "CELU", "Hardtanh", "Softplus", "Softmax", "LogSoftmax", "Softmin", "Softmax2d", "GLU", "Threshold",
           "Softshrink", "Hardshrink", "PReLU", "RReLU"]
_ = math
