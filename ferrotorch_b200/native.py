"""Python binding of the native CPU tensor / autograd core (``csrc/runtime/core.cpp``).

``Tensor`` wraps a handle of the C++ ``ft::Tensor`` (f32, strided, reference counted); the operations record ``ft::Node`` objects and
``Tensor.backward()`` runs the C++ engine (graph collection, Kahn ordering, reverse sweep, hooks; ``threads > 1`` selects the parallel sweep,
which produces the same bits). ``Linear`` / ``Conv2d`` / ``MaxPool2d`` / ``Flatten`` / activations / ``Sequential`` with ``Sgd`` / ``Adam`` /
``AdamW`` are the smallest framework layer over it: enough to train the MLP of the CPU data-parallel benchmark, or a small convolutional
network, without ``torch.nn`` / ``torch.autograd`` / ``torch.optim`` on the path. NumPy arrays are the interchange format
(``Tensor.numpy()`` of a contiguous tensor is a zero-copy view of the native storage).

Reference parity: ferrotorch-core/src/tensor.rs:46-103, autograd/graph.rs:20-458, ferrotorch-nn/src/{module,linear,loss}.rs,
ferrotorch-optim/src/sgd.rs.
"""
from __future__ import annotations

import ctypes
import math
from typing import Callable, Iterable, List, Optional

import numpy as np

from . import _lib
from .errors import InvalidArgument

_vp, _i, _i64, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
_GRAD_HOOK = ctypes.CFUNCTYPE(None, _vp, ctypes.POINTER(ctypes.c_float), _i64)
_POST_HOOK = ctypes.CFUNCTYPE(None, _vp, ctypes.c_uint64)
_SIGS = {
    "ftc_last_error": (ctypes.c_char_p, []), "ftc_tensor_new": (_vp, [_vp, _vp, _i, _i]), "ftc_free": (None, [_vp]), "ftc_ndim": (_i, [_vp]),
    "ftc_numel": (_i64, [_vp]), "ftc_shape": (None, [_vp, _vp]), "ftc_id": (ctypes.c_uint64, [_vp]), "ftc_requires_grad": (_i, [_vp]),
    "ftc_is_leaf": (_i, [_vp]), "ftc_grad_fn_name": (ctypes.c_char_p, [_vp]), "ftc_data_ptr": (_vp, [_vp]), "ftc_copy_out": (None, [_vp, _vp]),
    "ftc_grad": (_vp, [_vp]), "ftc_zero_grad": (None, [_vp]), "ftc_detach": (_vp, [_vp]), "ftc_set_grad_enabled": (_i, [_i]),
    "ftc_add": (_vp, [_vp, _vp]), "ftc_sub": (_vp, [_vp, _vp]), "ftc_mul": (_vp, [_vp, _vp]), "ftc_scale": (_vp, [_vp, _f]),
    "ftc_matmul": (_vp, [_vp, _vp]), "ftc_transpose": (_vp, [_vp]), "ftc_relu": (_vp, [_vp]), "ftc_tanh": (_vp, [_vp]), "ftc_sigmoid": (_vp, [_vp]),
    "ftc_sum": (_vp, [_vp]), "ftc_mean": (_vp, [_vp]), "ftc_linear": (_vp, [_vp, _vp, _vp]), "ftc_cross_entropy": (_vp, [_vp, _vp, _i64]),
    "ftc_backward": (_i, [_vp, _vp, _i]), "ftc_register_hook": (None, [_vp, _GRAD_HOOK, _vp]),
    "ftc_register_post_accumulate_hook": (None, [_vp, _POST_HOOK, _vp]),
    "ftc_sgd_new": (_vp, [_vp, _i, _f, _f, _f, _f, _i]), "ftc_sgd_step": (None, [_vp]), "ftc_sgd_set_lr": (None, [_vp, _f]),
    "ftc_sgd_zero_grad": (None, [_vp]), "ftc_sgd_free": (None, [_vp]),
    "ftc_unary": (_vp, [_vp, _i, _f]), "ftc_div": (_vp, [_vp, _vp]), "ftc_reshape": (_vp, [_vp, _vp, _i]), "ftc_sum_dim": (_vp, [_vp, _i, _i, _i]),
    "ftc_softmax": (_vp, [_vp, _i]), "ftc_conv2d": (_vp, [_vp, _vp, _vp, _i, _i, _i, _i]), "ftc_max_pool2d": (_vp, [_vp, _i, _i]),
    "ftc_adam_new": (_vp, [_vp, _i, _f, _f, _f, _f, _f, _i]), "ftc_adam_step": (None, [_vp]), "ftc_adam_set_lr": (None, [_vp, _f]),
    "ftc_adam_zero_grad": (None, [_vp]), "ftc_adam_free": (None, [_vp]),
    "ftc_permute": (_vp, [_vp, _vp, _i]), "ftc_bmm": (_vp, [_vp, _vp]), "ftc_layer_norm": (_vp, [_vp, _vp, _vp, _f]), "ftc_embedding": (_vp, [_vp, _vp, _vp, _i]),
    "ftc_narrow": (_vp, [_vp, _i, _i64, _i64]),
}
_UNARY = {"exp": 0, "log": 1, "sqrt": 2, "gelu": 3, "silu": 4, "leaky_relu": 5, "pow": 6, "abs": 7, "square": 8, "reciprocal": 9}
_bound = {}


def _fn(name: str):
    f = _bound.get(name)
    if f is None:
        f = getattr(_lib.runtime(), name)
        f.restype, f.argtypes = _SIGS[name]
        _bound[name] = f
    return f


def _check(h):
    if not h:
        raise InvalidArgument(_fn("ftc_last_error")().decode() or "native core: operation failed")
    return h


class Tensor:
    """A handle of a native ``ft::Tensor``."""

    __slots__ = ("_h", "_hooks")

    def __init__(self, data=None, requires_grad: bool = False, *, _handle=None):
        self._hooks: list = []            # keeps the ctypes callbacks alive as long as the tensor
        if _handle is not None:
            self._h = _handle
            return
        a = np.ascontiguousarray(np.asarray(data, dtype=np.float32))
        shape = (ctypes.c_int64 * max(a.ndim, 1))(*a.shape)
        self._h = _check(_fn("ftc_tensor_new")(a.ctypes.data, shape, a.ndim, int(requires_grad)))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _fn("ftc_free")(h)
            except Exception:
                pass

    # -- metadata ---------------------------------------------------------------------------------------------------------
    @property
    def shape(self) -> tuple:
        nd = _fn("ftc_ndim")(self._h)
        out = (ctypes.c_int64 * max(nd, 1))()
        _fn("ftc_shape")(self._h, out)
        return tuple(out[i] for i in range(nd))

    def numel(self) -> int:
        return _fn("ftc_numel")(self._h)

    @property
    def requires_grad(self) -> bool:
        return bool(_fn("ftc_requires_grad")(self._h))

    @property
    def is_leaf(self) -> bool:
        return bool(_fn("ftc_is_leaf")(self._h))

    @property
    def grad_fn(self) -> Optional[str]:
        n = _fn("ftc_grad_fn_name")(self._h).decode()
        return n or None

    @property
    def id(self) -> int:
        return _fn("ftc_id")(self._h)

    @property
    def grad(self) -> Optional["Tensor"]:
        h = _fn("ftc_grad")(self._h)
        return Tensor(_handle=h) if h else None

    def zero_grad(self) -> None:
        _fn("ftc_zero_grad")(self._h)

    def numpy(self) -> np.ndarray:
        """The values as a NumPy array: a zero-copy view of the native storage for a contiguous tensor (writes go through), else a copy."""
        p = _fn("ftc_data_ptr")(self._h)
        shape = self.shape
        if p:
            n = self.numel()
            arr = np.ctypeslib.as_array(ctypes.cast(p, ctypes.POINTER(ctypes.c_float)), shape=(n,)) if n else np.empty(0, np.float32)
            arr = arr.reshape(shape)
            arr_base = arr.base if arr.base is not None else arr
            try:
                arr_base._ft_owner = self          # keep the native tensor alive while the view is
            except AttributeError:
                pass
            return arr
        out = np.empty(shape, np.float32)
        _fn("ftc_copy_out")(self._h, out.ctypes.data)
        return out

    def item(self) -> float:
        return float(self.numpy().reshape(-1)[0])

    def detach(self) -> "Tensor":
        return Tensor(_handle=_check(_fn("ftc_detach")(self._h)))

    # -- operations -------------------------------------------------------------------------------------------------------
    def _bin(self, name, other):
        if not isinstance(other, Tensor):
            if np.isscalar(other) and name == "ftc_mul":
                return Tensor(_handle=_check(_fn("ftc_scale")(self._h, float(other))))
            other = Tensor(np.broadcast_to(np.asarray(other, np.float32), self.shape))
        a, b = self.shape, other.shape
        if len(a) < len(b) and tuple(b[len(b) - len(a):]) == tuple(a):
            # The kernels broadcast the SECOND operand over the first one's leading dimensions; with the smaller tensor first, rewrite.
            if name in ("ftc_add", "ftc_mul"):
                return other._bin(name, self)
            if name == "ftc_sub":
                return -(other._bin("ftc_sub", self))
            if name == "ftc_div":
                return other.reciprocal()._bin("ftc_mul", self)
        return Tensor(_handle=_check(_fn(name)(self._h, other._h)))

    def __add__(self, o): return self._bin("ftc_add", o)
    def __sub__(self, o): return self._bin("ftc_sub", o)
    def __mul__(self, o): return self._bin("ftc_mul", o)
    __rmul__ = __mul__
    __radd__ = __add__
    def __rsub__(self, o): return -(self._bin("ftc_sub", o))
    def __rtruediv__(self, o): return self.reciprocal() * o
    def __neg__(self): return Tensor(_handle=_check(_fn("ftc_scale")(self._h, -1.0)))
    def __matmul__(self, o):
        """Matrix product; tensors with leading (batch) dimensions multiply batch by batch."""
        return Tensor(_handle=_check(_fn("ftc_matmul" if len(self.shape) == 2 else "ftc_bmm")(self._h, o._h)))

    def permute(self, *dims):
        if len(dims) == 1 and isinstance(dims[0], (tuple, list)):
            dims = tuple(dims[0])
        arr = (ctypes.c_int64 * max(len(dims), 1))(*[int(d) for d in dims])
        return Tensor(_handle=_check(_fn("ftc_permute")(self._h, arr, len(dims))))

    def narrow(self, dim: int, start: int, length: int):
        """A view of ``length`` consecutive entries of dimension ``dim``."""
        return Tensor(_handle=_check(_fn("ftc_narrow")(self._h, int(dim), int(start), int(length))))

    def __getitem__(self, i):
        """``t[i]`` (an integer) or ``t[a:b]`` on the first dimension."""
        n = self.shape[0]
        if isinstance(i, slice):
            a, b, step = i.indices(n)
            if step != 1:
                raise InvalidArgument("native Tensor: slices have step 1")
            return self.narrow(0, a, max(b - a, 0))
        i = int(i) + (n if int(i) < 0 else 0)
        return self.narrow(0, i, 1).reshape(*self.shape[1:])

    def transpose(self, d0: int, d1: int):
        order = list(range(len(self.shape)))
        order[d0], order[d1] = order[d1], order[d0]
        return self.permute(*order)
    def t(self): return Tensor(_handle=_check(_fn("ftc_transpose")(self._h)))
    def relu(self): return Tensor(_handle=_check(_fn("ftc_relu")(self._h)))
    def tanh(self): return Tensor(_handle=_check(_fn("ftc_tanh")(self._h)))
    def sigmoid(self): return Tensor(_handle=_check(_fn("ftc_sigmoid")(self._h)))
    def __truediv__(self, o):
        if not isinstance(o, Tensor) and np.isscalar(o):
            return Tensor(_handle=_check(_fn("ftc_scale")(self._h, 1.0 / float(o))))
        return self._bin("ftc_div", o)

    def _un(self, kind: str, p: float = 0.0): return Tensor(_handle=_check(_fn("ftc_unary")(self._h, _UNARY[kind], float(p))))
    def exp(self): return self._un("exp")
    def log(self): return self._un("log")
    def sqrt(self): return self._un("sqrt")
    def gelu(self): return self._un("gelu")
    def silu(self): return self._un("silu")
    def leaky_relu(self, negative_slope: float = 0.01): return self._un("leaky_relu", negative_slope)
    def pow(self, p: float): return self._un("pow", p)
    __pow__ = pow
    def abs(self): return self._un("abs")
    def square(self): return self._un("square")
    def reciprocal(self): return self._un("reciprocal")

    def reshape(self, *shape):
        """A view with another shape (one entry may be -1); a non-contiguous tensor is copied first."""
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        arr = (ctypes.c_int64 * max(len(shape), 1))(*[int(v) for v in shape])
        return Tensor(_handle=_check(_fn("ftc_reshape")(self._h, arr, len(shape))))

    view = reshape

    def flatten(self, start_dim: int = 0):
        sh = self.shape
        start_dim %= max(len(sh), 1)
        return self.reshape(*sh[:start_dim], -1)

    def sum(self, dim: Optional[int] = None, keepdim: bool = False):
        if dim is None:
            return Tensor(_handle=_check(_fn("ftc_sum")(self._h)))
        return Tensor(_handle=_check(_fn("ftc_sum_dim")(self._h, int(dim), int(keepdim), 0)))

    def mean(self, dim: Optional[int] = None, keepdim: bool = False):
        if dim is None:
            return Tensor(_handle=_check(_fn("ftc_mean")(self._h)))
        return Tensor(_handle=_check(_fn("ftc_sum_dim")(self._h, int(dim), int(keepdim), 1)))

    def _softmax(self, dim: int, log: int):
        nd = len(self.shape)
        dim = int(dim) % max(nd, 1)
        if dim == nd - 1 or nd == 0:
            return Tensor(_handle=_check(_fn("ftc_softmax")(self._h, log)))
        moved = self.transpose(dim, nd - 1)           # the kernel normalises the last dimension
        return Tensor(_handle=_check(_fn("ftc_softmax")(moved._h, log))).transpose(dim, nd - 1)

    def softmax(self, dim: int = -1): return self._softmax(dim, 0)
    def log_softmax(self, dim: int = -1): return self._softmax(dim, 1)

    def backward(self, grad: Optional["Tensor"] = None, threads: int = 1) -> None:
        """Reverse sweep from this tensor. ``threads > 1`` runs independent nodes on worker threads (``backward_parallel``); gradients are
        summed per consuming edge in a fixed order, so the result does not depend on the number of threads."""
        if _fn("ftc_backward")(self._h, grad._h if grad is not None else None, int(threads)):
            raise InvalidArgument(_fn("ftc_last_error")().decode())

    def register_hook(self, fn: Callable[[np.ndarray], Optional[np.ndarray]]) -> None:
        """``fn(grad)`` sees every gradient that reaches this tensor during backward (a NumPy view; modify it in place or return a replacement)."""
        def cb(_user, ptr, n):
            g = np.ctypeslib.as_array(ptr, shape=(n,))
            r = fn(g)
            if r is not None:
                g[:] = np.asarray(r, np.float32).reshape(-1)
        c = _GRAD_HOOK(cb)
        self._hooks.append(c)
        _fn("ftc_register_hook")(self._h, c, None)

    def register_post_accumulate_grad_hook(self, fn: Callable[["Tensor"], None]) -> None:
        """``fn(tensor)`` runs once this leaf's ``.grad`` is complete for the current sweep (data-parallel wrappers launch a bucket here)."""
        def cb(_user, _tid):
            fn(self)
        c = _POST_HOOK(cb)
        self._hooks.append(c)
        _fn("ftc_register_post_accumulate_hook")(self._h, c, None)


class no_grad:
    def __enter__(self):
        self.prev = _fn("ftc_set_grad_enabled")(0)

    def __exit__(self, *exc):
        _fn("ftc_set_grad_enabled")(self.prev)
        return False


def linear(x: Tensor, w: Tensor, b: Optional[Tensor] = None) -> Tensor:
    return Tensor(_handle=_check(_fn("ftc_linear")(x._h, w._h, b._h if b is not None else None)))


def relu(x: Tensor) -> Tensor:
    return x.relu()


def cross_entropy(logits: Tensor, targets) -> Tensor:
    t = np.ascontiguousarray(np.asarray(targets, dtype=np.int64))
    return Tensor(_handle=_check(_fn("ftc_cross_entropy")(logits._h, t.ctypes.data, t.size)))


def layer_norm(x: Tensor, weight: Optional[Tensor] = None, bias: Optional[Tensor] = None, eps: float = 1e-5) -> Tensor:
    """Normalisation over the last dimension."""
    return Tensor(_handle=_check(_fn("ftc_layer_norm")(x._h, weight._h if weight is not None else None, bias._h if bias is not None else None, eps)))


def embedding(ids, table: Tensor) -> Tensor:
    """Rows ``ids`` (any integer array) of ``table`` [rows, dim]: the result has the shape of ``ids`` plus the row length."""
    a = np.ascontiguousarray(np.asarray(ids, dtype=np.int64))
    shape = (ctypes.c_int64 * max(a.ndim, 1))(*a.shape)
    return Tensor(_handle=_check(_fn("ftc_embedding")(table._h, a.ctypes.data, shape, a.ndim)))


def _pair(v):
    return (int(v), int(v)) if np.isscalar(v) else (int(v[0]), int(v[1]))


def conv2d(x: Tensor, w: Tensor, b: Optional[Tensor] = None, stride=1, padding=0) -> Tensor:
    """``x`` [N, C, H, W], ``w`` [O, C, kh, kw], ``b`` [O]: patch matrix times GEMM in the native core, with its backward rule."""
    (sh, sw), (ph, pw) = _pair(stride), _pair(padding)
    return Tensor(_handle=_check(_fn("ftc_conv2d")(x._h, w._h, b._h if b is not None else None, sh, sw, ph, pw)))


def max_pool2d(x: Tensor, kernel_size: int, stride: Optional[int] = None) -> Tensor:
    return Tensor(_handle=_check(_fn("ftc_max_pool2d")(x._h, int(kernel_size), int(stride or kernel_size))))


def mse_loss(a: Tensor, b: Tensor) -> Tensor:
    return (a - b).square().mean()


# ----------------------------------------------------------------------------------------------------------------------
# the smallest module layer
# ----------------------------------------------------------------------------------------------------------------------
class Module:
    def parameters(self) -> List[Tensor]:
        out = []
        for v in self.__dict__.values():
            if isinstance(v, Tensor) and v.requires_grad:
                out.append(v)
            elif isinstance(v, Module):
                out += v.parameters()
            elif isinstance(v, (list, tuple)):
                for m in v:
                    if isinstance(m, Module):
                        out += m.parameters()
        return out

    def zero_grad(self) -> None:
        for p in self.parameters():
            p.zero_grad()

    def __call__(self, *a):
        return self.forward(*a)


class Linear(Module):
    """``x W^T + b``; Kaiming-uniform weights for a ReLU network (bound ``sqrt(6 / fan_in)``) and zero bias, drawn from ``rng``."""

    def __init__(self, fan_in: int, fan_out: int, bias: bool = True, rng: Optional[np.random.Generator] = None, weight=None, bias_value=None):
        rng = rng or np.random.default_rng(0)
        bound = math.sqrt(6.0 / fan_in)
        w = rng.uniform(-bound, bound, size=(fan_out, fan_in)).astype(np.float32) if weight is None else np.asarray(weight, np.float32)
        self.weight = Tensor(w, requires_grad=True)
        self.bias = Tensor(np.zeros(fan_out, np.float32) if bias_value is None else np.asarray(bias_value, np.float32), requires_grad=True) if bias else None

    def forward(self, x: Tensor) -> Tensor:
        return linear(x, self.weight, self.bias)


class ReLU(Module):
    def forward(self, x: Tensor) -> Tensor:
        return x.relu()


class Conv2d(Module):
    """Kaiming-uniform weights (bound ``sqrt(6 / (C kh kw))``) and zero bias, like ``Linear``."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, bias: bool = True, rng: Optional[np.random.Generator] = None):
        rng = rng or np.random.default_rng(0)
        kh, kw = _pair(kernel_size)
        bound = math.sqrt(6.0 / (in_channels * kh * kw))
        self.weight = Tensor(rng.uniform(-bound, bound, size=(out_channels, in_channels, kh, kw)).astype(np.float32), requires_grad=True)
        self.bias = Tensor(np.zeros(out_channels, np.float32), requires_grad=True) if bias else None
        self.stride, self.padding = stride, padding

    def forward(self, x: Tensor) -> Tensor:
        return conv2d(x, self.weight, self.bias, self.stride, self.padding)


class MaxPool2d(Module):
    def __init__(self, kernel_size: int, stride: Optional[int] = None):
        self.kernel_size, self.stride = kernel_size, stride

    def forward(self, x: Tensor) -> Tensor:
        return max_pool2d(x, self.kernel_size, self.stride)


class Flatten(Module):
    def forward(self, x: Tensor) -> Tensor:
        return x.flatten(1)


class GELU(Module):
    def forward(self, x: Tensor) -> Tensor:
        return x.gelu()


class SiLU(Module):
    def forward(self, x: Tensor) -> Tensor:
        return x.silu()


class Tanh(Module):
    def forward(self, x: Tensor) -> Tensor:
        return x.tanh()


class Sigmoid(Module):
    def forward(self, x: Tensor) -> Tensor:
        return x.sigmoid()


class LayerNorm(Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        self.weight, self.bias, self.eps = Tensor(np.ones(dim, np.float32), requires_grad=True), Tensor(np.zeros(dim, np.float32), requires_grad=True), eps

    def forward(self, x: Tensor) -> Tensor:
        return layer_norm(x, self.weight, self.bias, self.eps)


class Embedding(Module):
    def __init__(self, rows: int, dim: int, rng: Optional[np.random.Generator] = None):
        rng = rng or np.random.default_rng(0)
        self.weight = Tensor(rng.standard_normal((rows, dim)).astype(np.float32), requires_grad=True)

    def forward(self, ids) -> Tensor:
        return embedding(ids, self.weight)


class Sequential(Module):
    def __init__(self, *mods: Module):
        self.mods = list(mods)

    def forward(self, x: Tensor) -> Tensor:
        for m in self.mods:
            x = m(x)
        return x


class Sgd:
    """Native SGD (momentum, dampening, Nesterov, coupled weight decay), the update rule of ferrotorch-optim/src/sgd.rs:210."""

    def __init__(self, params: Iterable[Tensor], lr: float, momentum: float = 0.0, dampening: float = 0.0, weight_decay: float = 0.0,
                 nesterov: bool = False):
        self.params = list(params)
        arr = (ctypes.c_void_p * len(self.params))(*[p._h for p in self.params])
        self._h = _fn("ftc_sgd_new")(arr, len(self.params), lr, momentum, dampening, weight_decay, int(nesterov))

    def step(self) -> None:
        _fn("ftc_sgd_step")(self._h)

    def zero_grad(self) -> None:
        _fn("ftc_sgd_zero_grad")(self._h)

    def set_lr(self, lr: float) -> None:
        _fn("ftc_sgd_set_lr")(self._h, lr)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _fn("ftc_sgd_free")(h)
            except Exception:
                pass


class Adam:
    """Native Adam; ``decoupled=True`` is AdamW (the weights shrink by ``1 - lr * weight_decay`` before the step), else the decay joins the
    gradient (ferrotorch-optim/src/adam.rs, adamw.rs:315)."""

    def __init__(self, params: Iterable[Tensor], lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, decoupled: bool = False):
        self.params = list(params)
        arr = (ctypes.c_void_p * len(self.params))(*[p._h for p in self.params])
        self._h = _fn("ftc_adam_new")(arr, len(self.params), lr, betas[0], betas[1], eps, weight_decay, int(decoupled))

    def step(self) -> None:
        _fn("ftc_adam_step")(self._h)

    def zero_grad(self) -> None:
        _fn("ftc_adam_zero_grad")(self._h)

    def set_lr(self, lr: float) -> None:
        _fn("ftc_adam_set_lr")(self._h, lr)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _fn("ftc_adam_free")(h)
            except Exception:
                pass


class AdamW(Adam):
    def __init__(self, params: Iterable[Tensor], lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2):
        super().__init__(params, lr, betas, eps, weight_decay, decoupled=True)
