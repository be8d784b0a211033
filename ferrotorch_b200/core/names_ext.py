"""Top-level functional names of the core package: elementwise / special functions, FFT family, cumulative and indexing operations, view
helpers, forward-mode dual arithmetic, anomaly mode, autocast debugging, dispatch-key sets, storage handles and the element-type groups.

Tensors are ``torch.Tensor`` and run on whatever device they live on (the reference refuses several of these on CUDA; here they work there).
Argument checks and error kinds follow the reference so that code written against it fails the same way.

Reference parity (ferrotorch-core/src): grad_fns/{transcendental,activation,arithmetic,reduction,shape,indexing,cumulative,fft}.rs, special.rs,
fft.rs, ops/{cumulative.rs:181, indexing.rs:334, scatter.rs:74, search.rs:140-260, tensor_ops.rs:292, higher_order.rs:142}, shape.rs:100,
autograd/{anomaly.rs:29-175, autocast.rs:18-60, autocast_ops.rs:73, graph.rs:30, forward_ad.rs}, dispatch.rs:137-291, storage.rs:63, tensor.rs:33,
dtype.rs (Element / Float / IntElement), einops.rs:33, quantize.rs (Observer, FakeQuantize, QAT).
"""
from __future__ import annotations

import abc
import enum
import itertools
import threading
import traceback
from dataclasses import dataclass
from typing import Any, Callable, List, NamedTuple, Optional, Sequence, Tuple, Union

import torch

from ..errors import FerrotorchError, InvalidArgument, ShapeMismatch

# -- element-type groups (dtype.rs) ------------------------------------------------------------------------------------------
Float = (torch.float32, torch.float64, torch.bfloat16, torch.float16)          # dtypes the differentiable operations accept
IntElement = (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)
Element = Float + IntElement + (torch.bool,)
FerrotorchResult = Any                                                         # results are returned directly; failures raise FerrotorchError


def is_float(t: torch.Tensor) -> bool:
    return t.dtype in Float


def normalize_axis(axis: int, ndim: int) -> int:
    if axis >= ndim or axis < -ndim:
        raise InvalidArgument(f"axis {axis} is out of bounds for tensor with {ndim} dimensions")
    return axis + ndim if axis < 0 else axis


def broadcast_shapes(a: Sequence[int], b: Sequence[int]) -> Tuple[int, ...]:
    try:
        return tuple(torch.broadcast_shapes(tuple(a), tuple(b)))
    except RuntimeError:
        raise ShapeMismatch(f"shapes {list(a)} and {list(b)} are not broadcast-compatible") from None


# -- elementwise and special functions ---------------------------------------------------------------------------------------------
exp, expm1, log, log1p, sin, cos, tanh, sigmoid = torch.exp, torch.expm1, torch.log, torch.log1p, torch.sin, torch.cos, torch.tanh, torch.sigmoid
erf, erfc, erfinv, lgamma, digamma, sinc, xlogy = torch.erf, torch.erfc, torch.erfinv, torch.lgamma, torch.digamma, torch.sinc, torch.xlogy


def clamp(x: torch.Tensor, lo: Optional[float] = None, hi: Optional[float] = None) -> torch.Tensor:
    if lo is None and hi is None:
        raise InvalidArgument("clamp: at least one bound is required")
    if lo is not None and hi is not None and lo > hi:
        raise InvalidArgument(f"clamp: min {lo} > max {hi}")
    return torch.clamp(x, lo, hi)


def where_cond(condition, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """``condition`` is a flat list of bools (or a bool tensor) with one entry per element of ``x``; ``x`` and ``y`` share a shape
    (ops/indexing.rs:334)."""
    if x.shape != y.shape:
        raise ShapeMismatch(f"where_cond: x shape {list(x.shape)} != y shape {list(y.shape)}")
    c = torch.as_tensor(condition, dtype=torch.bool, device=x.device)
    if c.numel() != x.numel():
        raise ShapeMismatch(f"where_cond: condition has {c.numel()} entries, tensors have {x.numel()}")
    return torch.where(c.reshape(x.shape), x, y)


# -- reductions / shape -------------------------------------------------------------------------------------------------------
def sum_dim(x: torch.Tensor, dim: int, keepdim: bool = False) -> torch.Tensor:
    return x.sum(normalize_axis(dim, x.dim()), keepdim=keepdim)


def mean_dim(x: torch.Tensor, dim: int, keepdim: bool = False) -> torch.Tensor:
    return x.mean(normalize_axis(dim, x.dim()), keepdim=keepdim)


def cat(tensors: Sequence[torch.Tensor], dim: int = 0) -> torch.Tensor:
    if len(tensors) == 0:
        raise InvalidArgument("cat: empty tensor list")
    d = normalize_axis(dim, tensors[0].dim())
    for t in tensors[1:]:
        if t.dim() != tensors[0].dim() or any(a != b for k, (a, b) in enumerate(zip(t.shape, tensors[0].shape)) if k != d):
            raise ShapeMismatch(f"cat: shapes {list(tensors[0].shape)} and {list(t.shape)} differ outside dim {d}")
    return torch.cat(list(tensors), d)


def expand(x: torch.Tensor, shape: Sequence[int]) -> torch.Tensor:
    try:
        return x.expand(tuple(shape))
    except RuntimeError as e:
        raise ShapeMismatch(f"expand: {list(x.shape)} cannot expand to {list(shape)}: {e}") from None


def view_t(x: torch.Tensor, shape: Sequence[int]) -> torch.Tensor:
    """Zero-copy reshape (one ``-1`` allowed); a non-contiguous source is refused rather than silently copied."""
    if list(shape).count(-1) > 1:
        raise InvalidArgument("view: only one dimension may be -1")
    try:
        return x.view(tuple(shape))
    except RuntimeError as e:
        raise ShapeMismatch(f"view: {list(x.shape)} -> {list(shape)}: {e}") from None


def permute_t(x: torch.Tensor, dims: Sequence[int]) -> torch.Tensor:
    nd = [normalize_axis(d, x.dim()) for d in dims]
    if sorted(nd) != list(range(x.dim())):
        raise InvalidArgument(f"permute: {list(dims)} is not a permutation of the {x.dim()} dimensions")
    return x.permute(nd)


def contiguous_t(x: torch.Tensor) -> torch.Tensor:
    return x.contiguous()


def chunk_t(x: torch.Tensor, chunks: int, dim: int = 0) -> List[torch.Tensor]:
    if chunks <= 0:
        raise InvalidArgument("chunk: chunks must be > 0")
    return list(x.chunk(chunks, normalize_axis(dim, x.dim())))


def split_t(x: torch.Tensor, split_sizes: Union[int, Sequence[int]], dim: int = 0) -> List[torch.Tensor]:
    d = normalize_axis(dim, x.dim())
    if not isinstance(split_sizes, int) and sum(split_sizes) != x.shape[d]:
        raise InvalidArgument(f"split: sizes {list(split_sizes)} do not sum to {x.shape[d]}")
    return list(x.split(split_sizes, d))


def roll(x: torch.Tensor, shifts: int, dim: int) -> torch.Tensor:
    return torch.roll(x, shifts, normalize_axis(dim, x.dim()))


def tril(x: torch.Tensor, diagonal: int = 0) -> torch.Tensor:
    if x.dim() < 2:
        raise InvalidArgument(f"tril: at least 2 dimensions required, got {x.dim()}")
    return torch.tril(x, diagonal)


def triu(x: torch.Tensor, diagonal: int = 0) -> torch.Tensor:
    if x.dim() < 2:
        raise InvalidArgument(f"triu: at least 2 dimensions required, got {x.dim()}")
    return torch.triu(x, diagonal)


def diag(x: torch.Tensor, diagonal: int = 0) -> torch.Tensor:
    if x.dim() not in (1, 2):
        raise InvalidArgument(f"diag: 1-D or 2-D input required, got {x.dim()}-D")
    return torch.diag(x, diagonal)


def diagflat(x: torch.Tensor, offset: int = 0) -> torch.Tensor:
    return torch.diagflat(x, offset)


def meshgrid(tensors: Sequence[torch.Tensor]) -> List[torch.Tensor]:
    """``ij`` indexing over 1-D inputs (ops/search.rs:228); an empty list gives an empty list."""
    if len(tensors) == 0:
        return []
    for t in tensors:
        if t.dim() != 1:
            raise InvalidArgument(f"meshgrid: all inputs must be 1-D, got shape {list(t.shape)}")
    return list(torch.meshgrid(*tensors, indexing="ij"))


def cdist(x1: torch.Tensor, x2: torch.Tensor, p: float = 2.0) -> torch.Tensor:
    if x1.dim() != x2.dim() or x1.dim() not in (2, 3) or x1.shape[-1] != x2.shape[-1] or (x1.dim() == 3 and x1.shape[0] != x2.shape[0]):
        raise ShapeMismatch(f"cdist: expected [P, M] x [R, M] or [B, P, M] x [B, R, M], got {list(x1.shape)} and {list(x2.shape)}")
    if p < 0:
        raise InvalidArgument(f"cdist: p must be >= 0, got {p}")
    return torch.cdist(x1, x2, p)


# -- indexing --------------------------------------------------------------------------------------------------------------------
def _index(idx, device) -> torch.Tensor:
    return idx.to(device=device, dtype=torch.long) if torch.is_tensor(idx) else torch.as_tensor(idx, dtype=torch.long, device=device)


def gather(x: torch.Tensor, dim: int, index) -> torch.Tensor:
    d, i = normalize_axis(dim, x.dim()), _index(index, x.device)
    if i.numel() and (int(i.min()) < 0 or int(i.max()) >= x.shape[d]):
        raise InvalidArgument(f"gather: index out of range for dimension {d} of size {x.shape[d]}")
    return torch.gather(x, d, i)


def scatter(x: torch.Tensor, dim: int, index, src: torch.Tensor) -> torch.Tensor:
    d, i = normalize_axis(dim, x.dim()), _index(index, x.device)
    if i.numel() and (int(i.min()) < 0 or int(i.max()) >= x.shape[d]):
        raise InvalidArgument(f"scatter: index out of range for dimension {d} of size {x.shape[d]}")
    return torch.scatter(x, d, i, src)


def scatter_add(x: torch.Tensor, dim: int, index, src: torch.Tensor) -> torch.Tensor:
    d, i = normalize_axis(dim, x.dim()), _index(index, x.device)
    if i.numel() and (int(i.min()) < 0 or int(i.max()) >= x.shape[d]):
        raise InvalidArgument(f"scatter_add: index out of range for dimension {d} of size {x.shape[d]}")
    return torch.scatter_add(x, d, i, src)


def scatter_add_segments(src: torch.Tensor, index, dim_size: int) -> torch.Tensor:
    """Rows of ``src [E, ...]`` summed into ``dim_size`` segments by ``index [E]``: the message-aggregation primitive of graph layers
    (ops/scatter.rs:74). Differentiable in ``src``."""
    i = _index(index, src.device)
    if src.dim() < 1 or i.dim() != 1 or i.numel() != src.shape[0]:
        raise ShapeMismatch(f"scatter_add_segments: {i.numel()} indices for source shape {list(src.shape)}")
    if i.numel() and (int(i.min()) < 0 or int(i.max()) >= dim_size):
        raise InvalidArgument(f"scatter_add_segments: index out of range for {dim_size} segments")
    return torch.zeros((dim_size,) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device).index_add(0, i, src)


def unique_consecutive(x: torch.Tensor) -> Tuple[torch.Tensor, List[int], List[int]]:
    """Values with adjacent repeats collapsed, plus for every input element the index of its run and the length of every run
    (ops/search.rs:140)."""
    vals, inv, counts = torch.unique_consecutive(x.reshape(-1), return_inverse=True, return_counts=True)
    return vals, inv.tolist(), counts.tolist()


# -- cumulative ------------------------------------------------------------------------------------------------------------------
class CumExtremeResult(NamedTuple):
    """Running extreme along a dimension with, for every position, the index (along that dimension) where it was attained
    (ops/cumulative.rs:181)."""
    values: torch.Tensor
    indices: torch.Tensor


def cummax(x: torch.Tensor, dim: int) -> CumExtremeResult:
    return CumExtremeResult(*torch.cummax(x, normalize_axis(dim, x.dim())))


def cummin(x: torch.Tensor, dim: int) -> CumExtremeResult:
    return CumExtremeResult(*torch.cummin(x, normalize_axis(dim, x.dim())))


def cumprod(x: torch.Tensor, dim: int) -> torch.Tensor:
    return torch.cumprod(x, normalize_axis(dim, x.dim()))


def logcumsumexp(x: torch.Tensor, dim: int) -> torch.Tensor:
    return torch.logcumsumexp(x, normalize_axis(dim, x.dim()))


# -- FFT family: complex values travel as a trailing dimension of size 2 (re, im), as in the reference's real-tensor API (fft.rs) -----------
def _c(x: torch.Tensor, who: str) -> torch.Tensor:
    if x.is_complex():
        return x
    if x.dim() == 0 or x.shape[-1] != 2:
        raise ShapeMismatch(f"{who}: complex input is a real tensor whose last dimension is 2 (re, im), got shape {list(x.shape)}")
    return torch.view_as_complex(x.contiguous())


def _r(z: torch.Tensor) -> torch.Tensor:
    return torch.view_as_real(z.resolve_conj())


def fft(x, n: Optional[int] = None): return _r(torch.fft.fft(_c(x, "fft"), n))                                    # noqa: E704
def ifft(x, n: Optional[int] = None): return _r(torch.fft.ifft(_c(x, "ifft"), n))                                 # noqa: E704
def rfft(x, n: Optional[int] = None): return _r(torch.fft.rfft(x, n))                                             # noqa: E704
def irfft(x, n: Optional[int] = None): return torch.fft.irfft(_c(x, "irfft"), n)                                  # noqa: E704
def fft2(x): return _r(torch.fft.fft2(_c(x, "fft2")))                                                             # noqa: E704
def ifft2(x): return _r(torch.fft.ifft2(_c(x, "ifft2")))                                                          # noqa: E704
def fftn(x, dims: Optional[Sequence[int]] = None): return _r(torch.fft.fftn(_c(x, "fftn"), dim=dims))             # noqa: E704
def ifftn(x, dims: Optional[Sequence[int]] = None): return _r(torch.fft.ifftn(_c(x, "ifftn"), dim=dims))          # noqa: E704
def rfftn(x, dims: Optional[Sequence[int]] = None): return _r(torch.fft.rfftn(x, dim=dims))                       # noqa: E704
def irfftn(x, s: Optional[Sequence[int]] = None, dims: Optional[Sequence[int]] = None): return torch.fft.irfftn(_c(x, "irfftn"), s=s, dim=dims)   # noqa: E704
def hfft(x, n: Optional[int] = None): return torch.fft.hfft(_c(x, "hfft"), n)                                     # noqa: E704
def ihfft(x, n: Optional[int] = None): return _r(torch.fft.ihfft(x, n))                                           # noqa: E704
def fftshift(x, dims: Optional[Sequence[int]] = None): return torch.fft.fftshift(x, dim=dims)                     # noqa: E704
def ifftshift(x, dims: Optional[Sequence[int]] = None): return torch.fft.ifftshift(x, dim=dims)                   # noqa: E704


def fftfreq(n: int, d: float = 1.0, dtype=torch.float32) -> torch.Tensor:
    if n <= 0:
        raise InvalidArgument("fftfreq: n must be > 0")
    return torch.fft.fftfreq(n, d, dtype=dtype)


def rfftfreq(n: int, d: float = 1.0, dtype=torch.float32) -> torch.Tensor:
    if n <= 0:
        raise InvalidArgument("rfftfreq: n must be > 0")
    return torch.fft.rfftfreq(n, d, dtype=dtype)


fft_differentiable, ifft_differentiable, rfft_differentiable, irfft_differentiable = fft, ifft, rfft, irfft          # every form here records autograd


# -- forward-mode dual arithmetic (autograd/forward_ad.rs) ----------------------------------------------------------------------------
def _dual(primal, tangent):
    from . import DualTensor
    return DualTensor(primal, tangent)


def dual_add(a, b): return _dual(a.primal + b.primal, a.tangent + b.tangent)                                       # noqa: E704
def dual_sub(a, b): return _dual(a.primal - b.primal, a.tangent - b.tangent)                                       # noqa: E704
def dual_mul(a, b): return _dual(a.primal * b.primal, a.tangent * b.primal + a.primal * b.tangent)                 # noqa: E704
def dual_div(a, b): return _dual(a.primal / b.primal, (a.tangent * b.primal - a.primal * b.tangent) / (b.primal * b.primal))   # noqa: E704
def dual_neg(a): return _dual(-a.primal, -a.tangent)                                                               # noqa: E704
def dual_matmul(a, b): return _dual(a.primal @ b.primal, a.tangent @ b.primal + a.primal @ b.tangent)              # noqa: E704


# -- backward with an explicit seed (autograd/graph.rs:30) -------------------------------------------------------------------------------
def backward_with_grad(root: torch.Tensor, gradient: Optional[torch.Tensor] = None) -> None:
    from ..errors import BackwardNonScalar, NoGradFn
    if gradient is None:
        if root.numel() != 1:
            raise BackwardNonScalar(root.shape)
    elif gradient.shape != root.shape:
        raise ShapeMismatch(f"gradient shape {list(gradient.shape)} does not match root shape {list(root.shape)}")
    if not root.requires_grad:
        raise NoGradFn("backward: the root does not require grad")
    root.backward(gradient)


# -- anomaly mode (autograd/anomaly.rs) ---------------------------------------------------------------------------------------------
_anomaly = threading.local()


class AnomalyMode:
    """Per-thread switch: while on, forward operations may record where they were called (:class:`ForwardBacktrace`) and gradients are
    checked for NaN / Inf by :func:`check_gradient_anomaly`. ``AnomalyMode.guard()`` is the scoped form."""

    @staticmethod
    def enable() -> None:
        _anomaly.on = True
        torch.autograd.set_detect_anomaly(True)

    @staticmethod
    def disable() -> None:
        _anomaly.on = False
        torch.autograd.set_detect_anomaly(False)

    @staticmethod
    def is_enabled() -> bool:
        return getattr(_anomaly, "on", False)

    class guard:  # noqa: N801
        def __enter__(self):
            self.prev = AnomalyMode.is_enabled()
            AnomalyMode.enable()
            return self

        def __exit__(self, *exc):
            AnomalyMode.enable() if self.prev else AnomalyMode.disable()
            return False


class ForwardBacktrace:
    """Where a forward operation ran, captured only while anomaly mode is on (anomaly.rs:86)."""

    def __init__(self, trace: str):
        self.trace = trace

    @classmethod
    def capture_if_enabled(cls) -> Optional["ForwardBacktrace"]:
        if not AnomalyMode.is_enabled():
            return None
        return cls("".join(traceback.format_stack()[:-1]))

    def __str__(self):
        return "forward pass backtrace:\n" + self.trace


def check_gradient_anomaly(grad: torch.Tensor, op_name: str, forward_bt: Optional[ForwardBacktrace] = None) -> None:
    """Raises when anomaly mode is on and ``grad`` holds NaN or Inf, naming the operation and where its forward ran (anomaly.rs:131)."""
    if not AnomalyMode.is_enabled() or not grad.is_floating_point():
        return
    has_nan, has_inf = bool(torch.isnan(grad).any()), bool(torch.isinf(grad).any())
    if has_nan or has_inf:
        kind = "NaN and Inf" if has_nan and has_inf else ("NaN" if has_nan else "Inf")
        bt = f"\n\n{forward_bt}" if forward_bt is not None else "\n\n(no forward backtrace available — was anomaly mode enabled during forward pass?)"
        raise InvalidArgument(f"anomaly detected: {kind} in gradient of {op_name}{bt}")


# -- autocast: dtype, guard, debug log (autograd/autocast.rs, autocast_ops.rs:73) ---------------------------------------------------
class AutocastDtype(enum.Enum):
    F16 = "f16"
    BF16 = "bf16"

    def torch_dtype(self) -> torch.dtype:
        return torch.float16 if self is AutocastDtype.F16 else torch.bfloat16


_autocast_debug = threading.local()


def set_autocast_debug(enabled: bool) -> None:
    _autocast_debug.on = bool(enabled)


def is_autocast_debug() -> bool:
    return getattr(_autocast_debug, "on", False)


def autocast_dtype() -> AutocastDtype:
    """The reduced dtype of the active autocast region (``BF16`` outside one, the default of :func:`autocast`)."""
    for dev in ("cuda", "cpu"):
        if torch.is_autocast_enabled(dev):
            return AutocastDtype.F16 if torch.get_autocast_dtype(dev) == torch.float16 else AutocastDtype.BF16
    return AutocastDtype.BF16


def autocast_guard(op_name: str):
    """``None`` outside an autocast region; inside one, the policy category of ``op_name`` — recorded in the event log when autocast
    debugging is on (autocast_ops.rs:73)."""
    from . import _autocast_log, autocast_category, is_autocast_enabled
    if not is_autocast_enabled():
        return None
    cat = autocast_category(op_name)
    if is_autocast_debug():
        _autocast_log.append((op_name, cat.value))
    return cat


# -- dispatch-key sets (dispatch.rs:137) ------------------------------------------------------------------------------------------
class DispatchKeySet:
    """Immutable bit set of :class:`DispatchKey`; ``highest()`` is the key a dispatcher serves first."""
    __slots__ = ("bits",)

    def __init__(self, bits: int = 0):
        object.__setattr__(self, "bits", int(bits))

    def __setattr__(self, *a):
        raise AttributeError("DispatchKeySet is immutable")

    @classmethod
    def empty(cls): return cls(0)                                                                                  # noqa: E704
    @classmethod
    def all(cls):                                                                                                  # noqa: A003
        from . import DispatchKey
        return cls(sum(1 << int(k) for k in DispatchKey))

    @classmethod
    def from_keys(cls, keys): return cls(sum({1 << int(k) for k in keys}))                                         # noqa: E704
    def contains(self, key) -> bool: return bool(self.bits >> int(key) & 1)                                        # noqa: E704
    def insert(self, key): return DispatchKeySet(self.bits | 1 << int(key))                                        # noqa: E704
    def remove(self, key): return DispatchKeySet(self.bits & ~(1 << int(key)))                                     # noqa: E704
    def union(self, other): return DispatchKeySet(self.bits | other.bits)                                          # noqa: E704
    def intersection(self, other): return DispatchKeySet(self.bits & other.bits)                                   # noqa: E704
    def is_empty(self) -> bool: return self.bits == 0                                                              # noqa: E704
    def __len__(self): return bin(self.bits).count("1")                                                            # noqa: E704
    def __eq__(self, o): return isinstance(o, DispatchKeySet) and o.bits == self.bits                              # noqa: E704
    def __hash__(self): return hash(self.bits)                                                                     # noqa: E704

    def keys(self):
        from . import DispatchKey
        return [k for k in sorted(DispatchKey, reverse=True) if self.contains(k)]

    def highest(self):
        ks = self.keys()
        return ks[0] if ks else None

    def __repr__(self):
        return "DispatchKeySet{" + ", ".join(k.name for k in self.keys()) + "}"


Kernel = Callable[..., torch.Tensor]                           # (inputs, key set, dispatcher) -> tensor: what a dispatcher table holds (dispatch.rs:287)


# -- identities and storage handles (tensor.rs:33, storage.rs:63) ------------------------------------------------------------------------
_ids = itertools.count(1)
_id_lock = threading.Lock()


@dataclass(frozen=True, order=True)
class TensorId:
    """Process-unique, monotonically increasing id; ``TensorId.of(t)`` gives the same id for every alias of one tensor object."""
    value: int

    @classmethod
    def next(cls) -> "TensorId":  # noqa: A003
        with _id_lock:
            return cls(next(_ids))

    @classmethod
    def of(cls, t: torch.Tensor) -> "TensorId":
        tid = getattr(t, "_ft_id", None)
        if tid is None:
            tid = cls.next()
            t._ft_id = tid
        return tid


class StorageBuffer(enum.Enum):
    """Where a tensor's bytes live (storage.rs:63). ``Cubecl`` (the reference's portable-GPU handle) has no counterpart here."""
    Cpu = "cpu"
    Gpu = "gpu"
    Meta = "meta"

    @classmethod
    def of(cls, t: torch.Tensor) -> "StorageBuffer":
        return cls.Gpu if t.is_cuda else (cls.Meta if t.is_meta else cls.Cpu)


class TensorStorage:
    """View of a tensor's allocation: device kind, byte size, base pointer, and whether two tensors share it."""

    def __init__(self, t: torch.Tensor):
        self._t = t

    @classmethod
    def cpu(cls, data: Sequence[float], dtype=torch.float32) -> "TensorStorage":
        return cls(torch.tensor(list(data), dtype=dtype))

    def buffer(self) -> StorageBuffer:
        return StorageBuffer.of(self._t)

    def is_cpu(self) -> bool:
        return self._t.device.type == "cpu"

    def is_gpu(self) -> bool:
        return self._t.is_cuda

    def len(self) -> int:  # noqa: A003
        st = self._t.untyped_storage()
        return st.nbytes() // max(self._t.element_size(), 1)

    def nbytes(self) -> int:
        return self._t.untyped_storage().nbytes()

    def data_ptr(self) -> int:
        return self._t.untyped_storage().data_ptr()

    def shares_with(self, other: "TensorStorage") -> bool:
        return not self._t.is_meta and self.data_ptr() == other.data_ptr() and self.data_ptr() != 0

    def tensor(self) -> torch.Tensor:
        return self._t


GradFn = torch.autograd.graph.Node                            # a node of the recorded backward graph (``tensor.grad_fn``)


class EinopsReduction(enum.Enum):
    """Reductions of the einops-style ``reduce`` (einops.rs:33)."""
    Sum = "sum"
    Mean = "mean"
    Max = "max"
    Min = "min"
    Prod = "prod"


def validate_cond_branches(true_outputs: Sequence[torch.Tensor], false_outputs: Sequence[torch.Tensor]) -> None:
    """Both branches of a ``cond`` must return the same number of tensors with pairwise equal shapes and dtypes (ops/higher_order.rs:142)."""
    if len(true_outputs) != len(false_outputs):
        raise InvalidArgument(f"cond: true branch returns {len(true_outputs)} tensors but false branch returns {len(false_outputs)}")
    for i, (a, b) in enumerate(zip(true_outputs, false_outputs)):
        if a.shape != b.shape:
            raise ShapeMismatch(f"cond: output {i} has shape {list(a.shape)} in the true branch and {list(b.shape)} in the false branch")
        if a.dtype != b.dtype:
            raise InvalidArgument(f"cond: output {i} has dtype {a.dtype} in the true branch and {b.dtype} in the false branch")


class AsStridedBackward(torch.autograd.Function):
    """``as_strided`` as an explicit autograd node (stride_tricks.rs): the gradient of the strided view is accumulated back into a zero tensor
    of the base's shape at the positions the view read, so overlapping windows add up."""

    @staticmethod
    def forward(ctx, base, size, stride, storage_offset=0):
        ctx.meta = (base.shape, base.stride(), base.storage_offset(), tuple(size), tuple(stride), storage_offset, base.dtype, base.device)
        return base.detach().as_strided(size, stride, storage_offset).clone()

    @staticmethod
    def backward(ctx, grad):
        shape, bstride, boff, size, stride, off, dtype, device = ctx.meta
        n = 1
        for d in shape:
            n *= d
        span = boff + sum((s - 1) * st for s, st in zip(shape, bstride)) + 1 if n else 0
        flat = torch.zeros(max(span, off + sum((s - 1) * st for s, st in zip(size, stride)) + 1), dtype=dtype, device=device)
        idx = torch.full((), off, dtype=torch.long, device=device)
        for s, st in zip(size, stride):
            idx = idx.unsqueeze(-1) + torch.arange(s, device=device) * st
        flat.index_add_(0, idx.reshape(-1), grad.reshape(-1))
        return flat.as_strided(shape, bstride, boff).clone(), None, None, None


class Observer(abc.ABC):
    """Interface of the range observers used for quantisation: ``observe(tensor)`` accumulates statistics, ``qparams(...)`` turns them into
    scale / zero point (quantize.rs). :class:`MinMaxObserver`, :class:`PerChannelMinMaxObserver` and :class:`HistogramObserver` implement it."""

    def observe(self, t: torch.Tensor) -> None:
        raise NotImplementedError

    def qparams(self, *a, **k):
        raise NotImplementedError

    @classmethod
    def __subclasshook__(cls, c):
        return all(callable(getattr(c, m, None)) for m in ("observe", "qparams")) if cls is Observer else NotImplemented


class _CallableNamespace:
    """A namespace (``core.fft.fft2``) that is also the function of the same name (``core.fft(x)``), as module and function share a name in
    the reference."""

    def __init__(self, ns, fn):
        self.__dict__.update({k: v for k, v in vars(ns).items() if not k.startswith("__")})
        self._fn, self.__doc__, self.__name__ = fn, fn.__doc__, getattr(ns, "__name__", "namespace")

    def __call__(self, *a, **k):
        return self._fn(*a, **k)


_NN_NAMES = {"FakeQuantize", "QatModel", "prepare_qat", "flex_attention", "gelu", "gelu_with", "GeluApproximate", "HookHandle"}


def nn_name(name: str):
    """Names the reference keeps in the core crate but that live with the layers here."""
    from .. import nn
    if name == "QatLayer":
        return nn.FakeQuantize
    if name == "fake_quantize_differentiable":
        return _fake_quantize_differentiable
    return getattr(nn, name)


def _fake_quantize_differentiable(x: torch.Tensor, scale: float, zero_point: int, qmin: int, qmax: int) -> torch.Tensor:
    """Quantise-dequantise with a straight-through gradient: inside the representable range the gradient passes unchanged, outside it is zero
    (quantize.rs)."""
    q = torch.clamp(torch.round(x / scale) + zero_point, qmin, qmax)
    y = (q - zero_point) * scale
    inside = ((x / scale + zero_point) >= qmin) & ((x / scale + zero_point) <= qmax)
    return x * inside + (y - x * inside).detach()


# -- meta-device shape propagation (meta_propagate.rs:36-230): ``None`` means "not meta, run the real kernel" -------------------------------
def _meta(shape, dtype) -> torch.Tensor:
    return torch.empty(tuple(shape), dtype=dtype, device="meta")


def full_meta(shape: Sequence[int], value=0.0, dtype=torch.float32) -> torch.Tensor:
    """A meta tensor of ``shape``: carries shape and dtype, no storage (the fill value is irrelevant by construction)."""
    return _meta(shape, dtype)


def meta_like(other: torch.Tensor) -> torch.Tensor:
    return _meta(other.shape, other.dtype)


def _both_meta(a: torch.Tensor, b: torch.Tensor) -> Optional[bool]:
    if a.is_meta != b.is_meta:
        from ..errors import DeviceMismatch
        raise DeviceMismatch(a.device, b.device)
    return a.is_meta


def meta_unary_same_shape(x: torch.Tensor) -> Optional[torch.Tensor]:
    return meta_like(x) if x.is_meta else None


def meta_binary_broadcast(a: torch.Tensor, b: torch.Tensor) -> Optional[torch.Tensor]:
    return _meta(broadcast_shapes(a.shape, b.shape), torch.result_type(a, b)) if _both_meta(a, b) else None


def meta_reduce_dim(x: torch.Tensor, dim: int, keepdim: bool = False) -> Optional[torch.Tensor]:
    if not x.is_meta:
        return None
    d = normalize_axis(dim, x.dim())
    shape = [1 if k == d else s for k, s in enumerate(x.shape)] if keepdim else [s for k, s in enumerate(x.shape) if k != d]
    return _meta(shape, x.dtype)


def meta_reduce_all(x: torch.Tensor) -> Optional[torch.Tensor]:
    return _meta((), x.dtype) if x.is_meta else None


def meta_matmul(a: torch.Tensor, b: torch.Tensor) -> Optional[torch.Tensor]:
    if not _both_meta(a, b):
        return None
    sa, sb = tuple(a.shape), tuple(b.shape)
    if not sa or not sb:
        raise InvalidArgument(f"meta_propagate::matmul: scalar operands not supported, got {list(sa)} and {list(sb)}")
    ka, kb = sa[-1], (sb[0] if len(sb) == 1 else sb[-2])
    if ka != kb:
        raise ShapeMismatch(f"meta_propagate::matmul: inner dimensions differ ({ka} vs {kb}) for {list(sa)} @ {list(sb)}")
    if len(sa) == 1 and len(sb) == 1:
        out: Tuple[int, ...] = ()
    elif len(sb) == 1:
        out = sa[:-1]
    elif len(sa) == 1:
        out = sb[:-2] + sb[-1:]
    else:
        out = broadcast_shapes(sa[:-2], sb[:-2]) + (sa[-2], sb[-1])
    return _meta(out, torch.result_type(a, b))
