"""Further core pieces: control-flow higher-order ops (``cond`` / ``scan``), search and sorting ops, boolean / integer tensor wrappers, the host
buffer pool, meta (shape-only) propagation, tensor display and the elementwise-fusion context.

Reference parity: ferrotorch-core/src/ops/higher_order.rs (cond / scan), ops/search.rs, bool_tensor.rs, int_tensor.rs, cpu_pool.rs,
meta_propagate.rs, display.rs, and the ``with_fusion`` thread-local of ferrotorch-jit/src/fusion.rs.
"""
from __future__ import annotations

import contextlib
import threading
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..errors import InvalidArgument, ShapeMismatch


# ---- control flow ------------------------------------------------------------------------------------------------------------------------
def cond(pred, true_fn: Callable, false_fn: Callable, operands: Sequence[torch.Tensor] = ()):
    """Evaluates exactly one branch (autograd flows through the branch taken). ``pred`` is a Python bool or a one-element tensor."""
    p = bool(pred.item()) if isinstance(pred, torch.Tensor) else bool(pred)
    return true_fn(*operands) if p else false_fn(*operands)


def scan(fn: Callable[[Any, torch.Tensor], Tuple[Any, torch.Tensor]], init, xs: torch.Tensor, reverse: bool = False):
    """``carry, y_t = fn(carry, x_t)`` over the leading dimension of ``xs``; returns ``(final_carry, stacked ys)``; differentiable."""
    carry, ys = init, []
    it = range(xs.shape[0] - 1, -1, -1) if reverse else range(xs.shape[0])
    for t in it:
        carry, y = fn(carry, xs[t])
        ys.append(y)
    if reverse:
        ys.reverse()
    return carry, (torch.stack(ys) if ys else xs.new_zeros((0,)))


# ---- creation ------------------------------------------------------------------------------------------------------------------------------
def empty(*shape, dtype=torch.float32, device=None):
    return torch.empty(*shape, dtype=dtype, device=device)


def tensor(data, dtype=None, device=None, requires_grad: bool = False):
    return torch.tensor(data, dtype=dtype, device=device, requires_grad=requires_grad)


def from_vec(data: Sequence[float], shape: Sequence[int], dtype=torch.float32, device=None):
    n = 1
    for s in shape:
        n *= s
    if len(data) != n:
        raise ShapeMismatch(f"{len(data)} values for shape {tuple(shape)}")
    return torch.tensor(list(data), dtype=dtype, device=device).reshape(tuple(shape))


# ---- search / sort -------------------------------------------------------------------------------------------------------------------------
def searchsorted(sorted_seq, values, right: bool = False): return torch.searchsorted(sorted_seq, values, right=right)   # noqa: E704
def bucketize(values, boundaries, right: bool = False): return torch.bucketize(values, boundaries, right=right)          # noqa: E704
def topk(x, k: int, dim: int = -1, largest: bool = True): return torch.topk(x, k, dim, largest)                         # noqa: E704
def sort(x, dim: int = -1, descending: bool = False, stable: bool = True): return torch.sort(x, dim=dim, descending=descending, stable=stable)  # noqa: E704
def argsort(x, dim: int = -1, descending: bool = False): return torch.argsort(x, dim, descending)                       # noqa: E704
def unique(x, return_inverse: bool = False, return_counts: bool = False): return torch.unique(x, return_inverse=return_inverse, return_counts=return_counts)  # noqa: E704
def histc(x, bins: int = 100, min: float = 0.0, max: float = 0.0): return torch.histc(x, bins, min=min, max=max)        # noqa: E704,A002
def nonzero(x): return torch.nonzero(x)                                                                                 # noqa: E704
def where(c, a, b): return torch.where(c, a, b)                                                                         # noqa: E704
def cumsum(x, dim): return torch.cumsum(x, dim)                                                                         # noqa: E704


# ---- bool / int tensors --------------------------------------------------------------------------------------------------------------------
class BoolTensor:
    """Boolean mask tensor with the logical op set (and / or / xor / not / any / all / count)."""

    def __init__(self, data):
        self.data = torch.as_tensor(data).bool()

    @property
    def shape(self): return tuple(self.data.shape)
    def __and__(self, o): return BoolTensor(self.data & o.data)
    def __or__(self, o): return BoolTensor(self.data | o.data)
    def __xor__(self, o): return BoolTensor(self.data ^ o.data)
    def __invert__(self): return BoolTensor(~self.data)
    def any(self) -> bool: return bool(self.data.any())                 # noqa: A003
    def all(self) -> bool: return bool(self.data.all())                 # noqa: A003
    def count(self) -> int: return int(self.data.sum())
    def to_float(self, dtype=torch.float32): return self.data.to(dtype)
    def select(self, t: torch.Tensor) -> torch.Tensor: return t[self.data]


class IntTensor:
    """Integer (index) tensor with checked conversion and the arithmetic indices need."""

    def __init__(self, data, dtype=torch.int64):
        t = torch.as_tensor(data)
        if t.is_floating_point() and not torch.equal(t, t.round()):
            raise InvalidArgument("IntTensor from non-integral values")
        self.data = t.to(dtype)

    @property
    def shape(self): return tuple(self.data.shape)
    def __add__(self, o): return IntTensor(self.data + (o.data if isinstance(o, IntTensor) else o), self.data.dtype)
    def __sub__(self, o): return IntTensor(self.data - (o.data if isinstance(o, IntTensor) else o), self.data.dtype)
    def __mul__(self, o): return IntTensor(self.data * (o.data if isinstance(o, IntTensor) else o), self.data.dtype)
    def __floordiv__(self, o): return IntTensor(torch.div(self.data, o.data if isinstance(o, IntTensor) else o, rounding_mode="floor"), self.data.dtype)
    def __mod__(self, o): return IntTensor(self.data % (o.data if isinstance(o, IntTensor) else o), self.data.dtype)
    def __eq__(self, o): return BoolTensor(self.data == (o.data if isinstance(o, IntTensor) else o))     # noqa: A003
    def __lt__(self, o): return BoolTensor(self.data < (o.data if isinstance(o, IntTensor) else o))
    def to_float(self, dtype=torch.float32): return self.data.to(dtype)
    def gather_from(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor: return t.index_select(dim, self.data.reshape(-1))


# ---- host buffer pool ------------------------------------------------------------------------------------------------------------------------
class CpuBufferPool:
    """Size-bucketed cache of host tensors (optionally pinned) so hot loops (loader collation, gradient staging) stop hitting the allocator."""

    def __init__(self, pinned: bool = False, max_cached_bytes: int = 1 << 30):
        self.pinned, self.max_cached = pinned and torch.cuda.is_available(), max_cached_bytes
        self._free: Dict[Tuple[torch.dtype, int], List[torch.Tensor]] = {}
        self._lock = threading.Lock()
        self.hits = self.misses = self.cached_bytes = 0

    @staticmethod
    def _bucket(n: int) -> int:
        return 1 if n <= 1 else 1 << (n - 1).bit_length()

    def take(self, numel: int, dtype=torch.float32) -> torch.Tensor:
        b = self._bucket(numel)
        with self._lock:
            lst = self._free.get((dtype, b))
            if lst:
                self.hits += 1
                t = lst.pop()
                self.cached_bytes -= t.numel() * t.element_size()
                return t[:numel]
            self.misses += 1
        return torch.empty(b, dtype=dtype, pin_memory=self.pinned)[:numel]

    def give(self, t: torch.Tensor) -> None:
        base = t._base if t._base is not None else t
        nbytes = base.numel() * base.element_size()
        with self._lock:
            if self.cached_bytes + nbytes > self.max_cached:
                return
            self._free.setdefault((base.dtype, base.numel()), []).append(base)
            self.cached_bytes += nbytes

    def stats(self) -> Dict[str, int]:
        return {"hits": self.hits, "misses": self.misses, "cached_bytes": self.cached_bytes}


cpu_pool = CpuBufferPool()


# ---- meta propagation ------------------------------------------------------------------------------------------------------------------------
def meta_propagate(fn: Callable, *shapes_dtypes: Tuple[Sequence[int], torch.dtype]) -> List[Tuple[Tuple[int, ...], torch.dtype]]:
    """Runs ``fn`` on meta tensors (no storage, no compute) and returns the output shapes and dtypes."""
    args = [torch.empty(tuple(s), dtype=d, device="meta") for s, d in shapes_dtypes]
    out = fn(*args)
    outs = out if isinstance(out, (tuple, list)) else [out]
    for o in outs:
        if not isinstance(o, torch.Tensor) or o.device.type != "meta":
            raise InvalidArgument("meta propagation needs a function of tensors built only from tensor ops")
    return [(tuple(o.shape), o.dtype) for o in outs]


# ---- display -------------------------------------------------------------------------------------------------------------------------------
def format_tensor(t: torch.Tensor, precision: int = 4, edge_items: int = 3, max_elements: int = 1000) -> str:
    """``tensor([...], shape=..., dtype=..., device=...)`` with summarisation of long dimensions; never moves more than the printed values."""
    def fmt(x) -> str:
        if isinstance(x, bool):
            return "true" if x else "false"
        if isinstance(x, int):
            return str(x)
        return f"{x:.{precision}f}"

    def rec(v: torch.Tensor) -> str:
        if v.dim() == 0:
            return fmt(v.item())
        n = v.shape[0]
        if v.numel() > max_elements and n > 2 * edge_items:
            parts = [rec(v[i]) for i in range(edge_items)] + ["..."] + [rec(v[i]) for i in range(n - edge_items, n)]
        else:
            parts = [rec(v[i]) for i in range(n)]
        return "[" + ", ".join(parts) + "]"
    body = "<meta>" if t.device.type == "meta" else rec(t.detach().cpu() if t.numel() <= max_elements else t.detach()[tuple(slice(None) for _ in range(t.dim()))].cpu())
    extra = f", grad_fn={type(t.grad_fn).__name__}" if t.grad_fn is not None else (", requires_grad=true" if t.requires_grad else "")
    return f"tensor({body}, shape={list(t.shape)}, dtype={str(t.dtype).replace('torch.', '')}, device={t.device}{extra})"


display = format_tensor


# ---- fusion context --------------------------------------------------------------------------------------------------------------------------
_fusion = threading.local()


def fusion_enabled() -> bool:
    return getattr(_fusion, "on", False)


@contextlib.contextmanager
def with_fusion(enabled: bool = True):
    """Inside the block, :func:`fused` callables run through the tracing JIT (elementwise regions become one generated kernel)."""
    prev = fusion_enabled()
    _fusion.on = enabled
    try:
        yield
    finally:
        _fusion.on = prev


def fused(fn: Callable) -> Callable:
    """Decorator: under ``with_fusion()`` the function is compiled on first use per input signature; otherwise it runs eagerly."""
    compiled = {}

    def run(*args):
        if not fusion_enabled() or not all(isinstance(a, torch.Tensor) for a in args):
            return fn(*args)
        if "cf" not in compiled:
            from ..jit import compile as jit_compile
            compiled["cf"] = jit_compile(fn)
        return compiled["cf"](*args)
    run.__wrapped__ = fn
    return run
