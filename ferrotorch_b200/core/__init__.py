"""Core runtime surface: devices, dtypes, tensor creation, grad modes, autograd utilities and functional transforms.

The tensor type is ``torch.Tensor`` (PyTorch is the host substrate); this package provides the reference's names on top of it:
``Device``, creation functions, ``no_grad/enable_grad/inference_mode``, ``backward``, tensor hooks, ``autocast`` with the
reference's policy table, activation checkpointing, anomaly mode, saved-tensor hooks, ``gradcheck``, higher-order
transforms (``grad``, ``jacobian``, ``hessian``, ``jvp``, ``vjp``, ``jacfwd``, forward-mode duals), ``vmap`` family, fixed-point
implicit differentiation, the dispatcher keys, and the op profiler hook.

Reference parity: ferrotorch-core/src/{device.rs, dtype.rs, tensor.rs, creation.rs, autograd/*.rs, vmap.rs, dispatch.rs,
profiler_hook.rs, error.rs}.
"""
from __future__ import annotations

import contextlib
import enum
import threading
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from ..errors import (BackwardNonScalar, DeviceMismatch, DeviceUnavailable, InvalidArgument, NoGradFn, ShapeMismatch,
                      NotImplementedOnCuda, FerrotorchError)

Tensor = torch.Tensor


# ----------------------------------------------------------------------------------------------------------------------
# Device / dtype
# ----------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Device:
    """``Cpu | Cuda(i) | Xpu(i) | Mps(i) | Meta`` with the ``"cuda:0"`` display form."""
    kind: str = "cpu"
    index: int = 0

    @staticmethod
    def Cpu():
        return Device("cpu")

    @staticmethod
    def Cuda(i: int = 0):
        return Device("cuda", i)

    @staticmethod
    def Xpu(i: int = 0):
        return Device("xpu", i)

    @staticmethod
    def Mps(i: int = 0):
        return Device("mps", i)

    @staticmethod
    def Meta():
        return Device("meta")

    def is_cuda(self) -> bool:
        return self.kind == "cuda"

    def is_cpu(self) -> bool:
        return self.kind == "cpu"

    def __str__(self):
        return self.kind if self.kind in ("cpu", "meta") else f"{self.kind}:{self.index}"

    def torch(self) -> torch.device:
        if self.kind in ("xpu", "mps"):
            # Intel XPU (wgpu/Vulkan) and Apple MPS (Metal) back ends need a graphics stack; these machines are CUDA-compute only.
            raise DeviceUnavailable(f"{self} is unavailable on this platform (no Vulkan/Metal stack); use cuda or cpu")
        return torch.device(str(self))

    @staticmethod
    def of(t: torch.Tensor) -> "Device":
        return Device(t.device.type, t.device.index or 0)


class DType(enum.Enum):
    F32 = torch.float32
    F64 = torch.float64
    BF16 = torch.bfloat16
    F16 = torch.float16
    I64 = torch.int64
    I32 = torch.int32
    U8 = torch.uint8
    Bool = torch.bool


class MemoryFormat(enum.Enum):
    Contiguous = torch.contiguous_format
    ChannelsLast = torch.channels_last
    ChannelsLast3d = torch.channels_last_3d


def _dev(device) -> torch.device:
    if isinstance(device, Device):
        return device.torch()
    return torch.device(device if device is not None else "cpu")


# creation (ferrotorch-core/src/creation.rs:7-309)
def zeros(*shape, dtype=torch.float32, device=None, requires_grad=False):
    return torch.zeros(*shape, dtype=dtype, device=_dev(device), requires_grad=requires_grad)


def ones(*shape, dtype=torch.float32, device=None, requires_grad=False):
    return torch.ones(*shape, dtype=dtype, device=_dev(device), requires_grad=requires_grad)


def full(shape, value, dtype=torch.float32, device=None):
    return torch.full(tuple(shape), value, dtype=dtype, device=_dev(device))


def _host_philox(kind: str, shape, generator):
    """Large f32 host tensors are filled by the native threaded Philox4x32-10 (the stream of the device kernels). The key of a call is one
    64-bit draw from the torch generator in charge, so ``torch.manual_seed`` / an explicit generator still makes the values reproducible."""
    import ctypes
    from .. import _lib
    if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
        shape = tuple(shape[0])
    out = torch.empty(*shape, dtype=torch.float32)
    seed = int(torch.empty((), dtype=torch.int64).random_(generator=generator)) & 0xFFFFFFFFFFFFFFFF
    fn = _lib.runtime().ft_philox_uniform_mt if kind == "uniform" else _lib.runtime().ft_philox_normal_mt
    fn(ctypes.c_uint64(seed), ctypes.c_uint64(0), ctypes.c_int64(out.numel()), ctypes.c_void_p(out.data_ptr()), ctypes.c_int(torch.get_num_threads()))
    return out


def _host_philox_ok(shape, dtype, device, generator) -> bool:
    if dtype != torch.float32 or _dev(device).type != "cpu" or (generator is not None and generator.device.type != "cpu"):
        return False
    dims = shape[0] if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)) else shape
    n = 1
    for d in dims:
        n *= int(d)
    return n >= (1 << 16)


def rand(*shape, dtype=torch.float32, device=None, generator=None):
    if _host_philox_ok(shape, dtype, device, generator):
        return _host_philox("uniform", shape, generator)
    return torch.rand(*shape, dtype=dtype, device=_dev(device), generator=generator)


def randn(*shape, dtype=torch.float32, device=None, generator=None):
    if _host_philox_ok(shape, dtype, device, generator):
        return _host_philox("normal", shape, generator)
    return torch.randn(*shape, dtype=dtype, device=_dev(device), generator=generator)


def arange(*a, dtype=None, device=None):
    return torch.arange(*a, dtype=dtype, device=_dev(device))


def linspace(start, end, steps, dtype=torch.float32, device=None):
    return torch.linspace(start, end, steps, dtype=dtype, device=_dev(device))


def eye(n, m=None, dtype=torch.float32, device=None):
    return torch.eye(n, m if m is not None else n, dtype=dtype, device=_dev(device))


def from_slice(data: Sequence, shape: Sequence[int], dtype=torch.float32, device=None):
    t = torch.tensor(list(data), dtype=dtype, device=_dev(device))
    if t.numel() != int(torch.tensor(list(shape)).prod()) if len(shape) else t.numel() != 1:
        raise ShapeMismatch(f"{t.numel()} elements do not fill shape {list(shape)}")
    return t.reshape(tuple(shape))


def scalar(v, dtype=torch.float32, device=None):
    return torch.tensor(v, dtype=dtype, device=_dev(device))


zeros_like, ones_like, full_like, rand_like, randn_like, empty_like = (torch.zeros_like, torch.ones_like, torch.full_like, torch.rand_like,
                                                                       torch.randn_like, torch.empty_like)


def zeros_meta(*shape, dtype=torch.float32):
    """Shape-only tensor for dry runs (no storage)."""
    return torch.zeros(*shape, dtype=dtype, device="meta")


ones_meta = lambda *shape, dtype=torch.float32: torch.ones(*shape, dtype=dtype, device="meta")  # noqa: E731


def to_pinned(t: torch.Tensor) -> torch.Tensor:
    return t.pin_memory() if torch.cuda.is_available() else t


# ----------------------------------------------------------------------------------------------------------------------
# grad modes, backward, hooks
# ----------------------------------------------------------------------------------------------------------------------
no_grad = torch.no_grad
enable_grad = torch.enable_grad
inference_mode = torch.inference_mode
set_grad_enabled = torch.set_grad_enabled
is_grad_enabled = torch.is_grad_enabled


def backward(t: torch.Tensor, gradient: Optional[torch.Tensor] = None, retain_graph: bool = False, create_graph: bool = False) -> None:
    """``t.backward()`` with the reference's error cases: a non-scalar root needs an explicit gradient; a root without history is an error."""
    if t.grad_fn is None and not t.requires_grad:
        raise NoGradFn("tensor has no grad_fn and does not require grad")
    if gradient is None and t.numel() != 1:
        raise BackwardNonScalar(t.shape)
    t.backward(gradient, retain_graph=retain_graph, create_graph=create_graph)


backward_with_gradient = backward


def backward_parallel(roots: Sequence[torch.Tensor], gradients: Optional[Sequence[Optional[torch.Tensor]]] = None) -> None:
    """Backward from several roots in one engine pass (the engine runs independent branches on its worker threads)."""
    torch.autograd.backward(list(roots), list(gradients) if gradients is not None else None)


def register_hook(t: torch.Tensor, fn: Callable[[torch.Tensor], Optional[torch.Tensor]]):
    """Gradient hook (may return a replacement gradient)."""
    return t.register_hook(fn)


def register_post_accumulate_grad_hook(t: torch.Tensor, fn: Callable[[torch.Tensor], None]):
    """Runs after ``t.grad`` has been accumulated - the hook a DDP/FSDP reducer uses to learn that a gradient is ready."""
    return t.register_post_accumulate_grad_hook(fn)


def detach(t):
    return t.detach()


# ----------------------------------------------------------------------------------------------------------------------
# autocast (policy of ferrotorch-core/src/autograd/autocast_ops.rs:29-45)
# ----------------------------------------------------------------------------------------------------------------------
class AutocastCategory(enum.Enum):
    Reduced = "reduced"       # run in the autocast dtype
    Full = "full"             # run in f32
    Passthrough = "passthrough"


AUTOCAST_POLICY: Dict[str, AutocastCategory] = {
    **{k: AutocastCategory.Reduced for k in ("mm", "matmul", "bmm", "linear", "conv1d", "conv2d", "conv3d", "conv_transpose2d", "addmm", "einsum")},
    **{k: AutocastCategory.Full for k in ("sum", "mean", "prod", "softmax", "log_softmax", "layer_norm", "batch_norm", "group_norm", "rms_norm",
                                          "cross_entropy", "mse_loss", "bce_loss", "bce_with_logits")},
}
_autocast_log: List[Tuple[str, str]] = []


def autocast_category(op: str) -> AutocastCategory:
    return AUTOCAST_POLICY.get(op, AutocastCategory.Passthrough)


def autocast(dtype: torch.dtype = torch.bfloat16, enabled: bool = True, device_type: Optional[str] = None):
    if dtype not in (torch.bfloat16, torch.float16):
        raise InvalidArgument("autocast dtype must be bf16 or f16")
    dt = device_type or ("cuda" if torch.cuda.is_available() else "cpu")
    return torch.autocast(dt, dtype=dtype, enabled=enabled)


def is_autocast_enabled() -> bool:
    return torch.is_autocast_enabled() or torch.is_autocast_enabled("cpu")


def autocast_cast(op: str, *tensors: torch.Tensor, dtype: torch.dtype = torch.bfloat16):
    """Cast the inputs of ``op`` per the policy table; records the decision in the autocast event log."""
    cat = autocast_category(op)
    _autocast_log.append((op, cat.value))
    if cat == AutocastCategory.Reduced:
        return tuple(t.to(dtype) if t.is_floating_point() else t for t in tensors)
    if cat == AutocastCategory.Full:
        return tuple(t.float() if t.is_floating_point() else t for t in tensors)
    return tensors


def autocast_events() -> List[Tuple[str, str]]:
    return list(_autocast_log)


# ----------------------------------------------------------------------------------------------------------------------
# checkpointing, anomaly mode, saved tensor hooks, gradcheck
# ----------------------------------------------------------------------------------------------------------------------
def checkpoint(fn: Callable, *args, preserve_rng_state: bool = True, **kwargs):
    """Recompute ``fn`` during backward instead of keeping its activations; RNG state (CPU and CUDA) is replayed."""
    from torch.utils.checkpoint import checkpoint as _c
    return _c(fn, *args, use_reentrant=False, preserve_rng_state=preserve_rng_state, **kwargs)


detect_anomaly = torch.autograd.detect_anomaly
set_detect_anomaly = torch.autograd.set_detect_anomaly
saved_tensors_hooks = torch.autograd.graph.saved_tensors_hooks
save_on_cpu = torch.autograd.graph.save_on_cpu


def has_inf_nan(t: torch.Tensor) -> bool:
    return not bool(torch.isfinite(t).all())


def gradcheck(fn: Callable, inputs: Sequence[torch.Tensor], eps: float = 1e-6, atol: float = 1e-5, rtol: float = 1e-3) -> bool:
    ins = tuple(i.detach().double().requires_grad_(True) for i in inputs)
    return torch.autograd.gradcheck(fn, ins, eps=eps, atol=atol, rtol=rtol)


# ----------------------------------------------------------------------------------------------------------------------
# functional transforms (higher_order.rs, grad_penalty.rs, forward_ad.rs, fixed_point.rs)
# ----------------------------------------------------------------------------------------------------------------------
def grad(outputs: torch.Tensor, inputs: Sequence[torch.Tensor], grad_outputs=None, create_graph: bool = False, retain_graph: Optional[bool] = None,
         allow_unused: bool = False):
    return torch.autograd.grad(outputs, list(inputs), grad_outputs, retain_graph=retain_graph, create_graph=create_graph, allow_unused=allow_unused)


def jacobian(fn: Callable, x: torch.Tensor, create_graph: bool = False) -> torch.Tensor:
    return torch.autograd.functional.jacobian(fn, x, create_graph=create_graph)


def hessian(fn: Callable, x: torch.Tensor) -> torch.Tensor:
    return torch.autograd.functional.hessian(fn, x)


def vjp(fn: Callable, x: torch.Tensor, v: torch.Tensor):
    return torch.autograd.functional.vjp(fn, x, v)


def jvp(fn: Callable, x: torch.Tensor, v: torch.Tensor):
    """Double-backward JVP (works for any reverse-differentiable ``fn``)."""
    return torch.autograd.functional.jvp(fn, x, v)


def grad_norm(outputs: torch.Tensor, inputs: Sequence[torch.Tensor], p: float = 2.0, create_graph: bool = True) -> torch.Tensor:
    gs = torch.autograd.grad(outputs, list(inputs), create_graph=create_graph)
    return torch.cat([g.reshape(-1) for g in gs]).norm(p)


def gradient_penalty(fn: Callable, x: torch.Tensor, target: float = 1.0) -> torch.Tensor:
    """WGAN-GP style penalty ``(||d fn/dx||_2 - target)^2`` averaged over the batch (differentiable)."""
    x = x.detach().requires_grad_(True)
    y = fn(x)
    (g,) = torch.autograd.grad(y.sum(), x, create_graph=True)
    return ((g.flatten(1).norm(2, dim=1) - target) ** 2).mean()


class DualTensor:
    """Forward-mode dual number ``primal + eps * tangent``."""

    def __init__(self, primal: torch.Tensor, tangent: Optional[torch.Tensor] = None):
        self.primal, self.tangent = primal, tangent if tangent is not None else torch.zeros_like(primal)

    def _bin(self, o, f, df):
        op, ot = (o.primal, o.tangent) if isinstance(o, DualTensor) else (o, 0.0)
        return DualTensor(f(self.primal, op), df(self.primal, self.tangent, op, ot))

    def __add__(self, o):
        return self._bin(o, lambda a, b: a + b, lambda a, da, b, db: da + db)

    __radd__ = __add__

    def __sub__(self, o):
        return self._bin(o, lambda a, b: a - b, lambda a, da, b, db: da - db)

    def __mul__(self, o):
        return self._bin(o, lambda a, b: a * b, lambda a, da, b, db: da * b + a * db)

    __rmul__ = __mul__

    def __truediv__(self, o):
        return self._bin(o, lambda a, b: a / b, lambda a, da, b, db: (da * b - a * db) / (b * b))

    def __matmul__(self, o):
        return self._bin(o, lambda a, b: a @ b, lambda a, da, b, db: da @ b + (a @ db if isinstance(db, torch.Tensor) else 0.0))

    def __neg__(self):
        return DualTensor(-self.primal, -self.tangent)


def dual_exp(d):
    e = d.primal.exp()
    return DualTensor(e, d.tangent * e)


def dual_log(d):
    return DualTensor(d.primal.log(), d.tangent / d.primal)


def dual_sin(d):
    return DualTensor(d.primal.sin(), d.tangent * d.primal.cos())


def dual_cos(d):
    return DualTensor(d.primal.cos(), -d.tangent * d.primal.sin())


def dual_tanh(d):
    t = d.primal.tanh()
    return DualTensor(t, d.tangent * (1 - t * t))


def dual_relu(d):
    return DualTensor(d.primal.relu(), d.tangent * (d.primal > 0))


def dual_sigmoid(d):
    s = d.primal.sigmoid()
    return DualTensor(s, d.tangent * s * (1 - s))


def dual_sum(d, dim=None):
    return DualTensor(d.primal.sum() if dim is None else d.primal.sum(dim), d.tangent.sum() if dim is None else d.tangent.sum(dim))


def jvp_exact(fn: Callable, x: torch.Tensor, v: torch.Tensor):
    """Single-pass forward-mode JVP."""
    import torch.autograd.forward_ad as fwad
    with fwad.dual_level():
        out = fn(fwad.make_dual(x, v))
        p, t = fwad.unpack_dual(out)
    return p, (t if t is not None else torch.zeros_like(p))


def jacfwd(fn: Callable, x: torch.Tensor) -> torch.Tensor:
    cols = []
    flat = x.reshape(-1)
    for i in range(flat.numel()):
        e = torch.zeros_like(flat)
        e[i] = 1
        cols.append(jvp_exact(fn, x, e.view_as(x))[1].reshape(-1))
    return torch.stack(cols, -1).reshape(*fn(x).shape, *x.shape)


def fixed_point(f: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], z0: torch.Tensor, theta: torch.Tensor, tol: float = 1e-6, max_iter: int = 200,
                bwd_iter: int = 200) -> torch.Tensor:
    """Solve ``z = f(z, theta)`` by iteration; the backward pass uses the implicit function theorem (Neumann iteration for
    ``(I - df/dz)^-T g``) instead of unrolling the solver."""

    class _FP(torch.autograd.Function):
        @staticmethod
        def forward(ctx, theta_):
            with torch.no_grad():
                z = z0
                for _ in range(max_iter):
                    zn = f(z, theta_)
                    if (zn - z).norm() <= tol * (1 + z.norm()):
                        z = zn
                        break
                    z = zn
            ctx.save_for_backward(z, theta_)
            return z

        @staticmethod
        def backward(ctx, g):
            z, th = ctx.saved_tensors
            with torch.enable_grad():
                zz = z.detach().requires_grad_(True)
                tt = th.detach().requires_grad_(True)
                fz = f(zz, tt)
                u = g
                for _ in range(bwd_iter):
                    (jt,) = torch.autograd.grad(fz, zz, u, retain_graph=True)
                    un = g + jt
                    if (un - u).norm() <= tol * (1 + u.norm()):
                        u = un
                        break
                    u = un
                (gt,) = torch.autograd.grad(fz, tt, u)
            return gt
    return _FP.apply(theta)


# ----------------------------------------------------------------------------------------------------------------------
# vmap family (vmap.rs:25-519)
# ----------------------------------------------------------------------------------------------------------------------
def select(t: torch.Tensor, dim: int, index: int) -> torch.Tensor:
    return t.select(dim, index)


def stack(ts: Sequence[torch.Tensor], dim: int = 0) -> torch.Tensor:
    return torch.stack(list(ts), dim)


def vmap(fn: Callable, in_dim: int = 0, out_dim: int = 0) -> Callable:
    return torch.vmap(fn, in_dims=in_dim, out_dims=out_dim)


def vmap2(fn: Callable, in_dims=(0, 0), out_dim: int = 0) -> Callable:
    return torch.vmap(fn, in_dims=tuple(in_dims), out_dims=out_dim)


def vmap3(fn: Callable, in_dims=(0, 0, 0), out_dim: int = 0) -> Callable:
    return torch.vmap(fn, in_dims=tuple(in_dims), out_dims=out_dim)


def vmap_many(fn: Callable, in_dims: Sequence[Optional[int]], out_dim: int = 0) -> Callable:
    return torch.vmap(fn, in_dims=tuple(in_dims), out_dims=out_dim)


def vmap_multi_output(fn: Callable, in_dim: int = 0, out_dims: Sequence[int] = (0, 0)) -> Callable:
    return torch.vmap(fn, in_dims=in_dim, out_dims=tuple(out_dims))


def per_sample_grad(model: torch.nn.Module, loss_fn: Callable, x: torch.Tensor, y: torch.Tensor) -> Dict[str, torch.Tensor]:
    """Per-example parameter gradients ``[B, *param.shape]`` via ``vmap(grad(...))`` over a functional call of the model."""
    from torch.func import functional_call, grad as fgrad, vmap as fvmap
    params = {k: v.detach() for k, v in model.named_parameters()}

    def one(p, xi, yi):
        return loss_fn(functional_call(model, p, (xi.unsqueeze(0),)), yi.unsqueeze(0))
    return fvmap(fgrad(one), in_dims=(None, 0, 0))(params, x, y)


# ----------------------------------------------------------------------------------------------------------------------
# dispatcher keys + op profiler hook
# ----------------------------------------------------------------------------------------------------------------------
class DispatchKey(enum.IntEnum):
    Cpu = 0
    Cuda = 1
    Meta = 2
    Sparse = 3
    Quantized = 4
    Nested = 5
    Autocast = 6
    Autograd = 7
    Vmap = 8


class Dispatcher:
    """Key-ordered kernel table with redispatch: the highest-priority key present on the inputs runs first and may call
    ``redispatch`` to fall through to the next (ferrotorch-core/src/dispatch.rs:70-99)."""

    def __init__(self):
        self._table: Dict[Tuple[str, DispatchKey], Callable] = {}

    def register(self, op: str, key: DispatchKey, fn: Callable) -> None:
        self._table[(op, key)] = fn

    @staticmethod
    def keys_of(*tensors: torch.Tensor) -> List[DispatchKey]:
        ks = set()
        for t in tensors:
            if not isinstance(t, torch.Tensor):
                continue
            ks.add(DispatchKey.Cuda if t.is_cuda else (DispatchKey.Meta if t.is_meta else DispatchKey.Cpu))
            if t.is_sparse:
                ks.add(DispatchKey.Sparse)
            if t.is_quantized:
                ks.add(DispatchKey.Quantized)
            if t.is_nested:
                ks.add(DispatchKey.Nested)
            if t.requires_grad and torch.is_grad_enabled():
                ks.add(DispatchKey.Autograd)
        if is_autocast_enabled():
            ks.add(DispatchKey.Autocast)
        return sorted(ks, reverse=True)

    def call(self, op: str, *args, _skip: int = 0, **kw):
        keys = self.keys_of(*args)
        for i, k in enumerate(keys[_skip:], start=_skip):
            fn = self._table.get((op, k))
            if fn is not None:
                return fn(*args, redispatch=lambda *a, **k2: self.call(op, *a, _skip=i + 1, **k2), **kw)
        raise InvalidArgument(f"no kernel registered for {op} with keys {[k.name for k in keys]}")


_prof = threading.local()


class OpProfiler:
    """Interface of the thread-local op hook: ``on_op(name, category, shapes, seconds)``."""

    def on_op(self, name: str, category: str, shapes, seconds: float) -> None:
        raise NotImplementedError


def set_current_profiler(p: Optional[OpProfiler]) -> None:
    _prof.cur = p


def current_profiler() -> Optional[OpProfiler]:
    return getattr(_prof, "cur", None)


def profile_op_scope(name: str, category: str, shapes, fn: Callable):
    """Run ``fn`` and report it to the installed profiler (if any)."""
    p = current_profiler()
    if p is None:
        return fn()
    import time
    t0 = time.perf_counter()
    out = fn()
    p.on_op(name, category, shapes, time.perf_counter() - t0)
    return out


def gpu_backend_available() -> bool:
    return torch.cuda.is_available()

from .tensor_ext import (linalg, fft, special, windows, einsum, einsum_differentiable, rearrange, rearrange_with, repeat, reduce, as_strided,
                         as_strided_copy, as_strided_scatter, magnitude_prune, apply_2_4_mask, sparsity_ratio, QuantScheme, QuantDtype, QParams,
                         QuantizedTensor, quantize, dequantize, quantized_matmul, quantize_named_tensors, MinMaxObserver,
                         PerChannelMinMaxObserver, HistogramObserver, CooTensor, CsrTensor, CscTensor, SparseTensor, SemiStructuredSparseTensor,
                         sparse_matmul_24, SparseGrad, NestedTensor, PackedNestedTensor, nested_scaled_dot_product_attention, MaskedTensor,
                         masked_sum, masked_mean, masked_min, masked_max, masked_count, masked_where, masked_invalid, masked_equal, NamedTensor,
                         ComplexTensor)

from .ops_ext import (cond, scan, empty, tensor, from_vec, searchsorted, bucketize, topk, sort, argsort, unique, histc, nonzero, where, cumsum,  # noqa: E402,F401
                      BoolTensor, IntTensor, CpuBufferPool, cpu_pool, meta_propagate, format_tensor, display, with_fusion, fusion_enabled, fused)

from . import names_ext as _nx  # noqa: E402
from .names_ext import (Float, IntElement, Element, FerrotorchResult, is_float, normalize_axis, broadcast_shapes, exp, expm1, log, log1p, sin, cos, tanh,  # noqa: E402,F401
                        sigmoid, erf, erfc, erfinv, lgamma, digamma, sinc, xlogy, clamp, where_cond, sum_dim, mean_dim, cat, expand, view_t, permute_t,
                        contiguous_t, chunk_t, split_t, roll, tril, triu, diag, diagflat, meshgrid, cdist, gather, scatter, scatter_add,
                        scatter_add_segments, unique_consecutive, CumExtremeResult, cummax, cummin, cumprod, logcumsumexp, ifft, rfft, irfft, fft2, ifft2,
                        fftn, ifftn, rfftn, irfftn, hfft, ihfft, fftshift, ifftshift, fftfreq, rfftfreq, fft_differentiable, ifft_differentiable,
                        rfft_differentiable, irfft_differentiable, dual_add, dual_sub, dual_mul, dual_div, dual_neg, dual_matmul, backward_with_grad,
                        AnomalyMode, ForwardBacktrace, check_gradient_anomaly, AutocastDtype, set_autocast_debug, is_autocast_debug, autocast_dtype,
                        autocast_guard, DispatchKeySet, Kernel, TensorId, StorageBuffer, TensorStorage, GradFn, EinopsReduction, validate_cond_branches,
                        AsStridedBackward, Observer)

for _n in ("unary_same_shape", "binary_broadcast", "reduce_dim", "reduce_all", "matmul"):      # ``core.meta_propagate.matmul(a, b)``: the per-operation shape rules
    setattr(meta_propagate, _n, getattr(_nx, "meta_" + _n))
full_meta, meta_like = _nx.full_meta, _nx.meta_like
fft = _nx._CallableNamespace(fft, _nx.fft)                   # ``core.fft(x)`` and ``core.fft.fft2(x)`` (torch complex forms) both work


def cuda_rng():
    """The process-wide Philox state manager of the CUDA generators (ferrotorch-core re-exports ferrotorch-gpu's)."""
    from ..gpu import CudaRngManager
    global _cuda_rng
    try:
        return _cuda_rng
    except NameError:
        _cuda_rng = CudaRngManager()
        return _cuda_rng


def __getattr__(name):
    if name in _nx._NN_NAMES or name in ("QatLayer", "fake_quantize_differentiable"):
        return _nx.nn_name(name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
