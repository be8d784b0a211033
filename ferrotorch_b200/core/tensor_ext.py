"""Linear algebra, FFT, special functions, einsum/einops, stride tricks, signal windows, pruning, quantization, sparse / nested /
masked / named / complex tensor types - the long tail of ferrotorch-core under the reference's names.

These are cold paths: they evaluate through PyTorch's reference implementations (cuSOLVER/cuFFT/cuSPARSE on CUDA tensors, exactly the
vendor libraries the reference wraps in ferrotorch-gpu/src/{cusolver,cufft,sparse}.rs) and are labelled "library path" in reports.

Reference parity: ferrotorch-core/src/{linalg.rs:121-2170, fft.rs, special.rs:675-905, einsum.rs, einops.rs, stride_tricks.rs,
signal/windows.rs, pruning.rs, quantize.rs, sparse.rs, nested.rs, masked.rs, named_tensor.rs, complex_tensor.rs}.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..errors import InvalidArgument, ShapeMismatch
from . import einops_impl as _einops_impl
from . import einsum_impl as _einsum_impl
from . import fft_impl as _fft_impl
from . import linalg_impl as _la
from . import special_fns as _sf



# -- linalg ---------------------------------------------------------------------------------------------------------------------
class linalg:
    """``core/linalg_impl.py``: factorisations in the host runtime library with the derivative formulas beside them, the rest composed from
    them (ferrotorch_core::linalg). CUDA / complex / half inputs and the general eigenproblem go to the substrate's library call."""
    svd = staticmethod(lambda a, full_matrices=False: _la.svd(a, full_matrices=full_matrices))
    lstsq = staticmethod(lambda a, b, rcond=None: _la.lstsq(a, b, rcond))
    for _n in ("solve", "det", "inv", "qr", "cholesky", "matrix_norm", "pinv", "eigh", "eigvalsh", "eig", "eigvals", "lu", "lu_factor", "svdvals", "lstsq_solve",
               "matrix_power", "tensorsolve", "tensorinv", "vector_norm", "slogdet", "matrix_rank", "cond", "cross", "multi_dot", "diagonal", "solve_triangular",
               "ldl_factor", "ldl_solve", "householder_product", "matrix_exp", "cholesky_ex", "inv_ex", "solve_ex"):
        locals()[_n] = staticmethod(getattr(_la, _n))
    del _n
    LinAlgError = _la.LinAlgError


# -- fft ------------------------------------------------------------------------------------------------------------------------
class fft:
    """Written out in ``core/fft_impl.py``: radix-2 butterflies for power-of-two lengths, Bluestein's chirp-z form for the others."""
    for _n in ("fft", "ifft", "rfft", "irfft", "fft2", "ifft2", "fftn", "ifftn", "rfftn", "irfftn", "hfft", "ihfft", "fftfreq", "rfftfreq", "fftshift", "ifftshift"):
        locals()[_n] = staticmethod(getattr(_fft_impl, _n))
    del _n


# -- special --------------------------------------------------------------------------------------------------------------------
class special:
    """Written out in ``core/special_fns.py`` (series, continued fractions, recurrences); ``log1p`` / ``expm1`` are the substrate's primitives."""
    erf, erfc, erfinv = staticmethod(_sf.erf), staticmethod(_sf.erfc), staticmethod(_sf.erfinv)
    lgamma, digamma = staticmethod(_sf.lgamma), staticmethod(_sf.digamma)
    log1p, expm1, sinc, xlogy = staticmethod(torch.log1p), staticmethod(torch.expm1), staticmethod(_sf.sinc), staticmethod(_sf.xlogy)
    for _n in ("chebyshev_polynomial_t", "chebyshev_polynomial_u", "chebyshev_polynomial_v", "chebyshev_polynomial_w", "hermite_polynomial_h",
               "hermite_polynomial_he", "laguerre_polynomial_l", "legendre_polynomial_p", "shifted_chebyshev_polynomial_t",
               "shifted_chebyshev_polynomial_u", "shifted_chebyshev_polynomial_v", "shifted_chebyshev_polynomial_w"):
        locals()[_n] = staticmethod(getattr(_sf, _n))
    del _n


# -- einsum / einops ------------------------------------------------------------------------------------------------------------------
def einsum(equation: str, *operands: torch.Tensor) -> torch.Tensor:
    """Einstein summation, planned and contracted in ``core/einsum_impl.py`` (diagonals, single-operand sums, pairwise batched products)."""
    return _einsum_impl.einsum(equation, *operands)


einsum_differentiable = einsum


def rearrange(t, pattern: str, **axes):
    return _einops_impl.rearrange(t, pattern, **axes)


rearrange_with = rearrange


def repeat(t, pattern: str, **axes):
    return _einops_impl.repeat(t, pattern, **axes)


def reduce(t, pattern: str, reduction: str = "mean", **axes):
    return _einops_impl.reduce(t, pattern, reduction, **axes)


# -- stride tricks ----------------------------------------------------------------------------------------------------------------
def as_strided(t, size, stride, storage_offset: int = 0):
    return torch.as_strided(t, tuple(size), tuple(stride), storage_offset)


def as_strided_copy(t, size, stride, storage_offset: int = 0):
    return torch.as_strided(t, tuple(size), tuple(stride), storage_offset).clone()


def as_strided_scatter(t, src, size, stride, storage_offset: int = 0):
    return torch.as_strided_scatter(t, src, tuple(size), tuple(stride), storage_offset)


# -- signal windows ------------------------------------------------------------------------------------------------------------------
def _win_n(M: int, sym: bool, dtype, device):
    """Sample positions 0..M-1 of a window of length M (a periodic window is the symmetric one of length M + 1 without its last sample)."""
    if M < 0:
        raise InvalidArgument("window length must be non-negative")
    dtype = dtype or torch.get_default_dtype()
    n = torch.arange(M, dtype=torch.float64, device=device)
    return n, float(M - 1 if sym else M), dtype


def _i0(x: torch.Tensor) -> torch.Tensor:
    """Modified Bessel function of order zero by its power series sum ((x/2)^2k / (k!)^2) (f64; enough terms for |x| up to a few hundred)."""
    q = (x * 0.5) ** 2
    term = torch.ones_like(x)
    total = torch.ones_like(x)
    for k in range(1, 400):
        term = term * q / (k * k)
        total = total + term
    return total


class windows:
    """Window functions from their formulas (ferrotorch-core/src/signal/windows.rs:35-170); ``sym=False`` gives the periodic form."""

    @staticmethod
    def general_cosine(M: int, *, a, sym: bool = True, dtype=None, device=None) -> torch.Tensor:
        n, L, dtype = _win_n(M, sym, dtype, device)
        if M == 1:
            return torch.ones(1, dtype=dtype, device=device)
        w = torch.zeros_like(n)
        for k, c in enumerate(a):
            w = w + ((-1) ** k) * float(c) * torch.cos(2 * math.pi * k * n / L)
        return w.to(dtype)

    @staticmethod
    def general_hamming(M: int, *, alpha: float = 0.54, sym: bool = True, dtype=None, device=None) -> torch.Tensor:
        return windows.general_cosine(M, a=[alpha, 1.0 - alpha], sym=sym, dtype=dtype, device=device)

    @staticmethod
    def hamming(M: int, *, sym: bool = True, dtype=None, device=None) -> torch.Tensor:
        return windows.general_hamming(M, alpha=0.54, sym=sym, dtype=dtype, device=device)

    @staticmethod
    def hann(M: int, *, sym: bool = True, dtype=None, device=None) -> torch.Tensor:
        return windows.general_hamming(M, alpha=0.5, sym=sym, dtype=dtype, device=device)

    hanning = hann

    @staticmethod
    def blackman(M: int, *, sym: bool = True, dtype=None, device=None) -> torch.Tensor:
        return windows.general_cosine(M, a=[0.42, 0.5, 0.08], sym=sym, dtype=dtype, device=device)

    @staticmethod
    def nuttall(M: int, *, sym: bool = True, dtype=None, device=None) -> torch.Tensor:
        return windows.general_cosine(M, a=[0.3635819, 0.4891775, 0.1365995, 0.0106411], sym=sym, dtype=dtype, device=device)

    @staticmethod
    def bartlett(M: int, *, sym: bool = True, dtype=None, device=None) -> torch.Tensor:
        n, L, dtype = _win_n(M, sym, dtype, device)
        if M == 1:
            return torch.ones(1, dtype=dtype, device=device)
        return (1.0 - (2.0 * n / L - 1.0).abs()).to(dtype)

    @staticmethod
    def cosine(M: int, *, sym: bool = True, dtype=None, device=None) -> torch.Tensor:
        n, L, dtype = _win_n(M, sym, dtype, device)
        if M == 1:
            return torch.ones(1, dtype=dtype, device=device)
        return torch.sin(math.pi * (n + 0.5) / (L + 1.0)).to(dtype)

    @staticmethod
    def exponential(M: int, *, center: Optional[float] = None, tau: float = 1.0, sym: bool = True, dtype=None, device=None) -> torch.Tensor:
        if sym and center is not None:
            raise InvalidArgument("a symmetric exponential window takes no centre")
        if tau <= 0:
            raise InvalidArgument("tau must be positive")
        n, L, dtype = _win_n(M, sym, dtype, device)
        if M == 1:
            return torch.ones(1, dtype=dtype, device=device)
        c = L / 2.0 if center is None else float(center)
        return torch.exp(-(n - c).abs() / tau).to(dtype)

    @staticmethod
    def gaussian(M: int, *, std: float = 1.0, sym: bool = True, dtype=None, device=None) -> torch.Tensor:
        if std <= 0:
            raise InvalidArgument("std must be positive")
        n, L, dtype = _win_n(M, sym, dtype, device)
        if M == 1:
            return torch.ones(1, dtype=dtype, device=device)
        return torch.exp(-0.5 * ((n - L / 2.0) / std) ** 2).to(dtype)

    @staticmethod
    def kaiser(M: int, *, beta: float = 12.0, sym: bool = True, dtype=None, device=None) -> torch.Tensor:
        if beta < 0:
            raise InvalidArgument("beta must be non-negative")
        n, L, dtype = _win_n(M, sym, dtype, device)
        if M == 1:
            return torch.ones(1, dtype=dtype, device=device)
        r = (2.0 * n / L - 1.0).clamp(-1.0, 1.0)
        return (_i0(beta * torch.sqrt(1.0 - r * r)) / _i0(torch.tensor(float(beta), dtype=torch.float64, device=device))).to(dtype)

    @staticmethod
    def parzen(n: int) -> torch.Tensor:
        k = torch.arange(n, dtype=torch.float64) - (n - 1) / 2
        a = k.abs() / (n / 2)
        return torch.where(a <= 0.5, 1 - 6 * a ** 2 + 6 * a ** 3, 2 * (1 - a).clamp(min=0) ** 3).float()

    @staticmethod
    def tukey(n: int, alpha: float = 0.5) -> torch.Tensor:
        if alpha <= 0:
            return torch.ones(n)
        x = torch.arange(n, dtype=torch.float64) / max(n - 1, 1)
        w = torch.ones(n, dtype=torch.float64)
        lo, hi = x < alpha / 2, x >= 1 - alpha / 2
        w[lo] = 0.5 * (1 + torch.cos(2 * math.pi / alpha * (x[lo] - alpha / 2)))
        w[hi] = 0.5 * (1 + torch.cos(2 * math.pi / alpha * (x[hi] - 1 + alpha / 2)))
        return w.float()

    @staticmethod
    def taylor(n: int, nbar: int = 4, sll: float = 30.0, norm: bool = True) -> torch.Tensor:
        """Taylor window with ``nbar`` nearly constant side lobes ``sll`` dB down; ``norm`` divides by the value at the centre (n - 1) / 2."""
        B = 10 ** (sll / 20)
        A = math.acosh(B) / math.pi
        s2 = nbar ** 2 / (A ** 2 + (nbar - 0.5) ** 2)
        ma = torch.arange(1, nbar, dtype=torch.float64)
        Fm = torch.empty(nbar - 1, dtype=torch.float64)
        for mi, m in enumerate(ma):
            numer = (-1) ** (mi) * torch.prod(1 - m ** 2 / s2 / (A ** 2 + (ma - 0.5) ** 2))
            denom = 2 * torch.prod(torch.tensor([1 - m ** 2 / j ** 2 for j in ma if j != m], dtype=torch.float64))
            Fm[mi] = numer / denom

        def W(pos: torch.Tensor) -> torch.Tensor:
            x = (pos - n / 2 + 0.5) / n
            return 1 + 2 * (Fm.view(-1, 1) * torch.cos(2 * math.pi * ma.view(-1, 1) * x.view(1, -1))).sum(0)
        w = W(torch.arange(n, dtype=torch.float64))
        if norm:
            w = w / W(torch.tensor([(n - 1) / 2], dtype=torch.float64))
        return w.float()


# -- pruning -------------------------------------------------------------------------------------------------------------------------
def magnitude_prune(t: torch.Tensor, sparsity: float) -> torch.Tensor:
    """Zero the ``sparsity`` fraction of smallest-magnitude entries; returns the mask."""
    k = int(t.numel() * sparsity)
    if k <= 0:
        return torch.ones_like(t, dtype=torch.bool)
    thr = t.abs().flatten().kthvalue(k).values
    return t.abs() > thr


def apply_2_4_mask(t: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Keep the two largest-magnitude values in every group of four along the last dim (2:4 structured sparsity)."""
    if t.shape[-1] % 4:
        raise ShapeMismatch("last dimension must be a multiple of 4 for 2:4 sparsity")
    g = t.reshape(-1, 4)
    idx = g.abs().topk(2, dim=1).indices
    mask = torch.zeros_like(g, dtype=torch.bool).scatter_(1, idx, True).reshape(t.shape)
    return t * mask, mask


def sparsity_ratio(t: torch.Tensor) -> float:
    return float((t == 0).sum()) / max(t.numel(), 1)


# -- quantization ----------------------------------------------------------------------------------------------------------------------
class QuantScheme(enum.Enum):
    PerTensorAffine = "per_tensor_affine"
    PerTensorSymmetric = "per_tensor_symmetric"
    PerChannelSymmetric = "per_channel_symmetric"


class QuantDtype(enum.Enum):
    Int8 = 8
    Int4 = 4


@dataclass
class QParams:
    scale: torch.Tensor
    zero_point: torch.Tensor
    qmin: int
    qmax: int
    axis: Optional[int] = None


@dataclass
class QuantizedTensor:
    data: torch.Tensor          # int8 storage (int4 values are kept one per byte)
    params: QParams
    shape: Tuple[int, ...]

    def dequantize(self) -> torch.Tensor:
        return dequantize(self)


def _qrange(dt: QuantDtype, symmetric: bool):
    b = dt.value
    return (-(2 ** (b - 1)) + (1 if symmetric else 0), 2 ** (b - 1) - 1)


def quantize(t: torch.Tensor, scheme: QuantScheme = QuantScheme.PerTensorSymmetric, dtype: QuantDtype = QuantDtype.Int8, axis: int = 0) -> QuantizedTensor:
    tf = t.detach().float()
    sym = scheme != QuantScheme.PerTensorAffine
    qmin, qmax = _qrange(dtype, sym)
    if scheme == QuantScheme.PerChannelSymmetric:
        red = [d for d in range(tf.dim()) if d != axis]
        amax = tf.abs().amax(red, keepdim=True).clamp(min=1e-12)
        scale, zp = amax / qmax, torch.zeros_like(amax)
    elif sym:
        scale, zp = (tf.abs().max().clamp(min=1e-12) / qmax).reshape(1), torch.zeros(1)
    else:
        lo, hi = tf.min(), tf.max()
        scale = ((hi - lo).clamp(min=1e-12) / (qmax - qmin)).reshape(1)
        zp = torch.round(qmin - lo / scale)
    q = torch.clamp(torch.round(tf / scale) + zp, qmin, qmax).to(torch.int8)
    return QuantizedTensor(q, QParams(scale, zp, qmin, qmax, axis if scheme == QuantScheme.PerChannelSymmetric else None), tuple(t.shape))


def dequantize(q: QuantizedTensor) -> torch.Tensor:
    return (q.data.float() - q.params.zero_point) * q.params.scale


def quantized_matmul(a: QuantizedTensor, b: QuantizedTensor) -> torch.Tensor:
    """Integer matmul with f32 rescale (symmetric per-tensor operands); falls back to dequantise-then-matmul otherwise."""
    if a.params.axis is None and b.params.axis is None and float(a.params.zero_point.abs().sum()) == 0 and float(b.params.zero_point.abs().sum()) == 0:
        acc = a.data.to(torch.int32) @ b.data.to(torch.int32) if not a.data.is_cuda else (a.data.float() @ b.data.float())
        return acc.float() * (a.params.scale * b.params.scale)
    return dequantize(a) @ dequantize(b)


def quantize_named_tensors(state: Dict[str, torch.Tensor], scheme=QuantScheme.PerChannelSymmetric, dtype=QuantDtype.Int8) -> Dict[str, QuantizedTensor]:
    return {k: quantize(v, scheme if v.dim() >= 2 else QuantScheme.PerTensorSymmetric, dtype) for k, v in state.items() if v.is_floating_point()}


class MinMaxObserver:
    def __init__(self):
        self.lo, self.hi = None, None

    def observe(self, t):
        lo, hi = float(t.min()), float(t.max())
        self.lo = lo if self.lo is None else min(self.lo, lo)
        self.hi = hi if self.hi is None else max(self.hi, hi)

    def qparams(self, dtype=QuantDtype.Int8, symmetric=True) -> QParams:
        qmin, qmax = _qrange(dtype, symmetric)
        if symmetric:
            return QParams(torch.tensor([max(abs(self.lo), abs(self.hi), 1e-12) / qmax]), torch.zeros(1), qmin, qmax)
        s = max(self.hi - self.lo, 1e-12) / (qmax - qmin)
        return QParams(torch.tensor([s]), torch.tensor([round(qmin - self.lo / s)]), qmin, qmax)


class PerChannelMinMaxObserver:
    def __init__(self, axis: int = 0):
        self.axis, self.amax = axis, None

    def observe(self, t):
        red = [d for d in range(t.dim()) if d != self.axis]
        a = t.detach().abs().amax(red)
        self.amax = a if self.amax is None else torch.maximum(self.amax, a)

    def qparams(self, dtype=QuantDtype.Int8) -> QParams:
        qmin, qmax = _qrange(dtype, True)
        return QParams(self.amax.clamp(min=1e-12) / qmax, torch.zeros_like(self.amax), qmin, qmax, self.axis)


class HistogramObserver:
    """Histogram of observed values; ``qparams`` picks the clipping range that keeps ``coverage`` of the mass."""

    def __init__(self, bins: int = 2048, coverage: float = 0.9999):
        self.bins, self.coverage, self.hist, self.range = bins, coverage, None, None

    def observe(self, t):
        a = float(t.detach().abs().max())
        if self.hist is None:
            self.range = max(a, 1e-12)
            self.hist = torch.histc(t.detach().abs().float(), self.bins, 0, self.range)
        else:
            if a > self.range:
                old = self.hist
                ratio = self.range / a
                idx = (torch.arange(self.bins) * ratio).long().clamp(max=self.bins - 1)
                self.hist = torch.zeros(self.bins).index_add_(0, idx, old)
                self.range = a
            self.hist += torch.histc(t.detach().abs().float(), self.bins, 0, self.range)

    def qparams(self, dtype=QuantDtype.Int8) -> QParams:
        c = self.hist.cumsum(0) / self.hist.sum()
        k = int((c >= self.coverage).nonzero()[0]) + 1
        qmin, qmax = _qrange(dtype, True)
        return QParams(torch.tensor([self.range * k / self.bins / qmax]), torch.zeros(1), qmin, qmax)


# -- sparse --------------------------------------------------------------------------------------------------------------------------
from .sparse_impl import CooTensor, CscTensor, CsrTensor, SparseTensor  # noqa: E402  (own storage and algorithms: core/sparse_impl.py)


class SemiStructuredSparseTensor:
    """2:4 structured-sparse matrix: two kept values and their 2-bit positions per group of four."""

    def __init__(self, dense: torch.Tensor):
        pruned, mask = apply_2_4_mask(dense)
        g = pruned.reshape(-1, 4)
        idx = mask.reshape(-1, 4).float().topk(2, dim=1).indices.sort(1).values
        self.values = g.gather(1, idx).reshape(*dense.shape[:-1], dense.shape[-1] // 2)
        self.meta = idx.to(torch.uint8).reshape(*dense.shape[:-1], dense.shape[-1] // 2)
        self.shape = tuple(dense.shape)

    def to_dense(self) -> torch.Tensor:
        out = torch.zeros(int(torch.tensor(self.shape).prod()) // 4, 4, dtype=self.values.dtype, device=self.values.device)
        out.scatter_(1, self.meta.reshape(-1, 2).long(), self.values.reshape(-1, 2))
        return out.reshape(self.shape)


def sparse_matmul_24(a: SemiStructuredSparseTensor, b: torch.Tensor) -> torch.Tensor:
    return a.to_dense() @ b


class SparseGrad:
    """Row-sparse gradient (embedding tables): ``indices`` rows hold ``values``."""

    def __init__(self, indices: torch.Tensor, values: torch.Tensor, num_rows: int):
        self.indices, self.values, self.num_rows = indices, values, num_rows

    def to_dense(self):
        out = torch.zeros(self.num_rows, *self.values.shape[1:], dtype=self.values.dtype, device=self.values.device)
        return out.index_add_(0, self.indices, self.values)

    def coalesce(self) -> "SparseGrad":
        u, inv = self.indices.unique(return_inverse=True)
        v = torch.zeros(len(u), *self.values.shape[1:], dtype=self.values.dtype, device=self.values.device).index_add_(0, inv, self.values)
        return SparseGrad(u, v, self.num_rows)


# -- nested / masked / named / complex ------------------------------------------------------------------------------------------------------
class NestedTensor:
    """A batch of variable-length sequences ``[len_i, ...]``."""

    def __init__(self, tensors: Sequence[torch.Tensor]):
        self.tensors = list(tensors)

    def to_padded(self, value: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor]:
        lens = torch.tensor([t.shape[0] for t in self.tensors])
        return torch.nn.utils.rnn.pad_sequence(self.tensors, batch_first=True, padding_value=value), lens

    def pack(self) -> "PackedNestedTensor":
        return PackedNestedTensor(torch.cat(self.tensors, 0), torch.tensor([0] + [t.shape[0] for t in self.tensors]).cumsum(0))

    def map(self, fn):
        return NestedTensor([fn(t) for t in self.tensors])

    def __len__(self):
        return len(self.tensors)


@dataclass
class PackedNestedTensor:
    data: torch.Tensor
    offsets: torch.Tensor

    def unpack(self) -> NestedTensor:
        o = self.offsets.tolist()
        return NestedTensor([self.data[a:b] for a, b in zip(o[:-1], o[1:])])


def nested_scaled_dot_product_attention(q: NestedTensor, k: NestedTensor, v: NestedTensor, causal: bool = False) -> NestedTensor:
    """Per-sequence attention on ``[len, heads, dim]`` entries (no padding waste)."""
    from ..nn.functional import scaled_dot_product_attention as sdpa      # this package's attention (the tcgen05 kernels for bf16 on a device)
    out = []
    for qi, ki, vi in zip(q.tensors, k.tensors, v.tensors):
        o = sdpa(qi.transpose(0, 1).unsqueeze(0), ki.transpose(0, 1).unsqueeze(0), vi.transpose(0, 1).unsqueeze(0), is_causal=causal)
        out.append(o.squeeze(0).transpose(0, 1))
    return NestedTensor(out)


class MaskedTensor:
    """Values with a validity mask (True = valid)."""

    def __init__(self, data: torch.Tensor, mask: torch.Tensor):
        self.data, self.mask = data, mask.bool()

    def filled(self, value=0.0):
        return torch.where(self.mask, self.data, torch.full_like(self.data, value))


def masked_sum(m: MaskedTensor, dim=None):
    return m.filled(0).sum() if dim is None else m.filled(0).sum(dim)


def masked_count(m: MaskedTensor, dim=None):
    return m.mask.sum() if dim is None else m.mask.sum(dim)


def masked_mean(m: MaskedTensor, dim=None):
    return masked_sum(m, dim) / masked_count(m, dim).clamp(min=1)


def masked_min(m: MaskedTensor, dim=None):
    f = m.filled(float("inf"))
    return f.min() if dim is None else f.min(dim).values


def masked_max(m: MaskedTensor, dim=None):
    f = m.filled(float("-inf"))
    return f.max() if dim is None else f.max(dim).values


def masked_where(cond: torch.Tensor, t: torch.Tensor) -> MaskedTensor:
    return MaskedTensor(t, ~cond)


def masked_invalid(t: torch.Tensor) -> MaskedTensor:
    return MaskedTensor(t, torch.isfinite(t))


def masked_equal(t: torch.Tensor, value) -> MaskedTensor:
    return MaskedTensor(t, t != value)


class NamedTensor:
    """Tensor with dimension names; ops align by name."""

    def __init__(self, data: torch.Tensor, names: Sequence[str]):
        if len(names) != data.dim() or len(set(names)) != len(names):
            raise InvalidArgument("need one distinct name per dimension")
        self.data, self.names = data, tuple(names)

    def dim_of(self, name: str) -> int:
        return self.names.index(name)

    def align_to(self, *names: str) -> "NamedTensor":
        return NamedTensor(self.data.permute(*[self.dim_of(n) for n in names]), names)

    def sum(self, name: str) -> "NamedTensor":
        d = self.dim_of(name)
        return NamedTensor(self.data.sum(d), [n for n in self.names if n != name])

    def rename(self, **m) -> "NamedTensor":
        return NamedTensor(self.data, [m.get(n, n) for n in self.names])

    def __add__(self, o: "NamedTensor") -> "NamedTensor":
        return NamedTensor(self.data + o.align_to(*self.names).data, self.names)


class ComplexTensor:
    """Complex tensor stored as separate real/imag parts (works for dtypes without native complex kernels, e.g. bf16)."""

    def __init__(self, re: torch.Tensor, im: torch.Tensor):
        self.re, self.im = re, im

    @staticmethod
    def from_torch(c: torch.Tensor) -> "ComplexTensor":
        return ComplexTensor(c.real.clone(), c.imag.clone())

    def to_torch(self) -> torch.Tensor:
        return torch.complex(self.re.float(), self.im.float())

    def __add__(self, o):
        return ComplexTensor(self.re + o.re, self.im + o.im)

    def __mul__(self, o):
        return ComplexTensor(self.re * o.re - self.im * o.im, self.re * o.im + self.im * o.re)

    def conj(self):
        return ComplexTensor(self.re, -self.im)

    def abs(self):
        return torch.sqrt(self.re * self.re + self.im * self.im)

    def matmul(self, o):
        return ComplexTensor(self.re @ o.re - self.im @ o.im, self.re @ o.im + self.im @ o.re)
