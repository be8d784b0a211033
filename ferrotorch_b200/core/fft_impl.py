"""Discrete Fourier transforms written out on complex tensor arithmetic: an iterative radix-2 transform for power-of-two lengths and
Bluestein's chirp-z re-expression (a convolution carried out by the radix-2 transform) for every other length; the real, Hermitian,
two- and n-dimensional forms, the frequency grids and the shifts are built on the one-dimensional complex transform.

Reference parity: ferrotorch-core/src/fft.rs:108-1141 (fft, ifft, rfft, irfft, fft2, ifft2, fftn, ifftn, rfftn, irfftn, hfft, ihfft, fftfreq,
rfftfreq, fftshift, ifftshift), same argument conventions as ``torch.fft`` (``n`` / ``s`` pad or trim, ``dim``, ``norm``). Every function
is differentiable because it is composed of differentiable tensor operations.
"""
from __future__ import annotations

import math
from functools import lru_cache
from typing import Optional, Sequence

import torch

from ..errors import InvalidArgument


def _complex(x: torch.Tensor) -> torch.Tensor:
    x = torch.as_tensor(x)
    if x.is_complex():
        return x
    if not x.is_floating_point():
        x = x.to(torch.get_default_dtype())
    if x.dtype in (torch.float16, torch.bfloat16):
        x = x.float()
    return torch.complex(x, torch.zeros_like(x))


@lru_cache(maxsize=64)
def _bit_reverse(n: int) -> torch.Tensor:
    bits = n.bit_length() - 1
    idx = torch.arange(n)
    rev = torch.zeros(n, dtype=torch.long)
    for b in range(bits):
        rev |= ((idx >> b) & 1) << (bits - 1 - b)
    return rev


def _twiddle(m: int, sign: float, dtype, device) -> torch.Tensor:
    """exp(sign * i * pi * k / m) for k < m, computed in f64."""
    ang = sign * math.pi * torch.arange(m, dtype=torch.float64, device=device) / m
    return torch.complex(torch.cos(ang), torch.sin(ang)).to(dtype)


def _radix2(x: torch.Tensor, sign: float) -> torch.Tensor:
    """Unnormalised transform along the last dim, whose length is a power of two: bit-reversal, then log2(n) butterfly stages."""
    n = x.shape[-1]
    if n == 1:
        return x
    x = x.index_select(-1, _bit_reverse(n).to(x.device))
    lead = x.shape[:-1]
    m = 1
    while m < n:
        x = x.reshape(*lead, n // (2 * m), 2, m)
        even, odd = x[..., 0, :], x[..., 1, :] * _twiddle(m, sign, x.dtype, x.device)
        x = torch.stack((even + odd, even - odd), dim=-2).reshape(*lead, n)
        m *= 2
    return x


def _bluestein(x: torch.Tensor, sign: float) -> torch.Tensor:
    """Any length: X_k = w_k * sum_j (x_j w_j) conj(w)_{k-j} with w_k = exp(sign * i * pi * k^2 / n); the sum is a convolution, done at a
    power-of-two length by ``_radix2``. k^2 is reduced modulo 2n in integers so the chirp keeps its accuracy for long inputs."""
    n = x.shape[-1]
    k = torch.arange(n, dtype=torch.long, device=x.device)
    ang = sign * math.pi * ((k * k) % (2 * n)).to(torch.float64) / n
    w = torch.complex(torch.cos(ang), torch.sin(ang)).to(x.dtype)
    size = 1 << (2 * n - 1).bit_length()
    a = torch.zeros(*x.shape[:-1], size, dtype=x.dtype, device=x.device)
    a[..., :n] = x * w
    b = torch.zeros(size, dtype=x.dtype, device=x.device)
    b[:n] = w.conj()
    b[size - n + 1:] = w.conj()[1:].flip(0)
    conv = _radix2(_radix2(a, -1.0) * _radix2(b, -1.0), +1.0) / size
    return conv[..., :n] * w


def _dft_last(x: torch.Tensor, sign: float) -> torch.Tensor:
    n = x.shape[-1]
    if n == 0:
        raise InvalidArgument("fft of an empty dimension")
    return _radix2(x, sign) if n & (n - 1) == 0 else _bluestein(x, sign)


def _resize(x: torch.Tensor, n: Optional[int], dim: int) -> torch.Tensor:
    if n is None or n == x.shape[dim]:
        return x
    if n < 1:
        raise InvalidArgument(f"invalid number of data points ({n})")
    if n < x.shape[dim]:
        return x.narrow(dim, 0, n)
    pad = list(x.shape)
    pad[dim] = n - x.shape[dim]
    return torch.cat([x, torch.zeros(pad, dtype=x.dtype, device=x.device)], dim)


def _scale(n: int, norm: Optional[str], inverse: bool) -> float:
    norm = norm or "backward"
    if norm not in ("backward", "ortho", "forward"):
        raise InvalidArgument(f"unknown normalisation '{norm}'")
    if norm == "ortho":
        return 1.0 / math.sqrt(n)
    return 1.0 / n if (norm == "backward") == inverse else 1.0


def _c2c(x: torch.Tensor, n: Optional[int], dim: int, norm: Optional[str], inverse: bool) -> torch.Tensor:
    x = _resize(_complex(x), n, dim)
    y = _dft_last(x.movedim(dim, -1), +1.0 if inverse else -1.0).movedim(-1, dim)
    s = _scale(x.shape[dim], norm, inverse)
    return y if s == 1.0 else y * s


def fft(x, n: Optional[int] = None, dim: int = -1, norm: Optional[str] = None) -> torch.Tensor:
    return _c2c(x, n, dim, norm, False)


def ifft(x, n: Optional[int] = None, dim: int = -1, norm: Optional[str] = None) -> torch.Tensor:
    return _c2c(x, n, dim, norm, True)


def rfft(x, n: Optional[int] = None, dim: int = -1, norm: Optional[str] = None) -> torch.Tensor:
    """Transform of a real signal: the non-negative-frequency half, n // 2 + 1 values."""
    x = torch.as_tensor(x)
    if x.is_complex():
        raise InvalidArgument("rfft takes a real input")
    y = _c2c(x, n, dim, norm, False)
    return y.narrow(dim, 0, y.shape[dim] // 2 + 1)


def _hermitian_full(x: torch.Tensor, n: int, dim: int) -> torch.Tensor:
    """The length-n spectrum whose first n // 2 + 1 values are (a trim / zero-pad of) ``x`` and whose rest is their mirrored conjugate."""
    half = n // 2 + 1
    x = _resize(_complex(x), half, dim)
    x0 = x.narrow(dim, 0, 1)
    x = torch.cat([torch.complex(x0.real, torch.zeros_like(x0.real)), x.narrow(dim, 1, half - 1)], dim) if half > 1 else torch.complex(x0.real, torch.zeros_like(x0.real))
    if n % 2 == 0 and half > 1:                     # the Nyquist term of a real signal is real
        ny = x.narrow(dim, half - 1, 1)
        x = torch.cat([x.narrow(dim, 0, half - 1), torch.complex(ny.real, torch.zeros_like(ny.real))], dim)
    tail = x.narrow(dim, 1, n - half).flip(dim).conj() if n - half > 0 else None
    return x if tail is None else torch.cat([x, tail], dim)


def irfft(x, n: Optional[int] = None, dim: int = -1, norm: Optional[str] = None) -> torch.Tensor:
    """Inverse of ``rfft``: a real signal of length n (default 2 * (m - 1))."""
    x = torch.as_tensor(x)
    n = 2 * (x.shape[dim] - 1) if n is None else n
    if n < 1:
        raise InvalidArgument(f"invalid number of data points ({n})")
    return _c2c(_hermitian_full(x, n, dim), None, dim, norm, True).real


def hfft(x, n: Optional[int] = None, dim: int = -1, norm: Optional[str] = None) -> torch.Tensor:
    """Transform of a signal that is Hermitian in time (given by its first half): a real spectrum of length n."""
    x = torch.as_tensor(x)
    n = 2 * (x.shape[dim] - 1) if n is None else n
    if n < 1:
        raise InvalidArgument(f"invalid number of data points ({n})")
    return _c2c(_hermitian_full(x, n, dim), None, dim, norm, False).real


def ihfft(x, n: Optional[int] = None, dim: int = -1, norm: Optional[str] = None) -> torch.Tensor:
    """Inverse of ``hfft``: the half of the Hermitian signal whose transform is the real input."""
    x = torch.as_tensor(x)
    if x.is_complex():
        raise InvalidArgument("ihfft takes a real input")
    y = _c2c(x, n, dim, norm, True)
    return y.narrow(dim, 0, y.shape[dim] // 2 + 1)


def _dims(x: torch.Tensor, s, dim, default_last: Optional[int] = None):
    if dim is None:
        if s is not None:
            dim = list(range(x.dim() - len(s), x.dim()))
        elif default_last is not None:
            dim = list(range(x.dim() - default_last, x.dim()))
        else:
            dim = list(range(x.dim()))
    dim = [d % x.dim() for d in ([dim] if isinstance(dim, int) else list(dim))]
    if len(set(dim)) != len(dim):
        raise InvalidArgument("fft dimensions must be distinct")
    if s is not None and len(s) != len(dim):
        raise InvalidArgument("s and dim must have the same length")
    return dim, (list(s) if s is not None else [None] * len(dim))


def fftn(x, s: Optional[Sequence[int]] = None, dim=None, norm: Optional[str] = None) -> torch.Tensor:
    x = torch.as_tensor(x)
    dims, sizes = _dims(x, s, dim)
    for d, n in zip(dims, sizes):
        x = fft(x, n, d, norm)
    return _complex(x)


def ifftn(x, s: Optional[Sequence[int]] = None, dim=None, norm: Optional[str] = None) -> torch.Tensor:
    x = torch.as_tensor(x)
    dims, sizes = _dims(x, s, dim)
    for d, n in zip(dims, sizes):
        x = ifft(x, n, d, norm)
    return _complex(x)


def fft2(x, s: Optional[Sequence[int]] = None, dim=(-2, -1), norm: Optional[str] = None) -> torch.Tensor:
    return fftn(x, s, dim, norm)


def ifft2(x, s: Optional[Sequence[int]] = None, dim=(-2, -1), norm: Optional[str] = None) -> torch.Tensor:
    return ifftn(x, s, dim, norm)


def rfftn(x, s: Optional[Sequence[int]] = None, dim=None, norm: Optional[str] = None) -> torch.Tensor:
    """Real input: the half transform along the last of ``dim``, full transforms along the others."""
    x = torch.as_tensor(x)
    dims, sizes = _dims(x, s, dim)
    y = rfft(x, sizes[-1], dims[-1], norm)
    for d, n in zip(dims[:-1], sizes[:-1]):
        y = fft(y, n, d, norm)
    return y


def irfftn(x, s: Optional[Sequence[int]] = None, dim=None, norm: Optional[str] = None) -> torch.Tensor:
    x = torch.as_tensor(x)
    dims, sizes = _dims(x, s, dim)
    for d, n in zip(dims[:-1], sizes[:-1]):
        x = ifft(x, n, d, norm)
    return irfft(x, sizes[-1], dims[-1], norm)


def fftfreq(n: int, d: float = 1.0, dtype=None, device=None) -> torch.Tensor:
    """Sample frequencies 0, 1, ..., ceil(n/2) - 1, -floor(n/2), ..., -1, each divided by n * d."""
    if n < 1:
        raise InvalidArgument("n must be positive")
    k = torch.arange(n, dtype=torch.float64, device=device)
    k = torch.where(k < (n + 1) // 2, k, k - n)
    return (k / (n * d)).to(dtype or torch.get_default_dtype())


def rfftfreq(n: int, d: float = 1.0, dtype=None, device=None) -> torch.Tensor:
    if n < 1:
        raise InvalidArgument("n must be positive")
    return (torch.arange(n // 2 + 1, dtype=torch.float64, device=device) / (n * d)).to(dtype or torch.get_default_dtype())


def fftshift(x, dim=None) -> torch.Tensor:
    """Moves the zero-frequency term to the middle (a roll by n // 2 along each of ``dim``)."""
    x = torch.as_tensor(x)
    dims = list(range(x.dim())) if dim is None else ([dim] if isinstance(dim, int) else list(dim))
    return torch.roll(x, [x.shape[d] // 2 for d in dims], dims)


def ifftshift(x, dim=None) -> torch.Tensor:
    x = torch.as_tensor(x)
    dims = list(range(x.dim())) if dim is None else ([dim] if isinstance(dim, int) else list(dim))
    return torch.roll(x, [-(x.shape[d] // 2) for d in dims], dims)
