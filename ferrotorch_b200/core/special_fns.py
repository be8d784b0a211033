"""Special functions written out on tensor primitives (series, continued fractions, recurrences), evaluated in f64 for f32 / f64 inputs
and cast back; every one is differentiable because it is composed of differentiable element-wise operations.

Reference parity: ferrotorch-core/src/special.rs:675-905 (erf, erfc, erfinv, lgamma, digamma, log1p, expm1, sinc, xlogy and the twelve
orthogonal-polynomial families). ``log1p`` / ``expm1`` stay the substrate's primitives (they are elementary operations like ``exp``).
"""
from __future__ import annotations

import math

import torch

from ..errors import InvalidArgument

_SQRT_PI = math.sqrt(math.pi)


def _wide(x: torch.Tensor):
    """The tensor in the precision the evaluation runs in, and a function that casts the result back."""
    x = torch.as_tensor(x)
    if not x.is_floating_point():
        x = x.to(torch.get_default_dtype())
    dt = x.dtype
    w = x.to(torch.float64) if dt in (torch.float32, torch.float64) else x.to(torch.float32)
    return w, (lambda y: y.to(dt))


def _erf_erfc(a: torch.Tensor):
    """erf and erfc of ``a >= 0``: Maclaurin series below 2, the continued fraction of erfc from 2 on."""
    small = a.clamp(max=2.0)
    s2 = small * small
    term = small.clone()
    total = small.clone()
    for n in range(60):
        term = term * (-s2) / (n + 1)
        total = total + term / (2 * n + 3)
    erf_small = total * (2.0 / _SQRT_PI)
    big = a.clamp(min=2.0)
    f = big.clone()
    for k in range(80, 0, -1):
        f = big + (0.5 * k) / f
    erfc_big = torch.exp(-big * big) / (_SQRT_PI * f)
    is_small = a < 2.0
    return torch.where(is_small, erf_small, 1.0 - erfc_big), torch.where(is_small, 1.0 - erf_small, erfc_big)


def erf(x) -> torch.Tensor:
    w, back = _wide(x)
    e, _ = _erf_erfc(w.abs())
    return back(torch.where(w < 0, -e, e))


def erfc(x) -> torch.Tensor:
    w, back = _wide(x)
    _, c = _erf_erfc(w.abs())
    return back(torch.where(w < 0, 2.0 - c, c))


class _ErfInv(torch.autograd.Function):
    """The value comes from an iteration, so the derivative is given in closed form: d/dx erfinv(x) = sqrt(pi)/2 * exp(erfinv(x)^2)."""

    @staticmethod
    def forward(ctx, x):
        y = _erfinv_value(x)
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, g):
        (y,) = ctx.saved_tensors
        return g * (0.5 * _SQRT_PI) * torch.exp(y.double() * y.double()).to(y.dtype)


def erfinv(x) -> torch.Tensor:
    """Inverse error function on (-1, 1): a polynomial first guess in ``w = -log(1 - x^2)`` (central and tail branch), then Newton steps
    on this module's own ``erf``. +-1 give +-inf, values outside [-1, 1] NaN."""
    x = torch.as_tensor(x)
    if not x.is_floating_point():
        x = x.to(torch.get_default_dtype())
    return _ErfInv.apply(x)


@torch.no_grad()
def _erfinv_value(x) -> torch.Tensor:
    w0, back = _wide(x)
    xs = w0.clamp(-1 + 1e-16, 1 - 1e-16)
    w = -torch.log((1.0 - xs) * (1.0 + xs))
    wc = w - 2.5
    pc = torch.full_like(w, 2.81022636e-08)
    for c in (3.43273939e-07, -3.5233877e-06, -4.39150654e-06, 0.00021858087, -0.00125372503, -0.00417768164, 0.246640727, 1.50140941):
        pc = c + pc * wc
    wt = torch.sqrt(w.clamp(min=5.0)) - 3.0
    pt = torch.full_like(w, -0.000200214257)
    for c in (0.000100950558, 0.00134934322, -0.00367342844, 0.00573950773, -0.0076224613, 0.00943887047, 1.00167406, 2.83297682):
        pt = c + pt * wt
    y = torch.where(w < 5.0, pc, pt) * xs
    for _ in range(3):
        e, _c = _erf_erfc(y.abs())
        err = torch.where(y < 0, -e, e) - xs
        y = y - err / ((2.0 / _SQRT_PI) * torch.exp(-y * y)).clamp(min=1e-300)
    y = torch.where(w0.abs() == 1.0, w0 * float("inf"), y)
    y = torch.where(w0.abs() > 1.0, torch.full_like(y, float("nan")), y)
    return back(y)


def _lgamma_pos(x: torch.Tensor) -> torch.Tensor:
    """log Gamma for x > 0: recurrence up to x >= 10, then the Stirling series."""
    shift = torch.zeros_like(x)
    for _ in range(10):
        low = x < 10.0
        shift = shift + torch.where(low, torch.log(x), torch.zeros_like(x))
        x = torch.where(low, x + 1.0, x)
    r = 1.0 / x
    r2 = r * r
    series = r * (1.0 / 12 + r2 * (-1.0 / 360 + r2 * (1.0 / 1260 + r2 * (-1.0 / 1680 + r2 * (1.0 / 1188 + r2 * (-691.0 / 360360 + r2 * (1.0 / 156)))))))
    return (x - 0.5) * torch.log(x) - x + 0.5 * math.log(2 * math.pi) + series - shift


def lgamma(x) -> torch.Tensor:
    """log |Gamma(x)|: the positive branch directly, x < 0.5 by reflection; +inf at zero and the negative integers."""
    w, back = _wide(x)
    refl = w < 0.5
    pos = torch.where(refl, 1.0 - w, w)
    lg = _lgamma_pos(pos)
    pole = (w <= 0) & (w == torch.floor(w))
    frac = torch.where(refl & ~pole, w - torch.floor(w), torch.full_like(w, 0.5))     # the unused branch gets a harmless argument (its gradient is discarded)
    s = torch.sin(math.pi * frac)                                   # sin(pi x) up to sign, with the argument reduced first; positive on (0, 1)
    out = torch.where(refl, math.log(math.pi) - torch.log(s) - lg, lg)
    return back(torch.where(pole, torch.full_like(out, float("inf")), out))


def digamma(x) -> torch.Tensor:
    """psi(x): recurrence up to x >= 10 and the asymptotic series; x < 0.5 by reflection; -inf at zero, NaN at the negative integers."""
    w, back = _wide(x)
    refl = w < 0.5
    p = torch.where(refl, 1.0 - w, w)
    acc = torch.zeros_like(p)
    for _ in range(10):
        low = p < 10.0
        acc = acc - torch.where(low, 1.0 / p, torch.zeros_like(p))
        p = torch.where(low, p + 1.0, p)
    r2 = 1.0 / (p * p)
    psi = torch.log(p) - 0.5 / p - r2 * (1.0 / 12 - r2 * (1.0 / 120 - r2 * (1.0 / 252 - r2 * (1.0 / 240 - r2 * (1.0 / 132 - r2 * (691.0 / 32760 - r2 / 12))))))
    psi = psi + acc
    frac = w - torch.floor(w)
    safe = torch.where(refl & (frac != 0), frac, torch.full_like(w, 0.25))
    out = torch.where(refl, psi - math.pi / torch.tan(math.pi * safe), psi)
    out = torch.where(w == 0, torch.full_like(out, float("-inf")), out)
    out = torch.where((w < 0) & (frac == 0), torch.full_like(out, float("nan")), out)
    return back(out)


def sinc(x) -> torch.Tensor:
    """sin(pi x) / (pi x), 1 at zero."""
    w, back = _wide(x)
    px = math.pi * w
    safe = torch.where(w == 0, torch.ones_like(px), px)
    return back(torch.where(w == 0, torch.ones_like(px), torch.sin(safe) / safe))


def xlogy(x, y) -> torch.Tensor:
    """x * log(y) with 0 where x == 0 (NaN in y still propagates)."""
    x, y = torch.as_tensor(x), torch.as_tensor(y)
    dt = torch.result_type(x, y)
    if not dt.is_floating_point:
        dt = torch.get_default_dtype()
    x, y = x.to(dt), y.to(dt)
    zero = (x == 0) & ~torch.isnan(y)
    out = x * torch.log(torch.where(zero, torch.ones_like(y), y))
    return torch.where(zero, torch.zeros_like(out), out)


# ---------------------------------------------------------------------------------------------------------------------
# orthogonal polynomials by their three-term recurrences; n is an int or an integer tensor that broadcasts against x
# ---------------------------------------------------------------------------------------------------------------------
def _recurrence(x, n, p0, p1, step):
    """P_n(x) from P_0, P_1 and ``step(k, x, P_k, P_{k-1}) -> P_{k+1}``; negative n gives 0 (as the substrate does)."""
    x, back = _wide(x)
    return back(_recurrence_wide(x, n, p0, p1, step))


def _recurrence_wide(x, n, p0, p1, step):
    if isinstance(n, torch.Tensor):
        if n.is_floating_point():
            n = n.to(torch.int64)
        x, nb = torch.broadcast_tensors(x, n.to(x.device))
        top = int(nb.max()) if nb.numel() else 0
    else:
        if int(n) != n:
            raise InvalidArgument("polynomial degree must be an integer")
        nb, top = None, int(n)
    a, b = p0(x), p1(x)
    if nb is None:
        if top < 0:
            return torch.zeros_like(x)
        if top == 0:
            return a
        for k in range(1, top):
            a, b = b, step(k, x, b, a)
        return b
    out = torch.where(nb == 0, a, torch.zeros_like(x))
    out = torch.where(nb == 1, b, out)
    for k in range(1, top):
        a, b = b, step(k, x, b, a)
        out = torch.where(nb == k + 1, b, out)
    return out


def _one(x):
    return torch.ones_like(x)


def chebyshev_polynomial_t(x, n):
    return _recurrence(x, n, _one, lambda x: x, lambda k, x, p, q: 2 * x * p - q)


def chebyshev_polynomial_u(x, n):
    return _recurrence(x, n, _one, lambda x: 2 * x, lambda k, x, p, q: 2 * x * p - q)


def chebyshev_polynomial_v(x, n):
    return _recurrence(x, n, _one, lambda x: 2 * x - 1, lambda k, x, p, q: 2 * x * p - q)


def chebyshev_polynomial_w(x, n):
    return _recurrence(x, n, _one, lambda x: 2 * x + 1, lambda k, x, p, q: 2 * x * p - q)


def shifted_chebyshev_polynomial_t(x, n):
    return chebyshev_polynomial_t(2 * torch.as_tensor(x) - 1, n)


def shifted_chebyshev_polynomial_u(x, n):
    return chebyshev_polynomial_u(2 * torch.as_tensor(x) - 1, n)


def shifted_chebyshev_polynomial_v(x, n):
    return chebyshev_polynomial_v(2 * torch.as_tensor(x) - 1, n)


def shifted_chebyshev_polynomial_w(x, n):
    return chebyshev_polynomial_w(2 * torch.as_tensor(x) - 1, n)


def hermite_polynomial_h(x, n):
    """Physicists' Hermite polynomials: H_{k+1} = 2x H_k - 2k H_{k-1}."""
    return _recurrence(x, n, _one, lambda x: 2 * x, lambda k, x, p, q: 2 * x * p - 2 * k * q)


def hermite_polynomial_he(x, n):
    """Probabilists' Hermite polynomials: He_{k+1} = x He_k - k He_{k-1}."""
    return _recurrence(x, n, _one, lambda x: x, lambda k, x, p, q: x * p - k * q)


def laguerre_polynomial_l(x, n):
    return _recurrence(x, n, _one, lambda x: 1 - x, lambda k, x, p, q: ((2 * k + 1 - x) * p - k * q) / (k + 1))


def legendre_polynomial_p(x, n):
    return _recurrence(x, n, _one, lambda x: x, lambda k, x, p, q: ((2 * k + 1) * x * p - k * q) / (k + 1))
