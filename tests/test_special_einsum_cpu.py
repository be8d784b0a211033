"""The special functions and the Einstein summation of ``core`` are written out in this package (series / continued fractions / recurrences;
parse + diagonal + pairwise batched products): values, gradients and edge cases against the substrate's library functions."""
import pytest
import torch

from ferrotorch_b200 import core as X
from ferrotorch_b200.core import einsum_impl, special_fns as S


def _rel(got, want, floor=1.0):
    fin = torch.isfinite(want) & torch.isfinite(got)
    return ((got - want)[fin].abs() / want[fin].abs().clamp(min=floor)).max().item()


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 2e-12), (torch.float32, 2e-6)])
def test_error_and_gamma_functions_match_the_library(dtype, tol):
    x = torch.cat([torch.linspace(-6, 6, 1201), torch.tensor([0.0, 1e-8, -1e-8, 1.9999, 2.0, 2.0001, 10.0, -10.0, 27.0])]).to(dtype)
    assert (S.erf(x) - torch.erf(x)).abs().max() < tol and (S.erfc(x) - torch.erfc(x)).abs().max() < tol
    big = torch.tensor([3.0, 5.0, 8.0, 12.0], dtype=dtype)
    assert _rel(S.erfc(big), torch.erfc(big), floor=torch.finfo(dtype).tiny) < (1e-11 if dtype == torch.float64 else 1e-5)      # the tail keeps its relative accuracy
    p = torch.cat([torch.linspace(-0.999999, 0.999999, 2001), torch.tensor([0.0, 1 - 1e-7, 1e-30])]).to(dtype)
    assert _rel(S.erfinv(p), torch.erfinv(p), floor=1e-30) < (1e-10 if dtype == torch.float64 else 1e-5)
    edge = S.erfinv(torch.tensor([1.0, -1.0, 1.5, -2.0], dtype=dtype))
    assert edge[0] == float("inf") and edge[1] == float("-inf") and torch.isnan(edge[2:]).all()
    g = torch.cat([torch.linspace(-9.7, 30, 1501), torch.tensor([1e-6, 0.5, 1.0, 2.0, 100.0, 1e5, -0.5, -2.5])]).to(dtype)
    assert _rel(S.lgamma(g), torch.lgamma(g)) < tol * 10 and _rel(S.digamma(g), torch.digamma(g)) < tol * 50
    poles = torch.tensor([0.0, -1.0, -3.0], dtype=dtype)
    assert torch.isinf(S.lgamma(poles)).all() and S.digamma(poles)[0] == float("-inf") and torch.isnan(S.digamma(poles)[1:]).all()
    z = torch.linspace(-3, 3, 601).to(dtype)
    assert (S.sinc(z) - torch.sinc(z)).abs().max() < tol
    a, b = torch.tensor([0.0, 2.0, 0.0, 3.0], dtype=dtype), torch.tensor([0.0, 3.0, float("nan"), 0.5], dtype=dtype)
    assert torch.allclose(S.xlogy(a, b), torch.xlogy(a, b), equal_nan=True)
    assert X.special.erf is not torch.erf and X.special.lgamma is not torch.lgamma                     # the namespace points at the own forms


def test_special_functions_are_differentiable():
    x = torch.tensor([-1.3, -0.2, 0.4, 1.7, 2.6], dtype=torch.float64, requires_grad=True)
    for ours, theirs in ((S.erf, torch.erf), (S.erfc, torch.erfc), (S.sinc, torch.sinc)):
        ga, = torch.autograd.grad(ours(x).sum(), x)
        gb, = torch.autograd.grad(theirs(x).sum(), x)
        assert torch.allclose(ga, gb, atol=1e-10)
    p = torch.tensor([0.7, 1.5, 3.2, 8.0, 15.0], dtype=torch.float64, requires_grad=True)
    for ours, theirs in ((S.lgamma, torch.lgamma), (S.digamma, torch.digamma)):
        ga, = torch.autograd.grad(ours(p).sum(), p)
        gb, = torch.autograd.grad(theirs(p).sum(), p)
        assert torch.allclose(ga, gb, atol=1e-9)
    q = torch.tensor([-0.8, -0.1, 0.3, 0.9], dtype=torch.float64, requires_grad=True)
    ga, = torch.autograd.grad(S.erfinv(q).sum(), q)
    gb, = torch.autograd.grad(torch.erfinv(q).sum(), q)
    assert torch.allclose(ga, gb, rtol=1e-6)


@pytest.mark.parametrize("name", ["chebyshev_polynomial_t", "chebyshev_polynomial_u", "chebyshev_polynomial_v", "chebyshev_polynomial_w", "hermite_polynomial_h",
                                  "hermite_polynomial_he", "laguerre_polynomial_l", "legendre_polynomial_p", "shifted_chebyshev_polynomial_t",
                                  "shifted_chebyshev_polynomial_u", "shifted_chebyshev_polynomial_v", "shifted_chebyshev_polynomial_w"])
def test_orthogonal_polynomials_match_the_library(name):
    ours, theirs = getattr(X.special, name), getattr(torch.special, name)
    xs = torch.linspace(-1.2, 1.2, 101, dtype=torch.float64)
    for n in (0, 1, 2, 3, 7, 12):
        assert _rel(ours(xs, n), theirs(xs, torch.tensor(n))) < 1e-11, n
    nt = torch.randint(0, 9, (101,), generator=torch.Generator().manual_seed(0))
    assert _rel(ours(xs, nt), theirs(xs, nt)) < 1e-11
    assert _rel(ours(xs.float(), 5), theirs(xs.float(), torch.tensor(5))) < 1e-5 and ours(xs.float(), 5).dtype == torch.float32
    assert torch.equal(ours(xs, -1), torch.zeros_like(xs))
    g = xs.clone().requires_grad_()
    ga, = torch.autograd.grad(ours(g, 4).sum(), g)
    eps = 1e-6
    assert torch.allclose(ga, (ours(xs + eps, 4) - ours(xs - eps, 4)) / (2 * eps), atol=1e-5)


EINSUM_CASES = [("ij,jk->ik", (3, 4), (4, 5)), ("ij,jk", (3, 4), (4, 5)), ("bij,bjk->bik", (2, 3, 4), (2, 4, 5)), ("ii->i", (4, 4)), ("ii", (4, 4)), ("ij->ji", (3, 4)),
                ("ij->", (3, 4)), ("i,j->ij", (3,), (4,)), ("...ij,...jk->...ik", (2, 5, 3, 4), (2, 5, 4, 6)), ("bhqd,bhkd->bhqk", (2, 3, 4, 8), (2, 3, 5, 8)),
                ("ij,ij,ij->i", (3, 4), (3, 4), (3, 4)), ("abc,cd,de->abe", (2, 3, 4), (4, 5), (5, 6)), ("i,i->", (5,), (5,)), ("...,...->...", (3, 4), (3, 4)),
                ("ij...,j->i...", (3, 4, 2, 2), (4,)), ("iji->j", (3, 4, 3)), ("bn,anm,bm->ba", (2, 3), (5, 3, 4), (2, 4)), ("ab,cd->abcd", (2, 3), (4, 5)),
                ("a...b,b->a...", (2, 3, 4), (4,)), ("ij,kj->ik", (3, 1), (5, 4)), ("i->", (6,)), ("ijk->kji", (2, 3, 4)), (" i j , j k -> i k ", (2, 3), (3, 2))]


@pytest.mark.parametrize("case", EINSUM_CASES, ids=[c[0].strip() for c in EINSUM_CASES])
def test_einsum_values_and_gradients(case):
    eq, *shapes = case
    torch.manual_seed(0)
    ops = [torch.randn(s, dtype=torch.float64, requires_grad=True) for s in shapes]
    got, want = X.einsum(eq, *ops), torch.einsum(eq, *ops)
    assert got.shape == want.shape and torch.allclose(got, want, atol=1e-12)
    w = torch.randn_like(want)
    ga, gb = torch.autograd.grad((got * w).sum(), ops), torch.autograd.grad((want * w).sum(), ops)
    assert all(torch.allclose(a, b, atol=1e-12) for a, b in zip(ga, gb))


def test_einsum_dtypes_lists_and_errors():
    ia, ib = torch.randint(0, 5, (3, 4)), torch.randint(0, 5, (4, 2))
    assert torch.equal(X.einsum("ij,jk->ik", ia, ib), ia @ ib)
    a, b = torch.randn(3, 4), torch.randn(4, 5, dtype=torch.float64)
    assert X.einsum("ij,jk->ik", a, b).dtype == torch.float64
    assert torch.allclose(X.einsum("ij,jk->ik", [a.double(), b]), a.double() @ b)
    c = torch.randn(2, 3, dtype=torch.complex64)
    assert torch.allclose(X.einsum("ij,kj->ik", c, c.conj()), c @ c.conj().t(), atol=1e-5)
    for eq, shapes in (("ij,jk->ik", [(3, 4), (5, 6)]), ("ij->k", [(2, 3)]), ("ij,jk", [(3, 4)]), ("ii->i", [(3, 4)]), ("ij->ii", [(2, 2)]), ("i.j->ij", [(2, 2)]),
                       ("ij", [(2, 3, 4)])):
        with pytest.raises(Exception):
            einsum_impl.einsum(eq, *[torch.randn(s) for s in shapes])
    assert X.einsum_differentiable is X.einsum


def test_einops_patterns_match_the_einops_package():
    einops = pytest.importorskip("einops")
    torch.manual_seed(0)
    x = torch.randn(2, 6, 8, 10, dtype=torch.float64, requires_grad=True)
    cases = [("rearrange", "b c h w -> b h w c", {}), ("rearrange", "b c (h p) (w q) -> b (h w) (p q c)", dict(p=2, q=5)), ("rearrange", "b c h w -> (b c) (h w)", {}),
             ("rearrange", "b (g c) h w -> g b c h w", dict(g=3)), ("rearrange", "... h w -> ... (h w)", {}), ("rearrange", "b ... -> ... b", {}),
             ("rearrange", "b c h w -> b c h w 1", {}), ("rearrange", "b c h w -> b 1 (c h w)", {}), ("rearrange", "b c h (w w2) -> b c (h w2) w", dict(w2=2)),
             ("repeat", "b c h w -> b c h w r", dict(r=3)), ("repeat", "b c h w -> b (c r) h w", dict(r=2)), ("repeat", "b c h w -> (r b) c (h s) w", dict(r=2, s=3)),
             ("repeat", "... -> ... 2", {}), ("reduce", "b c h w -> b c", "mean", {}), ("reduce", "b c h w -> b c", "max", {}),
             ("reduce", "b c (h p) (w q) -> b c h w", "sum", dict(p=2, q=2)), ("reduce", "b c h w -> b 1 h w", "min", {}), ("reduce", "b c h w -> (b c)", "prod", {}),
             ("reduce", "... w -> ...", "sum", {}), ("reduce", "b c h w -> b c h w", "mean", {})]
    for kind, pattern, *rest in cases:
        if kind == "reduce":
            got, want = X.reduce(x, pattern, rest[0], **rest[1]), einops.reduce(x, pattern, rest[0], **rest[1])
        else:
            got, want = getattr(X, kind)(x, pattern, **rest[0]), getattr(einops, kind)(x, pattern, **rest[0])
        assert got.shape == want.shape and torch.allclose(got, want), pattern
        w = torch.randn_like(want)
        ga, = torch.autograd.grad((got * w).sum(), x)
        gb, = torch.autograd.grad((want * w).sum(), x)
        assert torch.allclose(ga, gb), pattern
    y = torch.randn(3, 1, 5)
    assert torch.equal(X.rearrange(y, "a 1 c -> a c"), y[:, 0]) and torch.equal(X.rearrange(y, "a () c -> c a"), y[:, 0].t())
    assert torch.equal(X.rearrange_with(torch.arange(24.0).view(2, 12), "b (h w) -> b h w", h=3), torch.arange(24.0).view(2, 3, 4))
    for bad in ("b c -> b", "b c h w -> b c h", "b (c d) h w -> b c d h w", "b c h w -> b c h w z", "b (c h w -> b", "b b h w -> b h w", "b c h w"):
        with pytest.raises(Exception):
            X.rearrange(x, bad)
    with pytest.raises(Exception):
        X.repeat(x, "b c h w -> b c h")
    with pytest.raises(Exception):
        X.reduce(x, "b c h w -> b c", "median")


def test_window_functions_from_their_formulas():
    """Every window against ``torch.signal.windows`` (symmetric and periodic, lengths 0, 1, 2 and up) and, where the substrate has none,
    against scipy."""
    sw = pytest.importorskip("scipy.signal.windows")
    W, T = X.windows, torch.signal.windows
    for M in (0, 1, 2, 7, 16, 65):
        for sym in (True, False):
            for name, kw in (("hann", {}), ("hamming", {}), ("blackman", {}), ("nuttall", {}), ("bartlett", {}), ("cosine", {}), ("gaussian", {"std": 2.5}),
                             ("kaiser", {"beta": 8.6}), ("kaiser", {"beta": 0.0}), ("kaiser", {"beta": 40.0}), ("general_hamming", {"alpha": 0.6}),
                             ("general_cosine", {"a": [0.5, 0.3, 0.2]}), ("exponential", {"tau": 3.0})):
                got, want = getattr(W, name)(M, sym=sym, dtype=torch.float64, **kw), getattr(T, name)(M, sym=sym, dtype=torch.float64, **kw)
                assert got.shape == want.shape and torch.allclose(got, want, atol=1e-12), (name, M, sym)
    assert torch.allclose(W.exponential(9, center=2.0, tau=2.0, sym=False, dtype=torch.float64), T.exponential(9, center=2.0, tau=2.0, sym=False, dtype=torch.float64))
    assert W.hann(8).dtype == torch.float32 and W.hanning is W.hann and W.hann is not T.hann
    for M in (15, 16):
        assert torch.allclose(W.parzen(M).double(), torch.tensor(sw.parzen(M)), atol=1e-6)
        assert torch.allclose(W.tukey(M, 0.4).double(), torch.tensor(sw.tukey(M, 0.4)), atol=1e-6)
        assert torch.allclose(W.taylor(M).double(), torch.tensor(sw.taylor(M)), atol=1e-6)
        assert torch.allclose(W.taylor(M, 5, 40.0, False).double(), torch.tensor(sw.taylor(M, 5, 40, norm=False)), atol=1e-6)
    for bad in (lambda: W.gaussian(8, std=0.0), lambda: W.exponential(8, center=1.0), lambda: W.kaiser(8, beta=-1.0), lambda: W.hann(-1)):
        with pytest.raises(Exception):
            bad()


def _same(a, b, tol=1e-9):
    assert a.shape == b.shape and a.dtype == b.dtype, (a.shape, b.shape, a.dtype, b.dtype)
    assert torch.allclose(a, b, atol=tol, rtol=tol), (a - b).abs().max()


@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 7, 8, 12, 16, 17, 30, 64, 100, 127, 128, 243])
def test_one_dimensional_transforms_match_the_library(n):
    """Power-of-two lengths take the radix-2 butterflies, all others Bluestein's form; complex, real, half-spectrum and Hermitian variants,
    every normalisation, padding and trimming."""
    F, T = X.fft, torch.fft
    torch.manual_seed(n)
    x, r = torch.randn(3, n, dtype=torch.complex128), torch.randn(3, n, dtype=torch.float64)
    for norm in (None, "ortho", "forward"):
        _same(F.fft(x, norm=norm), T.fft(x, norm=norm))
        _same(F.ifft(x, norm=norm), T.ifft(x, norm=norm))
        _same(F.fft(r, norm=norm), T.fft(r, norm=norm))
        _same(F.rfft(r, norm=norm), T.rfft(r, norm=norm))
        _same(F.ihfft(r, norm=norm), T.ihfft(r, norm=norm))
        h = torch.randn(3, n // 2 + 1, dtype=torch.complex128)
        for m in (None, n, n + 1, max(1, n - 1)):
            if m is None and n // 2 + 1 < 2:
                continue
            _same(F.irfft(h, m, norm=norm), T.irfft(h, m, norm=norm))
            _same(F.hfft(h, m, norm=norm), T.hfft(h, m, norm=norm))
    for m in (max(1, n - 2), n + 3):
        _same(F.fft(x, m), T.fft(x, m))
        _same(F.rfft(r, m), T.rfft(r, m))
    _same(F.fft(x.t(), dim=0), T.fft(x.t(), dim=0))
    assert F.fft is not T.fft


def test_multi_dimensional_transforms_grids_shifts_and_gradients():
    F, T = X.fft, torch.fft
    torch.manual_seed(0)
    y, yr = torch.randn(2, 6, 5, 8, dtype=torch.complex128), torch.randn(2, 6, 5, 8, dtype=torch.float64)
    for ours, theirs in ((F.fft2, T.fft2), (F.ifft2, T.ifft2), (F.fftn, T.fftn), (F.ifftn, T.ifftn)):
        _same(ours(y), theirs(y))
    _same(F.fftn(y, s=(4, 9), dim=(1, 3)), T.fftn(y, s=(4, 9), dim=(1, 3)))
    _same(F.fftn(y, dim=(0, 2), norm="ortho"), T.fftn(y, dim=(0, 2), norm="ortho"))
    _same(F.fft2(yr), T.fft2(yr))
    _same(F.rfftn(yr), T.rfftn(yr))
    _same(F.rfftn(yr, s=(7, 6)), T.rfftn(yr, s=(7, 6)))
    _same(F.rfftn(yr, dim=(1, 2)), T.rfftn(yr, dim=(1, 2)))
    z = T.rfftn(yr)
    _same(F.irfftn(z), T.irfftn(z))
    _same(F.irfftn(z, s=(5, 8)), T.irfftn(z, s=(5, 8)))
    _same(F.irfftn(z, s=(5, 9), dim=(2, 3)), T.irfftn(z, s=(5, 9), dim=(2, 3)))
    for n in (1, 4, 7, 8):
        _same(F.fftfreq(n, 0.5), T.fftfreq(n, 0.5), 1e-7)
        _same(F.rfftfreq(n, 0.25), T.rfftfreq(n, 0.25), 1e-7)
    _same(F.fftshift(yr), T.fftshift(yr))
    _same(F.ifftshift(yr, dim=(1, 3)), T.ifftshift(yr, dim=(1, 3)))
    _same(F.fftshift(yr, dim=2), T.fftshift(yr, dim=2))
    x32 = torch.randn(4, 100)
    _same(F.rfft(x32), T.rfft(x32), 1e-4)
    _same(F.fft(x32.to(torch.complex64)), T.fft(x32.to(torch.complex64)), 1e-4)
    long = torch.randn(10007, dtype=torch.complex128)                     # a prime length: the chirp phases stay accurate
    assert (F.fft(long) - T.fft(long)).abs().max() < 1e-10
    a, w = torch.randn(2, 12, dtype=torch.float64, requires_grad=True), torch.randn(2, 7, dtype=torch.complex128)
    _same(*[torch.autograd.grad((f(a) * w).abs().sum(), a)[0] for f in (F.rfft, T.rfft)])
    c = torch.randn(2, 9, dtype=torch.complex128, requires_grad=True)
    _same(*[torch.autograd.grad(f(c).abs().sum(), c)[0] for f in (F.ifft, T.ifft)])
    hh = torch.randn(2, 7, dtype=torch.complex128, requires_grad=True)
    _same(*[torch.autograd.grad((f(hh, 12) ** 2).sum(), hh)[0] for f in (F.irfft, T.irfft)])
    for bad in (lambda: F.fft(torch.randn(4), norm="unitary"), lambda: F.rfft(y), lambda: F.fft(torch.randn(4), 0), lambda: F.fftn(y, dim=(1, 1)), lambda: F.fftfreq(0)):
        with pytest.raises(Exception):
            bad()
