"""``core.linalg`` on the host: the factorisations of the runtime library (Cholesky, pivoted LU, triangular solves, Householder QR, Jacobi
eigen- and singular value decompositions) and everything composed from them, values and gradients against ``torch.linalg`` in f64 and
f32, batched and unbatched, tall / wide / square / rank-deficient, with the error paths."""
import pytest
import torch

from ferrotorch_b200 import core as X
from ferrotorch_b200.core import linalg_impl as M

L = torch.linalg
D = torch.float64
INF = float("inf")


def close(a, b, tol=1e-9, msg=""):
    assert a.shape == b.shape, (msg, a.shape, b.shape)
    assert torch.allclose(a.double(), b.double(), atol=tol, rtol=tol), (msg, (a.double() - b.double()).abs().max().item())


def eye_like(n, ref):
    return torch.eye(n, dtype=ref.dtype).expand(*ref.shape[:-2], n, n)


def test_namespace_points_at_the_own_functions():
    assert X.linalg.cholesky is M.cholesky and X.linalg.qr is not L.qr and X.linalg.eig is M.eig
    a = torch.randn(3, 3, dtype=torch.complex64)
    close(torch.view_as_real(X.linalg.inv(a)), torch.view_as_real(L.inv(a)), 1e-5)          # complex input: the library route
    with pytest.raises(X.linalg.LinAlgError):
        X.linalg.cholesky(-torch.eye(3))


@pytest.mark.parametrize("dt,tol", [(torch.float64, 1e-9), (torch.float32, 2e-4)])
@pytest.mark.parametrize("shape", [(5, 5), (3, 6, 6), (2, 2, 1, 1), (40, 40)])
def test_square_matrix_functions_match_the_library(dt, tol, shape):
    torch.manual_seed(sum(shape))
    n = shape[-1]
    a = torch.randn(shape, dtype=dt)
    spd = a @ a.mT + n * torch.eye(n, dtype=dt)
    b = torch.randn(*shape[:-1], 3, dtype=dt)
    close(M.cholesky(spd), L.cholesky(spd), tol, "cholesky")
    close(M.cholesky(spd, upper=True), L.cholesky(spd, upper=True), tol)
    close(M.solve(a, b), L.solve(a, b), tol * 100, "solve")
    close(M.solve(a, b.mT, left=False), L.solve(a, b.mT, left=False), tol * 100, "solve right")
    close(M.inv(a), L.inv(a), tol * 100, "inv")
    close(M.det(a), L.det(a), tol * 100 * max(1.0, L.det(a).abs().max().item()), "det")
    (s1, l1), (s2, l2) = M.slogdet(a), L.slogdet(a)
    close(s1, s2)
    close(l1, l2, tol * 10)
    P, lo, up = M.lu(a)
    close(P @ lo @ up, a, tol * 10, "lu")
    assert torch.equal(lo, torch.tril(lo)) and torch.equal(up, torch.triu(up))
    (f1, p1), (f2, p2) = M.lu_factor(a), L.lu_factor(a)
    close(f1, f2, tol * 100, "lu_factor")
    assert torch.equal(p1, p2)                                                       # the same pivot choices as LAPACK
    t = torch.triu(a) + 3 * torch.eye(n, dtype=dt)
    close(M.solve_triangular(t, b, upper=True), L.solve_triangular(t, b, upper=True), tol * 10)
    close(M.solve_triangular(t.mT, b, upper=False, unitriangular=True), L.solve_triangular(t.mT, b, upper=False, unitriangular=True), tol * 100)
    bl = torch.randn(*shape[:-2], 3, n, dtype=dt)
    close(M.solve_triangular(t, bl, upper=True, left=False), L.solve_triangular(t, bl, upper=True, left=False), tol * 10)
    sym = a + a.mT
    (w1, v1), (w2, _) = M.eigh(sym), L.eigh(sym)
    close(w1, w2, tol * 10, "eigh")
    close(v1 @ torch.diag_embed(w1) @ v1.mT, sym, tol * 100)
    close(v1.mT @ v1, eye_like(n, sym), tol * 10)
    close(M.eigvalsh(sym, "U"), L.eigvalsh(sym, "U"), tol * 10)
    close(M.matrix_exp(a * 0.3), L.matrix_exp(a * 0.3), tol * 1000, "matrix_exp")
    big = L.matrix_exp(a * 3)
    close(M.matrix_exp(a * 3), big, tol * 1e3 * big.abs().max().item(), "matrix_exp with squaring")
    for k in (3, -2, 0):
        ref = L.matrix_power(a, k)
        close(M.matrix_power(a, k), ref, tol * 1e4 * max(1.0, ref.abs().max().item()), f"matrix_power {k}")
    for p in (None, 2, -2, "fro", "nuc", 1, -1, INF, -INF):
        ref = L.cond(a, p)
        close(M.cond(a, p), ref, tol * 1e4 * max(1.0, ref.abs().max().item()), f"cond {p}")


@pytest.mark.parametrize("dt,tol", [(torch.float64, 1e-9), (torch.float32, 2e-4)])
@pytest.mark.parametrize("shape", [(7, 4), (4, 7), (2, 5, 3), (2, 3, 5), (6, 6), (1, 4), (4, 1)])
def test_rectangular_matrix_functions_match_the_library(dt, tol, shape):
    torch.manual_seed(sum(shape))
    m, n = shape[-2:]
    k = min(m, n)
    a = torch.randn(shape, dtype=dt)
    for mode in ("reduced", "complete"):
        (q, r), (q2, r2) = M.qr(a, mode), L.qr(a, mode)
        assert q.shape == q2.shape and r.shape == r2.shape
        close(q @ r, a, tol * 10, "qr")
        close(q.mT @ q, eye_like(q.shape[-1], a), tol * 10)
        assert torch.equal(r, torch.triu(r))
    close(M.qr(a, "r")[1].abs(), L.qr(a, "r")[1].abs(), tol * 10)
    (u, s, vt), (u2, s2, vt2) = M.svd(a), L.svd(a, full_matrices=False)
    assert u.shape == u2.shape and vt.shape == vt2.shape
    close(s, s2, tol * 10, "svd")
    close(u @ torch.diag_embed(s) @ vt, a, tol * 10)
    close(u.mT @ u, eye_like(k, a), tol * 10)
    close(vt @ vt.mT, eye_like(k, a), tol * 10)
    uf, _, vf = M.svd(a, full_matrices=True)
    close(uf.mT @ uf, eye_like(m, a), tol * 10)
    close(vf @ vf.mT, eye_like(n, a), tol * 10)
    close(M.svdvals(a), L.svdvals(a), tol * 10)
    close(M.pinv(a), L.pinv(a), tol * 100, "pinv")
    assert torch.equal(M.matrix_rank(a), L.matrix_rank(a))
    b = torch.randn(*shape[:-1], 2, dtype=dt)
    close(M.lstsq(a, b).solution, L.lstsq(a, b).solution, tol * 100, "lstsq")
    close(M.lstsq_solve(a, b), L.lstsq(a, b).solution, tol * 100)
    for o in ("fro", "nuc", 2, -2, 1, -1, INF, -INF):
        close(M.matrix_norm(a, o), L.matrix_norm(a, o), tol * 10, f"matrix_norm {o}")
    close(M.matrix_norm(a, "fro", keepdim=True), L.matrix_norm(a, "fro", keepdim=True), tol * 10)
    for o in (2, 1, 0, 3.5, INF, -INF):
        close(M.vector_norm(a, o), L.vector_norm(a, o), tol * 10)
        close(M.vector_norm(a, o, dim=-1, keepdim=True), L.vector_norm(a, o, dim=-1, keepdim=True), tol * 10)


def test_rank_deficient_chains_tensors_and_error_paths():
    torch.manual_seed(0)
    a = torch.randn(6, 2, dtype=D) @ torch.randn(2, 5, dtype=D)
    assert int(M.matrix_rank(a)) == 2
    close(M.pinv(a), L.pinv(a), 1e-8, "pinv of a rank-2 matrix")
    u, s, vt = M.svd(a)
    close(u @ torch.diag_embed(s) @ vt, a, 1e-10)
    close(u.mT @ u, torch.eye(5, dtype=D), 1e-8, "left vectors of zero singular values are completed orthonormally")
    b = torch.randn(6, 3, dtype=D)
    close(M.lstsq(a, b).solution, L.lstsq(a, b, driver="gelsd").solution, 1e-8, "minimum-norm least squares")
    for shapes in (((4,), (4, 30), (30, 2), (2, 50), (50,)), ((3, 4), (4, 30), (30, 2))):
        ms = [torch.randn(sh, dtype=D) for sh in shapes]
        close(M.multi_dot(ms), L.multi_dot(ms), 1e-9)
    x, y = torch.randn(4, 3, dtype=D), torch.randn(4, 3, dtype=D)
    close(M.cross(x, y), L.cross(x, y))
    close(M.cross(x.t(), y.t(), dim=0), L.cross(x.t(), y.t(), dim=0))
    t = torch.randn(4, 6, 8, 3, dtype=D)
    close(M.tensorinv(t, 2), L.tensorinv(t, 2), 1e-8)
    ta, tb = torch.randn(2, 3, 6, 4, 9, dtype=D), torch.randn(2, 3, 6, dtype=D)
    close(M.tensorsolve(ta, tb), L.tensorsolve(ta, tb), 1e-7)
    sm = torch.randn(5, 5, dtype=D)
    sm = sm + sm.mT + 10 * torch.eye(5, dtype=D)
    ld, piv = M.ldl_factor(sm)
    lower = torch.tril(ld, -1) + torch.eye(5, dtype=D)
    close(lower @ torch.diag(torch.diagonal(ld)) @ lower.mT, sm, 1e-10, "ldl")
    bb = torch.randn(5, 2, dtype=D)
    close(M.ldl_solve(ld, piv, bb), L.solve(sm, bb), 1e-10)
    close(L.ldl_solve(ld, piv, bb), L.solve(sm, bb), 1e-10)                           # the compact form is the library's
    h, tau = torch.geqrf(torch.randn(6, 4, dtype=D))
    close(M.householder_product(h, tau), L.householder_product(h, tau), 1e-10)
    close(M.diagonal(t, 1, 0, 2), torch.diagonal(t, 1, 0, 2))
    for bad in (lambda: M.cholesky(-torch.eye(3)), lambda: M.solve(torch.zeros(3, 3), torch.ones(3)), lambda: M.inv(torch.ones(2, 2)), lambda: M.det(torch.randn(2, 3)),
                lambda: M.qr(torch.randn(3, 3), "x"), lambda: M.eigh(torch.eye(2), "X"), lambda: M.multi_dot([torch.eye(2)]), lambda: M.cross(torch.ones(2), torch.ones(2)),
                lambda: M.tensorinv(torch.randn(2, 3, 4)), lambda: M.ldl_factor(torch.zeros(2, 2)), lambda: M.matrix_norm(torch.eye(2), 3)):
        with pytest.raises(Exception):
            bad()
    assert int(M.cholesky_ex(-torch.eye(3))[1]) == 1 and int(M.inv_ex(torch.ones(2, 2))[1]) > 0 and int(M.solve_ex(torch.eye(2), torch.ones(2))[1]) == 0
    assert float(M.det(torch.ones(2, 2))) == 0.0


def _grads(f, *xs):
    xs = [x.clone().requires_grad_() for x in xs]
    return torch.autograd.grad(f(*xs), xs)


def _same_grads(name, ours, theirs, *xs, tol=1e-8):
    for a, b in zip(_grads(ours, *xs), _grads(theirs, *xs)):
        assert a.shape == b.shape and torch.allclose(a, b, atol=tol, rtol=tol), (name, (a - b).abs().max().item())


@pytest.mark.parametrize("shape", [(4, 4), (3, 5, 5)])
def test_gradients_of_square_matrix_functions(shape):
    torch.manual_seed(1)
    n = shape[-1]
    a = torch.randn(shape, dtype=D)
    spd = a @ a.mT + n * torch.eye(n, dtype=D)
    w, b = torch.randn(shape, dtype=D), torch.randn(*shape[:-1], 2, dtype=D)
    wb = torch.randn_like(b)
    _same_grads("cholesky", lambda x: (M.cholesky(x) * w).sum(), lambda x: (L.cholesky(x) * w).sum(), spd)
    _same_grads("cholesky upper", lambda x: (M.cholesky(x, upper=True) * w).sum(), lambda x: (L.cholesky(x, upper=True) * w).sum(), spd)
    _same_grads("solve", lambda x, y: (M.solve(x, y) * wb).sum(), lambda x, y: (L.solve(x, y) * wb).sum(), a, b)
    _same_grads("solve, vector", lambda x, y: (M.solve(x, y) * wb[..., 0]).sum(), lambda x, y: (L.solve(x, y) * wb[..., 0]).sum(), a, b[..., 0].contiguous())
    a0 = a if a.dim() == 2 else a[0]
    _same_grads("solve, broadcast", lambda x, y: (M.solve(x, y) ** 2).sum(), lambda x, y: (L.solve(x, y) ** 2).sum(), a0, b)
    _same_grads("inv", lambda x: (M.inv(x) * w).sum(), lambda x: (L.inv(x) * w).sum(), a)
    _same_grads("det", lambda x: M.det(x).sum(), lambda x: L.det(x).sum(), a)
    _same_grads("slogdet", lambda x: M.slogdet(x)[1].sum(), lambda x: L.slogdet(x)[1].sum(), a)
    t = torch.triu(a) + 3 * torch.eye(n, dtype=D)
    _same_grads("solve_triangular", lambda x, y: (M.solve_triangular(x, y, upper=True) * wb).sum(), lambda x, y: (L.solve_triangular(x, y, upper=True) * wb).sum(), t, b)
    _same_grads("solve_triangular, unit lower", lambda x, y: (M.solve_triangular(x, y, upper=False, unitriangular=True) * wb).sum(),
                lambda x, y: (L.solve_triangular(x, y, upper=False, unitriangular=True) * wb).sum(), t.mT.contiguous(), b)
    sym, ar = a + a.mT, torch.arange(n, dtype=D)
    _same_grads("eigh values", lambda x: (M.eigh(x)[0] ** 2 * ar).sum(), lambda x: (L.eigh(x)[0] ** 2 * ar).sum(), sym)
    _same_grads("eigh vectors", lambda x: ((M.eigh(x)[1] ** 2) * w).sum(), lambda x: ((L.eigh(x)[1] ** 2) * w).sum(), sym)     # squares: free of the sign choice
    _same_grads("matrix_exp", lambda x: (M.matrix_exp(x) * w).sum(), lambda x: (L.matrix_exp(x) * w).sum(), a * 0.5, tol=1e-7)
    _same_grads("matrix_power", lambda x: (M.matrix_power(x, 3) * w).sum(), lambda x: (L.matrix_power(x, 3) * w).sum(), a)
    _same_grads("cond", lambda x: M.cond(x).sum(), lambda x: L.cond(x).sum(), a, tol=1e-6)


@pytest.mark.parametrize("shape", [(6, 4), (4, 6), (2, 5, 3), (2, 3, 5), (4, 4)])
def test_gradients_of_rectangular_matrix_functions(shape):
    torch.manual_seed(2)
    m, n = shape[-2:]
    k = min(m, n)
    a = torch.randn(shape, dtype=D)
    wa, ar = torch.randn(shape, dtype=D), torch.arange(m, dtype=D)

    def qr_loss(fn):                                 # built from Q R, R^T R and Q Q^T: free of the sign choice of the columns
        return lambda x: (lambda q, r: ((q @ r) * wa).sum() + (r.mT @ r).pow(2).sum() + ((q @ q.mT) * ar).sum())(*fn(x))
    _same_grads("qr", qr_loss(M.qr), qr_loss(L.qr), a, tol=1e-7)
    ws, wu, wv = torch.randn(*shape[:-2], k, dtype=D), torch.randn(*shape[:-2], m, k, dtype=D), torch.randn(*shape[:-2], k, n, dtype=D)
    _same_grads("svd values", lambda x: (M.svd(x)[1] * ws).sum(), lambda x: (L.svd(x, full_matrices=False)[1] * ws).sum(), a)

    def svd_loss(fn):
        return lambda x: (lambda u, s, vt: ((u ** 2) * wu).sum() + ((vt ** 2) * wv).sum() + (s ** 3).sum())(*fn(x))
    _same_grads("svd vectors", svd_loss(M.svd), svd_loss(lambda x: L.svd(x, full_matrices=False)), a, tol=1e-7)
    wp = torch.randn(*shape[:-2], n, m, dtype=D)
    _same_grads("pinv", lambda x: (M.pinv(x) * wp).sum(), lambda x: (L.pinv(x) * wp).sum(), a, tol=1e-7)
    b = torch.randn(*shape[:-1], 2, dtype=D)
    _same_grads("lstsq", lambda x, y: (M.lstsq(x, y).solution ** 2).sum(), lambda x, y: (L.lstsq(x, y).solution ** 2).sum(), a, b, tol=1e-7)
    for o in ("fro", "nuc", 2, 1, INF):
        _same_grads(f"matrix_norm {o}", lambda x: M.matrix_norm(x, o).sum(), lambda x: L.matrix_norm(x, o).sum(), a, tol=1e-7)


def test_householder_product_gradient_and_dtype_of_gradients():
    torch.manual_seed(3)
    h, tau = torch.geqrf(torch.randn(6, 4, dtype=D))
    wh = torch.randn(6, 4, dtype=D)
    _same_grads("householder_product", lambda v, t: (M.householder_product(v, t) * wh).sum(), lambda v, t: (L.householder_product(v, t) * wh).sum(), h, tau)
    x = torch.randn(4, 4, requires_grad=True)
    M.inv(x).sum().backward()
    assert x.grad.dtype == torch.float32


def _sorted_eigs(w):
    flat = w.reshape(-1, w.shape[-1])
    rows = []
    for r in flat:
        order = sorted(range(len(r)), key=lambda i: (round(r[i].real.item(), 5), round(r[i].imag.item(), 5)))
        rows.append(r[order])
    return torch.stack(rows)


@pytest.mark.parametrize("dt,tol", [(torch.float64, 1e-9), (torch.float32, 2e-4)])
@pytest.mark.parametrize("shape", [(1, 1), (2, 2), (3, 3), (6, 6), (4, 5, 5), (30, 30), (64, 64)])
def test_general_eigenproblem_through_the_complex_schur_form(dt, tol, shape):
    """Eigenvalues equal the library's as a set; every returned pair satisfies A v = lambda v with a unit vector whose largest component
    is real and positive."""
    torch.manual_seed(sum(shape))
    a = torch.randn(shape, dtype=dt)
    (w, v), (w2, v2) = M.eig(a), L.eig(a)
    assert w.dtype == w2.dtype and v.shape == v2.shape and v.dtype == v2.dtype
    assert (a.to(v.dtype) @ v - v * w.unsqueeze(-2)).abs().max() < tol * 50 * max(1.0, a.abs().max().item() * shape[-1])
    assert ((v.abs() ** 2).sum(-2).sqrt() - 1).abs().max() < tol * 10
    assert (_sorted_eigs(w) - _sorted_eigs(w2)).abs().max() < tol * 1000
    assert (_sorted_eigs(M.eigvals(a)) - _sorted_eigs(w2)).abs().max() < tol * 1000
    big = v.abs().argmax(-2, keepdim=True)
    lead = v.gather(-2, big)
    assert lead.imag.abs().max() < tol * 10 and (lead.real > 0).all()


def test_general_eigenproblem_special_matrices_and_routes():
    rot = torch.tensor([[0.0, 1.0], [-1.0, 0.0]], dtype=D)
    w = M.eigvals(rot)
    assert torch.allclose(_sorted_eigs(w)[0], torch.tensor([-1j, 1j], dtype=torch.complex128))
    for a in (torch.zeros(3, 3, dtype=D), torch.eye(4, dtype=D), torch.tensor([[2.0, 1.0], [0.0, 2.0]], dtype=D), torch.triu(torch.randn(5, 5, dtype=D))):
        w, v = M.eig(a)
        assert (a.to(v.dtype) @ v - v * w.unsqueeze(-2)).abs().max() < 1e-12
        assert torch.allclose(_sorted_eigs(w)[0].real, torch.sort(torch.diagonal(a)).values)
    sym = torch.randn(6, 6, dtype=D)
    sym = sym + sym.T
    assert torch.allclose(torch.sort(M.eigvals(sym).real).values, M.eigvalsh(sym), atol=1e-10) and M.eigvals(sym).imag.abs().max() < 1e-10
    g = torch.randn(4, 4, dtype=D, requires_grad=True)                  # a derivative is asked: the library call carries it
    M.eig(g)[0].abs().sum().backward()
    assert g.grad is not None and g.grad.shape == (4, 4)
    with pytest.raises(Exception):
        M.eig(torch.randn(2, 3))
