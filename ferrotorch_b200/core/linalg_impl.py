"""Linear algebra of ``core.linalg``: the factorisations run in the host runtime library (``csrc/runtime/linalg.cpp``: Cholesky, pivoted LU,
triangular solves, Householder QR, Jacobi eigen- and singular value decompositions, f64, batched and threaded) with the derivative
formulas written here; everything else (determinants, inverses, least squares, pseudo-inverse, norms, rank, condition numbers, powers, the
matrix exponential, chain products, ...) is composed from them, so it is differentiable by composition.

Real f32 / f64 tensors on the host take this route (``eig`` / ``eigvals`` of general matrices too, through a complex Schur form, when no
derivative is asked of them). CUDA tensors, complex and half types go to the substrate's library call of the same name (cuSOLVER / LAPACK).

Reference parity: ferrotorch-core/src/linalg.rs:121-2170 (35 functions) and grad_fns/linalg.rs:777-1780 (their derivatives).
"""
from __future__ import annotations

import ctypes
import math
from typing import NamedTuple, Optional, Sequence

import torch
from torch.autograd.function import once_differentiable

from ..errors import InvalidArgument

L = torch.linalg


class LinAlgError(InvalidArgument):
    pass


# ---------------------------------------------------------------------------------------------------------------------
# plumbing
# ---------------------------------------------------------------------------------------------------------------------
_rt_cache = None


def _rt():
    global _rt_cache
    if _rt_cache is None:
        from .. import _lib
        rt = _lib.runtime()
        for n in ("ft_la_cholesky", "ft_la_lu", "ft_la_lu_solve", "ft_la_trsm", "ft_la_qr", "ft_la_eigh", "ft_la_svd"):
            getattr(rt, n).restype = ctypes.c_int
        _rt_cache = rt
    return _rt_cache


def _own(*ts: torch.Tensor) -> bool:
    """True when the native route takes these operands: real f32 / f64 on the host."""
    return all(isinstance(t, torch.Tensor) and t.device.type == "cpu" and t.dtype in (torch.float32, torch.float64) for t in ts)


def _p(t: torch.Tensor):
    return ctypes.c_void_p(t.data_ptr())


def _f64(t: torch.Tensor) -> torch.Tensor:
    """A private contiguous f64 copy (the kernels work in place)."""
    return t.detach().to(torch.float64).contiguous().clone()


def _square(a: torch.Tensor, name: str) -> None:
    if a.dim() < 2 or a.shape[-1] != a.shape[-2]:
        raise InvalidArgument(f"linalg.{name}: expected square matrices, got shape {tuple(a.shape)}")


def _batch(a: torch.Tensor) -> int:
    n = 1
    for s in a.shape[:-2]:
        n *= s
    return n


def _i64(v) -> ctypes.c_int64:
    return ctypes.c_int64(int(v))


def _trsm(t64: torch.Tensor, b64: torch.Tensor, upper: bool, trans: bool, unit: bool = False) -> torch.Tensor:
    """op(T)^-1 B for f64 contiguous [.., n, n] and [.., n, k] of equal batch shape; returns a new tensor."""
    out = b64.contiguous().clone()
    n, k = out.shape[-2], out.shape[-1]
    if n and k:
        _rt().ft_la_trsm(_p(t64.contiguous()), _p(out), _i64(_batch(out)), _i64(n), _i64(k), ctypes.c_int(upper), ctypes.c_int(trans), ctypes.c_int(unit))
    return out


def _lu_raw(a: torch.Tensor):
    lu = _f64(a)
    m, n = lu.shape[-2], lu.shape[-1]
    r = min(m, n)
    piv = torch.zeros(*lu.shape[:-2], r, dtype=torch.int32)
    info = torch.zeros(lu.shape[:-2], dtype=torch.int32)
    if m and n and _batch(lu):
        _rt().ft_la_lu(_p(lu), _i64(_batch(lu)), _i64(m), _i64(n), _p(piv), _p(info))
    return lu, piv, info


def _lu_solve_raw(lu: torch.Tensor, piv: torch.Tensor, b64: torch.Tensor, trans: bool) -> torch.Tensor:
    out = b64.contiguous().clone()
    n, k = out.shape[-2], out.shape[-1]
    if n and k and _batch(out):
        _rt().ft_la_lu_solve(_p(lu), _p(piv), _p(out), _i64(_batch(out)), _i64(n), _i64(k), ctypes.c_int(trans))
    return out


def _check(info: torch.Tensor, what: str) -> None:
    if bool((info != 0).any()):
        k = int(info[info != 0].flatten()[0])
        raise LinAlgError(f"linalg.{what}: the input is singular or not positive definite (order {k})")


# ---------------------------------------------------------------------------------------------------------------------
# Cholesky
# ---------------------------------------------------------------------------------------------------------------------
class _Cholesky(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, check):
        l64 = _f64(a)
        info = torch.zeros(a.shape[:-2], dtype=torch.int32)
        if a.shape[-1] and _batch(a):
            _rt().ft_la_cholesky(_p(l64), _i64(_batch(a)), _i64(a.shape[-1]), _p(info))
        if check:
            _check(info, "cholesky")
        ctx.save_for_backward(l64)
        ctx.dtype = a.dtype
        ctx.mark_non_differentiable(info)
        return l64.to(a.dtype), info

    @staticmethod
    @once_differentiable
    def backward(ctx, g, _ginfo):
        (l,) = ctx.saved_tensors
        g = g.to(torch.float64)
        p = torch.tril(l.mT @ g)
        p = p - 0.5 * torch.diag_embed(torch.diagonal(p, dim1=-2, dim2=-1))
        x = _trsm(l, p, upper=False, trans=True)                  # L^-T P
        s = _trsm(l, x.mT, upper=False, trans=True).mT            # (L^-T X^T)^T = X L^-1
        return (0.5 * (s + s.mT)).to(ctx.dtype), None


def cholesky(a: torch.Tensor, upper: bool = False) -> torch.Tensor:
    if not _own(a):
        return L.cholesky(a, upper=upper)
    _square(a, "cholesky")
    l, _ = _Cholesky.apply(a, True)
    return l.mT if upper else l


def cholesky_ex(a: torch.Tensor, upper: bool = False, check_errors: bool = False):
    if not _own(a):
        return L.cholesky_ex(a, upper=upper, check_errors=check_errors)
    _square(a, "cholesky_ex")
    l, info = _Cholesky.apply(a, check_errors)
    return (l.mT if upper else l), info


# ---------------------------------------------------------------------------------------------------------------------
# LU, solve, inverse, determinants
# ---------------------------------------------------------------------------------------------------------------------
def lu_factor(a: torch.Tensor, pivot: bool = True):
    """(LU, pivots): L (unit lower) and U packed into one matrix, pivots 1-based as LAPACK writes them."""
    if not _own(a) or not pivot:
        return L.lu_factor(a, pivot=pivot)
    if a.dim() < 2:
        raise InvalidArgument("linalg.lu_factor: expected a matrix")
    lu, piv, _ = _lu_raw(a)
    return lu.to(a.dtype), piv + 1


def lu(a: torch.Tensor, pivot: bool = True):
    """(P, L, U) with A = P L U."""
    if not _own(a) or not pivot:
        return L.lu(a, pivot=pivot)
    if a.dim() < 2:
        raise InvalidArgument("linalg.lu: expected a matrix")
    f, piv, _ = _lu_raw(a)
    m, n = a.shape[-2], a.shape[-1]
    r = min(m, n)
    lower = torch.tril(f[..., :, :r], -1) + torch.eye(m, r, dtype=torch.float64)
    upper = torch.triu(f[..., :r, :])
    perm = torch.arange(m).expand(*a.shape[:-2], m).clone()
    for k in range(r):                                          # replay the row exchanges on the identity permutation
        j = piv[..., k].long().unsqueeze(-1)
        pk = perm[..., k: k + 1].clone()
        pj = perm.gather(-1, j)
        perm[..., k: k + 1] = pj
        perm.scatter_(-1, j, pk)
    pmat = torch.zeros(*a.shape[:-2], m, m, dtype=torch.float64)
    pmat.scatter_(-2, perm.unsqueeze(-2), 1.0)                  # P[perm[k], k] = 1, so (P^T A)[k] = A[perm[k]]
    return pmat.to(a.dtype), lower.to(a.dtype), upper.to(a.dtype)


class _Solve(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, check):
        lu_, piv, info = _lu_raw(a)
        if check:
            _check(info, "solve")
        x = _lu_solve_raw(lu_, piv, b.detach().to(torch.float64), False)
        ctx.save_for_backward(lu_, piv, x)
        ctx.dtypes = (a.dtype, b.dtype)
        ctx.mark_non_differentiable(info)
        return x.to(torch.promote_types(a.dtype, b.dtype)), info

    @staticmethod
    @once_differentiable
    def backward(ctx, g, _ginfo):
        lu_, piv, x = ctx.saved_tensors
        gb = _lu_solve_raw(lu_, piv, g.to(torch.float64), True)   # A^-T g
        ga = -(gb @ x.mT)
        return ga.to(ctx.dtypes[0]), gb.to(ctx.dtypes[1]), None


def _solve_any(a: torch.Tensor, b: torch.Tensor, check: bool, name: str):
    _square(a, name)
    vec = b.dim() == 1 or (b.dim() == a.dim() - 1 and b.shape == a.shape[:-1])      # the substrate's rule for a vector right-hand side
    bm = b.unsqueeze(-1) if vec else b
    if bm.shape[-2] != a.shape[-1]:
        raise InvalidArgument(f"linalg.{name}: incompatible shapes {tuple(a.shape)} and {tuple(b.shape)}")
    shape = torch.broadcast_shapes(a.shape[:-2], bm.shape[:-2])
    x, info = _Solve.apply(a.expand(*shape, *a.shape[-2:]), bm.expand(*shape, *bm.shape[-2:]), check)
    return (x.squeeze(-1) if vec else x), info


def solve(a: torch.Tensor, b: torch.Tensor, left: bool = True) -> torch.Tensor:
    if not _own(a, b):
        return L.solve(a, b, left=left)
    if not left:                                                # X A = B  <=>  A^T X^T = B^T
        return _solve_any(a.mT, b.mT, True, "solve")[0].mT
    return _solve_any(a, b, True, "solve")[0]


def solve_ex(a: torch.Tensor, b: torch.Tensor, left: bool = True, check_errors: bool = False):
    if not _own(a, b):
        return L.solve_ex(a, b, left=left, check_errors=check_errors)
    if not left:
        x, info = _solve_any(a.mT, b.mT, check_errors, "solve_ex")
        return x.mT, info
    return _solve_any(a, b, check_errors, "solve_ex")


def inv(a: torch.Tensor) -> torch.Tensor:
    if not _own(a):
        return L.inv(a)
    _square(a, "inv")
    eye = torch.eye(a.shape[-1], dtype=a.dtype).expand_as(a)
    return _Solve.apply(a, eye, True)[0]


def inv_ex(a: torch.Tensor, check_errors: bool = False):
    if not _own(a):
        return L.inv_ex(a, check_errors=check_errors)
    _square(a, "inv_ex")
    eye = torch.eye(a.shape[-1], dtype=a.dtype).expand_as(a)
    return _Solve.apply(a, eye, check_errors)


class _SlogDet(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a):
        lu_, piv, _ = _lu_raw(a)
        d = torch.diagonal(lu_, dim1=-2, dim2=-1)
        swaps = (piv != torch.arange(piv.shape[-1], dtype=torch.int32)).sum(-1)
        sign = torch.sign(d).prod(-1) * (1.0 - 2.0 * (swaps % 2).to(torch.float64))
        logabs = torch.log(d.abs()).sum(-1)
        ctx.save_for_backward(lu_, piv, sign)
        ctx.dtype = a.dtype
        ctx.mark_non_differentiable(sign)
        return sign.to(a.dtype), logabs.to(a.dtype)

    @staticmethod
    @once_differentiable
    def backward(ctx, _gsign, glog):
        lu_, piv, sign = ctx.saved_tensors
        n = lu_.shape[-1]
        eye = torch.eye(n, dtype=torch.float64).expand_as(lu_)
        inv_t = _lu_solve_raw(lu_, piv, eye, True)               # A^-T
        inv_t = torch.where((sign == 0)[..., None, None], torch.zeros_like(inv_t), inv_t)
        return (glog.to(torch.float64)[..., None, None] * inv_t).to(ctx.dtype)


def slogdet(a: torch.Tensor):
    if not _own(a):
        return L.slogdet(a)
    _square(a, "slogdet")
    return _SlogDet.apply(a)


def det(a: torch.Tensor) -> torch.Tensor:
    if not _own(a):
        return L.det(a)
    _square(a, "det")
    sign, logabs = _SlogDet.apply(a)
    return sign * torch.exp(logabs)


# ---------------------------------------------------------------------------------------------------------------------
# triangular solves
# ---------------------------------------------------------------------------------------------------------------------
class _Trsm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, t, b, upper, unit):
        t64 = t.detach().to(torch.float64).contiguous()
        x = _trsm(t64, b.detach().to(torch.float64), upper, False, unit)
        ctx.save_for_backward(t64, x)
        ctx.cfg = (upper, unit, t.dtype, b.dtype)
        return x.to(torch.promote_types(t.dtype, b.dtype))

    @staticmethod
    @once_differentiable
    def backward(ctx, g):
        t64, x = ctx.saved_tensors
        upper, unit, dt, db = ctx.cfg
        gb = _trsm(t64, g.to(torch.float64), upper, True, unit)   # T^-T g
        ga = -(gb @ x.mT)
        ga = torch.triu(ga, 1 if unit else 0) if upper else torch.tril(ga, -1 if unit else 0)
        return ga.to(dt), gb.to(db), None, None


def solve_triangular(a: torch.Tensor, b: torch.Tensor, upper: bool = True, left: bool = True, unitriangular: bool = False) -> torch.Tensor:
    if not _own(a, b):
        return L.solve_triangular(a, b, upper=upper, left=left, unitriangular=unitriangular)
    _square(a, "solve_triangular")
    if not left:                                                # X A = B  <=>  A^T X^T = B^T, and A^T has the other triangle
        return solve_triangular(a.mT, b.mT, upper=not upper, left=True, unitriangular=unitriangular).mT
    if b.dim() < 2 or b.shape[-2] != a.shape[-1]:
        raise InvalidArgument(f"linalg.solve_triangular: incompatible shapes {tuple(a.shape)} and {tuple(b.shape)}")
    shape = torch.broadcast_shapes(a.shape[:-2], b.shape[:-2])
    return _Trsm.apply(a.expand(*shape, *a.shape[-2:]), b.expand(*shape, *b.shape[-2:]), upper, unitriangular)


# ---------------------------------------------------------------------------------------------------------------------
# QR
# ---------------------------------------------------------------------------------------------------------------------
def _copyltu(m: torch.Tensor) -> torch.Tensor:
    low = torch.tril(m, -1)
    return low + low.mT + torch.diag_embed(torch.diagonal(m, dim1=-2, dim2=-1))


def _qr_back_tall(q, r, gq, gr):
    """Gradient of A = Q R for m >= n (Q m x n, R n x n)."""
    mm = r @ gr.mT - gq.mT @ q
    rhs = gq + q @ _copyltu(mm)
    return _trsm(r.contiguous(), rhs.mT.contiguous(), upper=True, trans=False).mT       # rhs R^-T = (R^-1 rhs^T)^T


class _QR(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, complete):
        a64 = a.detach().to(torch.float64).contiguous()
        m, n = a.shape[-2], a.shape[-1]
        kq = m if complete else min(m, n)
        q = torch.zeros(*a.shape[:-2], m, kq, dtype=torch.float64)
        r = torch.zeros(*a.shape[:-2], kq, n, dtype=torch.float64)
        if m and n and _batch(a):
            _rt().ft_la_qr(_p(a64), _p(q), _p(r), _i64(_batch(a)), _i64(m), _i64(n), ctypes.c_int(complete))
        elif m and complete:
            q = torch.eye(m, dtype=torch.float64).expand(*a.shape[:-2], m, m).clone()
        ctx.save_for_backward(q, r)
        ctx.cfg = (complete, a.dtype, m, n)
        return q.to(a.dtype), r.to(a.dtype)

    @staticmethod
    @once_differentiable
    def backward(ctx, gq, gr):
        q, r = ctx.saved_tensors
        complete, dt, m, n = ctx.cfg
        if complete and m > n:
            raise InvalidArgument("linalg.qr: mode 'complete' is not differentiable for tall matrices")
        gq, gr = gq.to(torch.float64), gr.to(torch.float64)
        if m >= n:
            return _qr_back_tall(q, r, gq, gr).to(dt), None
        # wide: A = [X | Y] with X square; Q, R1 = qr(X), R2 = Q^T Y
        r1, r2 = r[..., :, :m], r[..., :, m:]
        g1, g2 = gr[..., :, :m], gr[..., :, m:]
        y = q @ r2
        gx = _qr_back_tall(q, r1.contiguous(), gq + y @ g2.mT, g1.contiguous())
        return torch.cat([gx, q @ g2], -1).to(dt), None


def qr(a: torch.Tensor, mode: str = "reduced"):
    if not _own(a):
        return L.qr(a, mode=mode)
    if mode not in ("reduced", "complete", "r"):
        raise InvalidArgument(f"linalg.qr: unknown mode '{mode}'")
    if a.dim() < 2:
        raise InvalidArgument("linalg.qr: expected a matrix")
    if mode == "r":
        with torch.no_grad():
            _, r = _QR.apply(a, False)
        return torch.empty(0, dtype=a.dtype), r
    return _QR.apply(a, mode == "complete")


def householder_product(v: torch.Tensor, tau: torch.Tensor) -> torch.Tensor:
    """The first n columns of H_1 H_2 ... H_k with H_i = I - tau_i v_i v_i^T, where v_i is column i of ``v`` with an implicit one on the
    diagonal and zeros above it."""
    if not _own(v, tau):
        return L.householder_product(v, tau)
    m, n = v.shape[-2], v.shape[-1]
    k = tau.shape[-1]
    if k > n or m < n:
        raise InvalidArgument("linalg.householder_product: needs rows >= columns >= number of reflectors")
    q = torch.eye(m, n, dtype=v.dtype).expand(*v.shape[:-2], m, n)
    rows = torch.arange(m)
    for i in range(k - 1, -1, -1):
        col = torch.where(rows > i, v[..., :, i], torch.zeros_like(v[..., :, i]))
        col = col + (rows == i).to(v.dtype)
        q = q - tau[..., i, None, None] * col.unsqueeze(-1) * (col.unsqueeze(-2) @ q)
    return q


# ---------------------------------------------------------------------------------------------------------------------
# symmetric eigenproblem, singular values
# ---------------------------------------------------------------------------------------------------------------------
class _Eigh(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, lower):
        a64 = a.detach().to(torch.float64).contiguous()
        n = a.shape[-1]
        w = torch.zeros(*a.shape[:-2], n, dtype=torch.float64)
        v = torch.zeros(*a.shape[:-2], n, n, dtype=torch.float64)
        if n and _batch(a):
            if _rt().ft_la_eigh(_p(a64), _p(w), _p(v), _i64(_batch(a)), _i64(n), ctypes.c_int(lower)) < 0:
                raise LinAlgError("linalg.eigh: the Jacobi sweeps did not converge")
        ctx.save_for_backward(w, v)
        ctx.dtype = a.dtype
        return w.to(a.dtype), v.to(a.dtype)

    @staticmethod
    @once_differentiable
    def backward(ctx, gw, gv):
        w, v = ctx.saved_tensors
        gw, gv = gw.to(torch.float64), gv.to(torch.float64)
        diff = w.unsqueeze(-2) - w.unsqueeze(-1)                  # [i, j] = w_j - w_i
        f = torch.where(diff == 0, torch.zeros_like(diff), 1.0 / torch.where(diff == 0, torch.ones_like(diff), diff))
        x = v.mT @ gv                                             # V^T dV is skew-symmetric, so only the skew part of V^T gV acts: the
        inner = torch.diag_embed(gw) + f * (0.5 * (x - x.mT))    # gradient comes out symmetric, as a symmetric input calls for
        return (v @ inner @ v.mT).to(ctx.dtype), None


def eigh(a: torch.Tensor, UPLO: str = "L"):
    if not _own(a):
        return L.eigh(a, UPLO=UPLO)
    _square(a, "eigh")
    if UPLO not in ("L", "U"):
        raise InvalidArgument("linalg.eigh: UPLO is 'L' or 'U'")
    return _Eigh.apply(a, UPLO == "L")


def eigvalsh(a: torch.Tensor, UPLO: str = "L") -> torch.Tensor:
    if not _own(a):
        return L.eigvalsh(a, UPLO=UPLO)
    return eigh(a, UPLO)[0]


class _SVD(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a):
        a64 = a.detach().to(torch.float64).contiguous()
        m, n = a.shape[-2], a.shape[-1]
        k = min(m, n)
        u = torch.zeros(*a.shape[:-2], m, k, dtype=torch.float64)
        s = torch.zeros(*a.shape[:-2], k, dtype=torch.float64)
        vt = torch.zeros(*a.shape[:-2], k, n, dtype=torch.float64)
        if k and _batch(a):
            if _rt().ft_la_svd(_p(a64), _p(u), _p(s), _p(vt), _i64(_batch(a)), _i64(m), _i64(n)) < 0:
                raise LinAlgError("linalg.svd: the Jacobi sweeps did not converge")
        ctx.save_for_backward(u, s, vt)
        ctx.dtype = a.dtype
        return u.to(a.dtype), s.to(a.dtype), vt.to(a.dtype)

    @staticmethod
    @once_differentiable
    def backward(ctx, gu, gs, gvt):
        u, s, vt = ctx.saved_tensors
        gu, gs, gv = gu.to(torch.float64), gs.to(torch.float64), gvt.to(torch.float64).mT
        v = vt.mT
        m, n, k = u.shape[-2], v.shape[-2], s.shape[-1]
        s2 = s * s
        diff = s2.unsqueeze(-2) - s2.unsqueeze(-1)                # [i, j] = s_j^2 - s_i^2
        f = torch.where(diff == 0, torch.zeros_like(diff), 1.0 / torch.where(diff == 0, torch.ones_like(diff), diff))
        sm = torch.diag_embed(s)
        sinv = torch.where(s == 0, torch.zeros_like(s), 1.0 / torch.where(s == 0, torch.ones_like(s), s))
        j = f * (u.mT @ gu)
        kk = f * (v.mT @ gv)
        core = (j + j.mT) @ sm + sm @ (kk + kk.mT) + torch.diag_embed(gs)
        ga = u @ core @ vt
        if m > k:
            ga = ga + (gu - u @ (u.mT @ gu)) @ torch.diag_embed(sinv) @ vt
        if n > k:
            ga = ga + u @ torch.diag_embed(sinv) @ (gv - v @ (v.mT @ gv)).mT
        return ga.to(ctx.dtype)


def svd(a: torch.Tensor, full_matrices: bool = False):
    """(U, S, Vh) with A = U diag(S) Vh, S descending. ``full_matrices`` completes U and Vh to square orthogonal matrices."""
    if not _own(a):
        return L.svd(a, full_matrices=full_matrices)
    if a.dim() < 2:
        raise InvalidArgument("linalg.svd: expected a matrix")
    u, s, vt = _SVD.apply(a)
    if full_matrices:
        m, n, k = a.shape[-2], a.shape[-1], s.shape[-1]
        if m > k:
            with torch.no_grad():
                rest = _QR.apply(u.detach(), True)[0][..., :, k:]
            u = torch.cat([u, rest], -1)
        if n > k:
            with torch.no_grad():
                rest = _QR.apply(vt.detach().mT, True)[0][..., :, k:]
            vt = torch.cat([vt, rest.mT], -2)
    return u, s, vt


def svdvals(a: torch.Tensor) -> torch.Tensor:
    if not _own(a):
        return L.svdvals(a)
    return svd(a)[1]


# ---------------------------------------------------------------------------------------------------------------------
# composed functions
# ---------------------------------------------------------------------------------------------------------------------
def _eps(dtype) -> float:
    return torch.finfo(dtype).eps


def pinv(a: torch.Tensor, rcond: Optional[float] = None, hermitian: bool = False) -> torch.Tensor:
    """Moore-Penrose pseudo-inverse: singular values below ``rcond`` times the largest are treated as zero."""
    if not _own(a):
        return L.pinv(a, rcond=rcond, hermitian=hermitian) if rcond is not None else L.pinv(a, hermitian=hermitian)
    u, s, vt = svd(a)
    rc = max(a.shape[-2], a.shape[-1]) * _eps(a.dtype) if rcond is None else rcond
    cutoff = rc * s.amax(-1, keepdim=True) if s.shape[-1] else s
    keep = s > cutoff
    sinv = torch.where(keep, 1.0 / torch.where(keep, s, torch.ones_like(s)), torch.zeros_like(s))
    return (vt.mT * sinv.unsqueeze(-2)) @ u.mT


class LstsqResult(NamedTuple):
    solution: torch.Tensor
    residuals: torch.Tensor
    rank: torch.Tensor
    singular_values: torch.Tensor


def lstsq(a: torch.Tensor, b: torch.Tensor, rcond: Optional[float] = None) -> LstsqResult:
    """Minimiser of ||A X - B||: through QR for tall full-rank systems, through the pseudo-inverse otherwise (minimum-norm solution)."""
    if not _own(a, b):
        return L.lstsq(a, b, rcond=rcond)
    m, n = a.shape[-2], a.shape[-1]
    if b.shape[-2] != m:
        raise InvalidArgument(f"linalg.lstsq: incompatible shapes {tuple(a.shape)} and {tuple(b.shape)}")
    s = svdvals(a.detach())
    rc = max(m, n) * _eps(a.dtype) if rcond is None else rcond
    rank = (s > rc * (s.amax(-1, keepdim=True) if s.shape[-1] else s)).sum(-1)
    if m >= n and bool((rank == n).all()):
        q, r = qr(a)
        x = solve_triangular(r, q.mT @ b, upper=True)
    else:
        x = pinv(a, rcond) @ b
    res = ((a @ x - b) ** 2).sum(-2) if m > n and bool((rank == n).all()) else torch.empty(0, dtype=a.dtype)
    return LstsqResult(x, res, rank, s)


def lstsq_solve(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return lstsq(a, b).solution


def matrix_rank(a: torch.Tensor, tol: Optional[float] = None, hermitian: bool = False) -> torch.Tensor:
    if not _own(a):
        return L.matrix_rank(a, tol=tol, hermitian=hermitian) if tol is not None else L.matrix_rank(a, hermitian=hermitian)
    s = svdvals(a.detach())
    if tol is None:
        t = max(a.shape[-2], a.shape[-1]) * _eps(a.dtype) * (s.amax(-1, keepdim=True) if s.shape[-1] else s)
    else:
        t = torch.as_tensor(tol, dtype=s.dtype)
        t = t.unsqueeze(-1) if t.dim() else t
    return (s > t).sum(-1)


def vector_norm(x: torch.Tensor, ord: float = 2, dim=None, keepdim: bool = False, dtype=None) -> torch.Tensor:
    if not _own(x):
        return L.vector_norm(x, ord=ord, dim=dim, keepdim=keepdim, dtype=dtype)
    if dtype is not None:
        x = x.to(dtype)
    dims = tuple(range(x.dim())) if dim is None else ((dim,) if isinstance(dim, int) else tuple(dim))
    a = x.abs()
    if ord == float("inf"):
        return a.amax(dims, keepdim=keepdim)
    if ord == float("-inf"):
        return a.amin(dims, keepdim=keepdim)
    if ord == 0:
        return (x != 0).to(x.dtype).sum(dims, keepdim=keepdim)
    if ord == 1:
        return a.sum(dims, keepdim=keepdim)
    if ord == 2:
        return torch.sqrt((x * x).sum(dims, keepdim=keepdim))
    return (a ** ord).sum(dims, keepdim=keepdim) ** (1.0 / ord)


def matrix_norm(a: torch.Tensor, ord="fro", dim=(-2, -1), keepdim: bool = False) -> torch.Tensor:
    if not _own(a):
        return L.matrix_norm(a, ord=ord, dim=dim, keepdim=keepdim)
    d0, d1 = (d % a.dim() for d in dim)
    if d0 == d1:
        raise InvalidArgument("linalg.matrix_norm: the two dims must differ")
    x = a.movedim((d0, d1), (-2, -1))
    if ord == "fro":
        out = torch.sqrt((x * x).sum((-2, -1)))
    elif ord == "nuc":
        out = svdvals(x).sum(-1)
    elif ord in (2, -2):
        s = svdvals(x)
        out = s.amax(-1) if ord == 2 else s.amin(-1)
    elif ord in (1, -1):
        c = x.abs().sum(-2)
        out = c.amax(-1) if ord == 1 else c.amin(-1)
    elif ord in (float("inf"), float("-inf")):
        r = x.abs().sum(-1)
        out = r.amax(-1) if ord > 0 else r.amin(-1)
    else:
        raise InvalidArgument(f"linalg.matrix_norm: unknown order {ord!r}")
    if keepdim:
        for d in sorted((d0, d1)):
            out = out.unsqueeze(d)
    return out


def cond(a: torch.Tensor, p=None) -> torch.Tensor:
    if not _own(a):
        return L.cond(a, p=p)
    if p in (None, 2, -2):
        s = svdvals(a)
        big, small = s.amax(-1), s.amin(-1)
        return big / small if p != -2 else small / big
    _square(a, "cond")
    _, info = inv_ex(a.detach())
    out = matrix_norm(a, p) * matrix_norm(_Solve.apply(a, torch.eye(a.shape[-1], dtype=a.dtype).expand_as(a), False)[0], p)
    return torch.where(info != 0, torch.full_like(out, float("inf")), out)


def matrix_power(a: torch.Tensor, n: int) -> torch.Tensor:
    if not _own(a):
        return L.matrix_power(a, n)
    _square(a, "matrix_power")
    if n < 0:
        a, n = inv(a), -n
    out = torch.eye(a.shape[-1], dtype=a.dtype).expand_as(a)
    base = a
    while n:
        if n & 1:
            out = out @ base
        n >>= 1
        if n:
            base = base @ base
    return out


_PADE13 = (64764752532480000.0, 32382376266240000.0, 7771770303897600.0, 1187353796428800.0, 129060195264000.0, 10559470521600.0, 670442572800.0,
           33522128640.0, 1323241920.0, 40840800.0, 960960.0, 16380.0, 182.0, 1.0)


def matrix_exp(a: torch.Tensor) -> torch.Tensor:
    """exp(A) by scaling and squaring around the degree-13 Pade approximant (each matrix is scaled until its 1-norm is below 5.37)."""
    if not _own(a):
        return L.matrix_exp(a)
    _square(a, "matrix_exp")
    n = a.shape[-1]
    if n == 0:
        return a.clone()
    norm1 = a.detach().abs().sum(-2).amax(-1)
    sq = torch.clamp(torch.ceil(torch.log2(torch.clamp(norm1 / 5.371920351148152, min=1e-300))), min=0).to(torch.int64)
    x = a * (2.0 ** (-sq.to(a.dtype)))[..., None, None]
    eye = torch.eye(n, dtype=a.dtype).expand_as(a)
    b = _PADE13
    x2 = x @ x
    x4 = x2 @ x2
    x6 = x4 @ x2
    u = x @ (x6 @ (b[13] * x6 + b[11] * x4 + b[9] * x2) + b[7] * x6 + b[5] * x4 + b[3] * x2 + b[1] * eye)
    v = x6 @ (b[12] * x6 + b[10] * x4 + b[8] * x2) + b[6] * x6 + b[4] * x4 + b[2] * x2 + b[0] * eye
    r = _Solve.apply(v - u, v + u, True)[0]
    for k in range(int(sq.max()) if sq.numel() else 0):
        r = torch.where((sq > k)[..., None, None], r @ r, r)
    return r


def multi_dot(tensors: Sequence[torch.Tensor]) -> torch.Tensor:
    """Product of a chain of matrices in the order that costs the fewest multiplications (first and last may be vectors)."""
    ts = list(tensors)
    if len(ts) < 2:
        raise InvalidArgument("linalg.multi_dot: needs at least two tensors")
    if not _own(*ts):
        return L.multi_dot(ts)
    first_vec, last_vec = ts[0].dim() == 1, ts[-1].dim() == 1
    if first_vec:
        ts[0] = ts[0].unsqueeze(0)
    if last_vec:
        ts[-1] = ts[-1].unsqueeze(-1)
    if any(t.dim() != 2 for t in ts):
        raise InvalidArgument("linalg.multi_dot: the inner tensors are matrices")
    dims = [ts[0].shape[0]] + [t.shape[1] for t in ts]
    for i, t in enumerate(ts):
        if t.shape[0] != dims[i]:
            raise InvalidArgument("linalg.multi_dot: shapes do not chain")
    k = len(ts)
    cost = [[0] * k for _ in range(k)]
    cut = [[0] * k for _ in range(k)]
    for span in range(1, k):
        for i in range(k - span):
            j = i + span
            cost[i][j] = None
            for s in range(i, j):
                c = cost[i][s] + cost[s + 1][j] + dims[i] * dims[s + 1] * dims[j + 1]
                if cost[i][j] is None or c < cost[i][j]:
                    cost[i][j], cut[i][j] = c, s

    def build(i, j):
        return ts[i] if i == j else build(i, cut[i][j]) @ build(cut[i][j] + 1, j)
    out = build(0, k - 1)
    if first_vec:
        out = out.squeeze(0)
    if last_vec:
        out = out.squeeze(-1)
    return out


def cross(a: torch.Tensor, b: torch.Tensor, dim: int = -1) -> torch.Tensor:
    if not _own(a, b):
        return L.cross(a, b, dim=dim)
    a, b = torch.broadcast_tensors(a, b)
    if a.shape[dim] != 3:
        raise InvalidArgument("linalg.cross: the dimension must have length 3")
    a0, a1, a2 = a.unbind(dim)
    b0, b1, b2 = b.unbind(dim)
    return torch.stack((a1 * b2 - a2 * b1, a2 * b0 - a0 * b2, a0 * b1 - a1 * b0), dim)


def diagonal(a: torch.Tensor, offset: int = 0, dim1: int = -2, dim2: int = -1) -> torch.Tensor:
    return torch.diagonal(a, offset=offset, dim1=dim1, dim2=dim2)


def tensorinv(a: torch.Tensor, ind: int = 2) -> torch.Tensor:
    if not _own(a):
        return L.tensorinv(a, ind=ind)
    if ind < 1:
        raise InvalidArgument("linalg.tensorinv: ind must be positive")
    lead, tail = a.shape[:ind], a.shape[ind:]
    rows, cols = math.prod(lead), math.prod(tail)
    if rows != cols:
        raise InvalidArgument("linalg.tensorinv: the two index groups must have the same total size")
    return inv(a.reshape(rows, cols)).reshape(*tail, *lead)


def tensorsolve(a: torch.Tensor, b: torch.Tensor, dims: Optional[Sequence[int]] = None) -> torch.Tensor:
    if not _own(a, b):
        return L.tensorsolve(a, b, dims=dims)
    if dims is not None:
        a = a.movedim(tuple(dims), tuple(range(a.dim() - len(dims), a.dim())))
    tail = a.shape[b.dim():]
    rows, cols = math.prod(b.shape), math.prod(tail)
    if rows != cols or a.shape[: b.dim()] != b.shape:
        raise InvalidArgument("linalg.tensorsolve: shapes do not match")
    return solve(a.reshape(rows, cols), b.reshape(rows)).reshape(tail)


def ldl_factor(a: torch.Tensor, hermitian: bool = False):
    """A = L D L^T of a symmetric matrix without pivoting, in the compact form (D on the diagonal, the unit-lower L below it) with the
    identity pivot vector 1..n, the form in which LAPACK reports a factorisation that needed no exchanges."""
    if not _own(a):
        return L.ldl_factor(a, hermitian=hermitian)
    _square(a, "ldl_factor")
    n = a.shape[-1]
    w = a.detach().to(torch.float64).clone()
    w = torch.tril(w) + torch.tril(w, -1).mT
    ld = torch.zeros_like(w)
    for j in range(n):
        d = w[..., j, j]
        if bool((d == 0).any()):
            raise LinAlgError(f"linalg.ldl_factor: zero pivot at position {j + 1} (this factorisation does not exchange rows)")
        col = w[..., j + 1:, j] / d.unsqueeze(-1)
        ld[..., j, j] = d
        ld[..., j + 1:, j] = col
        w[..., j + 1:, j + 1:] = w[..., j + 1:, j + 1:] - col.unsqueeze(-1) * w[..., j + 1:, j].unsqueeze(-2)
    piv = torch.arange(1, n + 1, dtype=torch.int32).expand(*a.shape[:-2], n).contiguous()
    return ld.to(a.dtype), piv


def ldl_solve(ld: torch.Tensor, pivots: torch.Tensor, b: torch.Tensor, hermitian: bool = False) -> torch.Tensor:
    n = ld.shape[-1]
    if not _own(ld, b) or not bool((pivots == torch.arange(1, n + 1, dtype=pivots.dtype)).all()):
        return L.ldl_solve(ld, pivots, b, hermitian=hermitian)
    y = solve_triangular(ld, b, upper=False, unitriangular=True)
    y = y / torch.diagonal(ld, dim1=-2, dim2=-1).unsqueeze(-1)
    return solve_triangular(ld.mT, y, upper=True, unitriangular=True)


def eig(a: torch.Tensor):
    """General (non-symmetric) eigenproblem: complex eigenvalues ``w`` [.., n] and unit eigenvectors in the columns of ``V`` [.., n, n] with
    ``A V = V diag(w)``, from the complex Schur form computed in the runtime library (the order of the eigenvalues is that form's, not
    LAPACK's). An input that takes part in differentiation goes to the substrate's library call, which carries the derivative."""
    if not _own(a) or a.requires_grad:
        return L.eig(a)
    _square(a, "eig")
    n = a.shape[-1]
    a64 = a.detach().to(torch.float64).contiguous()
    w = torch.zeros(*a.shape[:-2], n, 2, dtype=torch.float64)
    v = torch.zeros(*a.shape[:-2], n, n, 2, dtype=torch.float64)
    if n and _batch(a):
        _rt().ft_la_eig.restype = ctypes.c_int
        if _rt().ft_la_eig(_p(a64), _p(w), _p(v), _i64(_batch(a)), _i64(n)) < 0:
            raise LinAlgError("linalg.eig: the QR iterations did not converge")
    ct = torch.complex64 if a.dtype == torch.float32 else torch.complex128
    return torch.view_as_complex(w).to(ct), torch.view_as_complex(v).to(ct)


def eigvals(a: torch.Tensor):
    if not _own(a) or a.requires_grad:
        return L.eigvals(a)
    return eig(a)[0]
