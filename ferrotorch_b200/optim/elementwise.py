"""Adagrad, RMSprop, Adadelta, Adamax, NAdam, RAdam, Rprop, ASGD, SparseAdam and L-BFGS, implemented here (update rules as in PyTorch, which
the reference follows too: ferrotorch-optim/src/{adagrad,rmsprop,adadelta,adamax,nadam,radam,rprop,asgd,sparse_adam,lbfgs}.rs).

The eight element-wise ones share one CUDA kernel (``ft_foreach_opt``: one launch per parameter instead of a chain of a dozen tensor
operations; the step-dependent scalars are computed on the host); on CPU tensors, for sparse gradients and for dtypes the kernel does not
take, the same recurrences run as tensor operations, which is also the oracle the GPU test compares the kernel with.
"""
from __future__ import annotations

import ctypes
import math
from typing import Callable, Optional

import torch

from .. import _lib
from .optimizers import Optimizer

_ALGO = {"adagrad": 0, "rmsprop": 1, "adadelta": 2, "adamax": 3, "nadam": 4, "radam": 5, "rprop": 6, "asgd": 7}


def _kernel_ok(p: torch.Tensor, g: torch.Tensor) -> bool:
    return p.is_cuda and p.dtype == torch.float32 and g.dtype == torch.float32 and p.is_contiguous() and g.is_contiguous() and not g.is_sparse


def _launch(algo: str, p, g, states, hp, maximize: bool) -> None:
    s = list(states) + [None] * (3 - len(states))
    arr = (ctypes.c_float * 12)(*([float(x) for x in hp] + [0.0] * (12 - len(hp))))
    with torch.cuda.device(p.device):
        _lib.call("ft_foreach_opt", _ALGO[algo], p, g, s[0], s[1], s[2], p.numel(), arr, int(maximize), _lib.S())


class _Elementwise(Optimizer):
    """Shared driver: per parameter, build the state on first use, compute the step's scalars, run the kernel or the tensor-operation form."""

    def _cfg(self, params, config, defaults: dict, kw: dict):
        if config is not None and hasattr(config, "__dataclass_fields__"):
            import dataclasses
            kw = {**{k: v for k, v in dataclasses.asdict(config).items() if k in defaults}, **kw}
        elif config is not None:
            kw.setdefault("lr", config)
        self.config = config
        unknown = set(kw) - set(defaults) - {"foreach", "capturable", "differentiable", "fused"}
        if unknown:
            raise TypeError(f"{type(self).__name__}: unexpected arguments {sorted(unknown)}")
        super().__init__(params, {**defaults, **{k: v for k, v in kw.items() if k in defaults}})

    @torch.no_grad()
    def step(self, closure: Optional[Callable] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                self._update(p, p.grad, self.state[p], group)
        return loss


class Adagrad(_Elementwise):
    """Adagrad."""

    def __init__(self, params, config=None, **kw):
        self._cfg(params, config, dict(lr=1e-2, lr_decay=0.0, weight_decay=0.0, initial_accumulator_value=0.0, eps=1e-10, maximize=False), kw)

    def _update(self, p, g, st, h):
        if not st:
            st["step"] = 0
            st["sum"] = torch.full_like(p, h["initial_accumulator_value"], memory_format=torch.preserve_format)
        st["step"] += 1
        clr = h["lr"] / (1 + (st["step"] - 1) * h["lr_decay"])
        if _kernel_ok(p, g):
            return _launch("adagrad", p, g, [st["sum"]], [clr, h["weight_decay"], h["eps"]], h["maximize"])
        g = -g if h["maximize"] else g
        if g.is_sparse:
            g = g.coalesce()
            idx, val = g._indices(), g._values()
            st["sum"].add_(torch.sparse_coo_tensor(idx, val * val, g.shape))
            std = st["sum"].sparse_mask(g)._values().sqrt_().add_(h["eps"])
            p.add_(torch.sparse_coo_tensor(idx, val / std, g.shape), alpha=-clr)
            return
        if h["weight_decay"]:
            g = g.add(p, alpha=h["weight_decay"])
        st["sum"].addcmul_(g, g)
        p.addcdiv_(g, st["sum"].sqrt().add_(h["eps"]), value=-clr)


class Rmsprop(_Elementwise):
    """RMSprop (optionally centered, optionally with momentum)."""

    def __init__(self, params, config=None, **kw):
        self._cfg(params, config, dict(lr=1e-2, alpha=0.99, eps=1e-8, weight_decay=0.0, momentum=0.0, centered=False, maximize=False), kw)

    def _update(self, p, g, st, h):
        if not st:
            st["step"] = 0
            st["square_avg"] = torch.zeros_like(p)
            if h["momentum"] > 0:
                st["momentum_buffer"] = torch.zeros_like(p)
            if h["centered"]:
                st["grad_avg"] = torch.zeros_like(p)
        st["step"] += 1
        if _kernel_ok(p, g):
            return _launch("rmsprop", p, g, [st["square_avg"], st.get("momentum_buffer"), st.get("grad_avg")],
                           [h["lr"], h["alpha"], h["eps"], h["weight_decay"], h["momentum"], float(h["centered"])], h["maximize"])
        g = -g if h["maximize"] else g
        if h["weight_decay"]:
            g = g.add(p, alpha=h["weight_decay"])
        sq = st["square_avg"].mul_(h["alpha"]).addcmul_(g, g, value=1 - h["alpha"])
        if h["centered"]:
            ga = st["grad_avg"].lerp_(g, 1 - h["alpha"])
            avg = torch.addcmul(sq, ga, ga, value=-1).sqrt_().add_(h["eps"])
        else:
            avg = sq.sqrt().add_(h["eps"])
        if h["momentum"] > 0:
            p.add_(st["momentum_buffer"].mul_(h["momentum"]).addcdiv_(g, avg), alpha=-h["lr"])
        else:
            p.addcdiv_(g, avg, value=-h["lr"])


class Adadelta(_Elementwise):
    """Adadelta."""

    def __init__(self, params, config=None, **kw):
        self._cfg(params, config, dict(lr=1.0, rho=0.9, eps=1e-6, weight_decay=0.0, maximize=False), kw)

    def _update(self, p, g, st, h):
        if not st:
            st["step"] = 0
            st["square_avg"], st["acc_delta"] = torch.zeros_like(p), torch.zeros_like(p)
        st["step"] += 1
        if _kernel_ok(p, g):
            return _launch("adadelta", p, g, [st["square_avg"], st["acc_delta"]], [h["lr"], h["rho"], h["eps"], h["weight_decay"]], h["maximize"])
        g = -g if h["maximize"] else g
        if h["weight_decay"]:
            g = g.add(p, alpha=h["weight_decay"])
        sq, acc = st["square_avg"], st["acc_delta"]
        sq.mul_(h["rho"]).addcmul_(g, g, value=1 - h["rho"])
        delta = acc.add(h["eps"]).sqrt_().div_(sq.add(h["eps"]).sqrt_()).mul_(g)
        acc.mul_(h["rho"]).addcmul_(delta, delta, value=1 - h["rho"])
        p.add_(delta, alpha=-h["lr"])


class Adamax(_Elementwise):
    """Adamax (Adam with the infinity norm)."""

    def __init__(self, params, config=None, **kw):
        self._cfg(params, config, dict(lr=2e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, maximize=False), kw)

    def _update(self, p, g, st, h):
        if not st:
            st["step"] = 0
            st["exp_avg"], st["exp_inf"] = torch.zeros_like(p), torch.zeros_like(p)
        st["step"] += 1
        b1, b2 = h["betas"]
        clr = h["lr"] / (1 - b1 ** st["step"])
        if _kernel_ok(p, g):
            return _launch("adamax", p, g, [st["exp_avg"], st["exp_inf"]], [clr, b1, b2, h["eps"], h["weight_decay"]], h["maximize"])
        g = -g if h["maximize"] else g
        if h["weight_decay"]:
            g = g.add(p, alpha=h["weight_decay"])
        st["exp_avg"].lerp_(g, 1 - b1)
        torch.maximum(st["exp_inf"].mul_(b2), g.abs().add_(h["eps"]), out=st["exp_inf"])
        p.addcdiv_(st["exp_avg"], st["exp_inf"], value=-clr)


class NAdam(_Elementwise):
    """Adam with Nesterov momentum (momentum-decay schedule ``mu_t = beta1 (1 - 0.5 * 0.96^(t * momentum_decay))``)."""

    def __init__(self, params, config=None, **kw):
        self._cfg(params, config, dict(lr=2e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, momentum_decay=4e-3, decoupled_weight_decay=False,
                                       maximize=False), kw)

    def _update(self, p, g, st, h):
        if not st:
            st["step"], st["mu_product"] = 0, 1.0
            st["exp_avg"], st["exp_avg_sq"] = torch.zeros_like(p), torch.zeros_like(p)
        st["step"] += 1
        t, (b1, b2) = st["step"], h["betas"]
        bc2 = 1 - b2 ** t
        mu = b1 * (1 - 0.5 * 0.96 ** (t * h["momentum_decay"]))
        mu_next = b1 * (1 - 0.5 * 0.96 ** ((t + 1) * h["momentum_decay"]))
        st["mu_product"] *= mu
        c_grad = h["lr"] * (1 - mu) / (1 - st["mu_product"])
        c_mom = h["lr"] * mu_next / (1 - st["mu_product"] * mu_next)
        decay = 1 - h["lr"] * h["weight_decay"] if h["decoupled_weight_decay"] else 1.0
        wd = 0.0 if h["decoupled_weight_decay"] else h["weight_decay"]
        if _kernel_ok(p, g):
            return _launch("nadam", p, g, [st["exp_avg"], st["exp_avg_sq"]], [c_grad, c_mom, b1, b2, h["eps"], wd, bc2, decay], h["maximize"])
        g = -g if h["maximize"] else g
        p.mul_(decay)
        if wd:
            g = g.add(p, alpha=wd)
        st["exp_avg"].lerp_(g, 1 - b1)
        st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
        den = st["exp_avg_sq"].div(bc2).sqrt_().add_(h["eps"])
        p.addcdiv_(g, den, value=-c_grad)
        p.addcdiv_(st["exp_avg"], den, value=-c_mom)


class RAdam(_Elementwise):
    """Rectified Adam: the adaptive term is used once the variance of the second-moment estimate is tractable (``rho_t > 5``)."""

    def __init__(self, params, config=None, **kw):
        self._cfg(params, config, dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, decoupled_weight_decay=False, maximize=False), kw)

    def _update(self, p, g, st, h):
        if not st:
            st["step"] = 0
            st["exp_avg"], st["exp_avg_sq"] = torch.zeros_like(p), torch.zeros_like(p)
        st["step"] += 1
        t, (b1, b2) = st["step"], h["betas"]
        bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
        rho_inf = 2 / (1 - b2) - 1
        rho_t = rho_inf - 2 * t * (b2 ** t) / bc2
        rect = math.sqrt((rho_t - 4) * (rho_t - 2) * rho_inf / ((rho_inf - 4) * (rho_inf - 2) * rho_t)) if rho_t > 5 else 0.0
        decay = 1 - h["lr"] * h["weight_decay"] if h["decoupled_weight_decay"] else 1.0
        wd = 0.0 if h["decoupled_weight_decay"] else h["weight_decay"]
        if _kernel_ok(p, g):
            return _launch("radam", p, g, [st["exp_avg"], st["exp_avg_sq"]], [h["lr"], b1, b2, h["eps"], wd, bc1, bc2, rect, decay], h["maximize"])
        g = -g if h["maximize"] else g
        p.mul_(decay)
        if wd:
            g = g.add(p, alpha=wd)
        st["exp_avg"].lerp_(g, 1 - b1)
        st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
        mh = st["exp_avg"] / bc1
        if rect:
            p.addcdiv_(mh, st["exp_avg_sq"].sqrt().add_(h["eps"]), value=-h["lr"] * rect * math.sqrt(bc2))
        else:
            p.add_(mh, alpha=-h["lr"])


class Rprop(_Elementwise):
    """Resilient backpropagation: per-element step sizes grown / shrunk by the sign agreement of successive gradients."""

    def __init__(self, params, config=None, **kw):
        self._cfg(params, config, dict(lr=1e-2, etas=(0.5, 1.2), step_sizes=(1e-6, 50.0), maximize=False), kw)

    def _update(self, p, g, st, h):
        if not st:
            st["step"] = 0
            st["prev"] = torch.zeros_like(p)
            st["step_size"] = torch.full_like(p, h["lr"])
        st["step"] += 1
        (em, ep), (smin, smax) = h["etas"], h["step_sizes"]
        if _kernel_ok(p, g):
            return _launch("rprop", p, g, [st["prev"], st["step_size"]], [em, ep, smin, smax], h["maximize"])
        g = (-g if h["maximize"] else g).clone()
        sign = g.mul(st["prev"]).sign()
        factor = torch.where(sign > 0, ep, torch.where(sign < 0, em, 1.0)).to(p.dtype)
        st["step_size"].mul_(factor).clamp_(smin, smax)
        g[sign < 0] = 0
        p.addcmul_(g.sign(), st["step_size"], value=-1)
        st["prev"].copy_(g)


class Asgd(_Elementwise):
    """Averaged SGD (the running average of the iterates is kept in ``state[p]["ax"]``)."""

    def __init__(self, params, config=None, **kw):
        self._cfg(params, config, dict(lr=1e-2, lambd=1e-4, alpha=0.75, t0=1e6, weight_decay=0.0, maximize=False), kw)

    def _update(self, p, g, st, h):
        if not st:
            st["step"], st["eta"], st["mu"] = 0, h["lr"], 1.0
            st["ax"] = torch.zeros_like(p)
        st["step"] += 1
        eta, mu = st["eta"], st["mu"]
        if _kernel_ok(p, g):
            _launch("asgd", p, g, [st["ax"]], [eta, h["lambd"], h["weight_decay"], mu], h["maximize"])
        else:
            g = -g if h["maximize"] else g
            if h["weight_decay"]:
                g = g.add(p, alpha=h["weight_decay"])
            p.mul_(1 - h["lambd"] * eta).add_(g, alpha=-eta)
            if mu != 1:
                st["ax"].add_(p.sub(st["ax"]), alpha=mu)
            else:
                st["ax"].copy_(p)
        t = st["step"]
        st["eta"] = h["lr"] / ((1 + h["lambd"] * h["lr"] * t) ** h["alpha"])
        st["mu"] = 1 / max(1, t - h["t0"])


class SparseAdam(_Elementwise):
    """Adam for sparse gradients (embedding tables): moments and parameters are touched only at the rows present in the gradient."""

    def __init__(self, params, config=None, **kw):
        self._cfg(params, config, dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, maximize=False), kw)

    def _update(self, p, g, st, h):
        if not g.is_sparse:
            raise RuntimeError("SparseAdam does not support dense gradients, please consider Adam instead")
        if not st:
            st["step"] = 0
            st["exp_avg"], st["exp_avg_sq"] = torch.zeros_like(p), torch.zeros_like(p)
        st["step"] += 1
        g = g.coalesce()
        if h["maximize"]:
            g = -g
        idx, val = g._indices(), g._values()
        if val.numel() == 0:
            return
        b1, b2 = h["betas"]
        t = st["step"]

        def masked(dense):
            return dense.sparse_mask(g)._values()
        m_upd = val.sub(masked(st["exp_avg"])).mul_(1 - b1)
        st["exp_avg"].add_(torch.sparse_coo_tensor(idx, m_upd, g.shape))
        v_upd = val.pow(2).sub_(masked(st["exp_avg_sq"])).mul_(1 - b2)
        st["exp_avg_sq"].add_(torch.sparse_coo_tensor(idx, v_upd, g.shape))
        numer = masked(st["exp_avg"])
        denom = masked(st["exp_avg_sq"]).sqrt_().add_(h["eps"])
        step_size = h["lr"] * math.sqrt(1 - b2 ** t) / (1 - b1 ** t)
        p.add_(torch.sparse_coo_tensor(idx, -step_size * numer / denom, g.shape))


class Lbfgs(Optimizer):
    """Limited-memory BFGS over all parameters as one flat vector: two-loop recursion over the last ``history_size`` curvature pairs;
    ``line_search_fn=None`` takes fixed steps of ``lr`` (the first one scaled by ``min(1, 1/|g|_1)``), ``"strong_wolfe"`` runs a
    bracketing / zoom search for a step that satisfies the strong Wolfe conditions (c1 = 1e-4, c2 = 0.9)."""

    def __init__(self, params, config=None, **kw):
        defaults = dict(lr=1.0, max_iter=20, max_eval=None, tolerance_grad=1e-7, tolerance_change=1e-9, history_size=100, line_search_fn=None)
        if config is not None and hasattr(config, "__dataclass_fields__"):
            import dataclasses
            kw = {**{k: v for k, v in dataclasses.asdict(config).items() if k in defaults}, **kw}
        elif config is not None:
            kw.setdefault("lr", config)
        self.config = config
        d = {**defaults, **kw}
        if d["max_eval"] is None:
            d["max_eval"] = d["max_iter"] * 5 // 4
        super().__init__(params, d)
        if len(self.param_groups) != 1:
            raise ValueError("Lbfgs doesn't support per-parameter options (parameter groups)")
        self._params = self.param_groups[0]["params"]

    def _flat_grad(self):
        return torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in self._params])

    def _add(self, step, d):
        off = 0
        for p in self._params:
            n = p.numel()
            p.add_(d[off: off + n].view_as(p), alpha=step)
            off += n

    def _set(self, flat):
        off = 0
        for p in self._params:
            n = p.numel()
            p.copy_(flat[off: off + n].view_as(p))
            off += n

    @torch.no_grad()
    def step(self, closure):
        h = self.param_groups[0]
        closure = torch.enable_grad()(closure)
        st = self.state[self._params[0]]
        st.setdefault("n_iter", 0)
        loss = float(closure())
        evals = 1
        g = self._flat_grad()
        if g.abs().max() <= h["tolerance_grad"]:
            return loss
        d, t = st.get("d"), st.get("t")
        old_s, old_y, prev_g, H = st.setdefault("s", []), st.setdefault("y", []), st.get("prev_g"), st.get("H", 1.0)
        prev_loss = st.get("prev_loss")
        n_iter = 0
        while n_iter < h["max_iter"]:
            n_iter += 1
            st["n_iter"] += 1
            if st["n_iter"] == 1:
                d, H = g.neg(), 1.0
            else:
                y, s = g.sub(prev_g), d.mul(t)
                ys = float(y.dot(s))
                if ys > 1e-10:
                    if len(old_s) == h["history_size"]:
                        old_s.pop(0)
                        old_y.pop(0)
                    old_s.append(s)
                    old_y.append(y)
                    H = ys / float(y.dot(y))
                q = g.neg()
                al = [0.0] * len(old_s)
                for i in range(len(old_s) - 1, -1, -1):
                    al[i] = float(old_s[i].dot(q)) / float(old_y[i].dot(old_s[i]))
                    q.add_(old_y[i], alpha=-al[i])
                d = q.mul(H)
                for i in range(len(old_s)):
                    be = float(old_y[i].dot(d)) / float(old_y[i].dot(old_s[i]))
                    d.add_(old_s[i], alpha=al[i] - be)
            prev_g = g.clone()
            prev_loss = loss
            t = min(1.0, 1.0 / float(g.abs().sum())) * h["lr"] if st["n_iter"] == 1 else h["lr"]
            gtd = float(g.dot(d))
            if gtd > -h["tolerance_change"]:
                break
            if h["line_search_fn"] == "strong_wolfe":
                x0 = torch.cat([p.reshape(-1) for p in self._params]).clone()

                def phi(step):
                    self._set(x0.add(d, alpha=step))
                    l = float(closure())
                    return l, self._flat_grad()
                loss, g, t, n_ev = _strong_wolfe(phi, t, d, loss, g, gtd, h["tolerance_change"])
                self._set(x0.add(d, alpha=t))
                evals += n_ev
            elif h["line_search_fn"] is None:
                self._add(t, d)
                if n_iter != h["max_iter"]:
                    loss = float(closure())
                    g = self._flat_grad()
                    evals += 1
            else:
                raise RuntimeError("only 'strong_wolfe' is supported")
            if n_iter == h["max_iter"] or evals >= h["max_eval"] or g.abs().max() <= h["tolerance_grad"]:
                break
            if float(d.mul(t).abs().max()) <= h["tolerance_change"] or abs(loss - prev_loss) < h["tolerance_change"]:
                break
        st.update(d=d, t=t, prev_g=prev_g, H=H, prev_loss=prev_loss)
        return loss


def _strong_wolfe(phi, t, d, f0, g0, gtd0, tol, c1=1e-4, c2=0.9, max_ls=25):
    """Bracketing + bisection-with-cubic-guess search for a step satisfying the strong Wolfe conditions. Returns (loss, grad, step, evaluations)."""
    def cubic(x1, f1, d1, x2, f2, d2, lo, hi):
        dd1 = d1 + d2 - 3 * (f1 - f2) / (x1 - x2)
        sq = dd1 * dd1 - d1 * d2
        if sq >= 0:
            dd2 = math.sqrt(sq)
            x = x2 - (x2 - x1) * ((d2 + dd2 - dd1) / (d2 - d1 + 2 * dd2)) if x1 <= x2 else x1 - (x1 - x2) * ((d1 + dd2 - dd1) / (d1 - d2 + 2 * dd2))
            return min(max(x, lo), hi)
        return (lo + hi) / 2
    f_prev, g_prev, gtd_prev, t_prev = f0, g0, gtd0, 0.0
    f_new, g_new = phi(t)
    n = 1
    gtd_new = float(g_new.dot(d))
    bracket = None
    for it in range(max_ls):
        if f_new > f0 + c1 * t * gtd0 or (it > 0 and f_new >= f_prev):
            bracket = [(t_prev, f_prev, g_prev, gtd_prev), (t, f_new, g_new, gtd_new)]
            break
        if abs(gtd_new) <= -c2 * gtd0:
            return f_new, g_new, t, n
        if gtd_new >= 0:
            bracket = [(t_prev, f_prev, g_prev, gtd_prev), (t, f_new, g_new, gtd_new)]
            break
        lo, hi = t + 0.01 * (t - t_prev), t * 10
        t_next = cubic(t_prev, f_prev, gtd_prev, t, f_new, gtd_new, lo, hi)
        t_prev, f_prev, g_prev, gtd_prev = t, f_new, g_new, gtd_new
        t = t_next
        f_new, g_new = phi(t)
        n += 1
        gtd_new = float(g_new.dot(d))
    if bracket is None:
        return f_new, g_new, t, n
    for _ in range(max_ls):
        (ta, fa, ga, da), (tb, fb, gb, db) = bracket
        if abs(tb - ta) * float(d.abs().max()) < tol:
            break
        t = cubic(ta, fa, da, tb, fb, db, min(ta, tb), max(ta, tb))
        span = max(ta, tb) - min(ta, tb)
        if min(max(ta, tb) - t, t - min(ta, tb)) < 0.1 * span:      # too close to an end: bisect instead
            t = (ta + tb) / 2
        f_new, g_new = phi(t)
        n += 1
        gtd_new = float(g_new.dot(d))
        lo_i = 0 if fa <= fb else 1
        t_lo, f_lo = bracket[lo_i][0], bracket[lo_i][1]
        if f_new > f0 + c1 * t * gtd0 or f_new >= f_lo:
            bracket[1 - lo_i] = (t, f_new, g_new, gtd_new)
        else:
            if abs(gtd_new) <= -c2 * gtd0:
                return f_new, g_new, t, n
            if gtd_new * (bracket[1 - lo_i][0] - t_lo) >= 0:
                bracket[1 - lo_i] = bracket[lo_i]
            bracket[lo_i] = (t, f_new, g_new, gtd_new)
    best = min(bracket, key=lambda b: b[1])
    return best[1], best[2], best[0], n
