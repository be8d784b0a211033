"""Optimizers. ``Sgd``, ``Adam`` and ``AdamW`` update CUDA parameters with the flat fused kernels (one launch per
parameter tensor instead of ~12 elementwise launches plus scalar uploads); bf16 parameters get an f32 master copy in the
optimizer state. ``Muon`` runs its Newton-Schulz iteration on the tcgen05 GEMM for bf16 matrices. The remaining optimizers
carry PyTorch's reference update rules under the reference's names and config structs.

Reference parity: ferrotorch-optim/src/{optimizer.rs:8-101, sgd.rs:30-440, adam.rs:165-472, adamw.rs:31-430, adamax, nadam, radam,
adagrad, adadelta, adafactor, rmsprop, rprop, asgd, sparse_adam, lbfgs.rs:35-202, muon.rs:33-320, natural_gradient.rs:170}.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional

import torch

from .. import ops
from ..errors import InvalidArgument
from ..nn.compute_copy import mark_synced, optimizer_target


class _Cfg:
    """Builder-style configs: every field has a ``with_<field>(value)`` setter returning a new config."""

    def __getattr__(self, name):
        if name.startswith("with_") and name[5:] in self.__dataclass_fields__:
            def setter(v, _n=name[5:]):
                import dataclasses
                return dataclasses.replace(self, **{_n: v})
            return setter
        raise AttributeError(name)


@dataclass(frozen=True)
class SgdConfig(_Cfg):
    lr: float = 0.01
    momentum: float = 0.0
    dampening: float = 0.0
    weight_decay: float = 0.0
    nesterov: bool = False
    maximize: bool = False
    foreach: bool = True


@dataclass(frozen=True)
class AdamWConfig(_Cfg):
    lr: float = 1e-3
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.01
    amsgrad: bool = False
    maximize: bool = False
    foreach: bool = True


@dataclass(frozen=True)
class AdamConfig(_Cfg):
    lr: float = 1e-3
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.0
    amsgrad: bool = False
    maximize: bool = False


@dataclass(frozen=True)
class MuonConfig(_Cfg):
    lr: float = 0.02
    momentum: float = 0.95
    nesterov: bool = True
    ns_steps: int = 5
    weight_decay: float = 0.0
    adamw_lr: float = 3e-4          # for non-matrix parameters
    adamw_betas: tuple = (0.9, 0.95)
    adamw_eps: float = 1e-8


class Optimizer(torch.optim.Optimizer):
    """Common surface: ``step``, ``zero_grad``, ``lr`` / ``set_lr``, ``param_groups``, ``state_dict`` / ``load_state_dict``."""

    def lr(self) -> float:
        return self.param_groups[0]["lr"]

    def set_lr(self, lr: float) -> None:
        for g in self.param_groups:
            g["lr"] = lr

    def add_param_group_cfg(self, params, **overrides) -> None:
        self.add_param_group({"params": list(params), **overrides})


ParamGroup = dict


def _fused_ok(p: torch.Tensor, g: torch.Tensor) -> bool:
    return (p.is_cuda and p.is_contiguous() and g.is_contiguous() and not g.is_sparse and p.dtype in (torch.float32, torch.bfloat16)
            and g.dtype in (torch.float32, torch.bfloat16))


def _dense(t: torch.Tensor) -> bool:
    return t.is_contiguous() or (t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last))


def _flat(t: torch.Tensor) -> torch.Tensor:
    """1-D view over the storage of a dense tensor in memory order (row-major, or NHWC order for a channels-last tensor)."""
    return t.view(-1) if t.is_contiguous() else t.permute(0, 2, 3, 1).reshape(-1)


def _flat_pair_ok(p: torch.Tensor, g: torch.Tensor, need_cuda: bool = True) -> bool:
    """Parameters with a compute copy take the flat kernels in any dense layout (convolution weights of a channels-last model included):
    parameter, gradient, momentum buffer and compute copy are then all walked in the parameter's memory order."""
    return ((p.is_cuda or not need_cuda) and _dense(p) and not g.is_sparse and p.dtype in (torch.float32, torch.bfloat16)
            and g.dtype in (torch.float32, torch.bfloat16))


class Sgd(Optimizer):
    """SGD: weight decay folded into the gradient, momentum buffer seeded with the first gradient, dampening and Nesterov as in PyTorch."""

    def __init__(self, params, config: Optional[SgdConfig] = None, **kw):
        cfg = config or SgdConfig(**kw)
        if cfg.nesterov and (cfg.momentum <= 0 or cfg.dampening != 0):
            raise InvalidArgument("Nesterov momentum requires momentum > 0 and zero dampening")
        self.config = cfg
        super().__init__(params, dict(lr=cfg.lr, momentum=cfg.momentum, dampening=cfg.dampening, weight_decay=cfg.weight_decay,
                                      nesterov=cfg.nesterov, maximize=cfg.maximize))

    @torch.no_grad()
    def step(self, closure: Optional[Callable] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                first = "buf" not in st
                target = optimizer_target(p) if p.dtype == torch.float32 else None
                if _fused_ok(p, p.grad) or (target is not None and _flat_pair_ok(p, p.grad, need_cuda=False)):
                    grad = p.grad
                    if not (p.is_contiguous() and grad.is_contiguous()) and grad.stride() != p.stride():
                        grad = torch.empty_like(p, dtype=grad.dtype).copy_(grad)      # bring the gradient into the parameter's memory order
                    if first:
                        st["buf"] = torch.zeros(p.numel(), device=p.device, dtype=torch.float32) if g["momentum"] else None
                        if p.dtype == torch.bfloat16:
                            st["master"] = _flat(p.detach()).float().clone()
                    layout = None if p.is_contiguous() else p.stride()          # None: row-major order
                    if not first and st.get("layout") != layout and st["buf"] is not None:
                        # the parameter was re-laid-out since the last step: re-order the momentum buffer to match
                        old_stride = st.get("layout") or torch.empty(p.shape, device="meta").stride()
                        old = torch.as_strided(st["buf"], p.shape, old_stride)
                        st["buf"] = _flat(torch.empty_like(p, dtype=torch.float32).copy_(old)).clone()
                    st["layout"] = layout
                    master = st.get("master", _flat(p.detach()))
                    low = _flat(p.detach()) if p.dtype == torch.bfloat16 else (_flat(target) if target is not None else None)
                    ops.sgd_flat_(master, low, st["buf"], _flat(grad), lr=g["lr"],
                                  momentum=g["momentum"], dampening=g["dampening"], weight_decay=g["weight_decay"], nesterov=g["nesterov"],
                                  first_step=first, maximize=g["maximize"])
                    if target is not None:
                        mark_synced(p)
                    continue
                d = -p.grad if g["maximize"] else p.grad
                if g["weight_decay"]:
                    d = d.add(p, alpha=g["weight_decay"])
                if g["momentum"]:
                    if first:
                        st["buf"] = d.clone()
                    else:
                        st["buf"].mul_(g["momentum"]).add_(d, alpha=1 - g["dampening"])
                    d = d.add(st["buf"], alpha=g["momentum"]) if g["nesterov"] else st["buf"]
                elif first:
                    st["buf"] = None
                p.add_(d, alpha=-g["lr"])
        return loss


class AdamW(Optimizer):
    """AdamW with decoupled weight decay ``p *= 1 - lr*wd`` (ferrotorch-optim/src/adamw.rs:315,430)."""

    _decoupled = True

    def __init__(self, params, config=None, **kw):
        cfg = config or (AdamWConfig if self._decoupled else AdamConfig)(**kw)
        self.config = cfg
        super().__init__(params, dict(lr=cfg.lr, betas=tuple(cfg.betas), eps=cfg.eps, weight_decay=cfg.weight_decay, amsgrad=cfg.amsgrad,
                                      maximize=cfg.maximize))

    @torch.no_grad()
    def step(self, closure: Optional[Callable] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros(p.numel(), device=p.device, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros(p.numel(), device=p.device, dtype=torch.float32)
                    if g["amsgrad"]:
                        st["max_exp_avg_sq"] = torch.zeros(p.numel(), device=p.device, dtype=torch.float32)
                    if p.dtype != torch.float32:
                        st["master"] = p.detach().float().reshape(-1).clone()
                st["step"] += 1
                t = st["step"]
                grad = p.grad
                # a row-major f32 parameter with a compute copy takes the flat kernel on any device: the copy is rewritten with the master
                target = optimizer_target(p) if (p.dtype == torch.float32 and p.is_contiguous() and grad.is_contiguous()) else None
                if self._decoupled and not g["amsgrad"] and (_fused_ok(p, grad) or (target is not None and not grad.is_sparse)):
                    master = st.get("master", p.view(-1))
                    low = p.view(-1) if p.dtype == torch.bfloat16 else (target.view(-1) if target is not None else None)
                    ops.adamw_flat_(master, low, st["exp_avg"], st["exp_avg_sq"],
                                    grad.reshape(-1), lr=g["lr"], beta1=b1, beta2=b2, eps=g["eps"], weight_decay=g["weight_decay"], step=t,
                                    maximize=g["maximize"])
                    if target is not None:
                        mark_synced(p)
                    continue
                gr = grad.detach().float().reshape(-1)
                if g["maximize"]:
                    gr = -gr
                master = st.get("master", None)
                # moments and gradient are walked in logical (row-major) order; an f32 parameter whose memory is not row-major (the
                # convolution weights of a channels-last model) is updated through a row-major copy that is written back below
                writeback = master is None and not p.is_contiguous()
                w = master if master is not None else (p.detach().reshape(-1).clone() if writeback else p.view(-1))
                if self._decoupled:
                    w.mul_(1 - g["lr"] * g["weight_decay"])
                elif g["weight_decay"]:
                    gr = gr.add(w, alpha=g["weight_decay"])                    # coupled L2 (Adam)
                st["exp_avg"].mul_(b1).add_(gr, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(gr, gr, value=1 - b2)
                c1, c2 = 1 - b1 ** t, 1 - b2 ** t
                v = st["exp_avg_sq"]
                if g["amsgrad"]:
                    torch.maximum(st["max_exp_avg_sq"], v, out=st["max_exp_avg_sq"])
                    v = st["max_exp_avg_sq"]
                w.addcdiv_(st["exp_avg"], (v.sqrt() / math.sqrt(c2)).add_(g["eps"]), value=-g["lr"] / c1)
                if master is not None or writeback:
                    p.copy_(w.view_as(p))
        return loss


class Adam(AdamW):
    """Adam with (coupled) L2 weight decay added to the gradient, as ``FUSED_ADAM_PTX`` does (ferrotorch-gpu/src/kernels.rs:11907-11916)."""
    _decoupled = False


def _named(torch_cls, name, doc, cfg_cls=None):
    """A torch optimiser under this package's name and base class. Its second argument may be the matching ``<Name>Config`` (the reference's
    constructor form, ``Adamax::new(params, AdamaxConfig::default().with_lr(..))``); keyword arguments still work and override the config."""
    def __init__(self, params, config=None, **kw):
        if config is not None and hasattr(config, "__dataclass_fields__"):
            import dataclasses
            kw = {**dataclasses.asdict(config), **kw}
        elif config is not None:
            kw.setdefault("lr", config)                      # positional learning rate, as torch allows
        self.config = config
        torch_cls.__init__(self, params, **kw)
    return type(name, (torch_cls, Optimizer), {"__doc__": doc, "__module__": __name__, "__init__": __init__})


# -- configs of the remaining optimisers (defaults: ferrotorch-optim/src/{adadelta,adagrad,adamax,asgd,nadam,radam,rmsprop,rprop,sparse_adam,lbfgs}.rs) --
@dataclass(frozen=True)
class AdadeltaConfig(_Cfg):
    lr: float = 1.0
    rho: float = 0.9
    eps: float = 1e-6
    weight_decay: float = 0.0
    foreach: bool = False


@dataclass(frozen=True)
class AdagradConfig(_Cfg):
    lr: float = 0.01
    lr_decay: float = 0.0
    weight_decay: float = 0.0
    initial_accumulator_value: float = 0.0
    eps: float = 1e-10
    maximize: bool = False
    foreach: bool = False


@dataclass(frozen=True)
class AdamaxConfig(_Cfg):
    lr: float = 2e-3
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.0
    foreach: bool = False


@dataclass(frozen=True)
class AsgdConfig(_Cfg):
    lr: float = 1e-2
    lambd: float = 1e-4
    alpha: float = 0.75
    t0: float = 1e6
    weight_decay: float = 0.0
    foreach: bool = False


@dataclass(frozen=True)
class NAdamConfig(_Cfg):
    lr: float = 2e-3
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.0
    momentum_decay: float = 4e-3
    decoupled_weight_decay: bool = False
    foreach: bool = False


@dataclass(frozen=True)
class RAdamConfig(_Cfg):
    lr: float = 1e-3
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.0
    decoupled_weight_decay: bool = False
    foreach: bool = False


@dataclass(frozen=True)
class RmspropConfig(_Cfg):
    lr: float = 0.01
    alpha: float = 0.99
    eps: float = 1e-8
    weight_decay: float = 0.0
    momentum: float = 0.0
    centered: bool = False
    maximize: bool = False
    foreach: bool = False


@dataclass(frozen=True)
class RpropConfig(_Cfg):
    lr: float = 1e-2
    etas: tuple = (0.5, 1.2)
    step_sizes: tuple = (1e-6, 50.0)


@dataclass(frozen=True)
class SparseAdamConfig(_Cfg):
    lr: float = 1e-3
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8


@dataclass(frozen=True)
class LbfgsConfig(_Cfg):
    lr: float = 1.0
    max_iter: int = 20
    max_eval: Optional[int] = None
    tolerance_grad: float = 1e-7
    tolerance_change: float = 1e-9
    history_size: int = 10
    line_search_fn: Optional[str] = None                     # None or "strong_wolfe"


@dataclass(frozen=True)
class AdafactorConfig(_Cfg):
    """ferrotorch-optim/src/adafactor.rs:28-60. ``relative_step`` (default on) ignores ``lr`` and uses ``t^-0.5`` (with ``warmup_init``:
    ``min(t^-0.5, 1e-6 t)``) times ``max(rms(param), eps_rms)``."""
    lr: Optional[float] = None
    beta1: Optional[float] = None
    decay_rate: float = -0.8
    eps_sq: float = 1e-30
    eps_rms: float = 1e-3
    weight_decay: float = 0.0
    relative_step: bool = True
    warmup_init: bool = False


@dataclass(frozen=True)
class KfacConfig(_Cfg):
    """ferrotorch-optim/src/natural_gradient.rs:54-82: ``momentum`` is both the decay of the running Kronecker factors and the momentum of the
    preconditioned gradient; ``weight_decay`` is L2 (added to the gradient before preconditioning)."""
    lr: float = 1e-3
    damping: float = 1e-3
    momentum: float = 0.9
    update_freq: int = 10
    weight_decay: float = 0.0
    maximize: bool = False


@dataclass(frozen=True, order=True)
class ParamKey:
    """Position of a parameter: group index, index within the group; prints as ``g<group>_p<param>``, the key of a saved optimiser state
    (ferrotorch-optim/src/param_key.rs:43)."""
    group: int
    param: int

    def __str__(self):
        return f"g{self.group}_p{self.param}"

    @classmethod
    def parse(cls, s: str) -> "ParamKey":
        import re
        m = re.fullmatch(r"g(\d+)_p(\d+)", s)
        if not m:
            raise InvalidArgument(f"not a parameter key: {s!r}")
        return cls(int(m.group(1)), int(m.group(2)))


OptimizerState = Dict[str, Dict[str, List[float]]]           # saved form: parameter key -> named buffers as flat f64 lists (optimizer.rs:8)


# Adamax, NAdam, RAdam, Adagrad, Adadelta, Rmsprop, Rprop, Asgd, SparseAdam and Lbfgs are implemented in optim/elementwise.py (one shared
# element-wise CUDA kernel plus the tensor-operation forms) and re-exported at the end of this module.
LineSearchFn = str


class Adafactor(Optimizer):
    """Adafactor: factored second moments for matrices (row/column statistics), relative step size optional."""

    def __init__(self, params, lr: Optional[float] = 1e-3, eps=(1e-30, 1e-3), clip_threshold: float = 1.0, decay_rate: float = -0.8,
                 beta1: Optional[float] = None, weight_decay: float = 0.0, scale_parameter: bool = True, relative_step: bool = False,
                 warmup_init: bool = False):
        if isinstance(lr, AdafactorConfig):
            c = lr
            lr, eps, decay_rate, beta1, weight_decay = (c.lr if c.lr is not None else 1e-3), (c.eps_sq, c.eps_rms), c.decay_rate, c.beta1, c.weight_decay
            relative_step, warmup_init, scale_parameter = c.relative_step, c.warmup_init, c.relative_step      # the reference scales by rms(param)
            self.config = c                                                                                       # only on the relative path
        self._warmup_init = warmup_init
        super().__init__(params, dict(lr=lr, eps=eps, clip_threshold=clip_threshold, decay_rate=decay_rate, beta1=beta1,
                                      weight_decay=weight_decay, scale_parameter=scale_parameter, relative_step=relative_step))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad.float()
                st = self.state[p]
                factored = grad.dim() >= 2
                if not st:
                    st["step"] = 0
                    if factored:
                        st["row"] = torch.zeros(grad.shape[:-1], device=grad.device)
                        st["col"] = torch.zeros(grad.shape[:-2] + grad.shape[-1:], device=grad.device)
                    else:
                        st["sq"] = torch.zeros_like(grad)
                    if g["beta1"] is not None:
                        st["exp_avg"] = torch.zeros_like(grad)
                st["step"] += 1
                t = st["step"]
                pf = p.float()
                rms_p = pf.norm(2) / math.sqrt(pf.numel())
                lr = g["lr"]
                if g["relative_step"]:
                    lr = min(1e-2, 1.0 / math.sqrt(t))
                    if getattr(self, "config", None) is not None:                 # reference rule: no 1e-2 cap, optional linear warm-up
                        lr = min(t ** -0.5, 1e-6 * t) if self._warmup_init else t ** -0.5
                if g["scale_parameter"]:
                    lr = lr * max(g["eps"][1], float(rms_p))
                beta2t = 1.0 - t ** g["decay_rate"]
                upd = grad * grad + g["eps"][0]
                if factored:
                    st["row"].mul_(beta2t).add_(upd.mean(-1), alpha=1 - beta2t)
                    st["col"].mul_(beta2t).add_(upd.mean(-2), alpha=1 - beta2t)
                    r = (st["row"] / st["row"].mean(-1, keepdim=True)).rsqrt().unsqueeze(-1)
                    c = st["col"].unsqueeze(-2).rsqrt()
                    u = grad * r * c
                else:
                    st["sq"].mul_(beta2t).add_(upd, alpha=1 - beta2t)
                    u = grad * st["sq"].rsqrt()
                u = u / max(1.0, float(u.norm(2) / math.sqrt(u.numel())) / g["clip_threshold"])
                u = u * lr
                if g["beta1"] is not None:
                    st["exp_avg"].mul_(g["beta1"]).add_(u, alpha=1 - g["beta1"])
                    u = st["exp_avg"]
                if g["weight_decay"]:
                    pf = pf * (1 - g["weight_decay"] * lr)
                p.copy_((pf - u).to(p.dtype))
        return loss


def newton_schulz_cubic(G: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Orthogonalise a matrix: ``G <- G/||G||_F`` then ``steps`` times ``G <- 1/2 * G (3I - G^T G)``
    (ferrotorch-optim/src/muon.rs:182-228). bf16 CUDA matrices use the tcgen05 GEMM for both products."""
    transposed = G.shape[0] < G.shape[1]
    X = G.t() if transposed else G                      # tall: rows >= cols, so G^T G is the small square
    X = X / (X.norm() + 1e-7)
    n = X.shape[1]
    fast = X.is_cuda and X.dtype == torch.bfloat16 and n % 8 == 0 and X.shape[0] % 8 == 0
    eye3 = 3.0 * torch.eye(n, device=X.device, dtype=torch.float32)
    for _ in range(steps):
        if fast:
            Xc = X.contiguous()
            A = ops.gemm(Xc, Xc, a_mn=True, b_mn=True, out_dtype=torch.float32)       # X^T X  [n, n]
            M = (0.5 * (eye3 - A)).to(torch.bfloat16)
            X = ops.gemm(Xc, M, b_mn=True)                                             # X M
        else:
            Xf = X.float()
            X = (0.5 * Xf @ (eye3 - Xf.t() @ Xf)).to(G.dtype)
    return X.t() if transposed else X


class Muon(Optimizer):
    """Momentum + Newton-Schulz orthogonalised updates for 2-D parameters, AdamW for everything else."""

    def __init__(self, params, config: Optional[MuonConfig] = None, **kw):
        cfg = config or MuonConfig(**kw)
        self.config = cfg
        super().__init__(params, dict(lr=cfg.lr, momentum=cfg.momentum, nesterov=cfg.nesterov, ns_steps=cfg.ns_steps,
                                      weight_decay=cfg.weight_decay, adamw_lr=cfg.adamw_lr, adamw_betas=cfg.adamw_betas, adamw_eps=cfg.adamw_eps))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if p.dim() == 2:
                    if "buf" not in st:
                        st["buf"] = torch.zeros_like(p.grad)
                    buf = st["buf"]
                    buf.mul_(g["momentum"]).add_(p.grad)
                    upd = p.grad.add(buf, alpha=g["momentum"]) if g["nesterov"] else buf
                    o = newton_schulz_cubic(upd, g["ns_steps"])
                    if g["weight_decay"]:
                        p.mul_(1 - g["lr"] * g["weight_decay"])
                    p.add_(o.to(p.dtype), alpha=-g["lr"] * max(1.0, p.shape[0] / p.shape[1]) ** 0.5)
                else:
                    if "exp_avg" not in st:
                        st["step"], st["exp_avg"], st["exp_avg_sq"] = 0, torch.zeros_like(p, dtype=torch.float32), torch.zeros_like(p, dtype=torch.float32)
                    st["step"] += 1
                    b1, b2 = g["adamw_betas"]
                    gr = p.grad.float()
                    st["exp_avg"].mul_(b1).add_(gr, alpha=1 - b1)
                    st["exp_avg_sq"].mul_(b2).addcmul_(gr, gr, value=1 - b2)
                    c1, c2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
                    upd = st["exp_avg"] / c1 / ((st["exp_avg_sq"] / c2).sqrt() + g["adamw_eps"])
                    p.add_(upd.to(p.dtype), alpha=-g["adamw_lr"])
        return loss


class Kfac(Optimizer):
    """Kronecker-factored natural gradient for ``Linear`` layers: running covariances of layer inputs (A) and output gradients (G),
    preconditioned update ``G^-1 dW A^-1`` with Tikhonov damping; other parameters fall back to SGD."""

    def __init__(self, model: torch.nn.Module, lr=0.01, damping: float = 1e-3, ema: float = 0.95, update_freq: int = 1, momentum: float = 0.0,
                 weight_decay: float = 0.0, maximize: bool = False):
        self.config = lr if isinstance(lr, KfacConfig) else None
        if self.config is not None:
            c = lr
            lr, damping, ema, update_freq, momentum, weight_decay, maximize = c.lr, c.damping, c.momentum, c.update_freq, c.momentum, c.weight_decay, c.maximize
        self.momentum, self.weight_decay, self.maximize = momentum, weight_decay, maximize
        self._mom: Dict[torch.Tensor, torch.Tensor] = {}
        self.model, self.damping, self.ema, self.update_freq = model, damping, ema, update_freq
        self._layers: Dict[torch.nn.Module, dict] = {}
        super().__init__(model.parameters(), dict(lr=lr))
        for m in model.modules():
            if hasattr(m, "weight") and getattr(m, "weight", None) is not None and m.weight.dim() == 2 and hasattr(m, "in_features"):
                self._layers[m] = {}
                m.register_forward_pre_hook(self._save_input)
                m.register_full_backward_hook(self._save_grad)
        self._steps = 0

    def _save_input(self, mod, args):
        if mod.training and torch.is_grad_enabled():
            x = args[0].detach().reshape(-1, args[0].shape[-1]).float()
            if mod.bias is not None:
                x = torch.cat([x, torch.ones(x.shape[0], 1, device=x.device)], 1)
            a = x.t() @ x / x.shape[0]
            s = self._layers[mod]
            s["A"] = a if "A" not in s else s["A"] * self.ema + a * (1 - self.ema)

    def _save_grad(self, mod, gin, gout):
        g = gout[0].detach().reshape(-1, gout[0].shape[-1]).float()
        gg = g.t() @ g * g.shape[0]
        s = self._layers[mod]
        s["G"] = gg if "G" not in s else s["G"] * self.ema + gg * (1 - self.ema)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        lr = self.param_groups[0]["lr"]
        handled = set()
        for m, s in self._layers.items():
            if m.weight.grad is None or "A" not in s or "G" not in s:
                continue
            if self._steps % self.update_freq == 0 or "Ainv" not in s:
                s["Ainv"] = torch.linalg.inv(s["A"] + self.damping ** 0.5 * torch.eye(s["A"].shape[0], device=s["A"].device))
                s["Ginv"] = torch.linalg.inv(s["G"] + self.damping ** 0.5 * torch.eye(s["G"].shape[0], device=s["G"].device))
            sign = -1.0 if self.maximize else 1.0
            gw = sign * m.weight.grad.float() + self.weight_decay * m.weight.float()
            if m.bias is not None and m.bias.grad is not None:
                gw = torch.cat([gw, (sign * m.bias.grad.float() + self.weight_decay * m.bias.float()).unsqueeze(1)], 1)
            nat = s["Ginv"] @ gw @ s["Ainv"]
            if self.momentum > 0.0:
                buf = self._mom.get(m.weight)
                nat = nat.clone() if buf is None else buf.mul_(self.momentum).add_(nat)
                self._mom[m.weight] = nat
            if m.bias is not None and m.bias.grad is not None:
                m.weight.add_(nat[:, :-1].to(m.weight.dtype), alpha=-lr)
                m.bias.add_(nat[:, -1].to(m.bias.dtype), alpha=-lr)
                handled.add(m.bias)
            else:
                m.weight.add_(nat.to(m.weight.dtype), alpha=-lr)
            handled.add(m.weight)
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is not None and p not in handled:
                    d = (-p.grad if self.maximize else p.grad) + self.weight_decay * p
                    if self.momentum > 0.0:
                        buf = self._mom.get(p)
                        d = d.clone() if buf is None else buf.mul_(self.momentum).add_(d)
                        self._mom[p] = d
                    p.add_(d, alpha=-lr)
        self._steps += 1
        return loss


# -- differentiable SGD (ferrotorch-optim/src/differentiable.rs:55-110) ---------------------------------------------------------
def diff_sgd_step(params: List[torch.Tensor], grads: List[torch.Tensor], lr: float) -> List[torch.Tensor]:
    """Functional SGD step that stays in the autograd graph (for meta-learning / unrolled optimisation)."""
    return [p - lr * g for p, g in zip(params, grads)]


def diff_sgd_momentum_step(params, grads, bufs, lr: float, momentum: float):
    new_bufs = [momentum * b + g for b, g in zip(bufs, grads)]
    return [p - lr * b for p, b in zip(params, new_bufs)], new_bufs


# -- foreach helpers (ferrotorch-optim/src/foreach_utils.rs:15-31) ----------------------------------------------------------------
def elemwise_max(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return torch.maximum(a, b)


def scalar_on(value: float, like: torch.Tensor) -> torch.Tensor:
    return torch.full((), value, device=like.device, dtype=like.dtype)


from .elementwise import Adamax, NAdam, RAdam, Adagrad, Adadelta, Rmsprop, Rprop, Asgd, SparseAdam, Lbfgs  # noqa: E402,F401
