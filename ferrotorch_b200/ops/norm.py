"""RMSNorm / LayerNorm on the hand-written kernels (bf16 storage, f32 math) with autograd.

Reference parity: ``rmsnorm_f32`` (ferrotorch-core/src/gpu_dispatch.rs:1058), RMSNorm / LayerNorm modules
(ferrotorch-nn/src/norm.rs:53,850).
"""
from __future__ import annotations

import torch

from .. import _lib
from ._workspace import workspace


def _parts(rows: int) -> int:
    return min(rows, 296)


def rmsnorm_fwd(x2: torch.Tensor, w: torch.Tensor, eps: float, residual: torch.Tensor | None = None):
    """Returns (y, rstd, x_sum). With ``residual`` the kernel also writes x_sum = x + residual and normalises that."""
    rows, d = x2.shape
    y = torch.empty_like(x2)
    rstd = torch.empty(rows, device=x2.device, dtype=torch.float32)
    xs = torch.empty_like(x2) if residual is not None else None
    _lib.call("ft_rmsnorm_fwd", _lib.P(x2), _lib.P(residual), _lib.P(w), _lib.P(y), _lib.P(xs), _lib.P(rstd), rows, d,
              _lib.c_float(eps), _lib.S())
    return y, rstd, (xs if xs is not None else x2)


def rmsnorm_bwd(x2, w, dy2, rstd, dres=None, dw_out=None, accumulate=False):
    """Returns (dx, dw). ``dres`` is added into dx (the residual branch's gradient)."""
    rows, d = x2.shape
    dx = torch.empty_like(x2)
    part = workspace(x2.device, "norm_partial", _parts(rows) * d * 4)
    dw = dw_out if dw_out is not None else torch.empty(d, device=x2.device, dtype=torch.bfloat16)
    bf, f32 = (dw, None) if dw.dtype == torch.bfloat16 else (None, dw)
    _lib.call("ft_rmsnorm_bwd", _lib.P(x2), _lib.P(w), _lib.P(dy2), _lib.P(rstd), _lib.P(dres), _lib.P(dx), _lib.P(part),
              _lib.P(bf), _lib.P(f32), int(accumulate), rows, d, _lib.S())
    return dx, dw


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1]).contiguous()
        y, rstd, _ = rmsnorm_fwd(x2, w, eps)
        ctx.save_for_backward(x2, w, rstd)
        ctx.shp = shp
        return y.reshape(shp)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        dx, dw = rmsnorm_bwd(x2, w, dy.reshape(x2.shape).contiguous(), rstd)
        return dx.reshape(ctx.shp), dw, None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384:
        return _RMSNormFn.apply(x, weight.to(torch.bfloat16), eps)
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return y.to(x.dtype)


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1]).contiguous()
        rows, d = x2.shape
        y = torch.empty_like(x2)
        mean = torch.empty(rows, device=x.device, dtype=torch.float32)
        rstd = torch.empty_like(mean)
        _lib.call("ft_layernorm_fwd", _lib.P(x2), _lib.P(w), _lib.P(b), _lib.P(y), _lib.P(mean), _lib.P(rstd), rows, d,
                  _lib.c_float(eps), _lib.S())
        ctx.save_for_backward(x2, w, mean, rstd)
        ctx.shp, ctx.has_b = shp, b is not None
        return y.reshape(shp)

    @staticmethod
    def backward(ctx, dy):
        x2, w, mean, rstd = ctx.saved_tensors
        rows, d = x2.shape
        dy2 = dy.reshape(rows, d).contiguous()
        dx = torch.empty_like(x2)
        part = workspace(x2.device, "norm_partial2", 2 * _parts(rows) * d * 4)
        half = _parts(rows) * d * 4
        dw = torch.empty(d, device=x2.device, dtype=torch.bfloat16)
        db = torch.empty(d, device=x2.device, dtype=torch.bfloat16)
        _lib.call("ft_layernorm_bwd", _lib.P(x2), _lib.P(w), _lib.P(dy2), _lib.P(mean), _lib.P(rstd), _lib.P(dx),
                  _lib.c_void_p(part.data_ptr()), _lib.c_void_p(part.data_ptr() + half), _lib.P(dw), _lib.P(db), rows, d, _lib.S())
        return dx.reshape(ctx.shp), dw, (db if ctx.has_b else None), None


def layer_norm(x, weight, bias=None, eps: float = 1e-5):
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384 and weight is not None:
        return _LayerNormFn.apply(x, weight.to(torch.bfloat16), None if bias is None else bias.to(torch.bfloat16), eps)
    return torch.nn.functional.layer_norm(x, (x.shape[-1],), weight, bias, eps)
