"""Flat multi-tensor optimizer kernels (one launch per flat buffer instead of ~12 per parameter).

Reference parity: foreach AdamW/SGD op chains (ferrotorch-optim/src/adamw.rs:226-373, sgd.rs:210),
FUSED_ADAM_PTX (ferrotorch-gpu/src/kernels.rs:11918), clip_grad_norm_ (ferrotorch-nn/src/utils.rs:134),
GradScaler::unscale_ (ferrotorch-optim/src/grad_scaler.rs:200-240).
"""
from __future__ import annotations

import torch

from .. import _lib
from ._workspace import workspace


def adamw_flat_(master: torch.Tensor, p_bf16: torch.Tensor | None, m: torch.Tensor, v: torch.Tensor, grad: torch.Tensor, *, lr: float,
                beta1: float, beta2: float, eps: float, weight_decay: float, step: int, maximize: bool = False,
                grad_scale: torch.Tensor | None = None, skip: torch.Tensor | None = None, max_ctas: int = 0) -> None:
    n = master.numel()
    if master.is_cuda:
        _lib.call("ft_adamw_flat", master, p_bf16, m, v, grad, n, int(grad.dtype == torch.float32), lr, beta1, beta2, eps,
                  weight_decay, step, int(maximize), grad_scale, skip, max_ctas, _lib.S())
        return
    g = grad.float()
    if grad_scale is not None:
        g = g * grad_scale
    if maximize:
        g = -g
    master.mul_(1 - lr * weight_decay)
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    c1, c2 = 1 - beta1 ** step, 1 - beta2 ** step
    master.addcdiv_(m, (v.sqrt() / (c2 ** 0.5)).add_(eps), value=-lr / c1)
    if p_bf16 is not None:
        p_bf16.copy_(master)


def sgd_flat_(master: torch.Tensor, p_bf16: torch.Tensor | None, buf: torch.Tensor | None, grad: torch.Tensor, *, lr: float,
              momentum: float = 0.0, dampening: float = 0.0, weight_decay: float = 0.0, nesterov: bool = False,
              first_step: bool = False, maximize: bool = False, grad_scale: torch.Tensor | None = None) -> None:
    n = master.numel()
    if master.is_cuda:
        _lib.call("ft_sgd_flat", master, p_bf16, buf, grad, n, int(grad.dtype == torch.float32), lr, momentum, dampening,
                  weight_decay, int(nesterov), int(first_step), int(maximize), grad_scale, _lib.S())
        return
    g = grad.float()
    if grad_scale is not None:
        g = g * grad_scale
    if maximize:
        g = -g
    if weight_decay:
        g = g + weight_decay * master
    if momentum:
        if first_step:
            buf.copy_(g)
        else:
            buf.mul_(momentum).add_(g, alpha=1 - dampening)
        g = g + momentum * buf if nesterov else buf
    master.add_(g, alpha=-lr)
    if p_bf16 is not None:
        p_bf16.copy_(master)


def grad_norm_(buffers, max_norm: float = 0.0, found_inf: torch.Tensor | None = None):
    """Global L2 norm over a list of flat buffers, on device, no host sync.

    Returns (norm, clip_coef) as 0-d device tensors; ``clip_coef = min(1, max_norm/(norm+1e-6))``
    (1 when ``max_norm <= 0``) can be passed to the optimizer kernels as ``grad_scale``.
    """
    buffers = [b for b in buffers if b is not None and b.numel() > 0]
    dev = buffers[0].device
    if not buffers[0].is_cuda:
        tot = sum(float(b.float().pow(2).sum()) for b in buffers) ** 0.5
        nrm = torch.tensor(tot)
        coef = torch.tensor(min(1.0, max_norm / (tot + 1e-6)) if max_norm > 0 else 1.0)
        return nrm, coef
    out = torch.zeros(3, device=dev, dtype=torch.float32)
    part = workspace(dev, "sqnorm_partial", 2048 * 4)
    for i, b in enumerate(buffers):
        last = i == len(buffers) - 1
        _lib.call("ft_sqnorm", b, b.numel(), int(b.dtype == torch.float32), part, _lib.c_void_p(out.data_ptr()), int(i > 0),
                  int(last), float(max_norm), _lib.c_void_p(out.data_ptr() + 4), _lib.c_void_p(out.data_ptr() + 8), found_inf,
                  _lib.S())
    return out[1], out[2]


def scale_(x: torch.Tensor, scale: float = 1.0, scale_tensor: torch.Tensor | None = None) -> torch.Tensor:
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and x.is_contiguous():
        _lib.call("ft_scale_inplace", x, x.numel(), int(x.dtype == torch.float32), float(scale), scale_tensor, _lib.S())
        return x
    x.mul_(scale if scale_tensor is None else scale * scale_tensor)
    return x
