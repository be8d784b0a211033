"""Fused cross-entropy: loss and gradient from one pass over the logits.

Reference parity: CrossEntropyLoss (ferrotorch-nn/src/loss.rs:171-330; CUDA backward is NotImplementedOnCuda there).
"""
from __future__ import annotations

import torch

from .. import _lib


def cross_entropy_fwd_bwd(logits2: torch.Tensor, targets: torch.Tensor, *, ignore_index: int = -100, label_smoothing: float = 0.0,
                          grad_scale: float | None = None, inplace_grad: bool = True, want_grad: bool = True):
    """Returns (mean_loss [0-d f32 tensor], dlogits or None, n_valid tensor).

    The gradient is for the mean over valid rows (scaled by ``grad_scale`` if given, else by 1/rows
    when no row is ignored). ``inplace_grad`` overwrites the logits with the gradient.
    """
    rows, V = logits2.shape
    t = targets.reshape(-1).contiguous()
    # the kernel reads rows with 16-byte loads: the row pitch must be a multiple of 16 bytes (pad the vocabulary dimension otherwise)
    aligned = logits2.stride(1) == 1 and logits2.stride(0) % (8 if logits2.dtype == torch.bfloat16 else 4) == 0 and logits2.data_ptr() % 16 == 0
    if logits2.is_cuda and logits2.dtype in (torch.bfloat16, torch.float32) and aligned:
        loss_rows = torch.empty(rows, device=logits2.device, dtype=torch.float32)
        out = torch.empty(2, device=logits2.device, dtype=torch.float32)
        dl = None
        if want_grad:
            dl = logits2 if inplace_grad else torch.empty_strided(logits2.shape, logits2.stride(), device=logits2.device, dtype=logits2.dtype)
        gs = grad_scale if grad_scale is not None else 1.0 / rows
        _lib.call("ft_cross_entropy", logits2, t, loss_rows, None, dl, rows, V, logits2.stride(0), ignore_index,
                  float(label_smoothing), float(gs), None, int(logits2.dtype == torch.float32), _lib.S())
        _lib.call("ft_loss_mean", loss_rows, t, rows, ignore_index, _lib.c_void_p(out.data_ptr()),
                  _lib.c_void_p(out.data_ptr() + 4), _lib.S())
        return out[0], dl, out[1]
    lf = logits2.float().detach().requires_grad_(want_grad)
    loss = torch.nn.functional.cross_entropy(lf, t, ignore_index=ignore_index, label_smoothing=label_smoothing)
    dl = None
    if want_grad:
        (dl,) = torch.autograd.grad(loss, lf)
        dl = dl.to(logits2.dtype)
    return loss.detach(), dl, (t != ignore_index).sum().float()


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, ignore_index, label_smoothing):
        l2 = logits.reshape(-1, logits.shape[-1])
        if not l2.is_contiguous():
            l2 = l2.contiguous()
        n_valid = int((targets != ignore_index).sum().item()) if ignore_index is not None else l2.shape[0]
        loss, dl, _ = cross_entropy_fwd_bwd(l2, targets, ignore_index=ignore_index, label_smoothing=label_smoothing,
                                            grad_scale=1.0 / max(n_valid, 1), inplace_grad=False, want_grad=True)
        ctx.save_for_backward(dl)
        ctx.shp = logits.shape
        return loss.clone()

    @staticmethod
    def backward(ctx, g):
        (dl,) = ctx.saved_tensors
        return (dl * g.to(dl.dtype)).reshape(ctx.shp), None, None, None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100, label_smoothing: float = 0.0) -> torch.Tensor:
    """Mean cross-entropy over valid rows (differentiable w.r.t. ``logits``)."""
    if logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32):
        return _CrossEntropyFn.apply(logits, targets, ignore_index, label_smoothing)
    return torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1),
                                             ignore_index=ignore_index, label_smoothing=label_smoothing)
