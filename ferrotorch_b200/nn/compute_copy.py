"""bf16 compute copies of f32 master weights, kept current by the optimizer instead of being re-cast in every forward pass.

Mixed-precision training keeps f32 master weights and multiplies with bf16 copies. Casting inside ``forward`` costs one elementwise launch
per layer per step (a strided, non-vectorised one when the kernel wants another layout), and a second one in the backward pass to bring the
bf16 weight gradient back to f32. With a compute copy attached to a parameter

* the fused optimizer kernels (``optim.Sgd``) write the bf16 copy in the same pass that updates the f32 master (the copy has the master's
  memory layout, so a channels-last 3x3 weight is already in the ``[Cout, 3, 3, Cin]`` order the convolution kernel reads);
* the layers of ``ferrotorch_b200.vision`` multiply with the copy and hand the weight gradient back in f32, straight from the GEMM.

A copy that went stale because the master was changed behind the optimizer's back (``load_state_dict``, an initialiser, ``copy_``) is detected
through the tensor version counter and refreshed on its next use. The reference keeps f32 parameters and casts per call
(ferrotorch-core/src/autograd/autocast.rs:4-150, autocast_ops.rs:29-45); this is the same policy with the cast hoisted out of the step.
"""
from __future__ import annotations

from typing import Iterable, Optional

import torch

_ATTR = "_ft_compute"


class _Copy:
    __slots__ = ("tensor", "version")

    def __init__(self, tensor: torch.Tensor, version: int):
        self.tensor, self.version = tensor, version


def _fresh(p: torch.Tensor, dtype: torch.dtype) -> _Copy:
    t = torch.empty_like(p, dtype=dtype)           # preserves the memory format (dense tensors keep their strides)
    t.copy_(p.detach())
    return _Copy(t, p._version)


def attach_compute_copies(model_or_params, dtype: torch.dtype = torch.bfloat16, min_dim: int = 2) -> int:
    """Gives every f32 parameter with at least ``min_dim`` dimensions (weights, not biases or norm scales) a ``dtype`` compute copy.
    Accepts a module or an iterable of parameters; returns the number of copies attached."""
    params: Iterable[torch.Tensor] = model_or_params.parameters() if hasattr(model_or_params, "parameters") else model_or_params
    n = 0
    for p in params:
        if p.dtype == torch.float32 and p.dim() >= min_dim:
            setattr(p, _ATTR, _fresh(p, dtype))
            n += 1
    return n


def detach_compute_copies(model_or_params) -> None:
    params = model_or_params.parameters() if hasattr(model_or_params, "parameters") else model_or_params
    for p in params:
        if hasattr(p, _ATTR):
            delattr(p, _ATTR)


def compute_copy(p: torch.Tensor) -> Optional[torch.Tensor]:
    """The parameter's compute copy (refreshed first if the master changed outside the optimizer, moved or was re-laid-out), or ``None``."""
    c: Optional[_Copy] = getattr(p, _ATTR, None)
    if c is None:
        return None
    t = c.tensor
    if t.device != p.device or t.shape != p.shape or t.stride() != p.stride():
        c = _fresh(p, t.dtype)
        setattr(p, _ATTR, c)
    elif c.version != p._version:
        with torch.no_grad():
            t.copy_(p.detach())
        c.version = p._version
    return c.tensor


def optimizer_target(p: torch.Tensor) -> Optional[torch.Tensor]:
    """For optimizers: the copy to overwrite together with the master (same layout as ``p``), or ``None``. The caller updates the master
    through a raw kernel (no version bump) and the copy in the same pass, so the pair stays in step; call :func:`mark_synced` afterwards."""
    c: Optional[_Copy] = getattr(p, _ATTR, None)
    if c is None or c.tensor.device != p.device or c.tensor.shape != p.shape or c.tensor.stride() != p.stride():
        return None
    return c.tensor


def mark_synced(p: torch.Tensor) -> None:
    c: Optional[_Copy] = getattr(p, _ATTR, None)
    if c is not None:
        c.version = p._version
