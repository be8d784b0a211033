"""Dropout variants, embedding bags, reshaping layers and upsampling (ferrotorch-nn/src/dropout.rs, embedding.rs:236-520, identity.rs,
upsample.rs)."""
from __future__ import annotations

import math
from typing import Optional, Sequence, Union

import torch

from ..errors import InvalidArgument, ShapeMismatch
from .module import Module, Parameter


def _check_p(p: float) -> float:
    if not 0.0 <= p <= 1.0:
        raise InvalidArgument(f"dropout probability must lie in [0, 1], got {p}")
    return float(p)


def dropout(x, p: float = 0.5, training: bool = True, generator: Optional[torch.Generator] = None):
    """Zeroes each element with probability ``p`` and scales the survivors by ``1 / (1 - p)``."""
    p = _check_p(p)
    if not training or p == 0.0:
        return x
    if p == 1.0:
        return x * 0
    keep = torch.empty_like(x, dtype=torch.float32).uniform_(generator=generator) >= p
    return x * keep.to(x.dtype) / (1.0 - p)


def _channel_dropout(x, p: float, training: bool, nd: int, generator=None):
    """One decision per (sample, channel): the whole feature map is kept or dropped."""
    p = _check_p(p)
    if x.dim() not in (nd + 1, nd + 2):
        raise ShapeMismatch(f"expected a {nd + 1}-D or {nd + 2}-D input, got {list(x.shape)}")
    if not training or p == 0.0:
        return x
    shape = list(x.shape[: x.dim() - nd]) + [1] * nd
    keep = torch.empty(shape, device=x.device, dtype=torch.float32).uniform_(generator=generator) >= p
    return x * keep.to(x.dtype) / max(1e-12, 1.0 - p)


def alpha_dropout(x, p: float = 0.5, training: bool = True, generator=None):
    """Dropout that keeps the mean and variance of SELU activations: dropped units take the saturation value ``-scale * alpha`` and the
    result is rescaled by ``a`` and shifted by ``b``."""
    p = _check_p(p)
    if not training or p == 0.0:
        return x
    if p == 1.0:
        return x * 0
    sat = -1.0507009873554804934193349852946 * 1.6732632423543772848170429916717
    a = 1.0 / math.sqrt((1 - p) * (1 + p * sat * sat))
    b = -a * sat * p
    keep = (torch.empty_like(x, dtype=torch.float32).uniform_(generator=generator) >= p).to(x.dtype)
    return a * (x * keep + sat * (1 - keep)) + b


class _DropoutBase(Module):
    def __init__(self, p: float = 0.5, inplace: bool = False):
        super().__init__()
        self.p, self.inplace = _check_p(p), inplace

    def extra_repr(self):
        return f"p={self.p}"


class Dropout(_DropoutBase):
    def forward(self, x):
        return dropout(x, self.p, self.training)


class Dropout1d(_DropoutBase):
    def forward(self, x):
        return _channel_dropout(x, self.p, self.training, 1)


class Dropout2d(_DropoutBase):
    def forward(self, x):
        return _channel_dropout(x, self.p, self.training, 2)


class Dropout3d(_DropoutBase):
    def forward(self, x):
        return _channel_dropout(x, self.p, self.training, 3)


class AlphaDropout(_DropoutBase):
    def forward(self, x):
        return alpha_dropout(x, self.p, self.training)


class Identity(Module):
    def __init__(self, *args, **kwargs):
        super().__init__()

    def forward(self, x):
        return x


class Flatten(Module):
    def __init__(self, start_dim: int = 1, end_dim: int = -1):
        super().__init__()
        self.start_dim, self.end_dim = start_dim, end_dim

    def forward(self, x):
        return x.flatten(self.start_dim, self.end_dim)


class Unflatten(Module):
    def __init__(self, dim: int, unflattened_size: Sequence[int]):
        super().__init__()
        self.dim, self.unflattened_size = dim, tuple(unflattened_size)

    def forward(self, x):
        d = self.dim if self.dim >= 0 else x.dim() + self.dim
        known = math.prod(s for s in self.unflattened_size if s != -1)
        if (-1 not in self.unflattened_size and known != x.shape[d]) or (known and x.shape[d] % known):
            raise ShapeMismatch(f"Unflatten: cannot split dimension of size {x.shape[d]} into {list(self.unflattened_size)}")
        return x.reshape(*x.shape[:d], *self.unflattened_size, *x.shape[d + 1:])


class ChannelShuffle(Module):
    """``[N, g * c, ...] -> [N, c * g, ...]``: channels of the ``g`` groups are interleaved."""

    def __init__(self, groups: int):
        super().__init__()
        if groups <= 0:
            raise InvalidArgument("groups must be positive")
        self.groups = groups

    def forward(self, x):
        if x.dim() < 3 or x.shape[1] % self.groups:
            raise ShapeMismatch(f"ChannelShuffle: {x.shape[1] if x.dim() > 1 else '?'} channels are not divisible by {self.groups} groups")
        N, C = x.shape[:2]
        return x.reshape(N, self.groups, C // self.groups, *x.shape[2:]).transpose(1, 2).reshape(x.shape)


def embedding_bag(ids, weight, offsets=None, mode: str = "mean", per_sample_weights=None, padding_idx: Optional[int] = None,
                  include_last_offset: bool = False):
    """Reduces bags of embedding rows. ``ids`` is ``[B, L]`` (one fixed-length bag per row) or 1-D with ``offsets`` marking bag starts."""
    mode = getattr(mode, "value", mode)
    if mode not in ("sum", "mean", "max"):
        raise InvalidArgument(f"unknown mode {mode!r}")
    if per_sample_weights is not None and mode != "sum":
        raise InvalidArgument("per_sample_weights needs mode 'sum'")
    if ids.dim() == 2:
        if offsets is not None:
            raise InvalidArgument("offsets are only used with 1-D ids")
        B, L = ids.shape
        bag = torch.arange(B, device=ids.device).repeat_interleave(L)
        flat = ids.reshape(-1)
        psw = per_sample_weights.reshape(-1) if per_sample_weights is not None else None
    elif ids.dim() == 1:
        if offsets is None:
            raise InvalidArgument("1-D ids need offsets")
        off = offsets.to(ids.device).long()
        if off.numel() and int(off[0]) != 0:
            raise InvalidArgument("offsets must start at 0")
        B = off.numel() - (1 if include_last_offset else 0)
        flat, psw = ids, per_sample_weights
        bag = torch.searchsorted(off[:B].contiguous(), torch.arange(flat.numel(), device=ids.device), right=True) - 1
    else:
        raise ShapeMismatch("ids must be 1-D or 2-D")
    if flat.numel() and (int(flat.min()) < 0 or int(flat.max()) >= weight.shape[0]):
        raise InvalidArgument("embedding_bag: index out of range")
    rows = weight.index_select(0, flat)
    valid = torch.ones_like(flat, dtype=torch.bool) if padding_idx is None else flat != padding_idx
    if psw is not None:
        rows = rows * psw.unsqueeze(-1).to(rows.dtype)
    D = weight.shape[1]
    if mode == "max":
        rows = torch.where(valid.unsqueeze(-1), rows, torch.full_like(rows, float("-inf")))
        out = rows.new_full((B, D), float("-inf")).scatter_reduce(0, bag.unsqueeze(-1).expand(-1, D), rows, "amax", include_self=True)
        return torch.where(torch.isinf(out), torch.zeros_like(out), out)
    rows = rows * valid.unsqueeze(-1).to(rows.dtype)
    out = rows.new_zeros(B, D).index_add(0, bag, rows)
    if mode == "mean":
        cnt = torch.zeros(B, device=ids.device, dtype=rows.dtype).index_add(0, bag, valid.to(rows.dtype))
        out = out / torch.clamp_min(cnt, 1).unsqueeze(-1)
    return out


class EmbeddingBag(Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, mode: str = "mean", padding_idx: Optional[int] = None, include_last_offset: bool = False,
                 _weight: Optional[torch.Tensor] = None, device=None, dtype=None):
        super().__init__()
        mode = getattr(mode, "value", mode)
        if mode not in ("sum", "mean", "max"):
            raise InvalidArgument(f"unknown mode {mode!r}")
        self.num_embeddings, self.embedding_dim, self.mode, self.padding_idx = num_embeddings, embedding_dim, mode, padding_idx
        self.include_last_offset = include_last_offset
        self.weight = Parameter(torch.randn(num_embeddings, embedding_dim, device=device, dtype=dtype) if _weight is None else _weight)
        if padding_idx is not None and _weight is None:
            with torch.no_grad():
                self.weight[padding_idx].zero_()

    def forward(self, ids, offsets=None, per_sample_weights=None):
        return embedding_bag(ids, self.weight, offsets, self.mode, per_sample_weights, self.padding_idx, self.include_last_offset)


class Upsample(Module):
    """Resampling to ``size`` or by ``scale_factor`` with nearest, (bi/tri)linear or bicubic interpolation."""

    def __init__(self, size=None, scale_factor=None, mode: str = "nearest", align_corners: Optional[bool] = None):
        super().__init__()
        if size is None and scale_factor is None:
            raise InvalidArgument("Upsample needs size or scale_factor")
        self.size, self.scale_factor, self.mode, self.align_corners = size, scale_factor, getattr(mode, "value", mode), align_corners

    def forward(self, x):
        from .extras import interpolate
        return interpolate(x, self.size, self.scale_factor, self.mode, self.align_corners)


__all__ = ["dropout", "alpha_dropout", "embedding_bag", "Dropout", "Dropout1d", "Dropout2d", "Dropout3d", "AlphaDropout", "Identity", "Flatten",
           "Unflatten", "ChannelShuffle", "EmbeddingBag", "Upsample"]
_ = Union
