"""Padding layers (ferrotorch-nn/src/padding.rs:1-900): constant, zero, reflection, replication and circular padding in 1, 2 and 3
dimensions. Border modes are index maps evaluated with one ``index_select`` per padded dimension; negative amounts crop."""
from __future__ import annotations

from typing import List, Sequence, Tuple, Union

import torch

from ..errors import InvalidArgument, ShapeMismatch
from .module import Module


def _pad_dim(x: torch.Tensor, dim: int, left: int, right: int, mode: str, value: float) -> torch.Tensor:
    n = x.shape[dim]
    if left < 0:
        x, n, left = x.narrow(dim, -left, n + left), n + left, 0
    if right < 0:
        x, n, right = x.narrow(dim, 0, n + right), n + right, 0
    if left == 0 and right == 0:
        return x
    if mode in ("zeros", "constant"):
        parts: List[torch.Tensor] = []
        for amount, first in ((left, True), (right, False)):
            if first is False:
                parts.append(x)
            if amount:
                shp = list(x.shape)
                shp[dim] = amount
                parts.append(x.new_full(shp, value))
        return torch.cat(parts, dim)
    idx = torch.arange(-left, n + right, device=x.device)
    if mode == "reflect":
        if left >= n or right >= n:
            raise InvalidArgument(f"reflection padding ({left}, {right}) must be smaller than the padded dimension ({n})")
        idx = idx.abs()
        idx = torch.where(idx >= n, 2 * (n - 1) - idx, idx)
    elif mode == "replicate":
        if n == 0:
            raise InvalidArgument("replication padding of an empty dimension")
        idx = idx.clamp(0, n - 1)
    elif mode == "circular":
        if left > n or right > n:
            raise InvalidArgument(f"circular padding ({left}, {right}) must not exceed the padded dimension ({n})")
        idx = idx % n
    else:
        raise InvalidArgument(f"unknown padding mode {mode!r}")
    return x.index_select(dim, idx)


def pad_nd(x: torch.Tensor, pads: Sequence[Tuple[int, int]], mode: str = "zeros", value: float = 0.0) -> torch.Tensor:
    """Pads the trailing ``len(pads)`` dimensions; ``pads[i]`` is ``(before, after)`` of the i-th of those dimensions."""
    n = len(pads)
    if x.dim() < n:
        raise ShapeMismatch(f"cannot pad {n} dimensions of a {x.dim()}-D tensor")
    for i, (lo, hi) in enumerate(pads):
        x = _pad_dim(x, x.dim() - n + i, int(lo), int(hi), mode, value)
    return x


def pad(x: torch.Tensor, padding: Sequence[int], mode: str = "constant", value: float = 0.0) -> torch.Tensor:
    """Flat form ``(last_lo, last_hi, second_last_lo, second_last_hi, ...)``: the amounts start at the last dimension."""
    if hasattr(mode, "value"):
        mode = mode.value
    padding = [int(p) for p in padding]
    if len(padding) % 2:
        raise InvalidArgument("padding needs an even number of values")
    pairs = [(padding[i], padding[i + 1]) for i in range(0, len(padding), 2)][::-1]
    return pad_nd(x, pairs, mode, value)


def _amounts(padding: Union[int, Sequence[int]], nd: int) -> Tuple[int, ...]:
    if isinstance(padding, int):
        return (padding,) * (2 * nd)
    padding = tuple(int(p) for p in padding)
    if len(padding) != 2 * nd:
        raise InvalidArgument(f"expected {2 * nd} padding amounts, got {len(padding)}")
    return padding


class _PadNd(Module):
    _nd = 1
    _mode = "constant"

    def __init__(self, padding: Union[int, Sequence[int]], value: float = 0.0):
        super().__init__()
        self.padding = _amounts(padding, self._nd)
        self.value = value

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() not in (self._nd + 1, self._nd + 2):
            raise ShapeMismatch(f"{type(self).__name__} expects a {self._nd + 1}-D or {self._nd + 2}-D input, got {list(x.shape)}")
        return pad(x, self.padding, self._mode, self.value)

    def extra_repr(self) -> str:
        return f"{self.padding}" + (f", value={self.value}" if self._mode == "constant" and self.value else "")


def _mk(name: str, nd: int, mode: str, takes_value: bool):
    ns = {"_nd": nd, "_mode": mode, "__module__": __name__,
          "__doc__": f"{mode.capitalize()} padding of the last {nd} dimension(s); amounts run (left, right[, top, bottom[, front, back]])."}
    if not takes_value:
        def __init__(self, padding):
            _PadNd.__init__(self, padding, 0.0)
        ns["__init__"] = __init__
    return type(name, (_PadNd,), ns)


ConstantPad1d, ConstantPad2d, ConstantPad3d = (_mk(f"ConstantPad{n}d", n, "constant", True) for n in (1, 2, 3))
ZeroPad1d, ZeroPad2d, ZeroPad3d = (_mk(f"ZeroPad{n}d", n, "constant", False) for n in (1, 2, 3))
ReflectionPad1d, ReflectionPad2d, ReflectionPad3d = (_mk(f"ReflectionPad{n}d", n, "reflect", False) for n in (1, 2, 3))
ReplicationPad1d, ReplicationPad2d, ReplicationPad3d = (_mk(f"ReplicationPad{n}d", n, "replicate", False) for n in (1, 2, 3))
CircularPad1d, CircularPad2d, CircularPad3d = (_mk(f"CircularPad{n}d", n, "circular", False) for n in (1, 2, 3))

__all__ = ["pad", "pad_nd"] + [f"{k}Pad{n}d" for k in ("Constant", "Zero", "Reflection", "Replication", "Circular") for n in (1, 2, 3)]
