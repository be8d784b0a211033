"""The einops pattern language (``rearrange`` / ``repeat`` / ``reduce``) written out: both sides of the arrow are parsed into groups of named
axes, the input is reshaped to its elementary axes, reduced / permuted / expanded, and reshaped to the groups of the output.

Reference parity: ferrotorch-core/src/einops.rs:458 (rearrange), :482 (rearrange_with), :589 (repeat), :665 (reduce): parenthesised
groups, ``1`` axes, an ellipsis, axis lengths by keyword, reductions sum / mean / max / min / prod.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..errors import InvalidArgument


def _side(text: str) -> List[List[str]]:
    """``"b (h w) 1 ..."`` -> [["b"], ["h", "w"], [], ["..."]]; an empty group is a dimension of length one."""
    groups: List[List[str]] = []
    cur = None
    for tok in text.replace("(", " ( ").replace(")", " ) ").split():
        if tok == "(":
            if cur is not None:
                raise InvalidArgument("einops: nested parentheses")
            cur = []
        elif tok == ")":
            if cur is None:
                raise InvalidArgument("einops: unbalanced parentheses")
            groups.append(cur)
            cur = None
        else:
            if tok != "..." and tok != "1" and not (tok.isidentifier() or tok.isdigit()):
                raise InvalidArgument(f"einops: invalid axis name '{tok}'")
            item = [] if tok == "1" else [tok]
            if cur is None:
                groups.append(item)
            else:
                cur += item
    if cur is not None:
        raise InvalidArgument("einops: unbalanced parentheses")
    return groups


def _plan(t: torch.Tensor, pattern: str, axes: Dict[str, int]):
    if "->" not in pattern:
        raise InvalidArgument("einops: pattern needs '->'")
    left, right = (_side(s) for s in pattern.split("->"))
    n_ell = sum(g == ["..."] for g in left)
    if n_ell > 1 or any("..." in g and g != ["..."] for g in left):
        raise InvalidArgument("einops: the ellipsis stands alone and at most once on the left")
    if len(left) - n_ell > t.dim() or (not n_ell and len(left) != t.dim()):
        raise InvalidArgument(f"einops: pattern has {len(left)} input dimensions, the tensor {t.dim()}")
    ell = [f"…{k}" for k in range(t.dim() - (len(left) - n_ell))] if n_ell else []

    def expand(groups):
        out = []
        for g in groups:
            if g == ["..."]:
                out += [[e] for e in ell]
            else:
                out.append([a for x in g for a in (ell if x == "..." else [x])])
        return out
    left, right = expand(left), expand(right)
    sizes: Dict[str, int] = {k: int(v) for k, v in axes.items()}
    flat_left = [a for g in left for a in g]
    if len(set(flat_left)) != len(flat_left):
        raise InvalidArgument("einops: an axis appears twice on the left")
    for g, n in zip(left, t.shape):
        for a in g:
            if a.isdigit():
                sizes[a] = int(a)
        unknown = [a for a in g if a not in sizes]
        known = 1
        for a in g:
            if a in sizes:
                known *= sizes[a]
        if len(unknown) > 1:
            raise InvalidArgument(f"einops: cannot infer the lengths of {unknown}")
        if unknown:
            if known == 0 or n % known:
                raise InvalidArgument(f"einops: dimension {n} is not divisible by {known}")
            sizes[unknown[0]] = n // known
        elif known != n:
            raise InvalidArgument(f"einops: group {g} has length {known}, the dimension {n}")
    return left, right, flat_left, sizes


def _apply(t: torch.Tensor, pattern: str, axes: Dict[str, int], mode: str, reduction: str = "") -> torch.Tensor:
    left, right, flat_left, sizes = _plan(t, pattern, axes)
    flat_right = [a for g in right for a in g]
    if len(set(flat_right)) != len(flat_right):
        raise InvalidArgument("einops: an axis appears twice on the right")
    new = [a for a in flat_right if a not in flat_left]
    gone = [a for a in flat_left if a not in flat_right]
    if mode == "rearrange" and (new or gone):
        raise InvalidArgument(f"einops.rearrange: axes {new + gone} appear on one side only")
    if mode == "repeat" and gone:
        raise InvalidArgument(f"einops.repeat: axes {gone} vanish")
    if mode == "reduce" and new:
        raise InvalidArgument(f"einops.reduce: axes {new} appear on the right only")
    for a in new:
        if a.isdigit():
            sizes[a] = int(a)
        if a not in sizes:
            raise InvalidArgument(f"einops: length of the new axis '{a}' is not given")
    x = t.reshape([sizes[a] for a in flat_left])
    if gone:
        dims = [flat_left.index(a) for a in gone]
        if reduction == "sum":
            x = x.sum(dim=dims)
        elif reduction == "mean":
            x = x.mean(dim=dims)
        elif reduction == "prod":
            for d in sorted(dims, reverse=True):
                x = x.prod(dim=d)
        elif reduction in ("max", "min"):
            x = x.amax(dim=dims) if reduction == "max" else x.amin(dim=dims)
        else:
            raise InvalidArgument(f"einops.reduce: unknown reduction '{reduction}'")
    kept = [a for a in flat_left if a not in gone]
    x = x.permute([kept.index(a) for a in flat_right if a in kept])
    if new:
        order = [a for a in flat_right if a in kept]
        shape, index = [], []
        for a in flat_right:
            shape.append(sizes[a])
            index.append(slice(None) if a in kept else None)
        x = x[tuple(index)].expand(shape)
    return x.reshape([_prod(sizes[a] for a in g) for g in right])


def _prod(it) -> int:
    n = 1
    for v in it:
        n *= v
    return n


def rearrange(t: torch.Tensor, pattern: str, **axes) -> torch.Tensor:
    return _apply(t, pattern, axes, "rearrange")


def repeat(t: torch.Tensor, pattern: str, **axes) -> torch.Tensor:
    return _apply(t, pattern, axes, "repeat")


def reduce(t: torch.Tensor, pattern: str, reduction: str = "mean", **axes) -> torch.Tensor:
    return _apply(t, pattern, axes, "reduce", reduction)
