"""Support constraints of distributions: ``check(value)`` (scalar -> bool, tensor -> bool tensor), ``is_discrete``, ``event_dim``, ``name``.

Rules follow ferrotorch-distributions/src/constraints.rs:32-360: NaN satisfies nothing; ``Real`` accepts infinities; ``Simplex`` checks
per-element non-negativity (``event_dim`` 1) and :meth:`Simplex.check_event` adds the sum-to-one test over the last dimension. The lower-case
constructors mirror the module-level constants of ``torch.distributions.constraints``, whose dependent-property helpers are re-exported for the
distributions built on them.
"""
from __future__ import annotations

import math

import torch
from torch.distributions.constraints import *  # noqa: F401,F403  (dependent, independent, integer_interval, lower_cholesky, positive_definite ...)
from torch.distributions import constraints as _tc

from ..errors import InvalidArgument


class Constraint:
    def _ok(self, v: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def check(self, value):
        if torch.is_tensor(value):
            return self._ok(value) & ~torch.isnan(value) if value.is_floating_point() else self._ok(value)
        v = float(value)
        return (not math.isnan(v)) and bool(self._ok(torch.tensor(v, dtype=torch.float64)))

    def is_discrete(self) -> bool:
        return False

    def event_dim(self) -> int:
        return 0

    def name(self) -> str:
        return type(self).__name__

    def __repr__(self):
        return self.name()


class Real(Constraint):
    def _ok(self, v): return torch.ones_like(v, dtype=torch.bool)                              # noqa: E704


class Positive(Constraint):
    def _ok(self, v): return v > 0                                                             # noqa: E704


class NonNegative(Constraint):
    def _ok(self, v): return v >= 0                                                            # noqa: E704


class UnitInterval(Constraint):
    def _ok(self, v): return (v >= 0) & (v <= 1)                                               # noqa: E704


class BooleanConstraint(Constraint):
    def _ok(self, v): return (v == 0) | (v == 1)                                               # noqa: E704
    def is_discrete(self) -> bool: return True                                                 # noqa: E704
    def name(self) -> str: return "Boolean"                                                    # noqa: E704


class _Bounded(Constraint):
    def __init__(self, lower_bound=None, upper_bound=None):
        if lower_bound is not None and upper_bound is not None and not lower_bound <= upper_bound:
            raise InvalidArgument(f"{type(self).__name__}: lower bound {lower_bound} above upper bound {upper_bound}")
        self.lower_bound, self.upper_bound = lower_bound, upper_bound

    def __repr__(self):
        args = ", ".join(f"{k}={v}" for k, v in (("lower_bound", self.lower_bound), ("upper_bound", self.upper_bound)) if v is not None)
        return f"{self.name()}({args})"


class GreaterThan(_Bounded):
    def __init__(self, lower_bound): super().__init__(lower_bound, None)                       # noqa: E704
    def _ok(self, v): return v > self.lower_bound                                              # noqa: E704


class GreaterThanEq(_Bounded):
    def __init__(self, lower_bound): super().__init__(lower_bound, None)                       # noqa: E704
    def _ok(self, v): return v >= self.lower_bound                                             # noqa: E704


class LessThan(_Bounded):
    def __init__(self, upper_bound): super().__init__(None, upper_bound)                       # noqa: E704
    def _ok(self, v): return v < self.upper_bound                                              # noqa: E704


class OpenInterval(_Bounded):
    def _ok(self, v): return (v > self.lower_bound) & (v < self.upper_bound)                   # noqa: E704


class ClosedInterval(_Bounded):
    def _ok(self, v): return (v >= self.lower_bound) & (v <= self.upper_bound)                 # noqa: E704


class HalfOpenInterval(_Bounded):
    def _ok(self, v): return (v >= self.lower_bound) & (v < self.upper_bound)                  # noqa: E704


class Simplex(Constraint):
    def _ok(self, v): return v >= 0                                                            # noqa: E704
    def event_dim(self) -> int: return 1                                                       # noqa: E704

    def check_event(self, value: torch.Tensor, atol: float = 1e-6) -> torch.Tensor:
        """Whole-event test: every entry non-negative and the last dimension summing to one."""
        return (value >= 0).all(-1) & ((value.sum(-1) - 1.0).abs() <= atol)


def real() -> Real: return Real()                                                              # noqa: E704
def positive() -> Positive: return Positive()                                                  # noqa: E704
def nonnegative() -> NonNegative: return NonNegative()                                         # noqa: E704
def unit_interval() -> UnitInterval: return UnitInterval()                                     # noqa: E704
def boolean() -> BooleanConstraint: return BooleanConstraint()                                 # noqa: E704
def greater_than(lower_bound) -> GreaterThan: return GreaterThan(lower_bound)                  # noqa: E704
def greater_than_eq(lower_bound) -> GreaterThanEq: return GreaterThanEq(lower_bound)           # noqa: E704
def less_than(upper_bound) -> LessThan: return LessThan(upper_bound)                           # noqa: E704
def open_interval(lower_bound, upper_bound) -> OpenInterval: return OpenInterval(lower_bound, upper_bound)              # noqa: E704
def closed_interval(lower_bound, upper_bound) -> ClosedInterval: return ClosedInterval(lower_bound, upper_bound)        # noqa: E704
def half_open_interval(lower_bound, upper_bound) -> HalfOpenInterval: return HalfOpenInterval(lower_bound, upper_bound)  # noqa: E704
def simplex() -> Simplex: return Simplex()                                                     # noqa: E704


torch_constraints = _tc                                       # the library's objects, for code that needs their dependent-property machinery
