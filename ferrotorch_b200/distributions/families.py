"""Distribution families implemented here: parameters, sampling (reparameterised where a pathwise gradient exists), ``log_prob``, ``entropy``,
moments, ``cdf`` / ``icdf`` where closed forms exist, and a pairwise KL registry.

The classes derive from ``torch.distributions.Distribution`` only for its interface (batch / event shapes, ``expand`` bookkeeping,
argument validation hooks), so they compose with transforms and ``Independent``; all the arithmetic below is this module's. Sampling draws
from the substrate's generators (``torch.manual_seed``). Gamma-family reparameterised samples use the substrate's implicit-gradient sampler
(``torch._standard_gamma``), as the reference's use of a rejection sampler with reparameterisation does.

Reference parity: ferrotorch-distributions/src/lib.rs:138 (``Distribution`` trait) and one file per family (normal.rs, uniform.rs, bernoulli.rs,
categorical.rs, exponential.rs, laplace.rs, gumbel.rs, cauchy.rs, half_normal.rs, gamma.rs, beta.rs, dirichlet.rs, student_t.rs, poisson.rs,
weibull.rs, pareto.rs, kumaraswamy.rs, log_normal.rs, multivariate_normal.rs, one_hot_categorical.rs, independent.rs), kl.rs:66.
"""
from __future__ import annotations

import math
from numbers import Number
from typing import Callable, Dict, Tuple, Type

import torch
from torch.distributions import Distribution as _Base
from torch.distributions import constraints as _c
from torch.distributions.utils import broadcast_all

_EULER = 0.5772156649015329


def _shape(sample_shape, d):
    return torch.Size(sample_shape) + d.batch_shape + d.event_shape


class Distribution(_Base):
    """Interface base of the families below (``sample`` / ``rsample`` / ``log_prob`` / ``entropy`` / ``mean`` / ``variance`` / ``stddev``)."""

    def sample(self, sample_shape=torch.Size()):
        with torch.no_grad():
            return self.rsample(sample_shape)

    @property
    def stddev(self):
        return self.variance.sqrt()

    def perplexity(self):
        return self.entropy().exp()


class Normal(Distribution):
    arg_constraints = {"loc": _c.real, "scale": _c.positive}
    support = _c.real
    has_rsample = True

    def __init__(self, loc, scale, validate_args=None):
        self.loc, self.scale = broadcast_all(loc, scale)
        super().__init__(self.loc.shape, validate_args=validate_args)

    mean = property(lambda s: s.loc)
    mode = property(lambda s: s.loc)
    variance = property(lambda s: s.scale.pow(2))

    def rsample(self, sample_shape=torch.Size()):
        return self.loc + self.scale * torch.randn(_shape(sample_shape, self), dtype=self.loc.dtype, device=self.loc.device)

    def log_prob(self, value):
        z = (value - self.loc) / self.scale
        return -0.5 * z * z - self.scale.log() - 0.5 * math.log(2 * math.pi)

    def cdf(self, value):
        return 0.5 * (1 + torch.erf((value - self.loc) / (self.scale * math.sqrt(2))))

    def icdf(self, p):
        return self.loc + self.scale * torch.erfinv(2 * p - 1) * math.sqrt(2)

    def entropy(self):
        return 0.5 + 0.5 * math.log(2 * math.pi) + self.scale.log()


class LogNormal(Distribution):
    arg_constraints = {"loc": _c.real, "scale": _c.positive}
    support = _c.positive
    has_rsample = True

    def __init__(self, loc, scale, validate_args=None):
        self.base = Normal(loc, scale)
        self.loc, self.scale = self.base.loc, self.base.scale
        super().__init__(self.loc.shape, validate_args=validate_args)

    mean = property(lambda s: (s.loc + s.scale.pow(2) / 2).exp())
    mode = property(lambda s: (s.loc - s.scale.pow(2)).exp())
    variance = property(lambda s: (s.scale.pow(2).exp() - 1) * (2 * s.loc + s.scale.pow(2)).exp())

    def rsample(self, sample_shape=torch.Size()):
        return self.base.rsample(sample_shape).exp()

    def log_prob(self, value):
        return self.base.log_prob(value.log()) - value.log()

    def cdf(self, value):
        return self.base.cdf(value.log())

    def icdf(self, p):
        return self.base.icdf(p).exp()

    def entropy(self):
        return self.base.entropy() + self.loc


class Uniform(Distribution):
    arg_constraints = {"low": _c.dependent(is_discrete=False, event_dim=0), "high": _c.dependent(is_discrete=False, event_dim=0)}
    has_rsample = True

    def __init__(self, low, high, validate_args=None):
        self.low, self.high = broadcast_all(low, high)
        super().__init__(self.low.shape, validate_args=validate_args)

    @_c.dependent_property(is_discrete=False, event_dim=0)
    def support(self):
        return _c.interval(self.low, self.high)

    mean = property(lambda s: (s.low + s.high) / 2)
    variance = property(lambda s: (s.high - s.low).pow(2) / 12)

    def rsample(self, sample_shape=torch.Size()):
        u = torch.rand(_shape(sample_shape, self), dtype=self.low.dtype, device=self.low.device)
        return self.low + u * (self.high - self.low)

    def log_prob(self, value):
        inside = (value >= self.low) & (value < self.high)
        return torch.where(inside, -(self.high - self.low).log(), torch.full_like(self.low + value, -math.inf))

    def cdf(self, value):
        return ((value - self.low) / (self.high - self.low)).clamp(0, 1)

    def icdf(self, p):
        return self.low + p * (self.high - self.low)

    def entropy(self):
        return (self.high - self.low).log()


def _probs_logits(probs, logits, binary):
    if (probs is None) == (logits is None):
        raise ValueError("Either `probs` or `logits` must be specified, but not both.")
    if probs is not None:
        probs = torch.as_tensor(probs, dtype=torch.get_default_dtype()) if isinstance(probs, Number) else probs
        if binary:
            eps = torch.finfo(probs.dtype).eps
            pc = probs.clamp(eps, 1 - eps)
            return probs, pc.log() - (-pc).log1p()
        probs = probs / probs.sum(-1, keepdim=True)
        return probs, probs.clamp_min(torch.finfo(probs.dtype).tiny).log()
    logits = torch.as_tensor(logits, dtype=torch.get_default_dtype()) if isinstance(logits, Number) else logits
    if binary:
        return torch.sigmoid(logits), logits
    logits = logits - logits.logsumexp(-1, keepdim=True)
    return logits.exp(), logits


class Bernoulli(Distribution):
    arg_constraints = {"probs": _c.unit_interval, "logits": _c.real}
    support = _c.boolean
    has_enumerate_support = True

    def __init__(self, probs=None, logits=None, validate_args=None):
        self.probs, self.logits = _probs_logits(probs, logits, True)
        super().__init__(self.probs.shape, validate_args=validate_args)

    mean = property(lambda s: s.probs)
    variance = property(lambda s: s.probs * (1 - s.probs))

    def sample(self, sample_shape=torch.Size()):
        with torch.no_grad():
            return torch.bernoulli(self.probs.expand(_shape(sample_shape, self)))

    def log_prob(self, value):
        return -torch.nn.functional.binary_cross_entropy_with_logits(self.logits.expand_as(value + self.logits), value + 0 * self.logits, reduction="none")

    def entropy(self):
        return torch.nn.functional.binary_cross_entropy_with_logits(self.logits, self.probs, reduction="none")

    def enumerate_support(self, expand=True):
        v = torch.arange(2, dtype=self.probs.dtype, device=self.probs.device).view((-1,) + (1,) * len(self.batch_shape))
        return v.expand((-1,) + self.batch_shape) if expand else v


class Categorical(Distribution):
    arg_constraints = {"probs": _c.simplex, "logits": _c.real_vector}
    has_enumerate_support = True

    def __init__(self, probs=None, logits=None, validate_args=None):
        self.probs, self.logits = _probs_logits(probs, logits, False)
        self._n = self.probs.shape[-1]
        super().__init__(self.probs.shape[:-1], validate_args=validate_args)

    @_c.dependent_property(is_discrete=True, event_dim=0)
    def support(self):
        return _c.integer_interval(0, self._n - 1)

    @property
    def mean(self):
        return torch.full(self.batch_shape, math.nan, dtype=self.probs.dtype, device=self.probs.device)

    variance = mean
    mode = property(lambda s: s.probs.argmax(-1))

    def sample(self, sample_shape=torch.Size()):
        with torch.no_grad():
            n = torch.Size(sample_shape).numel()
            p2 = self.probs.reshape(-1, self._n)
            return torch.multinomial(p2, n, True).T.reshape(torch.Size(sample_shape) + self.batch_shape)

    def log_prob(self, value):
        value = value.long().unsqueeze(-1)
        value, lp = torch.broadcast_tensors(value, self.logits)
        return lp.gather(-1, value[..., :1]).squeeze(-1)

    def entropy(self):
        lg = self.logits.clamp_min(torch.finfo(self.logits.dtype).min)
        return -(lg * self.probs).sum(-1)

    def enumerate_support(self, expand=True):
        v = torch.arange(self._n, device=self.probs.device).view((-1,) + (1,) * len(self.batch_shape))
        return v.expand((-1,) + self.batch_shape) if expand else v


class OneHotCategorical(Distribution):
    arg_constraints = {"probs": _c.simplex, "logits": _c.real_vector}
    support = _c.one_hot

    def __init__(self, probs=None, logits=None, validate_args=None):
        self._cat = Categorical(probs, logits)
        self.probs, self.logits = self._cat.probs, self._cat.logits
        super().__init__(self._cat.batch_shape, self.probs.shape[-1:], validate_args=validate_args)

    mean = property(lambda s: s.probs)
    variance = property(lambda s: s.probs * (1 - s.probs))

    def sample(self, sample_shape=torch.Size()):
        return torch.nn.functional.one_hot(self._cat.sample(sample_shape), self.probs.shape[-1]).to(self.probs.dtype)

    def log_prob(self, value):
        return self._cat.log_prob(value.argmax(-1))

    def entropy(self):
        return self._cat.entropy()


class Exponential(Distribution):
    arg_constraints = {"rate": _c.positive}
    support = _c.nonnegative
    has_rsample = True

    def __init__(self, rate, validate_args=None):
        (self.rate,) = broadcast_all(rate)
        super().__init__(self.rate.shape, validate_args=validate_args)

    mean = property(lambda s: s.rate.reciprocal())
    variance = property(lambda s: s.rate.pow(-2))

    def rsample(self, sample_shape=torch.Size()):
        u = torch.rand(_shape(sample_shape, self), dtype=self.rate.dtype, device=self.rate.device)
        return -torch.log1p(-u) / self.rate

    def log_prob(self, value):
        return self.rate.log() - self.rate * value

    def cdf(self, value):
        return 1 - torch.exp(-self.rate * value)

    def icdf(self, p):
        return -torch.log1p(-p) / self.rate

    def entropy(self):
        return 1.0 - self.rate.log()


class Laplace(Distribution):
    arg_constraints = {"loc": _c.real, "scale": _c.positive}
    support = _c.real
    has_rsample = True

    def __init__(self, loc, scale, validate_args=None):
        self.loc, self.scale = broadcast_all(loc, scale)
        super().__init__(self.loc.shape, validate_args=validate_args)

    mean = property(lambda s: s.loc)
    variance = property(lambda s: 2 * s.scale.pow(2))

    def rsample(self, sample_shape=torch.Size()):
        eps = torch.finfo(self.loc.dtype).eps
        u = torch.rand(_shape(sample_shape, self), dtype=self.loc.dtype, device=self.loc.device) * (2 - 2 * eps) - (1 - eps)
        return self.loc - self.scale * u.sign() * torch.log1p(-u.abs())

    def log_prob(self, value):
        return -torch.log(2 * self.scale) - (value - self.loc).abs() / self.scale

    def cdf(self, value):
        z = (value - self.loc) / self.scale
        return 0.5 - 0.5 * z.sign() * torch.expm1(-z.abs())

    def icdf(self, p):
        t = p - 0.5
        return self.loc - self.scale * t.sign() * torch.log1p(-2 * t.abs())

    def entropy(self):
        return 1 + torch.log(2 * self.scale)


class Gumbel(Distribution):
    arg_constraints = {"loc": _c.real, "scale": _c.positive}
    support = _c.real
    has_rsample = True

    def __init__(self, loc, scale, validate_args=None):
        self.loc, self.scale = broadcast_all(loc, scale)
        super().__init__(self.loc.shape, validate_args=validate_args)

    mean = property(lambda s: s.loc + s.scale * _EULER)
    variance = property(lambda s: (math.pi ** 2 / 6) * s.scale.pow(2))

    def rsample(self, sample_shape=torch.Size()):
        fi = torch.finfo(self.loc.dtype)
        u = torch.rand(_shape(sample_shape, self), dtype=self.loc.dtype, device=self.loc.device).clamp(fi.tiny, 1 - fi.eps)
        return self.loc - self.scale * torch.log(-torch.log(u))

    def log_prob(self, value):
        z = (value - self.loc) / self.scale
        return -(z + torch.exp(-z)) - self.scale.log()

    def cdf(self, value):
        return torch.exp(-torch.exp(-(value - self.loc) / self.scale))

    def icdf(self, p):
        return self.loc - self.scale * torch.log(-torch.log(p))

    def entropy(self):
        return self.scale.log() + (1 + _EULER)


class Cauchy(Distribution):
    arg_constraints = {"loc": _c.real, "scale": _c.positive}
    support = _c.real
    has_rsample = True

    def __init__(self, loc, scale, validate_args=None):
        self.loc, self.scale = broadcast_all(loc, scale)
        super().__init__(self.loc.shape, validate_args=validate_args)

    @property
    def mean(self):
        return torch.full_like(self.loc, math.nan)

    @property
    def variance(self):
        return torch.full_like(self.loc, math.inf)

    def rsample(self, sample_shape=torch.Size()):
        u = torch.rand(_shape(sample_shape, self), dtype=self.loc.dtype, device=self.loc.device)
        return self.loc + self.scale * torch.tan(math.pi * (u - 0.5))

    def log_prob(self, value):
        return -math.log(math.pi) - self.scale.log() - torch.log1p(((value - self.loc) / self.scale).pow(2))

    def cdf(self, value):
        return torch.atan((value - self.loc) / self.scale) / math.pi + 0.5

    def icdf(self, p):
        return self.loc + self.scale * torch.tan(math.pi * (p - 0.5))

    def entropy(self):
        return math.log(4 * math.pi) + self.scale.log()


class HalfNormal(Distribution):
    arg_constraints = {"scale": _c.positive}
    support = _c.nonnegative
    has_rsample = True

    def __init__(self, scale, validate_args=None):
        (self.scale,) = broadcast_all(scale)
        super().__init__(self.scale.shape, validate_args=validate_args)

    mean = property(lambda s: s.scale * math.sqrt(2 / math.pi))
    variance = property(lambda s: s.scale.pow(2) * (1 - 2 / math.pi))

    def rsample(self, sample_shape=torch.Size()):
        return (self.scale * torch.randn(_shape(sample_shape, self), dtype=self.scale.dtype, device=self.scale.device)).abs()

    def log_prob(self, value):
        lp = Normal(torch.zeros_like(self.scale), self.scale).log_prob(value) + math.log(2)
        return torch.where(value >= 0, lp, torch.full_like(lp, -math.inf))

    def cdf(self, value):
        return torch.erf(value / (self.scale * math.sqrt(2)))

    def icdf(self, p):
        return self.scale * math.sqrt(2) * torch.erfinv(p)

    def entropy(self):
        return 0.5 * math.log(math.pi / 2) + 0.5 + self.scale.log()


class Gamma(Distribution):
    arg_constraints = {"concentration": _c.positive, "rate": _c.positive}
    support = _c.nonnegative
    has_rsample = True

    def __init__(self, concentration, rate, validate_args=None):
        self.concentration, self.rate = broadcast_all(concentration, rate)
        super().__init__(self.concentration.shape, validate_args=validate_args)

    mean = property(lambda s: s.concentration / s.rate)
    variance = property(lambda s: s.concentration / s.rate.pow(2))

    def rsample(self, sample_shape=torch.Size()):
        shape = _shape(sample_shape, self)
        v = torch._standard_gamma(self.concentration.expand(shape)) / self.rate.expand(shape)
        return v.detach().clamp_(min=torch.finfo(v.dtype).tiny) + (v - v.detach())

    def log_prob(self, value):
        return torch.xlogy(self.concentration, self.rate) + torch.xlogy(self.concentration - 1, value) - self.rate * value - torch.lgamma(self.concentration)

    def cdf(self, value):
        return torch.special.gammainc(self.concentration, self.rate * value)

    def entropy(self):
        a = self.concentration
        return a - self.rate.log() + torch.lgamma(a) + (1 - a) * torch.digamma(a)


class Beta(Distribution):
    arg_constraints = {"concentration1": _c.positive, "concentration0": _c.positive}
    support = _c.unit_interval
    has_rsample = True

    def __init__(self, concentration1, concentration0, validate_args=None):
        self.concentration1, self.concentration0 = broadcast_all(concentration1, concentration0)
        super().__init__(self.concentration1.shape, validate_args=validate_args)

    mean = property(lambda s: s.concentration1 / (s.concentration1 + s.concentration0))

    @property
    def variance(self):
        a, b = self.concentration1, self.concentration0
        return a * b / ((a + b).pow(2) * (a + b + 1))

    def rsample(self, sample_shape=torch.Size()):
        conc = torch.stack([self.concentration1, self.concentration0], -1)
        return Dirichlet(conc).rsample(sample_shape)[..., 0]

    def log_prob(self, value):
        a, b = self.concentration1, self.concentration0
        return torch.xlogy(a - 1, value) + torch.special.xlog1py(b - 1, -value) + torch.lgamma(a + b) - torch.lgamma(a) - torch.lgamma(b)

    def entropy(self):
        a, b = self.concentration1, self.concentration0
        return (torch.lgamma(a) + torch.lgamma(b) - torch.lgamma(a + b) - (a - 1) * torch.digamma(a) - (b - 1) * torch.digamma(b)
                + (a + b - 2) * torch.digamma(a + b))


class Dirichlet(Distribution):
    arg_constraints = {"concentration": _c.independent(_c.positive, 1)}
    support = _c.simplex
    has_rsample = True

    def __init__(self, concentration, validate_args=None):
        if concentration.dim() < 1:
            raise ValueError("`concentration` parameter must be at least one-dimensional.")
        self.concentration = concentration
        super().__init__(concentration.shape[:-1], concentration.shape[-1:], validate_args=validate_args)

    mean = property(lambda s: s.concentration / s.concentration.sum(-1, True))

    @property
    def variance(self):
        a0 = self.concentration.sum(-1, True)
        return self.concentration * (a0 - self.concentration) / (a0.pow(2) * (a0 + 1))

    def rsample(self, sample_shape=torch.Size()):
        shape = _shape(sample_shape, self)
        from torch.distributions.dirichlet import _Dirichlet          # the substrate's sampler with the implicit pathwise gradient
        return _Dirichlet.apply(self.concentration.expand(shape))

    def log_prob(self, value):
        a = self.concentration
        return torch.xlogy(a - 1.0, value).sum(-1) + torch.lgamma(a.sum(-1)) - torch.lgamma(a).sum(-1)

    def entropy(self):
        a = self.concentration
        k, a0 = a.shape[-1], a.sum(-1)
        return torch.lgamma(a).sum(-1) - torch.lgamma(a0) - (k - a0) * torch.digamma(a0) - ((a - 1.0) * torch.digamma(a)).sum(-1)


class StudentT(Distribution):
    arg_constraints = {"df": _c.positive, "loc": _c.real, "scale": _c.positive}
    support = _c.real
    has_rsample = True

    def __init__(self, df, loc=0.0, scale=1.0, validate_args=None):
        self.df, self.loc, self.scale = broadcast_all(df, loc, scale)
        super().__init__(self.df.shape, validate_args=validate_args)

    @property
    def mean(self):
        return torch.where(self.df > 1, self.loc, torch.full_like(self.loc, math.nan))

    @property
    def variance(self):
        v = torch.where(self.df > 2, self.scale.pow(2) * self.df / (self.df - 2), torch.full_like(self.df, math.inf))
        return torch.where(self.df > 1, v, torch.full_like(self.df, math.nan))

    def rsample(self, sample_shape=torch.Size()):
        shape = _shape(sample_shape, self)
        x = torch.randn(shape, dtype=self.df.dtype, device=self.df.device)
        z = Gamma(self.df / 2, torch.full_like(self.df, 0.5)).rsample(sample_shape)          # chi-square(df)
        return self.loc + self.scale * x * torch.rsqrt(z / self.df)

    def log_prob(self, value):
        y = (value - self.loc) / self.scale
        z = self.scale.log() + 0.5 * self.df.log() + 0.5 * math.log(math.pi) + torch.lgamma(0.5 * self.df) - torch.lgamma(0.5 * (self.df + 1))
        return -0.5 * (self.df + 1) * torch.log1p(y * y / self.df) - z

    def entropy(self):
        lbeta = torch.lgamma(0.5 * self.df) + math.lgamma(0.5) - torch.lgamma(0.5 * (self.df + 1))
        return self.scale.log() + 0.5 * (self.df + 1) * (torch.digamma(0.5 * (self.df + 1)) - torch.digamma(0.5 * self.df)) + 0.5 * self.df.log() + lbeta


class Poisson(Distribution):
    arg_constraints = {"rate": _c.nonnegative}
    support = _c.nonnegative_integer

    def __init__(self, rate, validate_args=None):
        (self.rate,) = broadcast_all(rate)
        super().__init__(self.rate.shape, validate_args=validate_args)

    mean = property(lambda s: s.rate)
    variance = property(lambda s: s.rate)

    def sample(self, sample_shape=torch.Size()):
        with torch.no_grad():
            return torch.poisson(self.rate.expand(_shape(sample_shape, self)))

    def log_prob(self, value):
        return torch.xlogy(value, self.rate) - self.rate - torch.lgamma(value + 1)


class Weibull(Distribution):
    arg_constraints = {"scale": _c.positive, "concentration": _c.positive}
    support = _c.positive
    has_rsample = True

    def __init__(self, scale, concentration, validate_args=None):
        self.scale, self.concentration = broadcast_all(scale, concentration)
        super().__init__(self.scale.shape, validate_args=validate_args)

    mean = property(lambda s: s.scale * torch.exp(torch.lgamma(1 + 1 / s.concentration)))

    @property
    def variance(self):
        k = self.concentration
        return self.scale.pow(2) * (torch.exp(torch.lgamma(1 + 2 / k)) - torch.exp(2 * torch.lgamma(1 + 1 / k)))

    def rsample(self, sample_shape=torch.Size()):
        e = Exponential(torch.ones_like(self.scale)).rsample(sample_shape)
        return self.scale * e.pow(1 / self.concentration)

    def log_prob(self, value):
        k, lam = self.concentration, self.scale
        return k.log() - lam.log() + (k - 1) * (value / lam).log() - (value / lam).pow(k)

    def cdf(self, value):
        return 1 - torch.exp(-(value / self.scale).pow(self.concentration))

    def icdf(self, p):
        return self.scale * (-torch.log1p(-p)).pow(1 / self.concentration)

    def entropy(self):
        k = self.concentration
        return _EULER * (1 - 1 / k) + (self.scale / k).log() + 1


class Pareto(Distribution):
    arg_constraints = {"scale": _c.positive, "alpha": _c.positive}
    has_rsample = True

    def __init__(self, scale, alpha, validate_args=None):
        self.scale, self.alpha = broadcast_all(scale, alpha)
        super().__init__(self.scale.shape, validate_args=validate_args)

    @_c.dependent_property(is_discrete=False, event_dim=0)
    def support(self):
        return _c.greater_than_eq(self.scale)

    @property
    def mean(self):
        a = self.alpha.clamp(min=1)
        return a * self.scale / (a - 1)

    @property
    def variance(self):
        a = self.alpha.clamp(min=2)
        return self.scale.pow(2) * a / ((a - 1).pow(2) * (a - 2))

    def rsample(self, sample_shape=torch.Size()):
        e = Exponential(self.alpha).rsample(sample_shape)
        return self.scale * e.exp()

    def log_prob(self, value):
        lp = self.alpha.log() + self.alpha * self.scale.log() - (self.alpha + 1) * value.log()
        return torch.where(value >= self.scale, lp, torch.full_like(lp, -math.inf))

    def cdf(self, value):
        return 1 - (self.scale / value).pow(self.alpha)

    def icdf(self, p):
        return self.scale * (1 - p).pow(-1 / self.alpha)

    def entropy(self):
        return (self.scale / self.alpha).log() + 1 + self.alpha.reciprocal()


class Kumaraswamy(Distribution):
    arg_constraints = {"concentration1": _c.positive, "concentration0": _c.positive}
    support = _c.unit_interval
    has_rsample = True

    def __init__(self, concentration1, concentration0, validate_args=None):
        self.concentration1, self.concentration0 = broadcast_all(concentration1, concentration0)
        super().__init__(self.concentration1.shape, validate_args=validate_args)

    def _moment(self, n):
        a, b = self.concentration1, self.concentration0
        return b * torch.exp(torch.lgamma(1 + n / a) + torch.lgamma(b) - torch.lgamma(1 + n / a + b))

    mean = property(lambda s: s._moment(1))
    variance = property(lambda s: s._moment(2) - s._moment(1).pow(2))

    def rsample(self, sample_shape=torch.Size()):
        fi = torch.finfo(self.concentration1.dtype)
        u = torch.rand(_shape(sample_shape, self), dtype=self.concentration1.dtype, device=self.concentration1.device).clamp(fi.eps, 1 - fi.eps)
        return (1 - (1 - u).pow(1 / self.concentration0)).pow(1 / self.concentration1)

    def log_prob(self, value):
        a, b = self.concentration1, self.concentration0
        return a.log() + b.log() + (a - 1) * value.log() + (b - 1) * torch.log1p(-value.pow(a))

    def cdf(self, value):
        return 1 - (1 - value.pow(self.concentration1)).pow(self.concentration0)

    def icdf(self, p):
        return (1 - (1 - p).pow(1 / self.concentration0)).pow(1 / self.concentration1)

    def entropy(self):
        a, b = self.concentration1, self.concentration0
        hb = torch.digamma(b + 1) + _EULER
        return (1 - 1 / b) + (1 - 1 / a) * hb - a.log() - b.log()


class MultivariateNormal(Distribution):
    arg_constraints = {"loc": _c.real_vector, "covariance_matrix": _c.positive_definite, "precision_matrix": _c.positive_definite,
                       "scale_tril": _c.lower_cholesky}
    support = _c.real_vector
    has_rsample = True

    def __init__(self, loc, covariance_matrix=None, precision_matrix=None, scale_tril=None, validate_args=None):
        if (covariance_matrix is not None) + (scale_tril is not None) + (precision_matrix is not None) != 1:
            raise ValueError("Exactly one of covariance_matrix or precision_matrix or scale_tril may be specified.")
        if scale_tril is None:
            cov = covariance_matrix if covariance_matrix is not None else torch.linalg.inv(precision_matrix)
            scale_tril = torch.linalg.cholesky(cov)
        batch = torch.broadcast_shapes(loc.shape[:-1], scale_tril.shape[:-2])
        self.loc = loc.expand(batch + loc.shape[-1:])
        self.scale_tril = scale_tril.expand(batch + scale_tril.shape[-2:])
        super().__init__(batch, loc.shape[-1:], validate_args=validate_args)

    mean = property(lambda s: s.loc)
    mode = property(lambda s: s.loc)
    covariance_matrix = property(lambda s: s.scale_tril @ s.scale_tril.transpose(-1, -2))
    precision_matrix = property(lambda s: torch.cholesky_inverse(s.scale_tril))
    variance = property(lambda s: s.scale_tril.pow(2).sum(-1))

    def rsample(self, sample_shape=torch.Size()):
        eps = torch.randn(_shape(sample_shape, self), dtype=self.loc.dtype, device=self.loc.device)
        return self.loc + (self.scale_tril @ eps.unsqueeze(-1)).squeeze(-1)

    def log_prob(self, value):
        diff = (value - self.loc).unsqueeze(-1)
        L = self.scale_tril.expand(diff.shape[:-2] + self.scale_tril.shape[-2:])
        z = torch.linalg.solve_triangular(L, diff, upper=False).squeeze(-1)
        half_logdet = self.scale_tril.diagonal(dim1=-2, dim2=-1).log().sum(-1)
        return -0.5 * (self.event_shape[0] * math.log(2 * math.pi) + z.pow(2).sum(-1)) - half_logdet

    def entropy(self):
        half_logdet = self.scale_tril.diagonal(dim1=-2, dim2=-1).log().sum(-1)
        return 0.5 * self.event_shape[0] * (1.0 + math.log(2 * math.pi)) + half_logdet


class Independent(Distribution):
    """Reinterprets the last ``n`` batch dimensions of ``base`` as event dimensions (log-probabilities and entropies are summed over them)."""
    arg_constraints: Dict = {}

    def __init__(self, base_distribution, reinterpreted_batch_ndims: int, validate_args=None):
        n = reinterpreted_batch_ndims
        if n > len(base_distribution.batch_shape):
            raise ValueError("Expected reinterpreted_batch_ndims <= len(base_distribution.batch_shape)")
        shape = base_distribution.batch_shape + base_distribution.event_shape
        ev = n + len(base_distribution.event_shape)
        self.base_dist, self.reinterpreted_batch_ndims = base_distribution, n
        super().__init__(shape[: len(shape) - ev], shape[len(shape) - ev:], validate_args=validate_args)

    has_rsample = property(lambda s: s.base_dist.has_rsample)
    mean = property(lambda s: s.base_dist.mean)
    variance = property(lambda s: s.base_dist.variance)

    @property
    def support(self):
        return _c.independent(self.base_dist.support, self.reinterpreted_batch_ndims) if self.reinterpreted_batch_ndims else self.base_dist.support

    def _sum(self, t):
        n = self.reinterpreted_batch_ndims
        return t.reshape(t.shape[: t.dim() - n] + (-1,)).sum(-1) if n else t

    def sample(self, sample_shape=torch.Size()):
        return self.base_dist.sample(sample_shape)

    def rsample(self, sample_shape=torch.Size()):
        return self.base_dist.rsample(sample_shape)

    def log_prob(self, value):
        return self._sum(self.base_dist.log_prob(value))

    def entropy(self):
        return self._sum(self.base_dist.entropy())


# ----------------------------------------------------------------------------------------------------------------------
# KL registry (ferrotorch-distributions/src/kl.rs:66): most specific registered pair along the two method resolution orders
# ----------------------------------------------------------------------------------------------------------------------
_KL: Dict[Tuple[Type, Type], Callable] = {}


def register_kl(p_cls: Type, q_cls: Type):
    def deco(fn):
        _KL[(p_cls, q_cls)] = fn
        return fn
    return deco


def kl_divergence(p, q) -> torch.Tensor:
    best = None
    for i, pc in enumerate(type(p).__mro__):
        for j, qc in enumerate(type(q).__mro__):
            fn = _KL.get((pc, qc))
            if fn is not None and (best is None or i + j < best[0]):
                best = (i + j, fn)
    if best is None:
        from torch.distributions import kl as _tkl                                  # families that are not implemented here
        return _tkl.kl_divergence(p, q)
    return best[1](p, q)


@register_kl(Normal, Normal)
def _kl_normal(p, q):
    vr = (p.scale / q.scale).pow(2)
    return 0.5 * (vr + ((p.loc - q.loc) / q.scale).pow(2) - 1 - vr.log())


@register_kl(Bernoulli, Bernoulli)
def _kl_bernoulli(p, q):
    t1 = p.probs * (torch.nn.functional.softplus(-q.logits) - torch.nn.functional.softplus(-p.logits))
    t2 = (1 - p.probs) * (torch.nn.functional.softplus(q.logits) - torch.nn.functional.softplus(p.logits))
    return t1 + t2


@register_kl(Categorical, Categorical)
def _kl_categorical(p, q):
    t = p.probs * (p.logits - q.logits)
    t = torch.where(q.probs == 0, torch.full_like(t, math.inf), t)
    return torch.where(p.probs == 0, torch.zeros_like(t), t).sum(-1)


@register_kl(OneHotCategorical, OneHotCategorical)
def _kl_onehot(p, q):
    return _kl_categorical(p._cat, q._cat)


@register_kl(Uniform, Uniform)
def _kl_uniform(p, q):
    r = ((q.high - q.low) / (p.high - p.low)).log()
    return torch.where((q.low > p.low) | (q.high < p.high), torch.full_like(r, math.inf), r)


@register_kl(Exponential, Exponential)
def _kl_exponential(p, q):
    r = q.rate / p.rate
    return r - r.log() - 1


@register_kl(Laplace, Laplace)
def _kl_laplace(p, q):
    sr = p.scale / q.scale
    d = (p.loc - q.loc).abs()
    return -sr.log() + d / q.scale + sr * torch.exp(-d / p.scale) - 1


@register_kl(Gamma, Gamma)
def _kl_gamma(p, q):
    return (q.concentration * (p.rate / q.rate).log() + torch.lgamma(q.concentration) - torch.lgamma(p.concentration)
            + (p.concentration - q.concentration) * torch.digamma(p.concentration) + (q.rate - p.rate) * (p.concentration / p.rate))


@register_kl(Beta, Beta)
def _kl_beta(p, q):
    sp, sq = p.concentration1 + p.concentration0, q.concentration1 + q.concentration0
    return (torch.lgamma(q.concentration1) + torch.lgamma(q.concentration0) + torch.lgamma(sp) - torch.lgamma(p.concentration1)
            - torch.lgamma(p.concentration0) - torch.lgamma(sq) + (p.concentration1 - q.concentration1) * torch.digamma(p.concentration1)
            + (p.concentration0 - q.concentration0) * torch.digamma(p.concentration0) + (sq - sp) * torch.digamma(sp))


@register_kl(Dirichlet, Dirichlet)
def _kl_dirichlet(p, q):
    a, b = p.concentration, q.concentration
    a0 = a.sum(-1)
    return (torch.lgamma(a0) - torch.lgamma(b.sum(-1)) - (torch.lgamma(a) - torch.lgamma(b)).sum(-1)
            + ((a - b) * (torch.digamma(a) - torch.digamma(a0).unsqueeze(-1))).sum(-1))


@register_kl(Poisson, Poisson)
def _kl_poisson(p, q):
    return p.rate * (p.rate.log() - q.rate.log()) - (p.rate - q.rate)


@register_kl(Gumbel, Gumbel)
def _kl_gumbel(p, q):
    ct1 = p.scale / q.scale
    ct2 = q.loc / q.scale
    ct3 = p.loc / q.scale
    return -ct1.log() - ct2 + ct3 + ct1 * _EULER + torch.exp(ct2 + (1 + ct1).lgamma() - ct3) - (1 + _EULER)


@register_kl(Normal, Uniform)
def _kl_normal_uniform(p, q):
    """A normal puts mass outside every bounded interval, so the divergence is infinite (kl.rs:334)."""
    return torch.full_like(p.loc + q.low, math.inf)


@register_kl(Uniform, Normal)
def _kl_uniform_normal(p, q):
    """E_p[log p - log q] with the second moment of a uniform about q's mean (kl.rs:367)."""
    width = p.high - p.low
    second = width.pow(2) / 12 + ((p.high + p.low) / 2 - q.loc).pow(2)
    return -width.log() + 0.5 * math.log(2 * math.pi) + q.scale.log() + second / (2 * q.scale.pow(2))


@register_kl(Gamma, Exponential)
def _kl_gamma_exponential(p, q):
    """Exponential(rate) is Gamma(1, rate) (kl.rs:533)."""
    return _kl_gamma(p, Gamma(torch.ones_like(q.rate), q.rate))


@register_kl(Exponential, Gamma)
def _kl_exponential_gamma(p, q):
    return _kl_gamma(Gamma(torch.ones_like(p.rate), p.rate), q)


@register_kl(HalfNormal, HalfNormal)
def _kl_half_normal(p, q):
    """Folding both normals at zero leaves the log-ratio of the densities unchanged on the support."""
    vr = (p.scale / q.scale).pow(2)
    return 0.5 * (vr - 1 - vr.log())


@register_kl(LogNormal, LogNormal)
def _kl_lognormal(p, q):
    """The divergence is invariant under the shared bijection exp, so it equals that of the underlying normals."""
    return _kl_normal(p.base, q.base)


@register_kl(Cauchy, Cauchy)
def _kl_cauchy(p, q):
    """Closed form of Chyzak and Nielsen (2019)."""
    return torch.log(((p.scale + q.scale).pow(2) + (p.loc - q.loc).pow(2)) / (4 * p.scale * q.scale))


@register_kl(Pareto, Pareto)
def _kl_pareto(p, q):
    """Infinite when p reaches below q's lower bound."""
    ratio = p.scale / q.scale
    ar = q.alpha / p.alpha
    out = q.alpha * ratio.log() - ar.log() + ar - 1
    return torch.where(p.scale < q.scale, torch.full_like(out, math.inf), out)


@register_kl(Normal, Laplace)
def _kl_normal_laplace(p, q):
    """-H(p) + log(2 b) + E_p|x - m| / b, with the mean absolute deviation of a normal about m in closed form."""
    d = p.loc - q.loc
    z = d / p.scale
    mad = p.scale * math.sqrt(2 / math.pi) * torch.exp(-0.5 * z.pow(2)) + d * torch.erf(z / math.sqrt(2))
    return -p.entropy() + torch.log(2 * q.scale) + mad / q.scale


@register_kl(Beta, Normal)
def _kl_beta_normal(p, q):
    """-H(p) minus the expected normal log-density, which needs only p's mean and variance."""
    second = p.variance + (p.mean - q.loc).pow(2)
    return -p.entropy() + 0.5 * math.log(2 * math.pi) + q.scale.log() + second / (2 * q.scale.pow(2))


@register_kl(MultivariateNormal, MultivariateNormal)
def _kl_mvn(p, q):
    n = p.event_shape[0]
    hl_p = p.scale_tril.diagonal(dim1=-2, dim2=-1).log().sum(-1)
    hl_q = q.scale_tril.diagonal(dim1=-2, dim2=-1).log().sum(-1)
    batch = torch.broadcast_shapes(p.batch_shape, q.batch_shape)
    Lq = q.scale_tril.expand(batch + (n, n))
    Lp = p.scale_tril.expand(batch + (n, n))
    m = torch.linalg.solve_triangular(Lq, Lp, upper=False)
    d = torch.linalg.solve_triangular(Lq, (q.loc - p.loc).expand(batch + (n,)).unsqueeze(-1), upper=False).squeeze(-1)
    return hl_q - hl_p + 0.5 * (m.pow(2).sum((-1, -2)) + d.pow(2).sum(-1) - n)


@register_kl(Independent, Independent)
def _kl_independent(p, q):
    if p.reinterpreted_batch_ndims != q.reinterpreted_batch_ndims:
        raise NotImplementedError("KL between Independent distributions with different event dimensions")
    return p._sum(kl_divergence(p.base_dist, q.base_dist))
