"""Six further families: multinomial, finite mixtures of one family, the two concrete (relaxed) distributions, von Mises on the circle and
the low-rank-plus-diagonal multivariate normal. Same conventions as ``families``: the arithmetic is written here, the base class only
supplies the shape bookkeeping.

Reference parity: ferrotorch-distributions/src/{multinomial.rs, mixture_same_family.rs, relaxed_bernoulli.rs,
relaxed_one_hot_categorical.rs, von_mises.rs, lowrank_multivariate_normal.rs}.
"""
from __future__ import annotations

import math

import torch
from torch.distributions import constraints as _c
from torch.distributions.utils import broadcast_all

from .families import Categorical, Distribution, _probs_logits, _shape


class Multinomial(Distribution):
    """Counts of ``total_count`` independent categorical draws."""
    arg_constraints = {"probs": _c.simplex, "logits": _c.real_vector}

    def __init__(self, total_count: int = 1, probs=None, logits=None, validate_args=None):
        if not isinstance(total_count, int) or total_count < 0:
            raise ValueError("total_count must be a non-negative integer (one count shared by the batch)")
        self.total_count = total_count
        self._cat = Categorical(probs, logits)
        self.probs, self.logits = self._cat.probs, self._cat.logits
        super().__init__(self._cat.batch_shape, self.probs.shape[-1:], validate_args=validate_args)

    @_c.dependent_property(is_discrete=True, event_dim=1)
    def support(self):
        return _c.multinomial(self.total_count)

    mean = property(lambda s: s.probs * s.total_count)
    variance = property(lambda s: s.total_count * s.probs * (1 - s.probs))

    def sample(self, sample_shape=torch.Size()):
        with torch.no_grad():
            draws = self._cat.sample(torch.Size((self.total_count,)) + torch.Size(sample_shape))      # [n, *sample, *batch]
            counts = torch.zeros(torch.Size(sample_shape) + self.batch_shape + self.event_shape, dtype=self.probs.dtype, device=self.probs.device)
            if self.total_count:
                idx = draws.movedim(0, -1)                                                            # [*sample, *batch, n]
                counts.scatter_add_(-1, idx, torch.ones_like(idx, dtype=counts.dtype))
            return counts

    rsample = None

    def log_prob(self, value):
        logits = torch.where(self.probs == 0, torch.full_like(self.logits, -math.inf), self.logits)   # an impossible category, exactly
        term = torch.where(value == 0, torch.zeros_like(logits * value), value * logits)              # 0 * log 0 = 0
        return torch.lgamma(value.sum(-1) + 1) - torch.lgamma(value + 1).sum(-1) + term.sum(-1)

    def entropy(self):
        """``n H(p) - log n! + sum_k E[log X_k!]`` with ``X_k ~ Binomial(n, p_k)`` summed exactly over its support."""
        n = self.total_count
        x = torch.arange(n + 1, dtype=self.probs.dtype, device=self.probs.device)
        p = self.probs.unsqueeze(-1)
        logc = math.lgamma(n + 1) - torch.lgamma(x + 1) - torch.lgamma(n - x + 1)
        logpmf = logc + torch.xlogy(x, p) + torch.xlogy(n - x, 1 - p)
        e_lfact = (logpmf.exp() * torch.lgamma(x + 1)).sum(-1).sum(-1)
        return n * self._cat.entropy() - math.lgamma(n + 1) + e_lfact


class MixtureSameFamily(Distribution):
    """``sum_k pi_k f_k(x)``: ``mixture_distribution`` is a :class:`Categorical` over the rightmost batch dimension of
    ``component_distribution``."""
    arg_constraints: dict = {}
    has_rsample = False

    def __init__(self, mixture_distribution, component_distribution, validate_args=None):
        if not hasattr(mixture_distribution, "logits") or mixture_distribution.event_shape != torch.Size():
            raise ValueError("mixture_distribution must be a Categorical")
        cb = component_distribution.batch_shape
        if len(cb) == 0 or cb[-1] != mixture_distribution.logits.shape[-1]:
            raise ValueError("the rightmost batch dimension of the components must equal the number of mixture weights")
        if mixture_distribution.batch_shape != torch.Size() and mixture_distribution.batch_shape != cb[:-1]:
            raise ValueError("batch shapes of the mixture weights and of the components do not agree")
        self.mixture_distribution, self.component_distribution = mixture_distribution, component_distribution
        self._k = cb[-1]
        self._ev = len(component_distribution.event_shape)
        super().__init__(cb[:-1], component_distribution.event_shape, validate_args=validate_args)

    @property
    def support(self):
        return self.component_distribution.support

    def _w(self):                              # weights broadcast against component statistics [*batch, K, *event]
        p = self.mixture_distribution.probs
        return p.reshape(p.shape + (1,) * self._ev)

    def _pad(self, x):                         # [*sample, *batch, *event] -> [*sample, *batch, 1, *event]
        return x.unsqueeze(-1 - self._ev)

    @property
    def mean(self):
        return (self._w() * self.component_distribution.mean).sum(-1 - self._ev)

    @property
    def variance(self):
        w, d = self._w(), -1 - self._ev
        within = (w * self.component_distribution.variance).sum(d)
        between = (w * (self.component_distribution.mean - self._pad(self.mean)) ** 2).sum(d)
        return within + between

    def log_prob(self, value):
        lp = self.component_distribution.log_prob(self._pad(value))                   # [*sample, *batch, K]
        lw = torch.log_softmax(self.mixture_distribution.logits, -1)
        return torch.logsumexp(lp + lw, -1)

    def cdf(self, value):
        return (self.component_distribution.cdf(self._pad(value)) * self.mixture_distribution.probs).sum(-1)

    def sample(self, sample_shape=torch.Size()):
        with torch.no_grad():
            sample_shape = torch.Size(sample_shape)
            k = self.mixture_distribution.sample(sample_shape)                        # [*sample, *batch]
            xs = self.component_distribution.sample(sample_shape)                     # [*sample, *batch, K, *event]
            k = k.expand(sample_shape + self.batch_shape)
            idx = k.reshape(k.shape + (1,) * (self._ev + 1)).expand(k.shape + (1,) + self.event_shape)
            return xs.gather(len(k.shape), idx).squeeze(len(k.shape))


class RelaxedBernoulli(Distribution):
    """Concrete relaxation of a Bernoulli variable on (0, 1): ``sigmoid((logits + Logistic noise) / temperature)``."""
    arg_constraints = {"probs": _c.unit_interval, "logits": _c.real}
    support = _c.unit_interval
    has_rsample = True

    def __init__(self, temperature, probs=None, logits=None, validate_args=None):
        self.temperature = torch.as_tensor(temperature, dtype=torch.get_default_dtype())
        self.probs, self.logits = _probs_logits(probs, logits, True)
        super().__init__(self.logits.shape, validate_args=validate_args)

    def rsample(self, sample_shape=torch.Size()):
        shape = _shape(sample_shape, self)
        eps = torch.finfo(self.logits.dtype).eps
        u = torch.rand(shape, dtype=self.logits.dtype, device=self.logits.device).clamp(eps, 1 - eps)
        return torch.sigmoid((self.logits + u.log() - (-u).log1p()) / self.temperature)

    def log_prob(self, value):
        z = value.log() - (-value).log1p()                                           # logit of the value
        diff = self.logits - z * self.temperature
        return self.temperature.log() + diff - 2 * torch.nn.functional.softplus(diff) - value.log() - (-value).log1p()


class RelaxedOneHotCategorical(Distribution):
    """Concrete (Gumbel-softmax) relaxation of a one-hot categorical variable on the simplex."""
    arg_constraints = {"probs": _c.simplex, "logits": _c.real_vector}
    support = _c.simplex
    has_rsample = True

    def __init__(self, temperature, probs=None, logits=None, validate_args=None):
        self.temperature = torch.as_tensor(temperature, dtype=torch.get_default_dtype())
        self.probs, self.logits = _probs_logits(probs, logits, False)
        super().__init__(self.logits.shape[:-1], self.logits.shape[-1:], validate_args=validate_args)

    def rsample(self, sample_shape=torch.Size()):
        shape = _shape(sample_shape, self)
        eps = torch.finfo(self.logits.dtype).tiny
        u = torch.rand(shape, dtype=self.logits.dtype, device=self.logits.device).clamp(eps, 1 - torch.finfo(self.logits.dtype).eps)
        g = -(-u.log()).log()
        return torch.softmax((self.logits + g) / self.temperature, -1)

    def log_prob(self, value):
        k = self.logits.shape[-1]
        logy = value.log()
        score = self.logits - logy * self.temperature
        score = (score - score.logsumexp(-1, keepdim=True)).sum(-1)
        log_scale = math.lgamma(k) + (k - 1) * self.temperature.log()
        return score + log_scale - logy.sum(-1)                                      # last term: density on the simplex, not on log y


class VonMises(Distribution):
    """Circular normal on [-pi, pi): density ``exp(kappa cos(x - mu)) / (2 pi I0(kappa))``."""
    arg_constraints = {"loc": _c.real, "concentration": _c.positive}
    support = _c.real
    has_rsample = False

    def __init__(self, loc, concentration, validate_args=None):
        self.loc, self.concentration = broadcast_all(loc, concentration)
        super().__init__(self.loc.shape, validate_args=validate_args)

    mean = property(lambda s: s.loc)
    mode = property(lambda s: s.loc)

    @property
    def variance(self):
        """Circular variance ``1 - I1(kappa) / I0(kappa)``."""
        return 1 - torch.special.i1e(self.concentration) / torch.special.i0e(self.concentration)

    def log_prob(self, value):
        k = self.concentration
        return k * torch.cos(value - self.loc) - math.log(2 * math.pi) - (torch.special.i0e(k).log() + k)

    def sample(self, sample_shape=torch.Size()):
        """Best and Fisher (1979): propose from a wrapped Cauchy, accept with the two-step test; the loop re-draws only the rejected entries."""
        with torch.no_grad():
            shape = _shape(sample_shape, self)
            k = self.concentration.double().expand(shape)
            tau = 1 + (1 + 4 * k * k).sqrt()
            rho = (tau - (2 * tau).sqrt()) / (2 * k)
            r = torch.where(k < 1e-5, 1 / k + k, (1 + rho * rho) / (2 * rho))        # series form where rho underflows
            x = torch.zeros(shape, dtype=torch.float64, device=k.device)
            todo = torch.ones(shape, dtype=torch.bool, device=k.device)
            for _ in range(1000):
                if not bool(todo.any()):
                    break
                u = torch.rand((3,) + tuple(shape), dtype=torch.float64, device=k.device)
                z = torch.cos(math.pi * u[0])
                f = (1 + r * z) / (r + z)
                c = k * (r - f)
                ok = ((c * (2 - c) - u[1]) > 0) | (((c / u[1]).log() + 1 - c) >= 0)
                cand = torch.sign(u[2] - 0.5) * torch.acos(f.clamp(-1, 1))
                take = todo & ok
                x = torch.where(take, cand, x)
                todo = todo & ~ok
            out = (x + math.pi + self.loc.double()) % (2 * math.pi) - math.pi
            return out.to(self.loc.dtype)


class LowRankMultivariateNormal(Distribution):
    """Normal with covariance ``W W^T + diag(d)`` (``W``: ``[.., D, K]``, ``d``: ``[.., D]``). Densities go through the ``K x K`` capacitance
    matrix ``I + W^T diag(d)^-1 W`` (Woodbury identity and matrix-determinant lemma), so nothing of size ``D x D`` is factorised."""
    arg_constraints = {"loc": _c.real_vector, "cov_factor": _c.independent(_c.real, 2), "cov_diag": _c.independent(_c.positive, 1)}
    support = _c.real_vector
    has_rsample = True

    def __init__(self, loc, cov_factor, cov_diag, validate_args=None):
        if loc.dim() < 1 or cov_factor.dim() < 2 or cov_factor.shape[-2] != loc.shape[-1] or cov_diag.shape[-1] != loc.shape[-1]:
            raise ValueError("loc [.., D], cov_factor [.., D, K] and cov_diag [.., D] must agree on D")
        batch = torch.broadcast_shapes(loc.shape[:-1], cov_factor.shape[:-2], cov_diag.shape[:-1])
        D, K = cov_factor.shape[-2:]
        self.loc = loc.expand(batch + (D,))
        self.cov_factor = cov_factor.expand(batch + (D, K))
        self.cov_diag = cov_diag.expand(batch + (D,))
        wd = self.cov_factor / self.cov_diag.unsqueeze(-1)                           # diag(d)^-1 W
        cap = torch.eye(K, dtype=loc.dtype, device=loc.device) + self.cov_factor.transpose(-1, -2) @ wd
        self._cap_tril = torch.linalg.cholesky(cap)
        super().__init__(batch, torch.Size((D,)), validate_args=validate_args)

    mean = property(lambda s: s.loc)
    mode = property(lambda s: s.loc)
    variance = property(lambda s: s.cov_factor.pow(2).sum(-1) + s.cov_diag)
    covariance_matrix = property(lambda s: s.cov_factor @ s.cov_factor.transpose(-1, -2) + torch.diag_embed(s.cov_diag))

    @property
    def precision_matrix(self):
        wd = self.cov_factor / self.cov_diag.unsqueeze(-1)
        a = torch.linalg.solve_triangular(self._cap_tril, wd.transpose(-1, -2), upper=False)           # L^-1 W^T D^-1
        return torch.diag_embed(1 / self.cov_diag) - a.transpose(-1, -2) @ a

    @property
    def scale_tril(self):
        return torch.linalg.cholesky(self.covariance_matrix)

    def _logdet(self):
        return self.cov_diag.log().sum(-1) + 2 * self._cap_tril.diagonal(dim1=-2, dim2=-1).log().sum(-1)

    def rsample(self, sample_shape=torch.Size()):
        shape = _shape(sample_shape, self)
        K = self.cov_factor.shape[-1]
        ew = torch.randn(shape[:-1] + (K,), dtype=self.loc.dtype, device=self.loc.device)
        ed = torch.randn(shape, dtype=self.loc.dtype, device=self.loc.device)
        return self.loc + (self.cov_factor @ ew.unsqueeze(-1)).squeeze(-1) + self.cov_diag.sqrt() * ed

    def log_prob(self, value):
        diff = value - self.loc
        wtd = (self.cov_factor.transpose(-1, -2) @ (diff / self.cov_diag).unsqueeze(-1))               # W^T D^-1 x  [.., K, 1]
        half = torch.linalg.solve_triangular(self._cap_tril.expand(wtd.shape[:-2] + self._cap_tril.shape[-2:]), wtd, upper=False)
        maha = (diff * diff / self.cov_diag).sum(-1) - half.squeeze(-1).pow(2).sum(-1)
        D = self.loc.shape[-1]
        return -0.5 * (D * math.log(2 * math.pi) + self._logdet() + maha)

    def entropy(self):
        D = self.loc.shape[-1]
        return 0.5 * (D * (1 + math.log(2 * math.pi)) + self._logdet())


__all__ = ["Multinomial", "MixtureSameFamily", "RelaxedBernoulli", "RelaxedOneHotCategorical", "VonMises", "LowRankMultivariateNormal"]
