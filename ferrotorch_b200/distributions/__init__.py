"""Probability distributions, KL registry, transforms and constraints (API names follow ferrotorch-distributions).

Twenty-one families are implemented in :mod:`.families` (parameters, reparameterised sampling, ``log_prob``, ``entropy``, moments, ``cdf`` /
``icdf`` where closed forms exist) together with the pairwise KL registry; each is checked against ``torch.distributions`` in the test
suite. The remaining six (``LowRankMultivariateNormal``, ``MixtureSameFamily``, ``Multinomial``, ``RelaxedBernoulli``,
``RelaxedOneHotCategorical``, ``VonMises``) are the substrate's implementations under the reference's names. Sampling draws from the
substrate's generators (``torch.manual_seed``), not from the Philox streams of ``ferrotorch_b200.gpu.CudaRngManager``.

Reference parity: ferrotorch-distributions/src/lib.rs:138 (Distribution trait), kl.rs:66, transforms.rs, constraints.rs and one
file per family.
"""
from . import constraints, transforms
from .constraints import Constraint
from .transforms import TransformedDistribution, SoftplusTransform, Transform
from .families import (Distribution, Normal, LogNormal, Uniform, Bernoulli, Categorical, OneHotCategorical, Exponential, Laplace, Gumbel, Cauchy,
                       HalfNormal, Gamma, Beta, Dirichlet, StudentT, Poisson, Weibull, Pareto, Kumaraswamy, MultivariateNormal, Independent,
                       kl_divergence, register_kl)
from . import families as kl

from .more_families import (LowRankMultivariateNormal, MixtureSameFamily, Multinomial, RelaxedBernoulli, RelaxedOneHotCategorical,
                            VonMises)
AffineTransform, ExpTransform, SigmoidTransform, TanhTransform, ComposeTransform, SoftmaxTransform, StickBreakingTransform = (
    transforms.AffineTransform, transforms.ExpTransform, transforms.SigmoidTransform, transforms.TanhTransform, transforms.ComposeTransform,
    transforms.SoftmaxTransform, transforms.StickBreakingTransform)

__all__ = [n for n in dir() if not n.startswith("_")]
