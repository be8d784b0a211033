"""Probability distributions, KL registry, transforms and constraints (API names follow ferrotorch-distributions).

The 27 distribution families, ``kl_divergence`` with its pairwise registry, bijective transforms and support constraints are PyTorch's
own implementations under the reference's names (``sample`` / ``rsample`` / ``log_prob`` / ``entropy``): this is a cold path that rides the
host substrate's tensor ops, on any device. Sampling draws from the substrate's generators (``torch.manual_seed``), not from the Philox
streams of ``ferrotorch_b200.gpu.CudaRngManager``.

Reference parity: ferrotorch-distributions/src/lib.rs:138 (Distribution trait), kl.rs:66, transforms.rs, constraints.rs and one
file per family.
"""
from torch import distributions as _d
from torch.distributions import kl
from . import constraints, transforms
from .constraints import Constraint
from .transforms import TransformedDistribution, SoftplusTransform, Transform
from torch.distributions.kl import kl_divergence, register_kl

Distribution = _d.Distribution
Bernoulli, Beta, Categorical, Cauchy, Dirichlet, Exponential, Gamma, Gumbel = (_d.Bernoulli, _d.Beta, _d.Categorical, _d.Cauchy, _d.Dirichlet,
                                                                               _d.Exponential, _d.Gamma, _d.Gumbel)
HalfNormal, Independent, Kumaraswamy, Laplace, LogNormal = _d.HalfNormal, _d.Independent, _d.Kumaraswamy, _d.Laplace, _d.LogNormal
LowRankMultivariateNormal, MixtureSameFamily, Multinomial, MultivariateNormal, Normal = (_d.LowRankMultivariateNormal, _d.MixtureSameFamily,
                                                                                         _d.Multinomial, _d.MultivariateNormal, _d.Normal)
OneHotCategorical, Pareto, Poisson, RelaxedBernoulli, RelaxedOneHotCategorical = (_d.OneHotCategorical, _d.Pareto, _d.Poisson,
                                                                                  _d.RelaxedBernoulli, _d.RelaxedOneHotCategorical)
StudentT, Uniform, VonMises, Weibull = _d.StudentT, _d.Uniform, _d.VonMises, _d.Weibull
AffineTransform, ExpTransform, SigmoidTransform, TanhTransform, ComposeTransform, SoftmaxTransform, StickBreakingTransform = (
    transforms.AffineTransform, transforms.ExpTransform, transforms.SigmoidTransform, transforms.TanhTransform, transforms.ComposeTransform,
    transforms.SoftmaxTransform, transforms.StickBreakingTransform)

__all__ = [n for n in dir() if not n.startswith("_")]
