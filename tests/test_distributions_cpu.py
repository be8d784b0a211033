"""The distribution families implemented in distributions/families.py against torch.distributions: log_prob, entropy, moments, cdf, KL,
sampling statistics and pathwise gradients."""
import math

import pytest
import torch
import torch.distributions as TD

td = TD

from ferrotorch_b200 import distributions as D

X = torch.tensor([0.3, 1.7, 0.05])
U = torch.tensor([0.2, 0.9, 0.55])
A, B = torch.tensor([0.7, 2.0, 3.5]), torch.tensor([1.3, 0.6, 2.2])
CASES = {
    "Normal": (lambda m: m.Normal(A, B), X), "LogNormal": (lambda m: m.LogNormal(A * 0.2, B * 0.5), X), "Uniform": (lambda m: m.Uniform(-A, B + 2), X),
    "Exponential": (lambda m: m.Exponential(A), X), "Laplace": (lambda m: m.Laplace(A, B), X), "Gumbel": (lambda m: m.Gumbel(A, B), X),
    "Cauchy": (lambda m: m.Cauchy(A, B), X), "HalfNormal": (lambda m: m.HalfNormal(B), X), "Gamma": (lambda m: m.Gamma(A, B), X),
    "Beta": (lambda m: m.Beta(A, B), U), "StudentT": (lambda m: m.StudentT(A + 2.5, B, A), X), "Weibull": (lambda m: m.Weibull(A, B), X),
    "Pareto": (lambda m: m.Pareto(A * 0.01, B), X), "Kumaraswamy": (lambda m: m.Kumaraswamy(A, B), U),
    "Bernoulli": (lambda m: m.Bernoulli(probs=U), torch.tensor([0.0, 1.0, 1.0])), "Poisson": (lambda m: m.Poisson(A), torch.tensor([0.0, 3.0, 2.0])),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_family_matches_torch(name):
    make, x = CASES[name]
    ours, ref = make(D), make(TD)
    assert type(ours).__module__.startswith("ferrotorch_b200")            # implemented here, not the torch class under another name
    assert torch.allclose(ours.log_prob(x), ref.log_prob(x), atol=1e-5, equal_nan=True), name
    if name != "Poisson":
        assert torch.allclose(ours.entropy(), ref.entropy(), atol=1e-5), name
    for attr in ("mean", "variance"):
        assert torch.allclose(getattr(ours, attr), getattr(ref, attr), atol=1e-5, equal_nan=True), (name, attr)
    if hasattr(ours, "cdf") and name not in ("Bernoulli", "Poisson"):
        try:
            r = ref.cdf(x)
        except NotImplementedError:
            r = None
        if r is not None:
            assert torch.allclose(ours.cdf(x), r, atol=1e-5), name
    assert ours.batch_shape == ref.batch_shape and ours.event_shape == ref.event_shape


def test_categorical_dirichlet_mvn_independent():
    lg = torch.tensor([[0.1, 0.5, -0.3], [1.0, -1.0, 0.0]])
    c, rc = D.Categorical(logits=lg), TD.Categorical(logits=lg)
    v = torch.tensor([1, 2])
    assert torch.allclose(c.log_prob(v), rc.log_prob(v)) and torch.allclose(c.entropy(), rc.entropy()) and torch.equal(c.mode, rc.mode)
    assert c.sample((5,)).shape == (5, 2) and c.enumerate_support().shape == (3, 2)
    oh, roh = D.OneHotCategorical(probs=lg.softmax(-1)), TD.OneHotCategorical(probs=lg.softmax(-1))
    one = torch.nn.functional.one_hot(v, 3).float()
    assert torch.allclose(oh.log_prob(one), roh.log_prob(one)) and oh.sample().sum(-1).eq(1).all()
    conc = torch.tensor([[0.7, 2.0, 3.5], [1.0, 1.0, 1.0]])
    d, rd = D.Dirichlet(conc), TD.Dirichlet(conc)
    p = torch.tensor([[0.2, 0.3, 0.5], [0.1, 0.1, 0.8]])
    assert torch.allclose(d.log_prob(p), rd.log_prob(p), atol=1e-5) and torch.allclose(d.entropy(), rd.entropy(), atol=1e-5)
    assert torch.allclose(d.mean, rd.mean) and torch.allclose(d.variance, rd.variance)
    cov = torch.tensor([[2.0, 0.3], [0.3, 1.0]])
    m, rm = D.MultivariateNormal(torch.tensor([0.5, -1.0]), covariance_matrix=cov), TD.MultivariateNormal(torch.tensor([0.5, -1.0]), covariance_matrix=cov)
    x = torch.tensor([[0.3, 1.7], [-1.0, 0.2]])
    assert torch.allclose(m.log_prob(x), rm.log_prob(x), atol=1e-5) and torch.allclose(m.entropy(), rm.entropy(), atol=1e-5)
    assert torch.allclose(m.covariance_matrix, cov, atol=1e-6) and torch.allclose(m.precision_matrix, torch.linalg.inv(cov), atol=1e-5)
    m2 = D.MultivariateNormal(torch.zeros(2), scale_tril=torch.tensor([[1.0, 0.0], [0.5, 0.8]]))
    r2 = TD.MultivariateNormal(torch.zeros(2), scale_tril=torch.tensor([[1.0, 0.0], [0.5, 0.8]]))
    assert torch.allclose(D.kl_divergence(m, m2), TD.kl_divergence(rm, r2), atol=1e-5)
    ind, rind = D.Independent(D.Normal(torch.zeros(3, 4), torch.ones(3, 4) * 2), 1), TD.Independent(TD.Normal(torch.zeros(3, 4), torch.ones(3, 4) * 2), 1)
    z = torch.randn(3, 4)
    assert ind.batch_shape == (3,) and ind.event_shape == (4,) and torch.allclose(ind.log_prob(z), rind.log_prob(z)) and torch.allclose(ind.entropy(), rind.entropy())
    with pytest.raises(ValueError):
        D.MultivariateNormal(torch.zeros(2))
    with pytest.raises(ValueError):
        D.Categorical()


KL_PAIRS = [(lambda m: m.Normal(A, B), lambda m: m.Normal(B, A)), (lambda m: m.Bernoulli(probs=U), lambda m: m.Bernoulli(probs=U.flip(0))),
            (lambda m: m.Exponential(A), lambda m: m.Exponential(B)), (lambda m: m.Laplace(A, B), lambda m: m.Laplace(B, A)),
            (lambda m: m.Gamma(A, B), lambda m: m.Gamma(B, A)), (lambda m: m.Beta(A, B), lambda m: m.Beta(B, A)),
            (lambda m: m.Poisson(A), lambda m: m.Poisson(B)), (lambda m: m.Gumbel(A, B), lambda m: m.Gumbel(B, A)),
            (lambda m: m.Uniform(-A, A), lambda m: m.Uniform(-A - 1, A + 2)), (lambda m: m.Dirichlet(A), lambda m: m.Dirichlet(B)),
            (lambda m: m.Categorical(probs=U), lambda m: m.Categorical(probs=U.flip(0)))]


@pytest.mark.parametrize("i", range(len(KL_PAIRS)))
def test_kl_registry_matches_torch(i):
    p, q = KL_PAIRS[i]
    assert torch.allclose(D.kl_divergence(p(D), q(D)), TD.kl_divergence(p(TD), q(TD)), atol=1e-5)


def test_sampling_statistics_and_pathwise_gradients():
    torch.manual_seed(0)
    n = 40000
    for make in (lambda: D.Normal(1.5, 0.7), lambda: D.Gamma(3.0, 2.0), lambda: D.Beta(2.0, 5.0), lambda: D.Laplace(-1.0, 0.5),
                 lambda: D.Gumbel(0.3, 1.2), lambda: D.Exponential(1.7), lambda: D.Weibull(1.5, 2.0), lambda: D.Uniform(-1.0, 3.0),
                 lambda: D.StudentT(8.0, 0.5, 1.5), lambda: D.Kumaraswamy(2.0, 3.0), lambda: D.HalfNormal(1.3), lambda: D.LogNormal(0.1, 0.4)):
        d = make()
        s = d.sample((n,))
        assert abs(float(s.mean()) - float(d.mean)) < 4 * float(d.stddev) / math.sqrt(n) + 1e-3, type(d).__name__
        assert abs(float(s.var()) / float(d.variance) - 1) < 0.08, type(d).__name__
    for d, ev in ((D.Bernoulli(probs=torch.tensor(0.3)), 0.3), (D.Poisson(torch.tensor(4.0)), 4.0)):
        assert abs(float(d.sample((n,)).mean()) - ev) < 0.05
    # reparameterised samples carry gradients to the parameters
    loc, scale = torch.tensor(0.5, requires_grad=True), torch.tensor(1.5, requires_grad=True)
    D.Normal(loc, scale).rsample((1000,)).mean().backward()
    assert abs(float(loc.grad) - 1.0) < 1e-5 and scale.grad is not None
    a = torch.tensor(2.0, requires_grad=True)
    D.Gamma(a, torch.tensor(1.0)).rsample((20000,)).mean().backward()
    assert abs(float(a.grad) - 1.0) < 0.05                               # d E[x] / d concentration = 1 / rate
    conc = torch.tensor([1.0, 2.0, 3.0], requires_grad=True)
    D.Dirichlet(conc).rsample((64,))[:, 0].mean().backward()
    assert conc.grad is not None and float(conc.grad[0]) > 0 > float(conc.grad[1])


# -- the six families of more_families.py ------------------------------------------------------------------------------------------------
def _tclose(a, b, tol=1e-5):
    assert a.shape == b.shape and torch.allclose(a, b, atol=tol, rtol=tol), (a.shape, b.shape, (a - b).abs().max().item() if a.shape == b.shape else None)


def test_further_families_are_this_packages():
    import ferrotorch_b200.distributions as FD
    for n in ("Multinomial", "MixtureSameFamily", "RelaxedBernoulli", "RelaxedOneHotCategorical", "VonMises", "LowRankMultivariateNormal"):
        assert getattr(FD, n).__module__ == "ferrotorch_b200.distributions.more_families", n


def test_multinomial_matches_torch():
    import ferrotorch_b200.distributions as FD
    torch.manual_seed(0)
    p = torch.softmax(torch.randn(3, 5), -1)
    ours, ref = FD.Multinomial(7, probs=p), td.Multinomial(7, probs=p)
    x = ref.sample((4,))
    _tclose(ours.log_prob(x), ref.log_prob(x))
    _tclose(ours.mean, ref.mean)
    _tclose(ours.variance, ref.variance)
    _tclose(ours.entropy(), ref.entropy(), 1e-4)
    s = ours.sample((2000,))
    assert s.shape == (2000, 3, 5) and torch.all(s.sum(-1) == 7) and (s.mean(0) - ours.mean).abs().max() < 0.15
    z = FD.Multinomial(3, probs=torch.tensor([0.5, 0.5, 0.0]))
    assert torch.isfinite(z.log_prob(torch.tensor([1.0, 2.0, 0.0]))) and z.log_prob(torch.tensor([1.0, 1.0, 1.0])) == -float("inf")
    _tclose(FD.Multinomial(4, logits=torch.randn(5)).probs.sum(), torch.tensor(1.0))


def test_mixture_same_family_matches_torch():
    import ferrotorch_b200.distributions as FD
    torch.manual_seed(1)
    w = torch.softmax(torch.randn(2, 3), -1)
    mu, sd = torch.randn(2, 3), torch.rand(2, 3) + 0.3
    ours = FD.MixtureSameFamily(FD.Categorical(probs=w), FD.Normal(mu, sd))
    ref = td.MixtureSameFamily(td.Categorical(probs=w), td.Normal(mu, sd))
    x = torch.randn(5, 2)
    _tclose(ours.log_prob(x), ref.log_prob(x))
    _tclose(ours.cdf(x), ref.cdf(x))
    _tclose(ours.mean, ref.mean)
    _tclose(ours.variance, ref.variance)
    s = ours.sample((20000,))
    assert s.shape == (20000, 2) and (s.mean(0) - ours.mean).abs().max() < 0.05 and (s.var(0) - ours.variance).abs().max() < 0.1
    # vector-valued components
    mu2 = torch.randn(3, 4)
    o2 = FD.MixtureSameFamily(FD.Categorical(probs=w[0]), FD.Independent(FD.Normal(mu2, torch.ones(3, 4)), 1))
    r2 = td.MixtureSameFamily(td.Categorical(probs=w[0]), td.Independent(td.Normal(mu2, torch.ones(3, 4)), 1))
    y = torch.randn(6, 4)
    _tclose(o2.log_prob(y), r2.log_prob(y))
    _tclose(o2.mean, r2.mean)
    assert o2.sample((7,)).shape == (7, 4)
    with pytest.raises(ValueError):
        FD.MixtureSameFamily(FD.Categorical(probs=torch.ones(4) / 4), FD.Normal(mu, sd))


def test_relaxed_distributions_match_torch():
    import ferrotorch_b200.distributions as FD
    torch.manual_seed(2)
    lg, T = torch.randn(4), torch.tensor(0.7)
    ours, ref = FD.RelaxedBernoulli(T, logits=lg), td.RelaxedBernoulli(T, logits=lg)
    y = torch.rand(6, 4) * 0.98 + 0.01
    _tclose(ours.log_prob(y), ref.log_prob(y), 1e-4)
    lgr = lg.clone().requires_grad_()
    s = FD.RelaxedBernoulli(T, logits=lgr).rsample((5000,))
    assert s.shape == (5000, 4) and 0 < s.min() and s.max() < 1
    s.mean().backward()
    assert lgr.grad is not None and (lgr.grad > 0).all()                   # larger logits push the relaxed sample towards one
    assert ((s > 0.5).float().mean(0) - torch.sigmoid(lg)).abs().max() < 0.04
    lg2 = torch.randn(3, 5)
    o2, r2 = FD.RelaxedOneHotCategorical(T, logits=lg2), td.RelaxedOneHotCategorical(T, logits=lg2)
    v = torch.softmax(torch.randn(6, 3, 5), -1)
    _tclose(o2.log_prob(v), r2.log_prob(v), 1e-4)
    s2 = o2.rsample((4000,))
    assert s2.shape == (4000, 3, 5) and torch.allclose(s2.sum(-1), torch.ones(4000, 3), atol=1e-5)
    freq = torch.zeros(3, 5).scatter_add_(1, s2.argmax(-1).T, torch.ones(3, 4000)) / 4000
    assert (freq - torch.softmax(lg2, -1)).abs().max() < 0.04                # the arg-max of a Gumbel-softmax sample is categorical


def test_von_mises_matches_torch():
    import ferrotorch_b200.distributions as FD
    torch.manual_seed(3)
    mu, k = torch.tensor([0.0, 1.0, -2.5]), torch.tensor([0.5, 4.0, 50.0])
    ours, ref = FD.VonMises(mu, k), td.VonMises(mu, k)
    x = torch.rand(7, 3) * 2 * math.pi - math.pi
    _tclose(ours.log_prob(x), ref.log_prob(x), 1e-5)
    _tclose(ours.variance, ref.variance, 1e-5)
    _tclose(ours.mean, ref.mean)
    s = ours.sample((20000,))
    assert s.shape == (20000, 3) and s.min() >= -math.pi and s.max() < math.pi
    circ_mean = torch.atan2(torch.sin(s).mean(0), torch.cos(s).mean(0))
    assert (torch.remainder(circ_mean - mu + math.pi, 2 * math.pi) - math.pi).abs().max() < 0.05
    resultant = torch.sqrt(torch.sin(s).mean(0) ** 2 + torch.cos(s).mean(0) ** 2)
    assert (1 - resultant - ours.variance).abs().max() < 0.02
    tiny = FD.VonMises(torch.tensor(0.0), torch.tensor(1e-8)).sample((4000,))
    assert abs(float(tiny.mean())) < 0.15 and float(tiny.std()) > 1.6           # nearly uniform on the circle


def test_low_rank_multivariate_normal_matches_torch():
    import ferrotorch_b200.distributions as FD
    torch.manual_seed(4)
    loc, W, d = torch.randn(2, 6), torch.randn(2, 6, 2), torch.rand(2, 6) + 0.2
    ours, ref = FD.LowRankMultivariateNormal(loc, W, d), td.LowRankMultivariateNormal(loc, W, d)
    x = torch.randn(5, 2, 6)
    _tclose(ours.log_prob(x), ref.log_prob(x), 1e-4)
    _tclose(ours.entropy(), ref.entropy(), 1e-4)
    _tclose(ours.variance, ref.variance)
    _tclose(ours.covariance_matrix, ref.covariance_matrix)
    _tclose(ours.precision_matrix, ref.precision_matrix, 1e-4)
    _tclose(ours.scale_tril, ref.scale_tril, 1e-4)
    dense = FD.MultivariateNormal(loc, covariance_matrix=ours.covariance_matrix)
    _tclose(ours.log_prob(x), dense.log_prob(x), 1e-4)
    Wg = W.clone().requires_grad_()
    s = FD.LowRankMultivariateNormal(loc, Wg, d).rsample((30000,))
    s.pow(2).mean().backward()
    assert Wg.grad is not None and s.shape == (30000, 2, 6)
    emp = torch.einsum("nbi,nbj->bij", s.detach() - loc, s.detach() - loc) / 30000
    assert (emp - ours.covariance_matrix).abs().max() < 0.15
    with pytest.raises(ValueError):
        FD.LowRankMultivariateNormal(loc, torch.randn(2, 5, 2), d)


def _params(name):
    g = torch.Generator().manual_seed(11)
    pos = lambda: torch.rand(4, dtype=torch.float64, generator=g) * 2 + 0.3
    real = lambda: torch.randn(4, dtype=torch.float64, generator=g)
    return {"LogNormal": (real(), pos()), "Laplace": (real(), pos()), "Gumbel": (real(), pos()), "HalfNormal": (pos(),), "Weibull": (pos(), pos()),
            "Pareto": (pos(), pos()), "Kumaraswamy": (pos(), pos()), "Normal": (real(), pos()), "Uniform": (real() - 3, real().abs() + 1),
            "Gamma": (pos(), pos()), "Exponential": (pos(),), "Cauchy": (real(), pos()), "Beta": (pos(), pos())}[name]


@pytest.mark.parametrize("name", ["LogNormal", "Laplace", "Gumbel", "HalfNormal", "Weibull", "Pareto", "Kumaraswamy"])
def test_quantile_functions_invert_the_cdf_and_match_torch(name):
    import ferrotorch_b200.distributions as D
    args = _params(name)
    mine, ref = getattr(D, name)(*args), getattr(torch.distributions, name)(*args)
    p = torch.rand(6, 4, dtype=torch.float64, generator=torch.Generator().manual_seed(2)) * 0.96 + 0.02
    x = mine.icdf(p)
    torch.testing.assert_close(mine.cdf(x), p, rtol=1e-9, atol=1e-9)
    try:
        want = ref.icdf(p)
    except NotImplementedError:
        return
    torch.testing.assert_close(x, want, rtol=1e-9, atol=1e-9)


@pytest.mark.parametrize("pn,qn", [("Uniform", "Normal"), ("Gamma", "Exponential"), ("Exponential", "Gamma"), ("HalfNormal", "HalfNormal"),
                                   ("LogNormal", "LogNormal"), ("Cauchy", "Cauchy"), ("Pareto", "Pareto"), ("Normal", "Laplace"), ("Beta", "Normal")])
def test_more_closed_form_kl_pairs_match_torch(pn, qn):
    import ferrotorch_b200.distributions as D
    a, b = _params(pn), tuple(t * 1.1 + 0.05 for t in _params(qn))
    if pn == qn == "Pareto":
        b = (a[0] * 0.6, b[1])                                  # q's support must contain p's for a finite value
    got = D.kl_divergence(getattr(D, pn)(*a), getattr(D, qn)(*b))
    want = torch.distributions.kl_divergence(getattr(torch.distributions, pn)(*a), getattr(torch.distributions, qn)(*b))
    assert torch.isfinite(want).all()
    torch.testing.assert_close(got, want, rtol=1e-8, atol=1e-9)


def test_kl_is_infinite_where_the_support_is_not_covered():
    import ferrotorch_b200.distributions as D
    one = torch.ones(2, dtype=torch.float64)
    assert torch.isinf(D.kl_divergence(D.Normal(0 * one, one), D.Uniform(-one, one))).all()
    assert torch.isinf(D.kl_divergence(D.Pareto(one, one), D.Pareto(2 * one, one))).all()
