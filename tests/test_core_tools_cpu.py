"""CPU checks of the core tensor extensions, autograd utilities, distributions, profiler, ml, tokenizer, grammar, hub cache and vision data."""
import json
import math

import numpy as np
import pytest
import torch


def test_autograd_utilities_and_vmap():
    from ferrotorch_b200 import core as C
    x = torch.tensor([0.5, -1.2, 2.0], dtype=torch.float64)
    f = lambda t: (t.sin() * t.exp()).sum()                        # noqa: E731
    J = C.jacobian(lambda t: t.sin() * t, x)
    assert torch.allclose(J, torch.diag(x.cos() * x + x.sin()))
    H = C.hessian(f, x)
    assert torch.allclose(H, torch.diag((2 * x.cos() * x.exp())), atol=1e-9)
    v = torch.ones_like(x)
    out, tangent = C.jvp(lambda t: t.sin(), x, v)
    assert torch.allclose(tangent, x.cos())
    out2, tang2 = C.jvp_exact(lambda t: t.sin(), x, v)
    assert torch.allclose(tang2, x.cos()) and torch.allclose(C.jacfwd(lambda t: t.exp(), x), torch.diag(x.exp()))
    d = C.dual_sin(C.DualTensor(x, v)) * C.dual_exp(C.DualTensor(x, v))
    assert torch.allclose(d.tangent, x.cos() * x.exp() + x.sin() * x.exp())
    _, cot = C.vjp(lambda t: t * t, x, v)
    assert torch.allclose(cot, 2 * x)
    assert C.gradcheck(lambda t: (t * t).sum(), [x.clone().requires_grad_()])
    batched = C.vmap(lambda r: r.dot(r))(torch.arange(6.0).view(2, 3))
    assert torch.allclose(batched, torch.tensor([5.0, 50.0]))
    m = torch.nn.Linear(3, 2)
    g = C.per_sample_grad(m, lambda o, y: ((o - y) ** 2).sum(), torch.randn(4, 3), torch.randn(4, 2))
    assert g["weight"].shape == (4, 2, 3)
    theta = torch.tensor([0.5], requires_grad=True)
    z = C.fixed_point(lambda z, th: torch.tanh(th * z + 1.0), torch.zeros(1), theta)
    z.sum().backward()
    assert abs(float(z) - math.tanh(0.5 * float(z) + 1.0)) < 1e-5 and theta.grad is not None and abs(float(theta.grad)) > 0
    assert C.has_inf_nan(torch.tensor([1.0, float("nan")])) and not C.has_inf_nan(torch.ones(3))
    with C.autocast(torch.bfloat16, device_type="cpu"):
        assert C.is_autocast_enabled()


def test_tensor_extensions():
    from ferrotorch_b200.core import tensor_ext as X
    a = torch.randn(5, 5, dtype=torch.float64)
    spd = a @ a.t() + 5 * torch.eye(5, dtype=torch.float64)
    L = X.linalg.cholesky(spd)
    assert torch.allclose(L @ L.t(), spd) and torch.allclose(X.linalg.inv(spd) @ spd, torch.eye(5, dtype=torch.float64), atol=1e-9)
    assert torch.allclose(X.linalg.det(spd), torch.linalg.det(spd)) and int(X.linalg.matrix_rank(spd)) == 5
    q, r = X.linalg.qr(a)
    assert torch.allclose(q @ r, a)
    assert torch.allclose(X.linalg.solve(spd, a), torch.linalg.solve(spd, a))
    sig = torch.randn(64)
    assert torch.allclose(X.fft.irfft(X.fft.rfft(sig), n=64), sig, atol=1e-5) and torch.allclose(X.fft.fftshift(X.fft.fftfreq(8)), torch.fft.fftshift(torch.fft.fftfreq(8)))
    xs = torch.linspace(-0.9, 0.9, 7)
    assert torch.allclose(X.special.erfinv(X.special.erf(xs)), xs, atol=1e-5)
    assert torch.allclose(X.special.chebyshev_polynomial_t(xs, 3), 4 * xs ** 3 - 3 * xs, atol=1e-6)
    assert torch.allclose(X.special.legendre_polynomial_p(xs, 2), 0.5 * (3 * xs ** 2 - 1), atol=1e-6)
    assert torch.allclose(X.windows.hann(16), torch.hann_window(16, periodic=False), atol=1e-6)
    assert torch.allclose(X.einsum("ij,jk->ik", a, a), a @ a)
    t = torch.arange(24.0).view(2, 3, 4)
    assert torch.equal(X.rearrange(t, "b h w -> b (h w)"), t.view(2, 12)) and X.repeat(t, "b h w -> b h w c", c=2).shape == (2, 3, 4, 2)
    assert torch.equal(X.reduce(t, "b h w -> b", "sum"), t.sum((1, 2)))
    dense = torch.tensor([[0.0, 2.0, 0.0], [3.0, 0.0, 4.0]])
    coo = X.CooTensor(torch.tensor([[0, 1, 1], [1, 0, 2]]), torch.tensor([2.0, 3.0, 4.0]), (2, 3))
    assert torch.equal(coo.to_dense(), dense)
    nt = X.NestedTensor([torch.ones(2, 3), torch.ones(4, 3)])
    assert len(nt.tensors) == 2
    mt = X.MaskedTensor(torch.tensor([1.0, 2.0, 3.0]), torch.tensor([True, False, True]))
    assert float(X.masked_sum(mt)) == 4.0 and float(X.masked_mean(mt)) == 2.0
    nm = X.NamedTensor(torch.zeros(2, 3), ["batch", "feat"])
    assert nm.names == ["batch", "feat"] or tuple(nm.names) == ("batch", "feat")
    w = torch.randn(16, 16)
    qt = X.quantize(w)
    assert (X.dequantize(qt) - w).abs().max() < w.abs().max() / 100
    pruned = X.magnitude_prune(w, 0.5)
    assert abs(X.sparsity_ratio(pruned) - 0.5) < 0.05
    m24, mask = X.apply_2_4_mask(w)
    assert torch.equal(mask.view(-1, 4).sum(1), torch.full((64,), 2, dtype=mask.view(-1, 4).sum(1).dtype))


def test_distributions_logprob_entropy_kl_and_transforms():
    from ferrotorch_b200 import distributions as D
    import torch.distributions as TD
    x = torch.tensor([0.3, 1.7])
    pairs = [(D.Normal(0.5, 2.0), TD.Normal(0.5, 2.0)), (D.Laplace(0.0, 1.5), TD.Laplace(0.0, 1.5)), (D.Gamma(2.0, 3.0), TD.Gamma(2.0, 3.0)),
             (D.Exponential(1.5), TD.Exponential(1.5)), (D.Gumbel(0.0, 1.0), TD.Gumbel(0.0, 1.0)), (D.StudentT(4.0), TD.StudentT(4.0)),
             (D.Weibull(1.2, 1.5), TD.Weibull(1.2, 1.5)), (D.LogNormal(0.0, 0.7), TD.LogNormal(0.0, 0.7))]
    for ours, ref in pairs:
        assert torch.allclose(ours.log_prob(x), ref.log_prob(x), atol=1e-5), type(ours).__name__
        assert torch.allclose(torch.as_tensor(ours.entropy()).float(), ref.entropy(), atol=1e-5), type(ours).__name__
    assert torch.allclose(D.kl_divergence(D.Normal(0.0, 1.0), D.Normal(1.0, 2.0)), TD.kl_divergence(TD.Normal(0.0, 1.0), TD.Normal(1.0, 2.0)))
    c = D.Categorical(logits=torch.tensor([0.1, 0.5, -0.3]))
    assert torch.allclose(c.log_prob(torch.tensor(1)), TD.Categorical(logits=torch.tensor([0.1, 0.5, -0.3])).log_prob(torch.tensor(1)))
    torch.manual_seed(0)
    s = D.Normal(torch.zeros(20000), torch.ones(20000)).rsample()
    assert abs(float(s.mean())) < 0.03 and abs(float(s.std()) - 1) < 0.03
    mvn = D.MultivariateNormal(torch.zeros(2), covariance_matrix=torch.tensor([[2.0, 0.3], [0.3, 1.0]]))
    ref = TD.MultivariateNormal(torch.zeros(2), covariance_matrix=torch.tensor([[2.0, 0.3], [0.3, 1.0]]))
    assert torch.allclose(mvn.log_prob(x), ref.log_prob(x), atol=1e-5)
    td = D.TransformedDistribution(D.Normal(0.0, 1.0), [D.ExpTransform()])
    assert torch.allclose(td.log_prob(x), TD.LogNormal(0.0, 1.0).log_prob(x), atol=1e-5)


def test_profiler_ml_tokenizer_grammar_hub_vision_data(tmp_path):
    from ferrotorch_b200 import grammar, hub, ml, profiler, tokenize
    from ferrotorch_b200.core import profile_op_scope
    from ferrotorch_b200.vision import data as VD

    def work():
        return profile_op_scope("matmul", "linalg", [(64, 64), (64, 64)], lambda: torch.randn(64, 64) @ torch.randn(64, 64))
    out, rep = profiler.with_profiler(profiler.ProfileConfig(), work)
    assert out.shape == (64, 64) and any(s.name == "matmul" for s in rep.summaries()) and "matmul" in rep.table()
    trace = json.loads(rep.chrome_trace_json())
    assert "traceEvents" in trace and rep.total_flops() >= 2 * 64 ** 3
    X, y = ml.make_classification(200, 10, 3, 2, seed=1)
    Xtr, Xte, ytr, yte = ml.train_test_split(X, y, test_size=0.25, seed=0)
    assert Xtr.shape == (150, 10) and ml.accuracy_score(yte, yte) == 1.0 and ml.confusion_matrix([0, 1, 1], [0, 1, 0]).tolist() == [[1, 0], [1, 1]]
    assert abs(ml.r2_score([1.0, 2.0, 3.0], [1.0, 2.0, 3.0]) - 1.0) < 1e-12 and torch.equal(ml.ndarray_to_tensor(np.ones((2, 2), np.float32)), torch.ones(2, 2))
    vocab = {c: i for i, c in enumerate(["h", "e", "l", "o", "he", "ll", "hell", "hello", "Ġ", "w", "r", "d", "<s>"])}
    tok = tokenize.Tokenizer(vocab, [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o")], bos_token="<s>")
    ids = tokenize.encode(tok, "hello")
    assert ids == [vocab["hello"]] and tokenize.decode(tok, ids) == "hello"
    assert "<|start_header_id|>user<|end_header_id|>" in tokenize.apply_chat_template([{"role": "user", "content": "hi"}])
    schema = grammar.Schema.from_json({"type": "object", "properties": {"a": {"type": "integer"}}, "required": ["a"]})
    g = grammar.JsonGrammar(schema)
    assert g.accepts_prefix('{"a": 1') and g.is_complete('{"a": 12}') and not g.accepts_prefix('{"b"')
    texts = ['{', '"a"', ':', ' ', '1', '2', '}', '"b"', 'x']
    proc = grammar.JsonSchemaProcessor(schema, texts, eos_id=None)
    m0 = proc.mask()
    assert bool(m0.allowed[0]) and not bool(m0.allowed[8]) and not bool(m0.allowed[7])
    logits = grammar.apply_mask(torch.zeros(len(texts)), m0)
    assert logits[0] == 0 and logits[8] == float("-inf")
    cache = hub.HubCache(tmp_path / "hub")
    assert cache.root.exists() or True
    assert isinstance(hub.list_models(), list) and len(hub.list_models()) > 0
    ds = VD.Mnist.synthetic(32) if hasattr(VD.Mnist, "synthetic") else None
    if ds is not None:
        img, lab = ds[0]
        assert img.shape[-2:] == (28, 28)
    tf = VD.Compose([VD.Resize(16), VD.CenterCrop(12), VD.RandomHorizontalFlip(0.5), VD.VisionNormalize([0.5] * 3, [0.5] * 3)])
    assert tf(torch.rand(3, 32, 32)).shape == (3, 12, 12)
    p = tmp_path / "im.ppm"
    VD.write_image(str(p), (torch.rand(3, 8, 9) * 255).to(torch.uint8))
    assert VD.read_image(str(p)).shape == (3, 8, 9)


def test_control_flow_search_wrappers_pool_meta_display_fusion():
    from ferrotorch_b200 import core as C
    x = torch.arange(1.0, 5.0, requires_grad=True)
    carry, ys = C.scan(lambda c, xt: (c * xt, c * xt), torch.tensor(1.0), x)
    ys[-1].backward()
    assert float(carry) == 24.0 and torch.allclose(x.grad, 24.0 / x.detach())
    _, rev = C.scan(lambda c, xt: (c + xt, c + xt), torch.tensor(0.0), x.detach(), reverse=True)
    assert rev.tolist() == [10.0, 9.0, 7.0, 4.0]
    assert C.cond(False, lambda a: a + 1, lambda a: a - 1, (torch.zeros(1),)).item() == -1
    assert C.meta_propagate(lambda a, b: (a @ b).sum(0), ((4, 8), torch.float32), ((8, 3), torch.float32)) == [((3,), torch.float32)]
    assert C.format_tensor(torch.tensor([1.5, 2.0])) == "tensor([1.5000, 2.0000], shape=[2], dtype=float32, device=cpu)"
    assert "..." in C.format_tensor(torch.zeros(5000))
    pool = C.CpuBufferPool()
    t = pool.take(100)
    pool.give(t)
    assert pool.take(120).shape == (120,) and pool.stats()["hits"] == 1
    f = C.fused(lambda a, b: torch.tanh(a) * b + 1)
    a, b = torch.randn(4, 8), torch.randn(4, 8)
    with C.with_fusion():
        assert C.fusion_enabled() and torch.allclose(f(a, b), torch.tanh(a) * b + 1, atol=1e-6)
    assert not C.fusion_enabled()
    assert (C.IntTensor([1, 2, 3]) * 2 == C.IntTensor([2, 4, 7])).data.tolist() == [True, True, False]
    with pytest.raises(Exception):
        C.IntTensor([1.5])
    assert (C.BoolTensor([1, 0, 1]) & ~C.BoolTensor([1, 1, 0])).data.tolist() == [False, False, True]
    assert C.searchsorted(torch.tensor([1.0, 3.0, 5.0]), torch.tensor([2.0, 5.0])).tolist() == [1, 2]
    assert C.from_vec([1, 2, 3, 4], (2, 2)).shape == (2, 2)
    with pytest.raises(Exception):
        C.from_vec([1, 2, 3], (2, 2))


def test_tokenizer_matches_hf_tokenizers_on_a_trained_byte_level_bpe(tmp_path):
    """A byte-level BPE trained with the HF ``tokenizers`` library on this package's own sources, saved as ``tokenizer.json`` and read back by
    ``tokenize.load_tokenizer``: identical ids (code, unicode, runs of whitespace, special tokens) and identical round trips."""
    import glob
    from pathlib import Path
    tk = pytest.importorskip("tokenizers")
    from tokenizers import decoders, models, pre_tokenizers, trainers
    from ferrotorch_b200 import tokenize
    root = Path(__file__).resolve().parents[1] / "ferrotorch_b200"
    files = sorted(glob.glob(str(root / "**" / "*.py"), recursive=True))[:25]
    hf = tk.Tokenizer(models.BPE())
    hf.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    hf.decoder = decoders.ByteLevel()
    hf.train(files, trainers.BpeTrainer(vocab_size=1200, special_tokens=["<|begin|>", "<|end|>"], initial_alphabet=pre_tokenizers.ByteLevel.alphabet(),
                                        show_progress=False))
    path = tmp_path / "tokenizer.json"
    hf.save(str(path))
    ours = tokenize.load_tokenizer(path)
    texts = ["hello world", "def f(x):\n    return x + 1  # comment", "naïve café — ünïcödé ✓ 你好", "  multiple   spaces\tand\ttabs\n\nnewlines",
             "<|begin|>special<|end|> tokens", "12345 67890 3.14159", Path(files[3]).read_text()[:4000]]
    for t in texts:
        a, b = ours.encode(t), hf.encode(t).ids
        assert a == b, t[:40]
        assert ours.decode(a, skip_special_tokens=False) == hf.decode(b, skip_special_tokens=False)


def test_ml_metrics_match_scikit_learn():
    """The metric functions of the sklearn-style adapter against scikit-learn itself on random multi-class and binary problems."""
    skm = pytest.importorskip("sklearn.metrics")
    import numpy as np
    from ferrotorch_b200 import ml
    rng = np.random.default_rng(0)
    y, p = rng.integers(0, 4, 500), rng.integers(0, 4, 500)
    assert abs(ml.accuracy_score(y, p) - skm.accuracy_score(y, p)) < 1e-12
    assert np.array_equal(ml.confusion_matrix(y, p), skm.confusion_matrix(y, p))
    for avg in ("macro", "micro", "weighted"):
        assert abs(ml.precision_score(y, p, average=avg) - skm.precision_score(y, p, average=avg, zero_division=0)) < 1e-9, avg
        assert abs(ml.recall_score(y, p, average=avg) - skm.recall_score(y, p, average=avg, zero_division=0)) < 1e-9, avg
        assert abs(ml.f1_score(y, p, average=avg) - skm.f1_score(y, p, average=avg, zero_division=0)) < 1e-9, avg
    yb, s = rng.integers(0, 2, 400), rng.random(400)
    s[:200:2] = s[1:200:2]                                              # some tied scores
    assert abs(ml.roc_auc_score(yb, s) - skm.roc_auc_score(yb, s)) < 1e-9
    proba = rng.dirichlet(np.ones(4), 500)
    assert abs(ml.log_loss(y, proba) - skm.log_loss(y, proba, labels=[0, 1, 2, 3])) < 1e-9
    t, q = rng.standard_normal(300), rng.standard_normal(300)
    assert abs(ml.r2_score(t, q) - skm.r2_score(t, q)) < 1e-9 and abs(ml.mean_squared_error(t, q) - skm.mean_squared_error(t, q)) < 1e-12
    assert abs(ml.mean_absolute_error(t, q) - skm.mean_absolute_error(t, q)) < 1e-12


def test_json_grammar_agrees_with_the_jsonschema_validator():
    """Random documents, valid and broken in five ways, serialised with both separator styles: the incremental grammar accepts exactly those
    the ``jsonschema`` validator accepts, and every prefix of an accepted document is an accepted prefix."""
    import json
    import random
    jsonschema = pytest.importorskip("jsonschema")
    from ferrotorch_b200 import grammar as G
    schema = {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"}, "tags": {"type": "array", "items": {"type": "string"}},
                                               "ok": {"type": "boolean"}, "score": {"type": "number"}, "kind": {"enum": ["a", "b"]},
                                               "inner": {"type": "object", "properties": {"x": {"type": "number"}}, "required": ["x"]}},
              "required": ["name", "age"]}
    g = G.JsonGrammar(G.Schema.from_json(schema))
    rnd = random.Random(0)

    def instance(valid):
        d = {"name": rnd.choice(["bob", "ali ce", 'é"q' + chr(92)]), "age": rnd.randint(-5, 99)}
        if rnd.random() < .5:
            d["tags"] = [rnd.choice(["x", "y z"]) for _ in range(rnd.randint(0, 3))]
        if rnd.random() < .5:
            d["ok"] = rnd.random() < .5
        if rnd.random() < .5:
            d["score"] = rnd.choice([1.5, -2e-3, 7, 0.0])
        if rnd.random() < .5:
            d["kind"] = rnd.choice(["a", "b"])
        if rnd.random() < .5:
            d["inner"] = {"x": rnd.random()}
        if not valid:
            k = rnd.choice(["age_str", "missing", "bad_enum", "bad_item", "inner_missing"])
            if k == "age_str":
                d["age"] = "12"
            elif k == "missing":
                d.pop("name")
            elif k == "bad_enum":
                d["kind"] = "c"
            elif k == "bad_item":
                d["tags"] = [1]
            else:
                d["inner"] = {}
        return d
    for i in range(300):
        inst = instance(i % 2 == 0)
        text = json.dumps(inst, ensure_ascii=False) if i % 4 < 2 else json.dumps(inst, separators=(",", ":"))
        try:
            jsonschema.validate(inst, schema)
            ok = True
        except jsonschema.ValidationError:
            ok = False
        assert g.is_complete(text) == ok, text
        if ok:
            assert all(g.accepts_prefix(text[:k]) for k in range(0, len(text) + 1, 3)), text


def test_resize_and_center_crop_follow_the_reference_rules():
    """Resize defaults to nearest neighbour with source index floor(dst * in / out); CenterCrop floors its offsets and refuses a crop larger
    than the image (ferrotorch-vision/src/transforms/resize.rs:44-52, center_crop.rs:43-53)."""
    from ferrotorch_b200.errors import InvalidArgument
    from ferrotorch_b200.vision import data as VD
    x = torch.arange(3 * 5 * 7.0).view(3, 5, 7)
    want = torch.stack([torch.stack([x[c, (oh * 5) // 3, [(ow * 7) // 4 for ow in range(4)]] for oh in range(3)]) for c in range(3)])
    assert torch.equal(VD.Resize((3, 4))(x), want)
    assert VD.Resize((3, 4), mode="bilinear")(x).shape == (3, 3, 4)
    assert torch.equal(VD.CenterCrop((2, 4))(x), x[:, 1:3, 1:5])
    with pytest.raises(InvalidArgument):
        VD.CenterCrop(9)(x)


def test_vision_rng_choice_and_to_tensor():
    """The augmentation stream is a splitmix64 counter keyed by (seed, draw) with default seed 42 (ferrotorch-vision/src/transforms/rng.rs:17-47);
    RandomChoice applies exactly one transform; VisionToTensor transposes [H, W, C] and always divides by 255 (to_tensor.rs:24-57)."""
    from ferrotorch_b200.errors import InvalidArgument
    from ferrotorch_b200 import vision as V
    from ferrotorch_b200.vision import data as VD

    def splitmix(seed, n):                                   # the published splitmix64 finaliser, written out independently
        m = (1 << 64) - 1
        z = (seed + n * 0x9E3779B97F4A7C15) & m
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        return (z ^ (z >> 31)) / float(m)

    V.vision_manual_seed(7)
    a = [VD._vision_rng.random() for _ in range(5)]
    assert a == [splitmix(7, n) for n in range(5)] and all(0.0 <= v <= 1.0 for v in a)
    V.vision_manual_seed(7)
    assert [VD._vision_rng.random() for _ in range(5)] == a
    V.vision_manual_seed(8)
    assert [VD._vision_rng.random() for _ in range(5)] != a
    assert all(0 <= VD._vision_rng.randint(3) < 3 for _ in range(50))

    x = torch.rand(3, 16, 16)
    aug = V.Compose([V.RandomCrop(8), V.RandomHorizontalFlip(), V.ColorJitter(0.3, 0.3, 0.3), V.GaussianNoise(0.1)])
    V.vision_manual_seed(3)
    y1 = aug(x)
    torch.manual_seed(999)                                  # the tensor RNG does not feed the augmentations
    V.vision_manual_seed(3)
    assert torch.equal(aug(x), y1)

    with pytest.raises(InvalidArgument):
        V.RandomChoice([])
    hits = [0, 0, 0]
    rc = V.RandomChoice([lambda t, i=i: (hits.__setitem__(i, hits[i] + 1), t + i)[1] for i in range(3)])
    V.vision_manual_seed(0)
    outs = [float(rc(torch.zeros(1))) for _ in range(300)]
    assert sum(hits) == 300 and min(hits) > 60 and set(outs) == {0.0, 1.0, 2.0}
    V.vision_manual_seed(0)
    want = [min(int(splitmix(0, n) * 3), 2) for n in range(300)]
    assert [int(o) for o in outs] == want

    img = torch.arange(4 * 5 * 3.0).view(4, 5, 3)
    t = V.VisionToTensor()(img)
    assert t.shape == (3, 4, 5) and torch.allclose(t, img.permute(2, 0, 1) / 255)
    assert V.VisionToTensor()(np.full((2, 2, 3), 255, np.uint8)).max() == 1.0
    with pytest.raises(InvalidArgument):
        V.VisionToTensor()(torch.zeros(4, 5))


def test_distribution_constraints_and_transformed_entropy():
    """Constraint objects follow ferrotorch-distributions/src/constraints.rs (NaN satisfies nothing, Real accepts infinities, Simplex is
    per-element with event_dim 1); TransformedDistribution.entropy uses H(Y) = H(X) + E[log|det J|] for affine and exponential maps."""
    import math
    from ferrotorch_b200 import distributions as D
    from ferrotorch_b200.errors import FerrotorchError, InvalidArgument
    C = D.constraints
    assert C.positive().check(1.0) and not C.positive().check(-1.0) and not C.positive().check(0.0) and C.nonnegative().check(0.0)
    assert C.real().check(float("inf")) and not C.real().check(float("nan")) and not C.unit_interval().check(1.5) and C.unit_interval().check(1.0)
    assert C.boolean().check(1.0) and not C.boolean().check(0.5) and C.boolean().is_discrete() and C.boolean().name() == "Boolean"
    assert C.greater_than(2.0).check(2.1) and not C.greater_than(2.0).check(2.0) and C.greater_than_eq(2.0).check(2.0) and C.less_than(0.0).check(-1.0)
    assert not C.open_interval(0.0, 1.0).check(0.0) and C.closed_interval(0.0, 1.0).check(0.0) and C.half_open_interval(0.0, 1.0).check(0.0) and not C.half_open_interval(0.0, 1.0).check(1.0)
    t = torch.tensor([0.2, float("nan"), -0.1, 0.9])
    assert C.unit_interval().check(t).tolist() == [True, False, False, True] and C.positive().event_dim() == 0 and C.simplex().event_dim() == 1
    assert C.simplex().check(torch.tensor([0.3, 0.7])).all() and C.simplex().check_event(torch.tensor([[0.3, 0.7], [0.5, 0.6]])).tolist() == [True, False]
    assert isinstance(C.positive(), D.Constraint) and repr(C.open_interval(0.0, 2.0)) == "OpenInterval(lower_bound=0.0, upper_bound=2.0)"
    with pytest.raises(InvalidArgument):
        C.closed_interval(2.0, 1.0)
    T = D.transforms
    x = torch.linspace(-3, 3, 7)
    sp = D.SoftplusTransform()
    assert torch.allclose(sp(x), torch.nn.functional.softplus(x)) and torch.allclose(sp.inv(sp(x)), x, atol=1e-5)
    assert torch.allclose(sp.log_abs_det_jacobian(x, sp(x)), -torch.nn.functional.softplus(-x), atol=1e-6)
    assert T.transform_name(T.ExpTransform()) == "ExpTransform" and T.is_exp_transform(T.ExpTransform()) and not T.is_exp_transform(sp)
    assert float(T.constant_entropy_contribution(T.AffineTransform(1.0, -3.0))) == pytest.approx(math.log(3.0)) and T.constant_entropy_contribution(sp) is None
    base = D.Normal(torch.tensor(0.5), torch.tensor(0.8))
    aff = D.TransformedDistribution(base, [T.AffineTransform(2.0, 3.0)])
    assert float(aff.entropy()) == pytest.approx(float(D.Normal(torch.tensor(3.5), torch.tensor(2.4)).entropy()), rel=1e-6)
    logn = D.TransformedDistribution(base, [T.AffineTransform(1.0, 2.0), T.ExpTransform()])       # exp(2 X + 1) is LogNormal(2 * 0.5 + 1, 1.6)
    assert float(logn.entropy()) == pytest.approx(float(D.LogNormal(torch.tensor(2.0), torch.tensor(1.6)).entropy()), rel=1e-6)
    scaled = D.TransformedDistribution(base, [T.ComposeTransform([T.ExpTransform(), T.AffineTransform(0.0, 5.0)])])
    assert float(scaled.entropy()) == pytest.approx(float(D.LogNormal(torch.tensor(0.5), torch.tensor(0.8)).entropy()) + math.log(5.0), rel=1e-6)
    for bad in ([T.SigmoidTransform()], [T.ExpTransform(), T.ExpTransform()]):
        with pytest.raises(FerrotorchError):
            D.TransformedDistribution(base, bad).entropy()
    y = logn.rsample((4,))
    assert y.shape == (4,) and (y > 0).all() and torch.isfinite(logn.log_prob(y)).all()


def test_chat_templates_jinja_ids_and_config_loading(tmp_path):
    """Jinja chat templates render as transformers renders them; id helpers, template-to-ids and tokenizer_config loading follow
    ferrotorch-tokenize/src/lib.rs:143-400."""
    import json
    from ferrotorch_b200 import tokenize as T
    from ferrotorch_b200.errors import Internal, InvalidArgument
    tpl = ("{{ bos_token }}{% for m in messages %}{% if m['role'] not in ['system', 'user', 'assistant'] %}{{ raise_exception('bad role ' + m['role']) }}{% endif %}"
           "<|{{ m['role'] }}|>\\n{{ m['content'] | trim }}{{ eos_token }}\\n{% endfor %}{% if add_generation_prompt %}<|assistant|>\\n{% endif %}")
    msgs = [T.ChatMessage("system", "Be brief."), T.ChatMessage("user", "  Hi there  ")]
    got = T.apply_chat_template(msgs, tpl, True, "<s>", "</s>")
    assert got.startswith("<s><|system|>") and got.endswith("<|assistant|>\\n") and "Hi there</s>" in got
    hf = pytest.importorskip("transformers")
    from transformers.utils.chat_template_utils import render_jinja_template
    want = render_jinja_template(conversations=[[{"role": m.role, "content": m.content} for m in msgs]], chat_template=tpl, add_generation_prompt=True,
                                 bos_token="<s>", eos_token="</s>")[0][0]
    assert got == want
    assert T.apply_chat_template(tpl, msgs, False, "<s>", "</s>") == T.apply_chat_template(msgs, tpl, False, "<s>", "</s>") != got      # reference argument order
    with pytest.raises(InvalidArgument, match="bad role tool"):
        T.apply_chat_template([T.ChatMessage("tool", "x")], tpl)
    with pytest.raises(InvalidArgument):
        T.apply_chat_template(msgs, "{{ undefined_variable }}")
    with pytest.raises(InvalidArgument):
        T.apply_chat_template(msgs, "{% for %}")
    assert T.apply_chat_template([{"role": "user", "content": "q"}], "chatml") == "<|im_start|>user\nq<|im_end|>\n<|im_start|>assistant\n"

    vocab = {chr(0x120 + 0): 0}
    tok = T.Tokenizer({"a": 0, "b": 1, "ab": 2, "<|user|>": 3}, [("a", "b")], {"<s>": 4, "</s>": 5}, bos_token="<s>", eos_token="</s>")
    assert T.vocab_size(tok) == 6 and T.vocab_size(tok, with_added_tokens=False) == 4 and T.token_to_id(tok, "ab") == 2 and T.token_to_id(tok, "zz") is None
    assert T.id_to_token(tok, 5) == "</s>" and T.id_to_token(tok, 99) is None
    text, ids = T.apply_chat_template_to_ids(tok, "{{ bos_token }}{% for m in messages %}{{ m['content'] }}{% endfor %}{{ eos_token }}", [T.ChatMessage("user", "abab")])
    assert text == "<s>abab</s>" and ids == [4, 2, 2, 5]

    (tmp_path / "a.json").write_text(json.dumps({"chat_template": tpl}))
    (tmp_path / "b.json").write_text(json.dumps({"chat_template": [{"name": "default", "template": "X"}, {"name": "tool_use", "template": "Y"}]}))
    (tmp_path / "c.json").write_text(json.dumps({"model_max_length": 4}))
    (tmp_path / "d.json").write_text(json.dumps({"chat_template": 7}))
    (tmp_path / "e.json").write_text("{nope")
    assert T.load_chat_template(tmp_path / "a.json") == tpl and T.load_chat_template(tmp_path / "b.json") == "X" and T.load_chat_template(tmp_path / "c.json") is None
    for bad in ("d.json", "e.json"):
        with pytest.raises(InvalidArgument):
            T.load_chat_template(tmp_path / bad)
    with pytest.raises(Internal):
        T.load_chat_template(tmp_path / "missing.json")
    from ferrotorch_b200 import profiler as P, vision as V
    assert P.flops.estimate("matmul", [[4, 5], [5, 6]]) == 240 and P.estimate("my_custom_op", [[3, 4]]) is None
    feat, rois = torch.randn(1, 2, 8, 8), torch.tensor([[0.0, 1.0, 1.0, 5.0, 6.0]])
    assert torch.equal(V.roi_align_with_aligned(feat, rois, 2, 1.0, 2, False), V.roi_align(feat, rois, 2, 1.0, 2, False))
    assert not torch.equal(V.roi_align_with_aligned(feat, rois, 2, 1.0, 2, True), V.roi_align(feat, rois, 2, 1.0, 2, False))
