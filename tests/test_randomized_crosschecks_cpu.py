"""Randomised cross-checks with fixed seeds: random elementwise programs through the tracing compiler against eager execution, random
graphs through the native autograd core against PyTorch autograd, random contraction strings through the own einsum against
``torch.einsum``, and random schemas and documents through the JSON grammar (Python matcher against the native vocabulary walk)."""
import json
import random

import numpy as np
import pytest
import torch

from ferrotorch_b200 import jit
from ferrotorch_b200 import native as N
from ferrotorch_b200.core import einsum_impl
from ferrotorch_b200.grammar import JsonGrammar, JsonSchemaProcessor, Schema

_UNARY = [torch.sigmoid, torch.tanh, torch.relu, torch.exp, torch.abs, torch.neg, lambda t: t * 0.5, lambda t: t + 1.0, torch.sin, torch.cos,
          lambda t: torch.log(t.abs() + 1.0), lambda t: torch.clamp(t, -0.5, 0.5), lambda t: t * t, torch.nn.functional.gelu, torch.nn.functional.silu,
          lambda t: torch.where(t > 0, t, t * 0.1), torch.erf, lambda t: 1.0 / (t.abs() + 1.0)]
_BINARY = [torch.add, torch.sub, torch.mul, lambda a, b: a / (b.abs() + 1.0), torch.maximum, torch.minimum]
_SHAPES = [((64, 33),) * 3, ((16, 8, 5), (8, 5), (5,)), ((7, 1), (1, 9), (7, 9)), ((1000,), (1000,), (1,))]


@pytest.mark.parametrize("seed", range(8))
def test_random_elementwise_programs_compile_to_the_eager_result(seed):
    rng = random.Random(seed)
    prog = [(rng.random() < 0.5, rng.randrange(len(_UNARY)), rng.randrange(len(_BINARY)), rng.randrange(3), rng.randrange(3)) for _ in range(rng.randint(2, 10))]
    red = rng.choice([None, None, "sum", "mean"])

    def f(x, y, z):
        vals = [x, y, z]
        for is_unary, ui, bi, a, b in prog:
            vals.append(_UNARY[ui](vals[a]) if is_unary else _BINARY[bi](vals[a], vals[b]))
        out = vals[-1]
        return out.sum(-1) if red == "sum" else out.mean(-1) if red == "mean" else out

    g = torch.Generator().manual_seed(seed)
    shapes = rng.choice(_SHAPES)
    xs = [torch.randn(s, generator=g) for s in shapes]
    compiled = jit.compile(f, example_inputs=xs)
    torch.testing.assert_close(compiled(*xs), f(*xs), rtol=1e-4, atol=1e-4, equal_nan=True)
    ys = [torch.randn(s, generator=g) for s in shapes]
    torch.testing.assert_close(compiled(*ys), f(*ys), rtol=1e-4, atol=1e-4, equal_nan=True)
    assert compiled.stats.traces == 1


_NATIVE_UNARY = {"exp": torch.exp, "tanh": torch.tanh, "sigmoid": torch.sigmoid, "relu": torch.relu, "gelu": torch.nn.functional.gelu, "silu": torch.nn.functional.silu,
                 "abs": torch.abs, "sqrt": torch.sqrt, "log": torch.log, "reciprocal": torch.reciprocal}


@pytest.mark.parametrize("seed", range(12))
def test_random_graphs_differentiate_like_pytorch(seed):
    rng = random.Random(100 + seed)
    g = torch.Generator().manual_seed(seed)
    a, b, w = torch.rand(6, 5, generator=g) + 0.5, torch.rand(5, generator=g) + 0.5, torch.rand(5, 4, generator=g) + 0.1
    ta, tb, tw = [t.clone().requires_grad_(True) for t in (a, b, w)]
    na, nb, nw = [N.Tensor(t.numpy().copy(), requires_grad=True) for t in (a, b, w)]
    tv, nv = [ta, tb], [na, nb]
    for _ in range(rng.randint(1, 6)):
        kind, i, j = rng.randrange(4), rng.randrange(len(tv)), rng.randrange(len(tv))
        if kind == 0:
            name = rng.choice(sorted(_NATIVE_UNARY))
            tv.append(_NATIVE_UNARY[name](tv[i])); nv.append(getattr(nv[i], name)())
        elif kind == 1:
            tv.append(tv[i] + tv[j]); nv.append(nv[i] + nv[j])
        elif kind == 2:
            tv.append(tv[i] * tv[j]); nv.append(nv[i] * nv[j])
        else:
            tv.append(tv[i] / tv[j]); nv.append(nv[i] / nv[j])
    to, no = tv[-1], nv[-1]
    if to.dim() == 2:
        to, no = (to @ tw).softmax(-1), (no @ nw).softmax(-1)
        to, no = (to * to).sum(), (no * no).sum()
    else:
        to, no = to.sum(), no.sum()
    assert no.item() == pytest.approx(to.item(), rel=1e-4, abs=1e-5)
    to.backward(); no.backward()
    for t, n in ((ta, na), (tb, nb), (tw, nw)):
        want = t.grad.numpy() if t.grad is not None else np.zeros(t.shape, np.float32)
        got = n.grad.numpy() if n.grad is not None else np.zeros(t.shape, np.float32)
        np.testing.assert_allclose(got, want, rtol=1e-3, atol=1e-4)


def test_random_contraction_strings_match_torch_einsum():
    rng = random.Random(3)
    letters = "abcdefg"
    sizes = {c: rng.randint(1, 4) for c in letters}
    g = torch.Generator().manual_seed(3)
    checked = 0
    for _ in range(200):
        subs = ["".join(rng.choice(letters) for _ in range(rng.randint(0, 4))) for _ in range(rng.randint(1, 3))]
        eq = ",".join(subs)
        if rng.random() > 0.3:
            out = [c for c in sorted(set("".join(subs))) if rng.random() < 0.5]
            rng.shuffle(out)
            eq += "->" + "".join(out)
        ops = [torch.randn([sizes[c] for c in s], dtype=torch.float64, generator=g) for s in subs]
        try:
            want = torch.einsum(eq, *ops)
        except Exception:
            continue
        torch.testing.assert_close(einsum_impl.einsum(eq, *ops), want, rtol=1e-9, atol=1e-9)
        checked += 1
    assert checked > 100


def _random_schema(rng, depth=0):
    kinds = ["string", "number", "integer", "boolean", "null", "enum", "object", "array", "nullable"] if depth < 3 else ["string", "integer", "boolean", "enum"]
    k = rng.choice(kinds)
    if k == "enum":
        return {"enum": rng.sample(["a", "b c", 1, 2.5, True, None, 'q"x', "é"], rng.randint(1, 4))}
    if k == "object":
        props = {f"k{i}": _random_schema(rng, depth + 1) for i in range(rng.randint(0, 3))}
        return {"type": "object", "properties": props, "required": [p for p in props if rng.random() < 0.6]}
    if k == "array":
        return {"type": "array", "items": _random_schema(rng, depth + 1)}
    if k == "nullable":
        return {"type": [rng.choice(["string", "integer", "boolean", "number"]), "null"]}
    return {"type": k}


def _random_value(rng, s):
    if "enum" in s:
        return rng.choice(s["enum"])
    t = s["type"]
    if isinstance(t, list):
        return None if rng.random() < 0.4 else _random_value(rng, {"type": t[0]})
    if t == "array":
        return [_random_value(rng, s["items"]) for _ in range(rng.randint(0, 3))]
    if t == "object":
        return {k: _random_value(rng, v) for k, v in s["properties"].items() if k in s["required"] or rng.random() < 0.5}
    return {"string": rng.choice(["", "x", 'he said "hi"\n', "tab\t\\", "é✓", "a b"]), "number": rng.choice([0, -1.5, 3.25e10, 1e-5, 12]),
            "integer": rng.choice([0, -7, 123456]), "boolean": rng.random() < 0.5, "null": None}[t]


_VOCAB = [chr(c) for c in range(32, 127)] + ['":', '",', '{"', "true", "false", "null", '"}', "]}", "k0", 'k1"', '\\"', "\\n", "é", "✓", "12", ".5", "e1", '": "',
                                              '", "', "tru", "nul", "[]", "{}", "[["]


def test_random_schemas_accept_their_documents_and_both_mask_engines_agree():
    rng = random.Random(5)
    for _ in range(80):
        schema = _random_schema(rng)
        grammar = JsonGrammar(Schema.from_json(schema))
        value = _random_value(rng, schema)
        for ensure_ascii in (False, True):
            doc = json.dumps(value, separators=(",", ":"), ensure_ascii=ensure_ascii)
            assert grammar.is_complete(doc), (schema, doc)
            assert all(grammar.accepts_prefix(doc[:i]) for i in range(len(doc) + 1)), (schema, doc)
        assert grammar.is_complete(json.dumps(value)), (schema, value)          # ", " and ": " separators
        proc = JsonSchemaProcessor(schema, _VOCAB)
        if proc._native is None:
            continue
        doc = json.dumps(value, separators=(",", ":"), ensure_ascii=False)
        for cut in sorted({0, len(doc) // 3, len(doc) // 2, max(0, len(doc) - 1), len(doc)}):
            proc.text = doc[:cut]
            assert torch.equal(proc.mask().allowed, proc._mask_py().allowed), (schema, doc[:cut])


def test_gradients_flow_through_generated_kernels_and_into_module_parameters():
    """A compiled function differentiates like the eager one although its fused region runs as a generated kernel, and a compiled module
    trains: its parameters receive gradients and the optimiser's in-place updates are seen by the next call."""
    import torch.nn.functional as F
    g = torch.Generator().manual_seed(0)
    f = lambda x, w1, b1, w2: (F.gelu(x @ w1 + b1) * torch.sigmoid(x @ w1) @ w2).pow(2).mean()      # noqa: E731
    xs = [torch.randn(8, 16, generator=g), torch.randn(16, 32, generator=g), torch.randn(32, generator=g), torch.randn(32, 4, generator=g)]
    a = [t.clone().requires_grad_(True) for t in xs]
    b = [t.clone().requires_grad_(True) for t in xs]
    compiled = jit.compile(f, example_inputs=a)
    out, ref = compiled(*a), f(*b)
    assert compiled.stats.fused_kernels >= 1 and compiled.stats.kernel_launches >= 1
    out.backward(); ref.backward()
    for p, q in zip(a, b):
        torch.testing.assert_close(p.grad, q.grad, rtol=1e-4, atol=1e-5)

    torch.manual_seed(0)
    mine = torch.nn.Sequential(torch.nn.Linear(4, 8), torch.nn.GELU(), torch.nn.Linear(8, 1))
    eager = torch.nn.Sequential(torch.nn.Linear(4, 8), torch.nn.GELU(), torch.nn.Linear(8, 1))
    eager.load_state_dict(mine.state_dict())
    cm = jit.compile(mine, example_inputs=[torch.randn(5, 4)])
    o1, o2 = torch.optim.SGD(mine.parameters(), lr=0.1), torch.optim.SGD(eager.parameters(), lr=0.1)
    x, y = torch.randn(32, 4, generator=g), torch.randn(32, 1, generator=g)
    for _ in range(10):
        o1.zero_grad(); l1 = ((cm(x) - y) ** 2).mean(); l1.backward(); o1.step()
        o2.zero_grad(); l2 = ((eager(x) - y) ** 2).mean(); l2.backward(); o2.step()
    assert all(p.grad is not None for p in mine.parameters())
    torch.testing.assert_close(l1, l2, rtol=1e-5, atol=1e-6)
    with torch.no_grad():
        torch.testing.assert_close(cm(x), eager(x), rtol=1e-5, atol=1e-6)


def test_functions_that_write_in_place_run_as_written():
    """Writes into a copy, through a view, into an intermediate and into an input: the compiled callable returns what the function returns
    and leaves (or changes) the caller's tensors exactly as the function does, once per call."""
    def into_copy(x):
        y = x.clone(); y.add_(1.0); y.mul_(2.0)
        return y

    def through_view(x):
        y = x.clone(); y[:, 0] = 0.0
        return y

    def into_intermediate(x):
        y = x + 0.5
        return y.relu_()

    def into_input(x):
        x.add_(1.0)
        return x * 2

    for fn in (into_copy, through_view, into_intermediate, into_input):
        compiled = jit.compile(fn, example_inputs=[torch.randn(3, 4)])
        x = torch.randn(3, 4, generator=torch.Generator().manual_seed(1))
        mine, theirs = x.clone(), x.clone()
        for _ in range(2):
            torch.testing.assert_close(compiled(mine), fn(theirs))
            torch.testing.assert_close(mine, theirs)
        assert compiled.stats.graph_breaks >= 1 and compiled.graph_for(x).mutations


def test_tracing_leaves_module_state_untouched_and_batch_norm_trains_like_eager():
    torch.manual_seed(0)
    mine, eager = torch.nn.BatchNorm1d(4), torch.nn.BatchNorm1d(4)
    compiled = jit.compile(mine, example_inputs=[torch.randn(8, 4)])
    assert int(mine.num_batches_tracked) == 0 and float(mine.running_mean.abs().sum()) == 0.0
    for _ in range(3):
        x = torch.randn(8, 4)
        torch.testing.assert_close(compiled(x), eager(x))
    assert int(mine.num_batches_tracked) == int(eager.num_batches_tracked) == 3
    torch.testing.assert_close(mine.running_mean, eager.running_mean)
    torch.testing.assert_close(mine.running_var, eager.running_var)
    with pytest.raises(Exception, match="take tensors"):
        jit.compile(lambda x, s: x * s, example_inputs=[torch.ones(3), 2.5])
