"""The native token-mask computation (``csrc/runtime/grammar.cpp``) against the Python prefix matcher it restates: random schemas, documents
cut at every position, vocabularies of structural fragments, and a constrained generation that runs to a complete document."""
import json
import random

import pytest
import torch

from ferrotorch_b200 import grammar as G


def _random_schema(rng, depth=0):
    kinds = ["string", "number", "integer", "boolean", "null", "enum", "any"] + (["object", "array"] * 2 if depth < 3 else [])
    k = rng.choice(kinds)
    if k == "object":
        names = rng.sample(["a", "b", "name", "x y", "k\"q", "é", "n1", "list"], rng.randint(0, 4))
        return {"type": "object", "properties": {n: _random_schema(rng, depth + 1) for n in names}, "required": [n for n in names if rng.random() < 0.5]}
    if k == "array":
        return {"type": "array", "items": _random_schema(rng, depth + 1)} if rng.random() < 0.8 else {"type": "array"}
    if rng.random() < 0.15 and k not in ("enum", "any", "null"):
        inner = _random_schema(rng, depth + 1)
        if "type" in inner and isinstance(inner["type"], str) and inner["type"] not in ("any", "null"):
            return {**inner, "type": [inner["type"], "null"]}
    if k == "enum":
        return {"enum": rng.sample(["red", "green", 1, 2.5, True, None, "a\"b", "é"], rng.randint(1, 4))}
    return {"type": k}


def _random_doc(rng, s, depth=0):
    if "enum" in s:
        return rng.choice(s["enum"])
    t = s.get("type", "any")
    if isinstance(t, list):
        return None if rng.random() < 0.4 else _random_doc(rng, {**s, "type": t[0]}, depth)
    if t == "object":
        out = {}
        for n, sub in s.get("properties", {}).items():
            if n in s.get("required", []) or rng.random() < 0.6:
                out[n] = _random_doc(rng, sub, depth + 1)
        return out
    if t == "array":
        return [_random_doc(rng, s.get("items", {"type": "any"}), depth + 1) for _ in range(rng.randint(0, 3))]
    if t == "string":
        return rng.choice(["", "hi", "a b", "q\"uote", "back\\slash", "né", "line\nbreak"])
    if t == "number":
        return rng.choice([0, -1, 3.25, 1e10, -2.5e-3, 12])
    if t == "integer":
        return rng.choice([0, 7, -13, 1000])
    if t == "boolean":
        return rng.random() < 0.5
    if t == "null":
        return None
    return rng.choice([1, "s", None, True, [1, "x"], {}]) if depth < 3 else 1


VOCAB = (["", "{", "}", "[", "]", ",", ":", ", ", ": ", "\"", "\\", "\\\"", "\\n", "\\u00e9", "\n", "\t", " ", "  ", "-", "0", "1", "12", "9.", ".", ".5", "e", "E+", "e-3",
          "true", "tr", "ue", "false", "fal", "null", "nu", "ll", "a", "b", "name", "x y", "é", "٣", "²", "\"a\"", "\"a\":", "\"b\": ", "{\"", "\"}", "\"]", "],", "},", "{}", "[]",
          "red", "\"red\"", "green", "2.5", "hello world", "<eos>", "}}", "]]", "\",\"", "\":\"", "1,", "1]", "1}", "0}", "00", "-0", "01", "n", "\"n\"", "tags", "t", "ags", "\"tags\":", "gre", "en", "r", "ed"])
EOS = VOCAB.index("<eos>")
VOCAB_ALL = VOCAB + [chr(c) for c in range(33, 127) if chr(c) not in VOCAB]        # with every printable character no prefix is a dead end


def test_native_mask_equals_python_mask_on_random_schemas_and_prefixes():
    rng = random.Random(0)
    checked = 0
    for trial in range(60):
        schema = _random_schema(rng)
        proc = G.JsonSchemaProcessor(schema, VOCAB, eos_id=EOS)
        assert proc._native is not None
        doc = json.dumps(_random_doc(rng, schema), separators=rng.choice([(",", ":"), (", ", ": ")]), ensure_ascii=rng.random() < 0.5)
        cuts = sorted(set([0, len(doc)] + [rng.randint(0, len(doc)) for _ in range(6)]))
        prefixes = [doc[:c] for c in cuts] + [doc[: cuts[len(cuts) // 2]] + rng.choice(["}", "x", ",", "\"", " "])]
        for text in prefixes:
            proc.text = text
            a, b = proc.mask().allowed, proc._mask_py().allowed
            assert torch.equal(a, b), (schema, text, [VOCAB[i] for i in (a != b).nonzero().flatten().tolist()])
            checked += 1
    assert checked > 300


def test_native_check_agrees_with_the_grammar_on_prefix_and_completion():
    import ctypes
    rng = random.Random(1)
    for _ in range(40):
        schema = _random_schema(rng)
        proc = G.JsonSchemaProcessor(schema, ["x"])
        doc = json.dumps(_random_doc(rng, schema), separators=(",", ":"))
        for c in range(len(doc) + 1):
            raw = doc[:c].encode()
            done = ctypes.c_int(0)
            ok = proc._rt.ft_json_grammar_check(proc._native, ctypes.c_char_p(raw), ctypes.c_int64(len(raw)), ctypes.byref(done))
            proc.text = doc[:c]
            assert bool(ok) == (proc._valid(doc[:c]) if c else True), (schema, doc[:c])
            assert bool(done.value) == proc._complete(), (schema, doc[:c])


def test_constrained_generation_reaches_a_complete_document_with_either_route(monkeypatch):
    schema = {"type": "object", "properties": {"name": {"type": "string"}, "n": {"type": "integer"}, "tags": {"type": "array", "items": {"enum": ["red", "green"]}}},
              "required": ["name", "n"]}
    outs = []
    for native in ("1", "0"):
        monkeypatch.setenv("FT_GRAMMAR_NATIVE", native)
        proc = G.JsonSchemaProcessor(schema, VOCAB_ALL, eos_id=EOS)
        assert (proc._native is not None) == (native == "1")
        g = torch.Generator().manual_seed(3)
        for _ in range(400):
            m = proc.mask()
            assert m.count() > 0
            logits = torch.randn(len(VOCAB_ALL), generator=g)
            logits[VOCAB.index("}")] += 2.0                        # pull towards closing
            logits[EOS] += 4.0
            tok = int(G.apply_mask(logits, m).argmax())
            if tok == EOS:
                break
            proc.advance(tok)
        outs.append(proc.text)
        doc = json.loads(proc.text)
        assert isinstance(doc["name"], str) and isinstance(doc["n"], int) and all(t in ("red", "green") for t in doc.get("tags", []))
    assert outs[0] == outs[1]


def test_numbers_take_ascii_digits_only():
    g = G.JsonGrammar(G.Schema.from_json({"type": "number"}))
    assert g.accepts_prefix("12") and not g.accepts_prefix("٣") and not g.accepts_prefix("1²")


def test_nullable_types_and_refused_keywords():
    s = G.Schema.from_json({"type": "object", "properties": {"a": {"type": ["integer", "null"]}, "b": {"type": ["null", "string"]}}, "required": ["a", "b"]})
    assert s.properties["a"].kind == "nullable" and s.properties["a"].items.kind == "integer" and s.properties["b"].items.kind == "string"
    g = G.JsonGrammar(s)
    for doc in ('{"a":null,"b":"x"}', '{"a":12,"b":null}', '{"a": null, "b": null}'):
        assert g.is_complete(doc) and all(g.accepts_prefix(doc[:c]) for c in range(1, len(doc)))
    assert not g.accepts_prefix('{"a":nul1') and not g.accepts_prefix('{"a":"x"')
    proc = G.JsonSchemaProcessor(s, ["n", "null", "1", "\"", "t", "nu", "x"])
    proc.text = '{"a":'
    assert proc.mask().allowed.tolist() == proc._mask_py().allowed.tolist() == [True, True, True, False, False, True, False]
    for word in ("oneOf", "anyOf", "allOf", "$ref"):
        with pytest.raises(Exception):
            G.Schema.from_json({word: [{"type": "string"}]})
    with pytest.raises(Exception):
        G.Schema.from_json({"type": ["string", "integer"]})


def test_batch_processor_constrains_every_sequence_of_a_serving_batch():
    schema = {"type": "object", "properties": {"n": {"type": "integer"}, "ok": {"type": "boolean"}}, "required": ["n", "ok"]}
    B = 4
    bp = G.BatchJsonSchemaProcessor(schema, VOCAB_ALL, B, eos_id=EOS)
    g = torch.Generator().manual_seed(11)
    for step in range(120):
        logits = torch.randn(B, len(VOCAB_ALL), generator=g)
        logits[:, EOS] += 6.0
        logits[:, VOCAB_ALL.index("}")] += 2.0
        masked = bp.apply(logits)
        single = G.JsonSchemaProcessor(schema, VOCAB_ALL, eos_id=EOS)
        for b in range(B):
            if not bp.finished[b]:
                single.text = bp.texts[b]
                assert torch.equal(torch.isfinite(masked[b]), single.mask().allowed)
            else:
                assert torch.equal(masked[b], logits[b])
        bp.advance(masked.argmax(-1))
        if all(bp.finished):
            break
    assert all(bp.finished)
    for b in range(B):
        doc = json.loads(bp.texts[b])
        assert isinstance(doc["n"], int) and isinstance(doc["ok"], bool) and bp.is_complete(b)
    assert len(set(bp.texts)) > 1                                    # the sequences went their own ways
    bp.reset()
    assert bp.texts == [""] * B and not any(bp.finished)
    with pytest.raises(Exception):
        bp.apply(torch.zeros(B + 1, len(VOCAB_ALL)))
    with pytest.raises(Exception):
        bp.advance([0])


def test_enum_values_and_property_names_outside_ascii_are_accepted_raw_and_escaped():
    import json
    from ferrotorch_b200.grammar import JsonGrammar, JsonSchemaProcessor, Schema
    schema = {"type": "object", "properties": {"né": {"enum": ["é✓", "plain", 3]}}, "required": ["né"]}
    g = JsonGrammar(Schema.from_json(schema))
    raw = json.dumps({"né": "é✓"}, ensure_ascii=False, separators=(",", ":"))
    assert g.is_complete(raw) and all(g.accepts_prefix(raw[:i]) for i in range(len(raw) + 1))
    assert g.is_complete('{"né":"\\u00e9\\u2713"}')
    assert not g.accepts_prefix('{"né":"è')
    vocab = ['{"', "né", '":', '"', "é", "✓", "è", "\\u00e9", "\\u2713", "}", "plain", "3"]
    proc = JsonSchemaProcessor(schema, vocab)
    for text in ("", '{"né":', '{"né":"', '{"né":"é', '{"né":"\\u00e9'):
        proc.text = text
        assert torch.equal(proc.mask().allowed, proc._mask_py().allowed), text
    proc.text = '{"né":"'
    allowed = {vocab[i] for i, ok in enumerate(proc.mask().allowed.tolist()) if ok}
    assert {"é", "\\u00e9", "plain"} <= allowed and "è" not in allowed and "✓" not in allowed
