"""The snippets of docs/GUIDE.md that are marked as checked, executed as written (host side)."""
import torch


def test_guide_snippets(tmp_path):
    from ferrotorch_b200 import gpu, jit, nn, optim, profiler, serialize, train
    torch.manual_seed(0)
    # 1. Learner
    model = nn.Sequential(nn.Linear(20, 64), nn.ReLU(), nn.Linear(64, 3))
    opt = optim.AdamW(model.parameters(), lr=1e-2)
    x, y = torch.randn(256, 20), torch.randint(0, 3, (256,))
    batches = [(x[i:i + 32], y[i:i + 32]) for i in range(0, 256, 32)]
    learner = train.Learner(model, opt, nn.CrossEntropyLoss()).with_metric(train.AccuracyMetric())
    history = learner.fit(batches, epochs=3, val_data=batches)
    assert history.epochs[-1].train_loss < history.epochs[0].train_loss
    # 2. compute copies under autocast
    assert nn.attach_compute_copies(model) == 2
    opt2 = optim.Sgd(model.parameters(), lr=0.1, momentum=0.9)
    with torch.autocast("cpu", dtype=torch.bfloat16):
        loss = torch.nn.functional.cross_entropy(model(x).float(), y)
    loss.backward()
    opt2.step()
    assert all(torch.equal(nn.compute_copy(p), p.detach().bfloat16()) for p in model.parameters() if p.dim() == 2)
    # 5. JIT
    def f(a, b):
        return torch.nn.functional.gelu(a + b) * 1.5 + torch.log(a * a + 1.0)
    x2, bias = torch.randn(256, 512), torch.randn(512)
    fast = jit.compile(f, example_inputs=[x2, bias])
    assert torch.allclose(fast(x2, bias), f(x2, bias), atol=1e-5)
    # 6. checkpoints
    path = tmp_path / "model.safetensors"
    serialize.save_safetensors(model.state_dict(), path)
    state = serialize.load_safetensors(path)
    assert set(state) == set(model.state_dict()) and all(torch.equal(state[k], v) for k, v in model.state_dict().items())
    # 7. profiler and memory guard
    result, report = profiler.with_profiler(profiler.ProfileConfig(), lambda: model(x))
    assert result.shape == (256, 3) and isinstance(report.table(), str)
    guard = gpu.MemoryGuardBuilder().with_budget(8 << 30).with_policy(gpu.OomPolicy.RETRY_AFTER_FREE).with_query(lambda: (0, 16 << 30)).build()
    with guard.reserve(1 << 20):
        assert guard.stats().reserved_by_guard == 1 << 20
    # 9. layers
    net = nn.Sequential(nn.Conv2d(3, 16, 3, padding=1, padding_mode="reflect"), nn.BatchNorm2d(16), nn.HardSwish(), nn.AdaptiveAvgPool2d(1), nn.Flatten(),
                        nn.Linear(16, 4))
    assert net(torch.randn(2, 3, 8, 8)).shape == (2, 4)
    lstm = nn.LSTM(32, 64, num_layers=2, bidirectional=True)
    out, (h, c) = lstm(torch.randn(5, 3, 32))
    assert out.shape == (5, 3, 128) and h.shape == (4, 3, 64)
    enc = nn.TransformerEncoder(nn.TransformerEncoderLayer(64, 4, 128, dropout=0.0, batch_first=True), 2)
    assert enc(torch.randn(2, 10, 64), src_key_padding_mask=torch.zeros(2, 10, dtype=torch.bool)).shape == (2, 10, 64)
    assert nn.attention_backend(torch.randn(1, 2, 8, 64)) == "standard"
    # 10. tokenizers and constrained decoding
    from ferrotorch_b200 import grammar, tokenize
    vocab = {c: i for i, c in enumerate(["<eos>"] + [tokenize._bytes_to_unicode()[b] for b in range(256)])}
    vocab.update({"he": 257, "ll": 258, "hell": 259, "hello": 260})
    tok = tokenize.Tokenizer(vocab, [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o")], {"<eos>": 0})
    ids = tok.encode("hello {\"n\": 7}")
    assert ids[0] == 260 and tok.decode(ids) == "hello {\"n\": 7}" and tok.encode_batch(["hello", "hi"])[0] == [260]
    texts = [tok.decode([i], skip_special_tokens=False) if i else "" for i in range(tok.vocab_size())]
    proc = grammar.JsonSchemaProcessor({"type": "object", "properties": {"n": {"type": ["integer", "null"]}}, "required": ["n"]}, texts, eos_id=0)
    for ch in "{\"n\": ":
        logits = proc.apply(torch.zeros(len(texts)))
        assert logits[vocab[tokenize._bytes_to_unicode()[ord(ch)]]] == 0
        proc.advance(vocab[tokenize._bytes_to_unicode()[ord(ch)]])
    allowed = {texts[i] for i in proc.mask().allowed.nonzero().flatten().tolist()}
    assert allowed == set("-0123456789n")
    # 11. native core
    import numpy as np
    from ferrotorch_b200 import native as N
    rng = np.random.default_rng(0)
    images, labels = rng.standard_normal((8, 1, 14, 14)).astype(np.float32), rng.integers(0, 10, 8)
    net = N.Sequential(N.Conv2d(1, 8, 3, padding=1), N.ReLU(), N.MaxPool2d(2), N.Flatten(), N.Linear(8 * 7 * 7, 10))
    opt = N.AdamW(net.parameters(), lr=3e-3)
    first = None
    for _ in range(5):
        opt.zero_grad()
        loss = N.cross_entropy(net(N.Tensor(images)), labels)
        loss.backward(threads=4)
        opt.step()
        first = first if first is not None else loss.item()
    assert loss.item() < first
    ids, table = rng.integers(0, 5, (2, 3)), N.Tensor(rng.standard_normal((5, 4)).astype(np.float32))
    hq = N.layer_norm(N.embedding(ids, table)).reshape(1, 2, 3, 4)
    att = (hq @ hq.transpose(2, 3) + N.Tensor(np.zeros((3, 3), np.float32))).softmax() @ hq
    assert att.shape == (1, 2, 3, 4)
