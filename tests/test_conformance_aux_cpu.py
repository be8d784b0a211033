"""Per-symbol behaviour checks of the auxiliary packages: ``ml`` (dataset generators, adapter, metrics), ``hub`` (registry, cache, offline
loading), ``train`` (callbacks, history, AMP bundle, segment checkpointing), ``profiler`` (events, report, FLOP estimates) and ``tokenize``."""
import hashlib
import json

import numpy as np
import pytest
import torch

import ferrotorch_b200.hub as H
import ferrotorch_b200.ml as M
import ferrotorch_b200.profiler as P
import ferrotorch_b200.tokenize as T
import ferrotorch_b200.train as TR
from ferrotorch_b200 import errors


def test_ml_generators_loaders_and_metrics():
    X, y = M.make_blobs(90, centers=3, n_features=2, cluster_std=0.3, seed=1)
    assert X.shape == (90, 2) and set(np.unique(y)) == {0, 1, 2}
    X2, y2 = M.make_blobs(90, centers=3, n_features=2, cluster_std=0.3, seed=1)
    assert np.array_equal(X, X2) and np.array_equal(y, y2)
    Xm, ym = M.make_moons(100, noise=0.0, seed=0)
    assert Xm.shape == (100, 2) and set(np.unique(ym)) == {0, 1}
    Xc, yc = M.make_circles(100, noise=0.0, factor=0.5, seed=0)
    r = np.linalg.norm(Xc, axis=1)
    assert abs(r[yc == 0].mean() - 1.0) < 1e-6 and abs(r[yc == 1].mean() - 0.5) < 1e-6
    Xr, yr = M.make_regression(200, n_features=5, noise=0.0, seed=0)
    coef = np.linalg.lstsq(Xr, yr, rcond=None)[0]
    assert np.allclose(Xr @ coef, yr, atol=1e-6)
    for loader, n, d in ((M.load_iris, 150, 4), (M.load_wine, 178, 13), (M.load_breast_cancer, 569, 30), (M.load_digits, 1797, 64)):
        Xd, yd = loader()
        assert Xd.shape == (n, d) and yd.shape == (n,)
    p, r_, f = M.precision_recall_f1([0, 0, 1, 1], [0, 1, 1, 1], "macro")
    assert abs(p - (1.0 + 2 / 3) / 2) < 1e-9 and abs(r_ - 0.75) < 1e-9 and abs(f - (2 / 3 + 0.8) / 2) < 1e-9
    a = M.tensor_to_ndarray(torch.arange(4.0).view(2, 2))
    assert isinstance(a, np.ndarray) and a.shape == (2, 2)
    ad = M.SklearnAdapter(torch.nn.Sequential(torch.nn.Linear(2, 16), torch.nn.ReLU(), torch.nn.Linear(16, 3)), lr=0.05, epochs=60, batch_size=32)
    ad.fit(X.astype(np.float32), y)
    assert ad.score(X.astype(np.float32), y) > 0.95 and ad.predict(X[:5].astype(np.float32)).shape == (5,)
    assert np.allclose(ad.predict_proba(X[:5].astype(np.float32)).sum(1), 1.0, atol=1e-5)


def test_hub_registry_cache_and_offline_loading(tmp_path, monkeypatch):
    monkeypatch.setenv("FT_HUB_OFFLINE", "1")
    monkeypatch.setenv("HF_TOKEN", "tok-123")
    assert H.hf_token() == "tok-123"
    cache = H.HubCache(tmp_path / "hub")
    f = tmp_path / "blob.bin"
    f.write_bytes(b"abc")
    assert H.sha256_file(f) == hashlib.sha256(b"abc").hexdigest()
    info = H.ModelInfo("unit-test-tiny", "unit/tiny", ["config.json", "model.safetensors"], "llama", params=10)
    H.register_model(info)
    assert H.model_info("unit-test-tiny") is info and info.weights_format is H.WeightsFormat.SafeTensors
    with pytest.raises(errors.InvalidArgument):
        H.model_info("no-such-model")
    with pytest.raises(errors.FerrotorchError):                      # nothing cached and the network is declared off
        H.download_weights("unit/tiny", "config.json", cache)
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps({"model_type": "llama", "hidden_size": 8, "n_layer": 2, "num_attention_heads": 2, "vocab_size": 16}))
    from ferrotorch_b200.serialize import save_safetensors
    w = tmp_path / "model.safetensors"
    save_safetensors({"w": torch.arange(4.0)}, w)
    cache.put("unit/tiny", "config.json", cfg)
    cache.put("unit/tiny", "model.safetensors", w)
    assert H.download_weights("unit/tiny", "config.json", cache) == cache.path("unit/tiny", "config.json")
    root = H.hf_download_model("unit/tiny", cache=cache)
    assert (root / "config.json").exists()
    c, sd = H.load_pretrained("unit-test-tiny", cache)
    assert isinstance(c, H.HfTransformerConfig) and c.hidden_size == 8 and c.num_hidden_layers == 2 and torch.equal(sd["w"], torch.arange(4.0))
    s = H.HfModelSummary("org/m", downloads=5, tags=["llama"])
    i = H.HfModelInfo("org/m", siblings=[H.HfRepoFile("config.json")]) if "siblings" in H.HfModelInfo.__dataclass_fields__ else H.HfModelInfo("org/m")
    assert s.model_id == i.model_id == "org/m" and H.HfRepoFile("a.bin").rfilename == "a.bin"


def test_training_callbacks_history_and_amp():
    ra = TR.RunningAverage(0.5)
    assert ra.value() == 0.0 and abs(ra.update(2.0) - 2.0) < 1e-12 and abs(ra.update(4.0) - (0.5 * 1.0 + 0.5 * 4.0) / 0.75) < 1e-12
    h = TR.TrainingHistory()
    h.push(TR.EpochResult(0, 1.0, 0.9))
    h.push(TR.EpochResult(1, 0.5, 0.95, metrics={"acc": 0.8}))
    assert h.losses() == [1.0, 0.5] and h.best().epoch == 0 and h.best("train_loss").epoch == 1
    lines = []
    pl = TR.ProgressLogger(every=2, printer=lines.append)
    assert isinstance(pl, TR.Callback) and pl.should_stop() is False
    for step in range(1, 5):
        pl.on_batch_end(None, step, 1.0)
    pl.on_epoch_end(None, 0, h.epochs[1])
    assert len(lines) == 3 and lines[0].startswith("step 2") and "acc=0.8000" in lines[2]

    class L:
        model = torch.nn.Linear(2, 1)
    ema = TR.EmaCallback(0.5)
    ema.on_train_start(L)
    w0 = L.model.weight.detach().clone()
    with torch.no_grad():
        L.model.weight.add_(1.0)
    ema.on_batch_end(L, 1, 0.0)
    shadow = ema.ema.shadow_params[0] if hasattr(ema.ema, "shadow_params") else None
    assert shadow is None or torch.allclose(shadow, w0 + 0.5)

    class Acc(TR.Metric):
        name = "acc"

        def __init__(self):
            self.reset()

        def update(self, output, target, loss=None):
            self.n += target.numel()
            self.ok += int((output.argmax(-1) == target).sum())

        def compute(self):
            return self.ok / self.n

        def reset(self):
            self.n = self.ok = 0
    m = Acc()
    m.update(torch.tensor([[0.1, 0.9], [0.8, 0.2]]), torch.tensor([1, 1]))
    assert m.compute() == 0.5
    with pytest.raises(NotImplementedError):
        TR.Metric().compute()
    amp = TR.AmpContext(torch.bfloat16, enabled=True, device_type="cpu")
    lin = torch.nn.Linear(4, 4)
    opt = torch.optim.SGD(lin.parameters(), 0.1)
    with amp.autocast():
        y = lin(torch.randn(2, 4))
    assert y.dtype == torch.bfloat16
    before = lin.weight.detach().clone()
    amp.backward(y.float().sum())
    amp.step(opt)
    assert not torch.equal(before, lin.weight)
    layers = [torch.nn.Linear(4, 4) for _ in range(4)]
    x = torch.randn(3, 4, requires_grad=True)
    out = TR.checkpoint_sequential(layers, 2, x)
    ref = x
    for l in layers:
        ref = l(ref)
    assert torch.allclose(out, ref)
    out.sum().backward()
    gx = x.grad.clone()
    x.grad = None
    ref.sum().backward()
    assert torch.allclose(gx, x.grad)


def test_profiler_events_report_and_flops():
    assert P.estimate_flops("matmul", [(4, 8), (8, 16)]) == 2.0 * 4 * 8 * 16
    assert P.estimate_flops("linear", [(4, 8), (16, 8)]) == 2.0 * 4 * 8 * 16
    assert P.estimate_flops("bmm", [(2, 3, 4), (2, 4, 5)]) == 2.0 * 2 * 3 * 4 * 5
    assert P.estimate_flops("attention", [(1, 2, 8, 4)]) == 4.0 * 1 * 2 * 8 * 8 * 4
    assert P.estimate_flops("unknown_op", [(1,)]) is None
    prof = P.Profiler()
    prof.record_with_duration("matmul", "op", 10.0, [(4, 8), (8, 16)])
    prof.record_with_duration("matmul", "op", 30.0, [(4, 8), (8, 16)])
    prof.record_with_duration("relu", "op", 5.0, [(4, 16)], P.DeviceType.Cpu)
    prof.record_memory("act", 1024, P.MemoryCategory.Other)
    with prof.scope("block"):
        pass
    ev = prof.events() if callable(getattr(prof, "events", None)) else prof.events
    assert all(isinstance(e, P.ProfileEvent) for e in ev)
    rep = P.ProfileReport(list(ev))
    top = rep.top_ops(1)[0]
    assert isinstance(top, P.OpSummary) and top.name == "matmul" and top.count == 2 and top.total_us == 40.0 and top.mean_us == 20.0
    assert rep.total_flops() >= 2 * 2.0 * 4 * 8 * 16 and rep.memory_by_category().get("other", rep.memory_by_category().get("Other", 0)) == 1024
    trace = json.loads(rep.chrome_trace_json())
    names = {e["name"] for e in (trace["traceEvents"] if isinstance(trace, dict) else trace)}
    assert {"matmul", "relu", "block"} <= names and "matmul" in rep.table()
    assert {a.value for a in P.ScheduleAction} == {"skip", "warmup", "record", "record_and_save"}
    pair = P.GpuTimingPair("k", None, None, 1.0)
    assert pair.category == "kernel"
    prof.push_gpu_event(pair)
    assert P.CudaKernelScope is not None and {d.value for d in P.DeviceType} >= {"cpu"}


def test_tokenizer_batch_encoding(tmp_path):
    tj = {"version": "1.0", "added_tokens": [], "normalizer": None, "pre_tokenizer": {"type": "ByteLevel", "add_prefix_space": False, "use_regex": True},
          "model": {"type": "BPE", "vocab": {"a": 0, "b": 1, "ab": 2, "Ġ": 3}, "merges": ["a b"]}}
    p = tmp_path / "tokenizer.json"
    p.write_text(json.dumps(tj))
    tok = T.load_tokenizer(p)
    batch = T.encode_batch(tok, ["ab", "ba", "ab ab"])
    assert batch == [T.encode(tok, "ab"), T.encode(tok, "ba"), T.encode(tok, "ab ab")] and batch[0] == [2]
