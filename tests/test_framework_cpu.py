"""CPU tests of the framework layers: nn (incl. derive_module diagnostics), optim, schedulers, data, serialize, train."""
import math
import os

import numpy as np
import pytest
import torch

import ferrotorch_b200.data as D
import ferrotorch_b200.nn as nn
import ferrotorch_b200.optim as O
import ferrotorch_b200.serialize as S
import ferrotorch_b200.train as T
from ferrotorch_b200 import errors


# ---------------------------------------------------------------- nn -------------------------------------------------------------
def test_linear_init_is_kaiming_uniform_relu_gain_zero_bias():
    torch.manual_seed(0)
    l = nn.Linear(784, 256)
    bound = math.sqrt(2.0) * math.sqrt(3.0 / 784)
    assert l.weight.abs().max().item() <= bound + 1e-6 and l.weight.abs().max().item() > 0.9 * bound
    assert torch.count_nonzero(l.bias) == 0


def test_module_api_names_and_state_dict_roundtrip():
    m = nn.Sequential(nn.Linear(4, 8), nn.ReLU(), nn.LayerNorm(8), nn.Linear(8, 2))
    assert m.is_training() and len(list(m.parameters_mut())) == 6
    m.eval()
    assert not m.is_training()
    sd = m.state_dict()
    m2 = nn.Sequential(nn.Linear(4, 8), nn.ReLU(), nn.LayerNorm(8), nn.Linear(8, 2))
    m2.load_state_dict(sd, strict=True)
    x = torch.randn(3, 4)
    assert torch.allclose(m(x), m2(x))
    with pytest.raises(RuntimeError):
        m2.load_state_dict({"bogus": torch.zeros(1)}, strict=True)


def test_derive_module_and_its_five_diagnostics():
    from ferrotorch_b200.nn import derive_module, param, submodule, skip, Module, DeriveError

    @derive_module
    class Aff(Module):
        weight: torch.Tensor = param()
        inner: Module = submodule()
        note: str = skip(default="n")
        training: bool = True
        T = float

        def forward(self, x):
            return self.inner(x) * self.weight
    a = Aff(torch.ones(4), nn.Linear(8, 4))
    assert [n for n, _ in a.named_parameters()] == ["weight", "inner.weight", "inner.bias"] and a.note == "n"
    import enum
    with pytest.raises(DeriveError, match="only supports structs$"):
        derive_module(enum.Enum("E", "a b"))
    with pytest.raises(DeriveError, match="requires a `training: bool` field"):
        @derive_module
        class B(Module):
            w: torch.Tensor = param()
            T = float
    with pytest.raises(DeriveError, match="more than one of"):
        @derive_module
        class C(Module):
            w: torch.Tensor = param() | submodule()
            training: bool = True
            T = float
    with pytest.raises(DeriveError, match="at least one type parameter"):
        @derive_module
        class Dd(Module):
            w: torch.Tensor = param()
            training: bool = True
    with pytest.raises(DeriveError, match="named fields"):
        @derive_module
        class Tup(Module):
            pass


def test_rope_conventions_and_swiglu_and_mha():
    torch.manual_seed(0)
    x = torch.randn(2, 6, 3, 8)
    half = nn.RotaryPositionEmbedding(8, 32, 10000.0, nn.RoPEConvention.HalfRotation)
    inter = nn.RotaryPositionEmbedding(8, 32, 10000.0, nn.RoPEConvention.Interleaved)
    yh, yi = half.apply(x), inter.apply(x)
    assert torch.allclose(yh.norm(dim=-1), x.norm(dim=-1), atol=1e-5) and torch.allclose(yi.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    assert torch.allclose(yh[:, 0], x[:, 0]) and not torch.allclose(yh[:, 1], x[:, 1])
    assert torch.allclose(half.apply(x[:, 2:3], offset=2), yh[:, 2:3], atol=1e-6)
    sw = nn.SwiGLU(8, 16)
    h = torch.randn(4, 8)
    gu = sw.gate_up(h)
    assert torch.allclose(sw(h), sw.down(torch.nn.functional.silu(gu[:, :16]) * gu[:, 16:]), atol=1e-6)
    mha = nn.MultiheadAttention.with_gqa(32, 4, 2)
    q = torch.randn(2, 5, 32)
    out = mha(q, causal=True)
    out2 = mha(torch.cat([q[:, :3], torch.randn(2, 2, 32)], 1), causal=True)
    assert torch.allclose(out[:, :3], out2[:, :3], atol=1e-5)       # causal: prefix outputs do not depend on later tokens


def test_paged_kv_cache_matches_contiguous_attention_and_cow():
    torch.manual_seed(1)
    mgr = nn.PagedAttentionManager(1, 16, 4, 2, 8)
    mgr.add_sequence(0)
    k, v = torch.randn(10, 2, 8), torch.randn(10, 2, 8)
    mgr.layers[0].append(0, k, v)
    q = torch.randn(4, 8)
    ref = nn.standard_attention(q.view(1, 4, 1, 8), k.transpose(0, 1).repeat_interleave(2, 0).unsqueeze(0), v.transpose(0, 1).repeat_interleave(2, 0).unsqueeze(0))
    assert torch.allclose(mgr.attend(0, 0, q), ref.view(4, 8), atol=1e-5)
    cache = mgr.layers[0]
    cache.fork(0, 1)
    free_before = cache.pool.num_free()
    cache.append(1, torch.randn(1, 2, 8), torch.randn(1, 2, 8))          # last page is shared -> copy on write
    assert cache.pool.num_free() == free_before - 1 and cache.tables[0][-1] != cache.tables[1][-1]
    assert torch.equal(cache.gather(0)[0], k)
    mgr.free_sequence(0)
    cache.free_sequence(1)
    assert cache.pool.num_free() == 16


def test_flex_attention_block_mask_and_lora_and_qat():
    torch.manual_seed(2)
    q, k, v = torch.randn(1, 2, 16, 8), torch.randn(1, 2, 16, 8), torch.randn(1, 2, 16, 8)
    bm = nn.BlockMask.causal(16, 16, block=4)
    assert abs(bm.sparsity() - 6 / 16) < 1e-6
    assert torch.allclose(nn.flex_attention(q, k, v, block_mask=bm), nn.standard_attention(q, k, v, causal=True), atol=1e-5)
    assert torch.allclose(nn.flex_attention(q, k, v, score_mod=nn.causal_score_mod), nn.standard_attention(q, k, v, causal=True), atol=1e-5)
    base = nn.Linear(8, 4)
    lora = nn.LoRALinear(base, rank=2)
    x = torch.randn(3, 8)
    assert torch.allclose(lora(x), base(x))                     # B starts at zero
    with torch.no_grad():
        lora.lora_b.normal_()
    y = lora(x)
    lora.merge()
    assert torch.allclose(lora(x), y, atol=1e-5)
    assert [n for n, p in lora.named_parameters() if p.requires_grad] == ["lora_a", "lora_b"]
    qm = nn.prepare_qat(nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 2)))
    out = qm(torch.randn(5, 8))
    out.sum().backward()
    assert out.shape == (5, 2)


def test_clip_grad_norm_cpu():
    p = [torch.nn.Parameter(torch.ones(4)), torch.nn.Parameter(torch.ones(3))]
    for t in p:
        t.grad = torch.full_like(t, 2.0)
    n = nn.clip_grad_norm_(p, 1.0)
    assert abs(float(n) - math.sqrt(7 * 4)) < 1e-5
    assert abs(math.sqrt(sum(float((t.grad ** 2).sum()) for t in p)) - 1.0) < 1e-4


# --------------------------------------------------------------- optim -----------------------------------------------------------
@pytest.mark.parametrize("ours,theirs,kw", [
    (O.Sgd, torch.optim.SGD, dict(lr=0.1, momentum=0.9, weight_decay=1e-4, nesterov=True)),
    (O.Sgd, torch.optim.SGD, dict(lr=0.1, momentum=0.9, dampening=0.1)),
    (O.AdamW, torch.optim.AdamW, dict(lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)),
    (O.Adam, torch.optim.Adam, dict(lr=1e-2, weight_decay=0.1)),
])
def test_optimizers_match_pytorch_trajectories(ours, theirs, kw):
    torch.manual_seed(3)
    p = torch.nn.Parameter(torch.randn(7, 5))
    q = torch.nn.Parameter(p.detach().clone())
    a, b = ours([p], **kw), theirs([q], **kw)
    for _ in range(6):
        g = torch.randn(7, 5)
        p.grad, q.grad = g.clone(), g.clone()
        a.step()
        b.step()
    assert (p - q).abs().max().item() < 1e-6


def test_muon_orthogonalises_and_learns():
    torch.manual_seed(4)
    G = torch.randn(16, 8)
    X = O.newton_schulz_cubic(G, steps=12)
    assert torch.allclose(X.t() @ X, torch.eye(8), atol=5e-2)
    m = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 1))
    opt = O.Muon(m.parameters())
    x, y = torch.randn(64, 8), torch.randn(64, 1)
    l0 = None
    for _ in range(40):
        opt.zero_grad()
        l = ((m(x) - y) ** 2).mean()
        l.backward()
        opt.step()
        l0 = l0 or l.item()
    assert l.item() < 0.6 * l0


def test_grad_scaler_skips_on_inf_and_backs_off():
    p = torch.nn.Parameter(torch.ones(3))
    opt = O.Sgd([p], lr=0.1)
    sc = O.GradScaler(init_scale=8.0, growth_interval=2)
    p.grad = torch.tensor([float("inf"), 1.0, 1.0])
    sc.step(opt)
    sc.update()
    assert torch.equal(p.detach(), torch.ones(3)) and sc.get_scale() == 4.0
    for _ in range(2):
        p.grad = torch.full((3,), 4.0)        # scaled gradient; true gradient 1.0
        sc.step(opt)
        sc.update()
    assert torch.allclose(p.detach(), torch.full((3,), 0.8)) and sc.get_scale() == 8.0
    st = sc.state_dict()
    sc2 = O.GradScaler()
    sc2.load_state_dict(st)
    assert sc2.get_scale() == 8.0


def test_schedulers_and_ema_swa():
    p = torch.nn.Parameter(torch.zeros(1))
    opt = O.Sgd([p], lr=1.0)
    s = O.cosine_warmup_scheduler(opt, 2, 10, 0.1)
    lrs = []
    for _ in range(10):
        lrs.append(opt.lr())
        opt.step()
        s.step()
    assert lrs[0] == 0.0 and abs(lrs[2] - 1.0) < 1e-9 and abs(opt.lr() - 0.1) < 1e-9 and all(a >= b for a, b in zip(lrs[2:], lrs[3:]))
    w = O.LinearWarmup(O.Sgd([p], lr=2.0), 4)
    assert w.get_last_lr()[0] == 0.0
    ema = O.ExponentialMovingAverage([p], decay=0.5, use_num_updates=False)
    with torch.no_grad():
        p.fill_(2.0)
    ema.update()
    assert abs(float(ema.shadow[0]) - 1.0) < 1e-6
    am = O.AveragedModel(torch.nn.Linear(1, 1, bias=False))
    for v in (1.0, 3.0):
        src = torch.nn.Linear(1, 1, bias=False)
        with torch.no_grad():
            src.weight.fill_(v)
        am.update_parameters(src)
    assert abs(float(am.module.weight) - 2.0) < 1e-6
    acc = O.GradientAccumulator(3)
    assert [acc.accumulate() for _ in range(6)] == [False, False, True, False, False, True]


# ---------------------------------------------------------------- data -----------------------------------------------------------
def test_distributed_sampler_partitions_and_pads():
    parts = [D.DistributedSampler(10, 4, r, seed=5).indices(3) for r in range(4)]
    assert all(len(p) == 3 for p in parts)
    flat = sum(parts, [])
    assert set(flat) == set(range(10)) and len(flat) == 12
    assert D.DistributedSampler(10, 4, 1, seed=5).indices(3) == parts[1]
    assert D.DistributedSampler(10, 4, 1, seed=5).indices(4) != parts[1]
    assert D.DistributedSampler(8, 2, 1, shuffle=False).indices(0) == [1, 3, 5, 7]


def test_dataloader_workers_order_and_errors():
    ds = D.TensorDataset(torch.arange(40.).view(20, 2), torch.arange(20))
    seq = [b[1].tolist() for b in D.DataLoader(ds, batch_size=6, num_workers=3)]
    assert seq == [list(range(0, 6)), list(range(6, 12)), list(range(12, 18)), [18, 19]]
    assert len(D.DataLoader(ds, batch_size=6, drop_last=True)) == 3

    class Bad(D.Dataset):
        def __len__(self):
            return 4

        def __getitem__(self, i):
            if i == 2:
                raise ValueError("boom")
            return torch.zeros(1)
    with pytest.raises(errors.WorkerPanic):
        list(D.DataLoader(Bad(), batch_size=1, num_workers=2))
    cat = D.ConcatDataset([D.VecDataset([1, 2]), D.VecDataset([3])])
    assert [cat[i] for i in range(3)] == [1, 2, 3]
    with pytest.raises(errors.IndexOutOfBounds):
        cat[3]


# ------------------------------------------------------------- serialize ---------------------------------------------------------
def test_safetensors_roundtrip_and_interop(tmp_path):
    sd = {"a.w": torch.randn(3, 4), "b": torch.randn(5).to(torch.bfloat16), "c": torch.arange(6).reshape(2, 3), "e": torch.empty(0, 2),
          "h": torch.randn(2, 2).half()}
    S.save_safetensors(sd, tmp_path / "x.safetensors", {"k": "v"})
    for kw in ({}, {"use_mmap": False}, {"parallel": True}):
        ld = S.load_safetensors(tmp_path / "x.safetensors", **kw)
        assert all(torch.equal(sd[k], ld[k]) for k in sd)
    from safetensors.torch import load_file, save_file
    ref = load_file(str(tmp_path / "x.safetensors"))
    assert all(torch.equal(sd[k], ref[k]) for k in sd)
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "y.safetensors"))
    assert all(torch.equal(sd[k], v) for k, v in S.load_safetensors(tmp_path / "y.safetensors").items())
    cast = S.load_safetensors(tmp_path / "x.safetensors", dtype=torch.float32)
    assert cast["b"].dtype == torch.float32 and cast["c"].dtype == torch.int64
    only = S.load_safetensors_filtered(tmp_path / "x.safetensors", lambda n: n.startswith("a."))
    assert list(only) == ["a.w"]
    idx = S.save_safetensors_sharded(sd, tmp_path / "sh", max_shard_bytes=40)
    assert all(torch.equal(sd[k], v) for k, v in S.load_safetensors_sharded(idx).items())


def test_native_pt_checkpoint_gguf_onnx(tmp_path):
    sd = {"w": torch.randn(4, 3), "b": torch.randn(3).to(torch.bfloat16), "i": torch.arange(4)}
    S.save_state_dict(sd, tmp_path / "n.ftsd")
    assert all(torch.equal(sd[k], v) for k, v in S.load_state_dict(tmp_path / "n.ftsd").items())
    S.save_pytorch_state_dict(sd, tmp_path / "p.pt")
    assert all(torch.equal(sd[k], v) for k, v in S.load_pytorch_state_dict(tmp_path / "p.pt").items())
    assert all(torch.equal(v, torch.load(tmp_path / "p.pt")[k]) for k, v in sd.items())
    torch.save({"evil": os.system}, tmp_path / "evil.pt")
    with pytest.raises(errors.InvalidArgument):
        S.load_pytorch_state_dict(tmp_path / "evil.pt")
    m = torch.nn.Linear(4, 2)
    o = torch.optim.Adam(m.parameters())
    m(torch.randn(3, 4)).sum().backward()
    o.step()
    S.save_checkpoint(tmp_path / "c.ftc", m, o, epoch=3, step=7)
    m2, o2 = torch.nn.Linear(4, 2), torch.optim.Adam(m.parameters())
    ck = S.load_checkpoint(tmp_path / "c.ftc", m2, o2)
    assert (ck.epoch, ck.step) == (3, 7) and torch.equal(m2.weight, m.weight)
    assert torch.allclose(o2.state_dict()["state"][0]["exp_avg"], o.state_dict()["state"][0]["exp_avg"])
    # q8_0 / q4_0 dequantisation against a direct evaluation of the block formulas
    rng = np.random.default_rng(0)
    d = np.float16(0.5)
    q8 = rng.integers(-127, 127, 32, dtype=np.int8)
    raw = d.tobytes() + q8.tobytes()
    assert torch.allclose(S.dequantize_gguf(raw, 8, 32), torch.from_numpy(q8.astype(np.float32) * 0.5))
    q4 = rng.integers(0, 255, 16, dtype=np.uint8)
    raw = d.tobytes() + q4.tobytes()
    exp = np.concatenate([(q4 & 15).astype(np.float32) - 8, (q4 >> 4).astype(np.float32) - 8]) * 0.5
    assert torch.allclose(S.dequantize_gguf(raw, 2, 32), torch.from_numpy(exp))
    seq = torch.nn.Sequential(torch.nn.Linear(4, 8), torch.nn.ReLU(), torch.nn.Linear(8, 2))
    S.export_onnx(seq, torch.randn(1, 4), tmp_path / "m.onnx")
    blob = (tmp_path / "m.onnx").read_bytes()
    assert b"Gemm" in blob and b"Relu" in blob and b"ferrotorch_b200" in blob
    with pytest.raises(errors.InvalidArgument):
        S.export_onnx(torch.nn.Sequential(torch.nn.Conv2d(1, 1, 1)), torch.randn(1, 1, 2, 2), tmp_path / "bad.onnx")


# ---------------------------------------------------------------- train ----------------------------------------------------------
def test_learner_fit_checkpoint_resume_tensorboard(tmp_path):
    torch.manual_seed(0)
    X = torch.randn(256, 10)
    Y = (X @ torch.randn(10, 3)).argmax(1)
    dl = D.DataLoader(D.TensorDataset(X, Y), batch_size=32, shuffle=True)
    m = nn.Sequential(nn.Linear(10, 32), nn.ReLU(), nn.Linear(32, 3))
    L = T.Learner(m, O.AdamW(m.parameters(), lr=1e-2), nn.CrossEntropyLoss(), metrics=[T.AccuracyMetric(), T.TopKAccuracy(2)],
                  callbacks=[T.EarlyStopping(patience=3), T.TensorBoardCallback(tmp_path / "tb")]).with_checkpointing(tmp_path)
    h = L.fit(dl, 4, dl)
    assert h.losses()[-1] < 0.9 * h.losses()[0] and h.epochs[-1].metrics["accuracy"] > 0.6
    ev = list((tmp_path / "tb").glob("events.out.tfevents.*"))
    assert ev and ev[0].stat().st_size > 100
    m2 = nn.Sequential(nn.Linear(10, 32), nn.ReLU(), nn.Linear(32, 3))
    L2 = T.Learner(m2, O.AdamW(m2.parameters(), lr=1e-2), nn.CrossEntropyLoss())
    L2.load_checkpoint(tmp_path / "checkpoint_epoch_3.ftc")
    assert L2.epoch == 4 and L2.step == L.step and torch.equal(m2[0].weight, m[0].weight)
    assert T.crc32c(b"123456789") == 0xE3069283


def test_host_philox_streams_do_not_depend_on_the_vector_path_or_thread_count():
    """Large host rand / randn come from the native Philox fill: same seed -> same values, with the AVX2 code or the generic code (no FMA
    contraction in either), with one thread or eight; the normal stream has unit moments."""
    import subprocess
    import sys
    code = ("import torch, hashlib\nfrom ferrotorch_b200 import core\ntorch.manual_seed(123)\n"
            "a = core.rand([300, 1001]); b = core.randn([300, 1001])\n"
            "print(hashlib.sha256(a.numpy().tobytes() + b.numpy().tobytes()).hexdigest())\n")
    import os
    outs = []
    for env in ({}, {"FT_NO_AVX2": "1"}):
        r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, env=dict(os.environ, **env),
                           cwd=str(__import__("pathlib").Path(__file__).resolve().parents[1]))
        assert r.returncode == 0, r.stderr[-2000:]
        outs.append(r.stdout.strip().splitlines()[-1])
    assert outs[0] == outs[1]
    import torch
    from ferrotorch_b200 import core
    torch.manual_seed(5)
    one = core.randn([512, 513])
    torch.set_num_threads(1)
    try:
        torch.manual_seed(5)
        assert torch.equal(one, core.randn([512, 513]))
    finally:
        torch.set_num_threads(max(1, os.cpu_count() or 1))
    assert abs(float(one.mean())) < 0.01 and abs(float(one.std()) - 1.0) < 0.01 and abs(float((one ** 4).mean()) - 3.0) < 0.1


def test_gguf_reader_matches_the_official_writer(tmp_path):
    """A file written by the ``gguf`` package (metadata of every kind used by Llama exports, f32 / f16 / q4_0 / q4_1 / q5_0 / q5_1 / q8_0 tensors):
    metadata read back as written, tensors dequantised to exactly what the package's own dequantiser gives."""
    import numpy as np
    gguf = pytest.importorskip("gguf")
    from gguf import GGMLQuantizationType as T, quants
    from ferrotorch_b200 import serialize as S
    rng = np.random.default_rng(0)
    path = tmp_path / "parity.gguf"
    w = gguf.GGUFWriter(str(path), "llama")
    w.add_uint32("llama.block_count", 2)
    w.add_string("general.name", "parity")
    w.add_float32("llama.rope.freq_base", 500000.0)
    w.add_array("tokenizer.ggml.tokens", ["a", "b", "c"])
    want = {}
    for name, q, shape in (("f32", T.F32, (3, 64)), ("f16", T.F16, (2, 64)), ("q4_0", T.Q4_0, (4, 64)), ("q4_1", T.Q4_1, (4, 64)), ("q5_0", T.Q5_0, (2, 128)),
                           ("q5_1", T.Q5_1, (2, 128)), ("q8_0", T.Q8_0, (5, 32))):
        x = rng.standard_normal(shape).astype(np.float32)
        if q == T.F32:
            data, want[name] = x, x
            w.add_tensor(name, data)
        elif q == T.F16:
            data = x.astype(np.float16)
            want[name] = data.astype(np.float32)
            w.add_tensor(name, data)
        else:
            data = quants.quantize(x, q)
            want[name] = quants.dequantize(data, q)
            w.add_tensor(name, data, raw_shape=data.shape, raw_dtype=q)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    g = S.parse_gguf(path)
    assert g.metadata["llama.block_count"] == 2 and g.metadata["general.name"] == "parity" and g.metadata["tokenizer.ggml.tokens"] == ["a", "b", "c"]
    assert abs(g.metadata["llama.rope.freq_base"] - 500000.0) < 1e-3
    for k, v in want.items():
        t = g.load_tensor(k)
        assert tuple(t.shape) == v.shape and np.array_equal(t.numpy(), v), k


def test_tensorboard_event_files_are_read_by_tensorboard(tmp_path):
    """The hand-written event-file writer (record framing with masked CRC32C, Event / Summary protobufs) against TensorBoard's own reader."""
    pytest.importorskip("tensorboard")
    from tensorboard.backend.event_processing.event_accumulator import EventAccumulator
    w = T.TensorBoardWriter(tmp_path / "run")
    for s in range(5):
        w.add_scalar("loss", 1.0 / (s + 1), s)
    w.add_scalars("m", {"a": 1.5, "b": -2.0}, 3)
    w.add_histogram("h", torch.arange(100.0), 7)
    for name in ("flush", "close"):
        getattr(w, name, lambda: None)()
    ea = EventAccumulator(str(tmp_path / "run"), size_guidance={"histograms": 0, "scalars": 0})
    ea.Reload()
    tags = ea.Tags()
    assert sorted(tags["scalars"]) == ["loss", "m/a", "m/b"] and tags["histograms"] == ["h"]
    assert [(e.step, round(e.value, 4)) for e in ea.Scalars("loss")] == [(0, 1.0), (1, 0.5), (2, 0.3333), (3, 0.25), (4, 0.2)]
    assert [(e.step, e.value) for e in ea.Scalars("m/b")] == [(3, -2.0)]
    h = ea.Histograms("h")[0]
    assert h.step == 7 and h.histogram_value.min == 0.0 and h.histogram_value.max == 99.0 and h.histogram_value.num == 100 and h.histogram_value.sum == 4950.0


@pytest.mark.parametrize("kw", [dict(lr=1e-3, scale_parameter=True, relative_step=False),
                                dict(lr=1e-2, scale_parameter=False, relative_step=False, beta1=0.9, weight_decay=0.01),
                                dict(lr=None, scale_parameter=True, relative_step=True)])
def test_adafactor_matches_the_transformers_implementation(kw):
    """Factored second moments, update clipping, parameter-scaled and relative step sizes: six steps on a matrix and a vector against
    ``transformers.optimization.Adafactor``."""
    hf = pytest.importorskip("transformers.optimization")
    torch.manual_seed(0)
    w0, b0 = torch.randn(6, 5), torch.randn(5)
    pa = [torch.nn.Parameter(w0.clone()), torch.nn.Parameter(b0.clone())]
    pb = [torch.nn.Parameter(w0.clone()), torch.nn.Parameter(b0.clone())]
    a = O.Adafactor(pa, **kw)
    b = hf.Adafactor(pb, **dict(kw, warmup_init=False) if kw.get("relative_step") else kw)
    for _ in range(6):
        for p, q, g in zip(pa, pb, (torch.randn(6, 5), torch.randn(5))):
            p.grad, q.grad = g.clone(), g.clone()
        a.step()
        b.step()
    assert max(float((p - q).abs().max()) for p, q in zip(pa, pb)) < 2e-6


def test_tensorboard_event_files_are_read_by_the_tensorboard_package(tmp_path):
    """Scalars, grouped scalars, a histogram and a text record, written by ``TensorBoardWriter`` and read back by TensorBoard's own event
    loader (which checks the record framing and both checksums)."""
    pytest.importorskip("tensorboard")
    from tensorboard.backend.event_processing.event_accumulator import EventAccumulator
    from ferrotorch_b200.train import TensorBoardWriter
    w = TensorBoardWriter(str(tmp_path))
    for i in range(5):
        w.add_scalar("loss", 1.0 / (i + 1), i)
    w.add_scalars("m", {"a": 1.0, "b": 2.0}, 3)
    w.add_histogram("h", torch.linspace(-2, 3, 1000), 1)
    w.add_text("note", "hello ✓", 0)
    w.close() if hasattr(w, "close") else w.flush()
    ea = EventAccumulator(str(tmp_path), size_guidance={"histograms": 0, "tensors": 0, "scalars": 0})
    ea.Reload()
    tags = ea.Tags()
    assert set(tags["scalars"]) == {"loss", "m/a", "m/b"} and tags["histograms"] == ["h"] and tags["tensors"] == ["note"]
    assert [(e.step, round(e.value, 6)) for e in ea.Scalars("loss")] == [(i, round(1.0 / (i + 1), 6)) for i in range(5)]
    h = ea.Histograms("h")[0].histogram_value
    assert h.num == 1000 and abs(h.min + 2) < 1e-6 and abs(h.max - 3) < 1e-6 and abs(sum(h.bucket) - 1000) < 1e-6
    assert ea.Tensors("note")[0].tensor_proto.string_val == ["hello ✓".encode()]
