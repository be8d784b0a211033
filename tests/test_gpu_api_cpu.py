"""Buffer-level device API: every wrapper refuses host tensors; with the device check lifted the arithmetic and the size checks are
verified on the host. Capture-pool handles, memory statistics / watchdog and the host Philox generator need no device at all."""
import threading

import numpy as np
import pytest
import torch

from ferrotorch_b200 import gpu as G
from ferrotorch_b200.errors import DeviceMismatch, FerrotorchError, InvalidArgument, ShapeMismatch


def test_wrappers_refuse_host_tensors():
    a = torch.ones(4)
    for call in (lambda: G.gpu_add(a, a), lambda: G.gpu_softmax(a, 1, 4), lambda: G.gpu_matmul_f32(a, a, 2, 2, 2), lambda: G.gpu_slice_read(a, 1, 1, 1, 4),
                 lambda: G.gpu_rmsnorm_bf16(a.bfloat16(), a.bfloat16(), 1, 4, 1e-5), lambda: G.gpu_neg(a)):
        with pytest.raises(DeviceMismatch):
            call()
    if not torch.cuda.is_available():
        with pytest.raises(FerrotorchError):
            G.get_cuda_device(0)
        assert G.cached_bytes() == 0 and G.capture_status() is G.CaptureStatus.None_ and not G.is_stream_capturing()
        G.empty_cache_all()


@pytest.fixture
def host(monkeypatch):
    monkeypatch.setattr(G.api_ext, "_require_cuda", False)


def test_elementwise_norm_and_products(host):
    g = torch.Generator().manual_seed(0)
    a, b = torch.randn(12, generator=g), torch.randn(12, generator=g)
    assert torch.equal(G.gpu_add(a, b), a + b) and torch.equal(G.gpu_sub(a, b), a - b) and torch.equal(G.gpu_mul(a, b), a * b) and torch.equal(G.gpu_neg(a), -a)
    out = torch.empty(12)
    G.gpu_add_into(a, b, out)
    assert torch.equal(out, a + b)
    G.gpu_add_into_on_stream(a, b, out, None, None)
    G.gpu_scale_into(a, 3.0, out)
    assert torch.equal(out, a * 3)
    G.gpu_gelu_into(a, out)
    assert torch.allclose(out, torch.nn.functional.gelu(a)) and torch.equal(G.gpu_relu(a), a.relu())
    with pytest.raises(ShapeMismatch):
        G.gpu_add(a, b[:5])
    with pytest.raises(InvalidArgument):
        G.gpu_add(a.double(), b.double())
    hb = a.bfloat16()
    assert torch.equal(G.gpu_fatrelu_bf16(hb, 0.3), torch.where(hb >= 0.3, hb, torch.zeros_like(hb))) and G.gpu_silu_bf16(hb).dtype == torch.bfloat16
    assert torch.equal(G.gpu_add_bf16(hb, hb), hb + hb) and torch.equal(G.gpu_scale_bf16(hb, 2.0), hb * 2) and torch.equal(G.gpu_relu_bf16(hb), hb.relu())
    r = G.gpu_broadcast_add(a[:3], b[:4], [3, 1], [1, 4], [3, 4])
    assert torch.equal(r.view(3, 4), a[:3, None] + b[None, :4]) and torch.equal(G.gpu_broadcast_mul(a[:3], b[:4], [3, 1], [4], [3, 4]).view(3, 4), a[:3, None] * b[:4])
    with pytest.raises(ShapeMismatch):
        G.gpu_broadcast_sub(a[:3], b[:4], [3], [4], [3, 4])
    with pytest.raises(ShapeMismatch):
        G.gpu_broadcast_add(a[:3], b[:4], [3, 1], [1, 4], [4, 3])
    x = torch.randn(10000, generator=g)
    d1, d2 = G.gpu_dropout(x, 1 << 30, 4 / 3, 7), G.gpu_dropout(x, 1 << 30, 4 / 3, 7)
    kept = d1 != 0
    assert torch.equal(d1, d2) and abs(float(kept.float().mean()) - 0.75) < 0.02 and torch.allclose(d1[kept], x[kept] * 4 / 3)
    assert not torch.equal(d1, G.gpu_dropout(x, 1 << 30, 4 / 3, 8))
    m = torch.randn(3, 8, generator=g)
    assert torch.allclose(G.gpu_softmax(m.reshape(-1), 3, 8).view(3, 8), m.softmax(-1))
    so = torch.empty(24)
    G.gpu_softmax_into(m.reshape(-1), so, 3, 8)
    assert torch.allclose(so.view(3, 8), m.softmax(-1)) and torch.allclose(G.gpu_softmax_bf16(m.bfloat16(), 3, 8).float(), m.bfloat16().float().softmax(-1), atol=1e-2)
    w, bb = torch.rand(8, generator=g) + 0.5, torch.randn(8, generator=g)
    assert torch.allclose(G.gpu_layernorm(m, w, bb, 3, 8, 1e-5), torch.nn.functional.layer_norm(m, (8,), w, bb, 1e-5), atol=1e-6)
    lo = torch.empty(3, 8)
    G.gpu_layernorm_into(m, w, bb, lo, 3, 8, 1e-5)
    assert torch.allclose(lo, torch.nn.functional.layer_norm(m, (8,), w, bb, 1e-5), atol=1e-6)
    mb = m.bfloat16()
    want = (mb.float() * torch.rsqrt(mb.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w.bfloat16().float()).bfloat16()
    assert torch.equal(G.gpu_rmsnorm_bf16(mb, w.bfloat16(), 3, 8, 1e-5), want)
    gn = torch.randn(2, 4, 6, generator=g)
    assert torch.allclose(G.gpu_group_norm_f32(gn.reshape(-1), torch.ones(4), torch.zeros(4), 2, 4, 2, 6, 1e-5).view(2, 4, 6),
                          torch.nn.functional.group_norm(gn, 2, torch.ones(4), torch.zeros(4), 1e-5), atol=1e-6)
    with pytest.raises(InvalidArgument):
        G.gpu_group_norm_f32(gn.reshape(-1), torch.ones(4), torch.zeros(4), 2, 4, 3, 6, 1e-5)
    blk = torch.randn(2, 12, generator=g).bfloat16()
    assert torch.equal(G.gpu_block_reduce_max_abs_bf16(blk, 2, 3, 4), blk.view(2, 3, 4).abs().amax(-1).float().reshape(-1))
    A, B = torch.randn(3, 5, generator=g), torch.randn(5, 4, generator=g)
    assert torch.allclose(G.gpu_matmul_f32(A.reshape(-1), B.reshape(-1), 3, 5, 4).view(3, 4), A @ B) and torch.allclose(G.gpu_small_matmul(A, B, 3, 5, 4).view(3, 4), A @ B)
    mo = torch.empty(12)
    G.gpu_matmul_f32_into(A, B, mo, 3, 5, 4)
    assert torch.allclose(mo.view(3, 4), A @ B) and torch.allclose(G.gpu_matmul_f64(A.double(), B.double(), 3, 5, 4).view(3, 4), A.double() @ B.double())
    with pytest.raises(ShapeMismatch):
        G.gpu_matmul_f32(A, B, 3, 4, 4)
    Ab, Bb = torch.randn(2, 3, 5, generator=g), torch.randn(2, 5, 4, generator=g)
    assert torch.allclose(G.gpu_bmm_f32(Ab, Bb, 2, 3, 5, 4).view(2, 3, 4), Ab @ Bb) and torch.allclose(G.gpu_small_bmm(Ab, Bb, 2, 3, 5, 4).view(2, 3, 4), Ab @ Bb)
    ah, bh = A.bfloat16(), B.bfloat16()
    assert torch.allclose(G.gpu_matmul_bf16_bf16(ah, bh, 3, 5, 4).float().view(3, 4), ah.float() @ bh.float(), atol=0.05)
    assert torch.allclose(G.gpu_matmul_bf16_bf16_nt(ah, bh.t().contiguous(), 3, 5, 4).float().view(3, 4), ah.float() @ bh.float(), atol=0.05)
    sb = G.gpu_matmul_bf16_bf16_strided_batched(Ab.bfloat16(), bh, 3, 5, 4, 2, 15, 0, 0.5)            # stride 0: one B for both batches
    assert torch.allclose(sb.float().view(2, 3, 4), 0.5 * (Ab.bfloat16().float() @ bh.float()), atol=0.05)
    snt = G.gpu_matmul_bf16_bf16_strided_batched_nt(Ab.bfloat16(), Bb.transpose(1, 2).contiguous().bfloat16(), 3, 5, 4, 2, 15, 20)
    assert torch.allclose(snt.float().view(2, 3, 4), Ab.bfloat16().float() @ Bb.bfloat16().float(), atol=0.05)
    with pytest.raises(FerrotorchError):
        G.gpu_matmul_bf16_bf16_strided_batched(Ab.bfloat16(), bh, 3, 5, 4, 2, 7, 0)
    img, ker = torch.randn(1, 4, 6, 6, generator=g), torch.randn(6, 2, 3, 3, generator=g)
    assert torch.allclose(G.gpu_conv2d_f32(img.reshape(-1), ker.reshape(-1), None, [1, 4, 6, 6], [6, 2, 3, 3], (1, 1), (1, 1), (1, 1), 2),
                          torch.nn.functional.conv2d(img, ker, None, 1, 1, 1, 2), atol=1e-5)
    with pytest.raises(ShapeMismatch):
        G.gpu_conv2d_f32(img, ker, None, [1, 4, 6, 6], [6, 2, 3, 3], groups=1)
    q, k, v = torch.randn(4, 5, 8, generator=g), torch.randn(4, 7, 8, generator=g), torch.randn(4, 7, 6, generator=g)
    got = G.gpu_flash_attention_f32(q.reshape(-1), k.reshape(-1), v.reshape(-1), 5, 7, 8, 6, 4, 0.3, False).view(4, 5, 6)
    assert torch.allclose(got, torch.softmax(q @ k.transpose(1, 2) * 0.3, -1) @ v, atol=1e-5)
    assert G.gpu_flash_attention_f64(q.double(), q.double(), q.double(), 5, 5, 8, 8, 4, 0.3, True).dtype == torch.float64


def test_layout_indexing_and_cache_ops(host):
    x = torch.arange(24.0)
    assert torch.equal(G.gpu_transpose_2d(x, 4, 6).view(6, 4), x.view(4, 6).t()) and torch.equal(G.gpu_permute_0213(x, 2, 3, 2, 2).view(2, 2, 3, 2), x.view(2, 3, 2, 2).permute(0, 2, 1, 3))
    o = torch.empty(24)
    G.gpu_transpose_2d_into(x, o, 4, 6)
    assert torch.equal(o.view(6, 4), x.view(4, 6).t())
    G.gpu_permute_0213_into(x, o, 2, 3, 2, 2)
    assert torch.equal(o.view(2, 2, 3, 2), x.view(2, 3, 2, 2).permute(0, 2, 1, 3))
    h = G.gpu_transpose_to_heads_bf16(x, 2, 3, 4)
    assert torch.equal(h.view(2, 3, 4), x.view(3, 2, 4).transpose(0, 1)) and torch.equal(G.gpu_transpose_from_heads_bf16(h, 2, 3, 4), x)
    assert torch.equal(G.gpu_repeat_kv_bf16(x, 2, 3, 3, 4).view(6, 3, 4)[4], x.view(2, 3, 4)[1])
    pos = torch.arange(10.0)[:, None] * (1.0 / 10000 ** (torch.arange(0, 2) / 2.0))
    t = torch.randn(2, 3, 4)
    got = G.gpu_rope_half_bf16(t.reshape(-1), pos.cos(), pos.sin(), 2, 3, 4, 5).view(2, 3, 4)
    c, s = pos.cos()[5:8], pos.sin()[5:8]
    assert torch.allclose(got, torch.cat([t[..., :2] * c - t[..., 2:] * s, t[..., 2:] * c + t[..., :2] * s], -1), atol=1e-6)
    with pytest.raises(ShapeMismatch):
        G.gpu_rope_half_bf16(t.reshape(-1), pos.cos(), pos.sin(), 2, 3, 4, 8)
    sc = torch.zeros(2, 3, 5)
    G.gpu_causal_mask_bf16(sc, 2, 3, 5)
    assert sc[0].isinf().tolist() == [[False, False, False, True, True], [False, False, False, False, True], [False] * 5]
    mk = torch.empty(2, 6)
    G.gpu_causal_mask_indirect(torch.tensor([4], dtype=torch.int32), 2, 6, mk)
    assert mk[1].tolist() == [0, 0, 0, 0, -1e9, -1e9]
    W = torch.arange(12.0).view(4, 3)
    assert G.gpu_embed_lookup(torch.tensor([2.0, 0.0]), W.reshape(-1), 3).tolist() == [6, 7, 8, 0, 1, 2]
    eo = torch.empty(6)
    G.gpu_embed_lookup_into(torch.tensor([1.0, 1.0]), W, eo, 3)
    assert eo.tolist() == [3, 4, 5, 3, 4, 5]
    with pytest.raises(InvalidArgument):
        G.gpu_embed_lookup(torch.tensor([4.0]), W, 3)
    assert torch.equal(G.gpu_embedding_gather_bf16(W.bfloat16(), torch.tensor([3, 1], dtype=torch.int32), 3).view(2, 3), W.bfloat16()[[3, 1]])
    assert G.gpu_embedding_gather_bf16_to_f32(W.bfloat16(), torch.tensor([0], dtype=torch.int32), 3).dtype == torch.float32
    cache = torch.zeros(2, 4, 3)
    G.gpu_slice_write(torch.ones(2, 3), cache, 2, 3, 4, 1)
    G.gpu_slice_write_indirect(torch.full((2, 3), 2.0), cache, 2, 3, 4, torch.tensor([2], dtype=torch.int32))
    G.gpu_slice_write_indirect(torch.full((2, 3), 9.0), cache, 2, 3, 4, torch.tensor([7], dtype=torch.int32))      # outside the cache: nothing is written
    assert cache[:, :, 0].tolist() == [[0, 1, 2, 0], [0, 1, 2, 0]]
    assert G.gpu_slice_read(cache, 2, 3, 3, 4).view(2, 3, 3)[1, :, 0].tolist() == [0, 1, 2]
    ro = torch.empty(2, 2, 3)
    G.gpu_slice_read_into(cache, ro, 2, 3, 2, 4)
    assert ro[0, 1].tolist() == [1, 1, 1]
    for bad in (lambda: G.gpu_slice_write(torch.ones(2, 3), cache, 2, 3, 4, 4), lambda: G.gpu_slice_read(cache, 2, 3, 5, 4)):
        with pytest.raises(InvalidArgument):
            bad()
    assert torch.equal(G.gpu_roll_f32(x, 2, 4, 3, 1).view(2, 4, 3), torch.roll(x.view(2, 4, 3), 1, 1))
    up = G.gpu_nearest_upsample2x_f32(torch.arange(4.0), 1, 1, 2, 2).view(4, 4)
    assert up[0].tolist() == [0, 0, 1, 1] and up[3].tolist() == [2, 2, 3, 3]
    assert G.tensor_to_cpu(x) is x and G.round_len(1000) >= 1000


def test_pool_handles_memory_stats_watchdog_and_philox():
    class _Pool:
        handle = object()
    real = G.CapturePool
    G.CapturePool = _Pool                                    # pool handles are bookkeeping; the pool itself needs a device
    try:
        h1, h2 = G.graph_pool_handle(), G.graph_pool_handle()
        assert h1 != h2 and isinstance(G.capture_pool_for_handle(h1), _Pool) and G.capture_pool_for_handle(h1) is G.capture_pool_for_handle(h1)
        G.release_graph_pool_handle(h1)
        assert G.capture_pool_for_handle(h1) is None and G.capture_pool_for_handle(h2) is not None
    finally:
        G.CapturePool = real
    assert G.CaptureStatus.Active.is_capturing() and not G.CaptureStatus.Invalidated.is_capturing()
    with pytest.raises(FerrotorchError):
        G.end_capture(object())

    used = [100]
    guard = G.MemoryGuardBuilder().with_budget(1000).with_query(lambda: (used[0], 4000)).build()

    class Drop(G.MemoryHook):
        name, priority, calls = "drop-cache", 5, 0

        def on_pressure(self, need):
            Drop.calls += 1
            used[0] = 0
            return 100
    G.register_hook(guard, Drop())
    levels = []

    class L(G.MemoryPressureListener):
        def on_pressure_change(self, old, new):
            levels.append((old, new))
    guard.add_pressure_listener(L())
    r = guard.reserve(950)                                   # 100 used + 950 > budget: the hook frees the 100
    st = G.MemoryStats.of(guard)
    assert Drop.calls == 1 and st.budget_bytes == 1000 and st.total_device_bytes == 4000 and st.used_bytes >= 950 and st.peak_bytes >= 950
    r.release()
    dev = G.MemoryGuardedDevice("dev0", guard)
    assert dev.device() == "dev0" and dev.stats().budget_bytes == 1000

    free = [10_000]
    wd = G.MemoryWatchdog(lambda: (free[0], 100_000), pressure_threshold_bytes=5_000, check_interval_s=0.01)
    assert not wd.check_pressure() and wd.wait_if_paused(0.01)
    free[0] = 1_000
    assert wd.check_pressure() and wd.is_paused() and not wd.wait_if_paused(0.05)
    wd.start()
    woke = []
    t = threading.Thread(target=lambda: woke.append(wd.wait_if_paused(5.0)))
    t.start()
    free[0] = 50_000                                         # memory recovers: the polling thread lifts the pause
    t.join(5.0)
    wd.stop()
    assert woke == [True] and not wd.is_paused()

    p = G.PhiloxGenerator(1234)
    a = [p.next_u32() for _ in range(8)]
    st = p.get_state()
    b = [p.next_u32() for _ in range(4)]
    p.set_state(st)
    assert [p.next_u32() for _ in range(4)] == b and st.offset == 2 and len(set(a)) == 8
    q = G.PhiloxGenerator(1234)
    q.advance(1)
    assert [q.next_u32() for _ in range(4)] == a[4:]         # skipping one counter skips four draws
    q.set_seed(1234)
    u = q.generate_uniform(10_001)
    assert u.dtype == np.float32 and 0.0 <= u.min() and u.max() < 1.0 and abs(float(u.mean()) - 0.5) < 0.02 and q.get_state().offset == 2501
    assert 0.0 <= G.PhiloxGenerator(5).next_f32() < 1.0 and G.PhiloxGenerator(5).next_u32() != G.PhiloxGenerator(6).next_u32()
    # Philox-4x32-10 known-answer test (Random123 kat_vectors: zero counter / zero key, and the all-ones vector)
    z = G.api_ext._philox4x32(np.zeros((1, 4), np.uint32), (0, 0))[0].tolist()
    assert z == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    o = G.api_ext._philox4x32(np.full((1, 4), 0xFFFFFFFF, np.uint32), (0xFFFFFFFF, 0xFFFFFFFF))[0].tolist()
    assert o == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    with pytest.raises(ShapeMismatch):
        G.join_rng([0, 1], [G.PhiloxState(0, 0)])
    assert G.cuda_rng_manager() is G.rng_manager
