"""Device path of the buffer-level API: the wrappers that route to this framework's kernels against f32 PyTorch references, and explicit
begin / end stream capture."""
import os

import pytest
import torch

from ferrotorch_b200 import gpu as G

pytestmark = [pytest.mark.gpu]


def test_kernel_backed_wrappers_match_f32_references():
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(256, 512, device=dev, generator=g).bfloat16()
    w = (torch.rand(512, device=dev, generator=g) + 0.5).bfloat16()
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    assert (G.gpu_rmsnorm_bf16(x.reshape(-1), w, 256, 512, 1e-5).view(256, 512).float() - ref).abs().max() < 0.06
    b = torch.randn(512, device=dev, generator=g).bfloat16()
    ln = torch.nn.functional.layer_norm(x.float(), (512,), w.float(), b.float(), 1e-5)
    assert (G.gpu_layernorm(x.reshape(-1), w, b, 256, 512, 1e-5).view(256, 512).float() - ln).abs().max() < 0.08
    A = torch.randn(256, 512, device=dev, generator=g).bfloat16()
    Wt = torch.randn(384, 512, device=dev, generator=g).bfloat16()
    want = A.float() @ Wt.float().t()
    got = G.gpu_matmul_bf16_bf16_nt(A.reshape(-1), Wt.reshape(-1), 256, 512, 384).view(256, 384).float()
    assert (got - want).abs().max() / want.abs().max() < 0.02
    got2 = G.gpu_matmul_bf16_bf16(A.reshape(-1), Wt.t().contiguous().reshape(-1), 256, 512, 384).view(256, 384).float()
    assert (got2 - want).abs().max() / want.abs().max() < 0.02
    table = torch.randn(1000, 256, device=dev, generator=g).bfloat16()
    idx = torch.randint(0, 1000, (77,), device=dev, generator=g, dtype=torch.int32)
    assert torch.equal(G.gpu_embedding_gather_bf16(table.reshape(-1), idx, 256).view(77, 256), table[idx.long()])
    f = torch.randn(1 << 16, device=dev, generator=g)
    assert torch.equal(G.gpu_add(f, f), f + f) and torch.allclose(G.gpu_softmax(f, 64, 1024).view(64, 1024), f.view(64, 1024).softmax(-1), atol=1e-6)
    with pytest.raises(Exception):
        G.gpu_add(f.cpu(), f.cpu())
    d = G.gpu_dropout(f, 1 << 31, 2.0, 3)
    assert torch.equal(d, G.gpu_dropout(f, 1 << 31, 2.0, 3)) and abs(float((d != 0).float().mean()) - 0.5) < 0.02
    sms = G.get_cuda_device(0).sm_count
    assert int(sms() if callable(sms) else sms) > 0 and G.cached_bytes() >= 0


def test_explicit_capture_replays_the_recorded_work():
    dev = "cuda"
    a, b, out = torch.ones(1024, device=dev), torch.full((1024,), 2.0, device=dev), torch.zeros(1024, device=dev)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        G.gpu_add_into(a, b, out)                             # warm-up outside the capture
    torch.cuda.synchronize()
    h = G.graph_pool_handle()
    assert G.capture_status(side) is G.CaptureStatus.None_
    G.begin_capture_with_mode(side, G.CaptureMode.THREAD_LOCAL, G.capture_pool_for_handle(h))
    assert G.is_stream_capturing(side)
    G.gpu_add_into(a, b, out)
    graph = G.end_capture_with_pool(side, G.capture_pool_for_handle(h))
    assert not G.is_stream_capturing(side)
    a.fill_(5.0)
    graph.launch()
    torch.cuda.synchronize()
    assert float(out[0]) == 7.0 and graph.launches == 1
    G.release_graph_pool_handle(h)
    with pytest.raises(Exception):
        G.end_capture(side)


def test_buffer_transfers_small_math_and_plain_capture():
    dev = G.cuda_default()
    assert isinstance(dev, G.GpuDevice) and dev.sm_count > 0 and dev.total_memory > 0
    z = G.alloc_zeros(1000)
    assert isinstance(z, G.CudaBuffer) and z.tensor().is_cuda and float(z.tensor().abs().sum()) == 0 and z.device_ptr() != 0
    assert G.alloc_zeros_f32(8).tensor().dtype == torch.float32 and G.alloc_zeros_f64(8).tensor().dtype == torch.float64
    z.release()
    h = torch.arange(16.0)
    d = G.cpu_to_gpu(h)
    dp = G.cpu_to_gpu_pinned(h)
    torch.cuda.synchronize()
    assert d.is_cuda and torch.equal(d.cpu(), h) and torch.equal(dp.cpu(), h) and G.tensor_to_gpu(d) is d and G.tensor_to_gpu(h).is_cuda
    back = G.gpu_to_cpu(d, pinned=True)
    assert back.is_pinned() and torch.equal(back, h) and torch.equal(G.gpu_to_cpu(d), h)
    a, b = torch.randn(512, device="cuda"), torch.randn(512, device="cuda")
    out = torch.empty(512, device="cuda")
    G.gpu_mul_into(a, b, out)
    assert torch.equal(out, a * b)
    assert torch.equal(G.gpu_mul_bf16(a.bfloat16(), b.bfloat16()), a.bfloat16() * b.bfloat16())
    assert torch.allclose(G.gpu_gelu(a), torch.nn.functional.gelu(a), atol=1e-6)
    A, B = torch.randn(8 * 16, device="cuda"), torch.randn(16 * 4, device="cuda")
    mm = torch.empty(8 * 4, device="cuda")
    G.gpu_small_matmul_into(A, B, mm, 8, 16, 4)
    assert torch.allclose(mm.view(8, 4), A.view(8, 16) @ B.view(16, 4), atol=1e-4)
    bA, bB = torch.randn(3 * 8 * 16, device="cuda"), torch.randn(3 * 16 * 4, device="cuda")
    bo = torch.empty(3 * 8 * 4, device="cuda")
    G.gpu_bmm_f32_into(bA, bB, bo, 3, 8, 16, 4)
    assert torch.allclose(bo.view(3, 8, 4), torch.bmm(bA.view(3, 8, 16), bB.view(3, 16, 4)), atol=1e-4)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        G.gpu_mul_into(a, b, out)
    torch.cuda.synchronize()
    G.begin_capture(side)
    G.gpu_mul_into(a, b, out)
    graph = G.end_capture(side)
    assert isinstance(graph, G.CapturedGraph)
    a.fill_(2.0)
    graph.launch()
    torch.cuda.synchronize()
    assert torch.equal(out, 2.0 * b)
    assert G.StreamPriority.HIGH < G.StreamPriority.NORMAL
