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
