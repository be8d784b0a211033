"""tcgen05 GEMM against an f32 PyTorch reference, every operand-layout combination, ragged sizes."""
import pytest
import torch

from ferrotorch_b200 import ops

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn, bias=None):
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    r = A @ B
    if bias is not None:
        r = r + bias.float()
    return r


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (200, 328, 136), (1024, 1024, 1024), (72, 8, 8)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    torch.manual_seed(M * 7 + N * 3 + K)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda").to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda").to(torch.bfloat16)
    d = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    ref = _ref(a, b, a_mn, b_mn)
    err = (d.float() - ref).abs().max().item()
    tol = 0.02 * ref.abs().max().item() + 1e-2
    assert err <= tol, f"max err {err} > {tol}"


def test_gemm_f32_out_and_bias():
    torch.manual_seed(0)
    M, N, K = 384, 520, 320
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    d = ops.gemm(a, b, bias=bias, out_dtype=torch.float32)
    ref = _ref(a, b, False, False, bias)
    assert d.dtype == torch.float32
    assert (d - ref).abs().max().item() <= 2e-3 * ref.abs().max().item() + 1e-3


def test_gemm_deterministic_and_large():
    torch.manual_seed(1)
    M, N, K = 2048, 4096, 2048
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    d1 = ops.gemm(a, b)
    d2 = ops.gemm(a, b)
    assert torch.equal(d1, d2)
    ref = (a.float() @ b.float().t())
    rel = (d1.float() - ref).norm() / ref.norm()
    assert rel.item() < 5e-3


def test_linear_autograd_matches_reference():
    torch.manual_seed(2)
    x = torch.randn(4, 96, 256, device="cuda").to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(512, 256, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    bias = torch.randn(512, device="cuda").to(torch.bfloat16).requires_grad_(True)
    y = ops.linear(x, w, bias)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, bias))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    for got, ref in ((y, yr), (x.grad, xr.grad), (w.grad, wr.grad), (bias.grad, br.grad)):
        rel = (got.float() - ref).norm() / (ref.norm() + 1e-6)
        assert rel.item() < 1e-2
