"""tcgen05 GEMM against an f32 PyTorch reference, every operand-layout combination, ragged sizes."""
import os

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


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("act", [None, "relu", "gelu", "gelu_tanh", "silu"])
def test_gemm_epilogue_activation_residual_and_fp16(dtype, act):
    from ferrotorch_b200 import ops
    import torch.nn.functional as F
    g = torch.Generator(device="cuda").manual_seed(0)
    M, N, K = 300, 520, 264
    a, b = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(dtype), (torch.randn(N, K, device="cuda", generator=g) * 0.5).to(dtype)
    bias, res = torch.randn(N, device="cuda", generator=g).to(dtype), torch.randn(M, N, device="cuda", generator=g).to(dtype)
    out = ops.gemm(a, b, bias=bias, act=act, residual=res)
    ref = a.float() @ b.float().t() + bias.float()
    ref = {None: lambda t: t, "relu": F.relu, "gelu": F.gelu, "gelu_tanh": lambda t: F.gelu(t, approximate="tanh"), "silu": F.silu}[act](ref) + res.float()
    assert out.dtype == dtype and (out.float() - ref).abs().max() < (0.08 if dtype == torch.bfloat16 else 0.02)
    o32 = ops.gemm(a, b, act=act, out_dtype=torch.float32, residual=res.float())
    ref32 = {None: lambda t: t, "relu": F.relu, "gelu": F.gelu, "gelu_tanh": lambda t: F.gelu(t, approximate="tanh"), "silu": F.silu}[act](a.float() @ b.float().t()) + res.float()
    assert (o32 - ref32).abs().max() < 2e-3


def test_exact_gemm_gemv_and_split_k_path():
    from ferrotorch_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(1)
    for dtype, tol in ((torch.float32, 2e-4), (torch.float64, 1e-11)):
        a, b = torch.randn(3, 70, 45, device="cuda", generator=g).to(dtype), torch.randn(3, 45, 90, device="cuda", generator=g).to(dtype)
        assert (ops.matmul_exact(a, b) - a @ b).abs().max() < tol
        assert (ops.matmul_exact(a.transpose(1, 2).contiguous().transpose(1, 2), b.transpose(1, 2).contiguous().transpose(1, 2)) - a @ b).abs().max() < tol
        assert (ops.matmul_exact(a[0], b) - a[0] @ b).abs().max() < tol                       # broadcast over the batch
        m, x = torch.randn(77, 130, device="cuda", generator=g).to(dtype), torch.randn(130, device="cuda", generator=g).to(dtype)
        assert (ops.mv(m, x) - m @ x).abs().max() < tol * 10 and (ops.mv(m, torch.ones(77, device="cuda", dtype=dtype), trans=True) - m.sum(0)).abs().max() < tol * 10
        assert abs(float(ops.dot(x, x)) - float((x * x).sum())) < tol * 100
    # weight-gradient shape: tiny output, very long K -> split over the SMs
    dy, x = (torch.randn(200_000, 64, device="cuda", generator=g) * 0.1).bfloat16(), (torch.randn(200_000, 256, device="cuda", generator=g) * 0.1).bfloat16()
    from ferrotorch_b200.ops.gemm import _auto_splits
    assert _auto_splits(64, 256, 200_000) > 1
    dw = ops.gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32)
    ref = dy.float().t() @ x.float()
    assert (dw - ref).abs().max() < 0.05 * ref.abs().max().clamp_min(1)
    bb = ops.bmm(torch.randn(4, 128, 64, device="cuda", generator=g).bfloat16(), torch.randn(4, 64, 96, device="cuda", generator=g).bfloat16())
    assert bb.shape == (4, 128, 96)


@pytest.mark.skipif(os.environ.get("FT_GEMM_TAIL") != "1", reason="tail slices are opt-in (FT_GEMM_TAIL=1)")
@pytest.mark.parametrize("M,N,K,f32_out", [(4096, 4096, 512, False), (4096, 6144, 1024, False), (4096, 4096, 768, True), (4000, 4072, 520, False)])
def test_gemm_tail_slices_match_unsplit(M, N, K, f32_out):
    """Output-tile counts that leave a short last round: the K-sliced tail tiles must reproduce the unsplit result (f32 sums in a different
    order: equal up to rounding of the output dtype) and stay deterministic."""
    from ferrotorch_b200 import _lib
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    res = torch.randn(M, N, device="cuda").to(torch.float32 if f32_out else torch.bfloat16)
    kw = dict(bias=bias, residual=res, act="relu", out_dtype=torch.float32 if f32_out else None)
    _lib.call("ft_gemm_set_tail", 0)
    try:
        plain = ops.gemm(a, b, **kw)
        _lib.call("ft_gemm_set_tail", 1)
        t1 = ops.gemm(a, b, **kw)
        t2 = ops.gemm(a, b, **kw)
    finally:
        _lib.call("ft_gemm_set_tail", 1)
    assert _lib.read_status() == 0
    assert torch.equal(t1, t2)
    ref = torch.relu(a.float() @ b.float().t() + bias.float()) + res.float()
    scale = ref.abs().max().item()
    assert (t1.float() - ref).abs().max().item() <= (2e-3 if f32_out else 1e-2) * scale + 1e-2
    assert (t1.float() - plain.float()).abs().max().item() <= (1e-5 if f32_out else 8e-3) * scale
