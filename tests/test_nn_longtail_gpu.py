"""CUDA routes of the long-tail layers: element-wise activation kernels (contiguous and channels-last), fused batch norm, the two convolution
shapes that run on this package's kernels, the fused recurrent cells and channels-last max pooling, each against PyTorch evaluated in f32."""
import pytest
import torch

import ferrotorch_b200.nn as nn

pytestmark = pytest.mark.gpu
tnn = torch.nn


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("name,tname,kw", [("ReLU", "ReLU", {}), ("Sigmoid", "Sigmoid", {}), ("Tanh", "Tanh", {}), ("SiLU", "SiLU", {}), ("Mish", "Mish", {}),
                                           ("ELU", "ELU", {"alpha": 1.3}), ("LeakyReLU", "LeakyReLU", {"negative_slope": 0.2}),
                                           ("Softplus", "Softplus", {"beta": 2.0, "threshold": 3.0}), ("HardSwish", "Hardswish", {}),
                                           ("Hardtanh", "Hardtanh", {"min_val": -0.5, "max_val": 0.8}), ("ReLU6", "ReLU6", {}), ("GELU", "GELU", {})])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("channels_last", [False, True])
def test_activation_kernels_forward_backward(name, tname, kw, dtype, channels_last):
    torch.manual_seed(0)
    x = (torch.randn(4, 16, 9, 7, device="cuda") * 3).to(dtype)
    for kink in (-3.0, -0.5, 0.0, 0.8, 3.0, 6.0):          # at a kink the one-sided derivative is a convention: keep the inputs off them
        x = torch.where((x.float() - kink).abs() < 0.06, x + 0.125, x)
    if channels_last:
        x = x.contiguous(memory_format=torch.channels_last)
    a = x.clone().requires_grad_()
    b = x.float().clone().requires_grad_()
    ya, yb = getattr(nn, name)(**kw)(a), getattr(tnn, tname)(**kw)(b)
    assert ya.dtype == dtype and ya.stride() == a.stride()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert _rel(ya, yb) < tol
    w = torch.randn_like(yb)
    (ya.float() * w).sum().backward()
    (yb * w).sum().backward()
    assert a.grad.stride() == a.stride() and _rel(a.grad, b.grad) < tol


def test_batch_norm2d_channels_last_matches_torch_in_train_and_eval():
    torch.manual_seed(1)
    ours, theirs = nn.BatchNorm2d(32).cuda(), tnn.BatchNorm2d(32).cuda()
    with torch.no_grad():
        theirs.weight.uniform_(0.5, 1.5)
        theirs.bias.uniform_(-0.5, 0.5)
    ours.load_state_dict(theirs.state_dict())
    for _ in range(3):
        x = (torch.randn(8, 32, 14, 14, device="cuda") * 2 + 1).contiguous(memory_format=torch.channels_last)
        a, b = x.clone().requires_grad_(), x.clone().requires_grad_()
        ya, yb = ours(a), theirs(b)
        assert _rel(ya, yb) < 1e-4
        w = torch.randn_like(yb)
        (ya * w).sum().backward()
        (yb * w).sum().backward()
        assert _rel(a.grad, b.grad) < 1e-3
    assert _rel(ours.running_mean, theirs.running_mean) < 1e-4 and _rel(ours.running_var, theirs.running_var) < 1e-4
    assert int(ours.num_batches_tracked) == 3
    ours.eval(), theirs.eval()
    assert _rel(ours(x), theirs(x)) < 1e-4
    # NCHW input takes the written-out statistics
    xn = torch.randn(4, 32, 5, 5, device="cuda")
    ours.train(), theirs.train()
    assert _rel(ours(xn), theirs(xn)) < 1e-4


@pytest.mark.parametrize("k,stride,cin,cout", [(3, 1, 64, 128), (1, 1, 64, 96), (1, 2, 64, 96)])
def test_conv2d_kernel_routes_match_f32_convolution(k, stride, cin, cout):
    torch.manual_seed(2)
    conv = nn.Conv2d(cin, cout, k, stride, k // 2, bias=True).cuda().to(torch.bfloat16)
    with torch.no_grad():
        conv.bias.uniform_(-0.5, 0.5)
    x = torch.randn(2, cin, 20, 18, device="cuda", dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    a = x.clone().requires_grad_()
    y = conv(a)
    b = x.float().clone().requires_grad_()
    wf = conv.weight.detach().float().requires_grad_()
    ref = torch.nn.functional.conv2d(b, wf, conv.bias.float(), stride, k // 2)
    assert y.shape == ref.shape and _rel(y, ref) < 1e-2
    w = torch.randn_like(ref)
    (y.float() * w).sum().backward()
    (ref * w).sum().backward()
    assert _rel(a.grad, b.grad) < 2e-2
    assert _rel(conv.weight.grad, wf.grad) < 2e-2


@pytest.mark.parametrize("name", ["LSTM", "GRU"])
def test_recurrent_layers_on_fused_cells_match_host_evaluation(name):
    """The device path (one GEMM for the input projections, fused cell kernels per step) against the same layer evaluated on the host in f32
    (the library's device RNN runs its GEMMs in TF32, which is looser than what is checked here)."""
    torch.manual_seed(3)
    kw = dict(num_layers=2, bidirectional=True)
    theirs = getattr(tnn, name)(24, 32, **kw)
    ours = getattr(nn, name)(24, 32, **kw)
    ours.load_state_dict(theirs.state_dict())
    ours = ours.cuda()
    x = torch.randn(9, 5, 24)
    a, b = x.cuda().requires_grad_(), x.clone().requires_grad_()
    (ya, sa), (yb, sb) = ours(a), theirs(b)
    assert _rel(ya.cpu(), yb) < 1e-5
    w = torch.randn_like(yb)
    (ya * w.cuda()).sum().backward()
    (yb * w).sum().backward()
    assert _rel(a.grad.cpu(), b.grad) < 1e-4
    for (n, pa), (_, pb) in zip(ours.named_parameters(), theirs.named_parameters()):
        assert _rel(pa.grad.cpu(), pb.grad) < 1e-4, n


def test_max_pool2d_channels_last_kernel_and_window_views_agree():
    torch.manual_seed(4)
    x = torch.randn(4, 16, 15, 13, device="cuda").contiguous(memory_format=torch.channels_last)
    a, b = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya = nn.MaxPool2d(3, 2, 1)(a)                           # channels-last kernel
    yb = tnn.MaxPool2d(3, 2, 1)(b)
    assert torch.equal(ya, yb)
    ya.sum().backward(), yb.sum().backward()
    assert torch.equal(a.grad, b.grad)
    yc = nn.MaxPool2d(3, 2, 1, ceil_mode=True)(x)           # window views
    assert torch.equal(yc, tnn.MaxPool2d(3, 2, 1, ceil_mode=True)(x))


def test_derivatives_at_the_kinks_follow_pytorch():
    """Exactly at a kink the derivative is a convention; the kernels take PyTorch's (outer pieces at the hard-swish kinks, no gradient at the
    bounds of hardtanh / ReLU6, zero at the origin of ReLU)."""
    x = torch.tensor([-3.0, 3.0, 0.0, 6.0, -1.0, 1.0, 7.0, -4.0], device="cuda")
    for ours, theirs in ((nn.HardSwish(), tnn.Hardswish()), (nn.ReLU6(), tnn.ReLU6()), (nn.Hardtanh(-3.0, 3.0), tnn.Hardtanh(-3.0, 3.0)), (nn.ReLU(), tnn.ReLU())):
        for dtype in (torch.float32, torch.bfloat16):
            a, b = x.clone().to(dtype).requires_grad_(), x.clone().to(dtype).requires_grad_()
            ya, yb = ours(a), theirs(b)
            tol = 1e-6 if dtype == torch.float32 else 1e-2
            assert torch.allclose(ya.float(), yb.float(), atol=tol), type(ours).__name__
            ya.sum().backward()
            yb.sum().backward()
            assert torch.equal(a.grad[:4], b.grad[:4]), (type(ours).__name__, a.grad.tolist(), b.grad.tolist())       # the four kink points
            assert torch.allclose(a.grad.float(), b.grad.float(), atol=tol)


def test_global_average_pool_channels_last_kernel_route():
    torch.manual_seed(5)
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        x = torch.randn(6, 32, 7, 5, device="cuda").to(dtype).contiguous(memory_format=torch.channels_last)
        a, b = x.clone().requires_grad_(), x.float().clone().requires_grad_()
        ya, yb = nn.AdaptiveAvgPool2d(1)(a), tnn.AdaptiveAvgPool2d(1)(b)
        assert ya.shape == (6, 32, 1, 1) and torch.allclose(ya.float(), yb, atol=tol)
        w = torch.randn_like(yb)
        (ya.float() * w).sum().backward()
        (yb * w).sum().backward()
        assert a.grad.is_contiguous(memory_format=torch.channels_last) and torch.allclose(a.grad.float(), b.grad, atol=tol)
