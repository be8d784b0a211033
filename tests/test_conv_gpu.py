"""Implicit-GEMM 3x3 convolution kernel against an f32 PyTorch convolution (forward, fused ReLU, data gradient, ragged patches)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,Cin,Cout,H,W", [(2, 64, 64, 56, 56), (3, 128, 128, 28, 28), (2, 256, 256, 14, 14), (4, 512, 512, 7, 7), (1, 64, 200, 19, 13),
                                            (1, 192, 24, 5, 40)])
def test_conv3x3_forward_and_input_gradient(N, Cin, Cout, H, W):
    from ferrotorch_b200 import _lib, ops
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(N, Cin, H, W, device="cuda", generator=g).bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_()
    w = (torch.randn(Cout, Cin, 3, 3, device="cuda", generator=g) * (2.0 / (9 * Cin)) ** 0.5).requires_grad_()
    y = ops.conv3x3(x, w)
    ref = F.conv2d(x.detach().float(), w.detach().bfloat16().float(), padding=1)
    assert y.shape == ref.shape and y.is_contiguous(memory_format=torch.channels_last)
    assert (y.float() - ref).abs().max() < 0.06, float((y.float() - ref).abs().max())
    dy = torch.randn(N, Cout, H, W, device="cuda", generator=g).bfloat16().contiguous(memory_format=torch.channels_last)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().bfloat16().float().requires_grad_()
    F.conv2d(xr, wr, padding=1).backward(dy.float())
    tol = 0.08 * max(1.0, float(xr.grad.abs().max()))
    assert (x.grad.float() - xr.grad).abs().max() < tol
    assert (w.grad - wr.grad).abs().max() < 0.05 * float(wr.grad.abs().max()) + 0.05
    yr = ops.conv3x3_nhwc_raw(x.detach(), w.detach().bfloat16().permute(0, 2, 3, 1).contiguous(), relu=True)
    assert (yr.float() - ref.relu()).abs().max() < 0.06
    assert _lib.read_status() == 0


def test_resnet_block_uses_the_kernel_and_matches_library_path():
    from ferrotorch_b200 import _lib
    from ferrotorch_b200.vision.models import BasicBlock
    torch.manual_seed(0)
    blk = BasicBlock(64, 64).cuda().to(memory_format=torch.channels_last)
    x = torch.randn(4, 64, 28, 28, device="cuda").contiguous(memory_format=torch.channels_last)
    l0 = _lib.launch_calls
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = blk(x)
    assert _lib.launch_calls > l0
    ref_blk = torch.nn.Sequential()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        o = torch.relu(F.batch_norm(F.conv2d(x, blk.conv1.weight, padding=1), None, None, blk.bn1.weight, blk.bn1.bias, True))
        o = F.batch_norm(F.conv2d(o, blk.conv2.weight, padding=1), None, None, blk.bn2.weight, blk.bn2.bias, True)
        ref = torch.relu(o + x)
    assert (y.float() - ref.float()).abs().max() < 0.1


@pytest.mark.parametrize("N,C,Co,H,W", [(4, 64, 64, 56, 56), (8, 128, 256, 14, 14), (2, 64, 128, 7, 9)])
def test_conv3x3_weight_gradient_as_shifted_gemms_on_device(N, C, Co, H, W):
    from ferrotorch_b200 import _lib, ops
    torch.manual_seed(C + H)
    x = torch.randn(N, C, H, W, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    dy = torch.randn(N, Co, H, W, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    got = ops.conv.conv3x3_wgrad_gemm(x, dy)
    ref = torch.nn.grad.conv2d_weight(x.float(), (Co, C, 3, 3), dy.float(), padding=1).permute(0, 2, 3, 1)
    assert (got - ref).abs().max().item() <= 2e-3 * ref.abs().max().item() + 1e-2
    assert _lib.read_status() == 0


@pytest.mark.parametrize("N,C,Co,H,W", [(4, 64, 64, 56, 56), (8, 128, 256, 14, 14), (2, 64, 128, 7, 9), (3, 256, 72, 5, 5)])
def test_conv3x3_weight_gradient_fused_gemm_on_device(N, C, Co, H, W):
    from ferrotorch_b200 import _lib, ops
    torch.manual_seed(C + W)
    x = torch.randn(N, C, H, W, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    dy = torch.randn(N, Co, H, W, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    got = ops.conv.conv3x3_wgrad_fused(x, dy)
    ref = torch.nn.grad.conv2d_weight(x.float(), (Co, C, 3, 3), dy.float(), padding=1).permute(0, 2, 3, 1)
    assert (got - ref).abs().max().item() <= 2e-3 * ref.abs().max().item() + 1e-2
    assert torch.equal(got, ops.conv.conv3x3_wgrad_fused(x, dy))            # planes summed in a fixed order
    assert _lib.read_status() == 0


@pytest.mark.parametrize("stride", [1, 2])
@pytest.mark.parametrize("N,C,Co,H,W", [(4, 64, 64, 56, 56), (8, 128, 256, 14, 14), (2, 256, 128, 6, 10)])
def test_conv3x3_rows_forward_and_gradients_on_device(N, C, Co, H, W, stride):
    from ferrotorch_b200 import _lib, ops
    torch.manual_seed(C + W + stride)
    x = (torch.randn(N, C, H, W, device="cuda") * 0.5).bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True)
    w = (torch.randn(Co, C, 3, 3, device="cuda") * 0.05).requires_grad_(True)
    y = ops.conv.conv3x3_autograd_rows(x, w, stride)
    g = torch.randn_like(y)
    y.backward(g)
    x2 = x.detach().float().requires_grad_(True)
    w2 = w.detach().bfloat16().float().requires_grad_(True)
    y2 = F.conv2d(x2, w2, stride=stride, padding=1)
    y2.backward(g.float())
    for got, ref, what in ((y, y2, "y"), (x.grad, x2.grad, "dx"), (w.grad, w2.grad, "dw")):
        err, scale = (got.float() - ref).abs().max().item(), ref.abs().max().item()
        assert err <= 2e-2 * scale + 2e-2, (what, err, scale)
    assert _lib.read_status() == 0


@pytest.mark.parametrize("N,C,H,W,Co,k,s,p", [(4, 3, 64, 48, 64, 7, 2, 3), (2, 3, 33, 35, 32, 7, 2, 3), (3, 1, 28, 28, 16, 5, 1, 2), (2, 4, 17, 19, 24, 3, 2, 1)])
def test_first_layer_convolution_as_patch_gemm(N, C, H, W, Co, k, s, p):
    """The few-input-channel route (patch matrix + tcgen05 GEMM, f32 weight gradient from the split-K form) against the f32 convolution."""
    import ferrotorch_b200.nn as nn
    from ferrotorch_b200.ops import conv as C_
    torch.manual_seed(0)
    conv = nn.Conv2d(C, Co, k, s, p, bias=False).cuda()
    x = torch.randn(N, C, H, W, device="cuda")
    assert C_.conv_stem_eligible(x.bfloat16(), conv.weight, conv.stride, conv.padding, conv.dilation, conv.groups)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = conv(x)
    assert y.dtype == torch.bfloat16 and y.is_contiguous(memory_format=torch.channels_last)
    wf = conv.weight.detach().bfloat16().float().requires_grad_()
    ref = torch.nn.functional.conv2d(x.bfloat16().float(), wf, None, s, p)
    assert y.shape == ref.shape and ((y.float() - ref).norm() / ref.norm()).item() < 1e-2
    g = torch.randn_like(ref)
    y.backward(g.to(y.dtype))
    ref.backward(g.bfloat16().float())
    assert conv.weight.grad.dtype == torch.float32 and ((conv.weight.grad - wf.grad).norm() / wf.grad.norm()).item() < 1e-2


def test_autocast_linear_with_f32_master_runs_on_the_package_gemm():
    import ferrotorch_b200.nn as nn
    torch.manual_seed(1)
    lin = nn.Linear(256, 1000).cuda()
    with torch.no_grad():
        lin.bias.uniform_(-0.5, 0.5)
    x = torch.randn(96, 256, device="cuda", requires_grad=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = lin(x)
    assert y.dtype == torch.bfloat16
    xr = x.detach().bfloat16().float().requires_grad_()
    wr = lin.weight.detach().bfloat16().float().requires_grad_()
    ref = torch.nn.functional.linear(xr, wr, lin.bias.detach().bfloat16().float())
    assert ((y.float() - ref).norm() / ref.norm()).item() < 1e-2
    g = torch.randn_like(ref)
    y.backward(g.to(y.dtype))
    ref.backward(g.bfloat16().float())
    assert lin.weight.grad.dtype == torch.float32 and ((lin.weight.grad - wr.grad).norm() / wr.grad.norm()).item() < 1e-2
    assert ((x.grad - xr.grad).norm() / xr.grad.norm()).item() < 1e-2 and ((lin.bias.grad - g.bfloat16().float().sum(0)).abs().max() < 0.1)
