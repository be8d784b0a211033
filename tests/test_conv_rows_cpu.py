"""3x3 convolutions expressed through the GEMM's row-shift tables, checked on the host against torch.nn.functional.conv2d and its gradients:
weight gradient as nine shifted products (stride 1 and 2), the producer's atom arithmetic of the fused launch, forward and input gradient as
row GEMMs on the padded (stride 2: parity-split) activation."""
import pytest
import torch

from ferrotorch_b200 import ops


@pytest.mark.parametrize("N,C,Co,H,W", [(2, 8, 16, 5, 7), (3, 16, 8, 4, 4), (1, 8, 8, 1, 1), (2, 8, 8, 3, 9)])
def test_conv3x3_weight_gradient_as_shifted_gemms(N, C, Co, H, W):
    """dW of a padded 3x3 convolution = nine products of the zero-padded output gradient with row-shifted views of the zero-padded input."""
    torch.manual_seed(N + C + H)
    x = torch.randn(N, C, H, W).bfloat16().contiguous(memory_format=torch.channels_last)
    dy = torch.randn(N, Co, H, W).bfloat16().contiguous(memory_format=torch.channels_last)
    got = ops.conv.conv3x3_wgrad_gemm(x, dy)
    ref = torch.nn.grad.conv2d_weight(x.float(), (Co, C, 3, 3), dy.float(), padding=1).permute(0, 2, 3, 1)
    assert got.shape == (Co, 3, 3, C) and got.dtype == torch.float32
    assert torch.allclose(got, ref, rtol=1e-5, atol=1e-4)


def test_row_shift_table_of_the_fused_weight_gradient_gemm():
    """Host restatement of what the GEMM's producer does for the fused 3x3 weight gradient: 64-channel atom g of the N axis belongs to tap
    g // atoms_per_tap, reads channel block g % atoms_per_tap of the padded input at rows k + (r-1) * pitch + (s-1) (zeros outside, zeros for
    atoms past the ninth tap); the [Cout, 9 Cin] product must be the convolution's weight gradient in [Cout, 3, 3, Cin] order."""
    torch.manual_seed(11)
    N, C, Co, H, W = 2, 128, 16, 5, 6
    x = torch.randn(N, C, H, W).bfloat16().contiguous(memory_format=torch.channels_last)
    dy = torch.randn(N, Co, H, W).bfloat16().contiguous(memory_format=torch.channels_last)
    xp = torch.nn.functional.pad(x.permute(0, 2, 3, 1), (0, 0, 1, 1, 1, 1)).reshape(-1, C).float()
    dyp = torch.nn.functional.pad(dy.permute(0, 2, 3, 1), (0, 0, 1, 1, 1, 1)).reshape(-1, Co).float()
    J, apt, pitch = xp.shape[0], C // 64, W + 2
    n_tiles = -(-9 * C // 256)
    out = torch.zeros(Co, n_tiles * 256)
    for n0 in range(0, n_tiles * 256, 256):
        for j in range(4):
            g = n0 // 64 + j
            tap = g // apt
            if tap >= 9:
                continue                                             # zero-filled box
            col = (g % apt) * 64
            shift = (tap // 3 - 1) * pitch + (tap % 3 - 1)
            b = torch.zeros(J, 64)
            lo, hi = max(0, -shift), J - max(0, shift)
            b[lo:hi] = xp[lo + shift: hi + shift, col: col + 64]
            out[:, n0 + j * 64: n0 + (j + 1) * 64] = dyp.t() @ b
    got = out[:, : 9 * C].reshape(Co, 3, 3, C)
    ref = torch.nn.grad.conv2d_weight(x.float(), (Co, C, 3, 3), dy.float(), padding=1).permute(0, 2, 3, 1)
    assert torch.allclose(got, ref, rtol=1e-5, atol=1e-4)
    from ferrotorch_b200.ops.conv import _wgrad_splits
    for co, ci, j in [(64, 64, 861184), (128, 128, 230400), (512, 512, 20736), (8, 64, 100)]:
        s = _wgrad_splits(co, ci, j)
        nkb = -(-j // 64)
        assert 1 <= s <= 64 and (s == 1 or -(-nkb // s) * (s - 1) < nkb)


@pytest.mark.parametrize("stride", [1, 2])
@pytest.mark.parametrize("N,C,Co,H,W", [(2, 64, 16, 6, 8), (1, 128, 8, 4, 4), (3, 64, 24, 2, 10)])
def test_conv3x3_as_one_row_gemm(N, C, Co, H, W, stride):
    """Stride 1 and stride 2 convolutions as a sum of row-shifted products on the padded (for stride 2: parity-split) activation."""
    torch.manual_seed(N * 7 + H + stride)
    x = torch.randn(N, C, H, W).bfloat16().contiguous(memory_format=torch.channels_last)
    w = (torch.randn(Co, C, 3, 3) * 0.1).bfloat16()
    bias = torch.randn(Co).bfloat16()
    y = ops.conv.conv3x3_rows(x, w.permute(0, 2, 3, 1).contiguous(), stride=stride, bias=bias, relu=True)
    ref = torch.relu(torch.nn.functional.conv2d(x.float(), w.float(), bias.float(), stride=stride, padding=1))
    assert y.shape == ref.shape and y.is_contiguous(memory_format=torch.channels_last)
    assert torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("stride", [1, 2])
def test_conv3x3_weight_gradient_by_row_shifts_both_strides(stride):
    torch.manual_seed(20 + stride)
    N, C, Co, H, W = 2, 64, 16, 6, 8
    x = torch.randn(N, C, H, W).bfloat16().contiguous(memory_format=torch.channels_last)
    dy = torch.randn(N, Co, H // stride, W // stride).bfloat16().contiguous(memory_format=torch.channels_last)
    got = ops.conv.conv3x3_wgrad_fused(x, dy, stride=stride)
    ref = torch.nn.grad.conv2d_weight(x.float(), (Co, C, 3, 3), dy.float(), stride=stride, padding=1).permute(0, 2, 3, 1)
    assert got.shape == (Co, 3, 3, C) and torch.allclose(got, ref, rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("stride", [1, 2])
def test_conv3x3_rows_autograd_matches_reference(stride):
    """Forward, input gradient (stride 2: one product per pixel-parity plane) and weight gradient of the row-GEMM convolution."""
    torch.manual_seed(30 + stride)
    N, C, Co, H, W = 2, 64, 64, 6, 8
    x = (torch.randn(N, C, H, W) * 0.5).bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True)
    w = (torch.randn(Co, C, 3, 3) * 0.05).requires_grad_(True)
    y = ops.conv.conv3x3_autograd_rows(x, w, stride)
    g = torch.randn_like(y)
    y.backward(g)
    x2 = x.detach().float().requires_grad_(True)
    w2 = w.detach().bfloat16().float().requires_grad_(True)
    y2 = torch.nn.functional.conv2d(x2, w2, stride=stride, padding=1)
    y2.backward(g.float())
    assert torch.allclose(y.float(), y2, rtol=2e-2, atol=2e-2)
    assert torch.allclose(x.grad.float(), x2.grad, rtol=3e-2, atol=3e-2)
    assert w.grad.dtype == torch.float32 and torch.allclose(w.grad, w2.grad, rtol=2e-2, atol=2e-2)


def test_row_shift_launchers_refuse_bad_arguments_before_touching_the_device():
    """Argument checks of the new launchers run on the host (no GPU needed): misaligned channel counts, too many taps, missing tables."""
    import ctypes
    from ferrotorch_b200 import _lib
    from ferrotorch_b200.errors import FerrotorchError
    buf = torch.zeros(64 * 64, dtype=torch.bfloat16)
    out = torch.zeros(64 * 9 * 64, dtype=torch.float32)
    shifts = (ctypes.c_int * 9)(*range(9))
    for args in (("ft_conv_rows_gemm", buf, buf, buf, None, 64, 64, 63, 64, 9, shifts, 0, 0),          # Cin not a multiple of 64
                 ("ft_conv_rows_gemm", buf, buf, buf, None, 64, 64, 64, 64, 10, shifts, 0, 0),         # more than nine taps
                 ("ft_conv_rows_gemm", buf, buf, buf, None, 64, 64, 64, 60, 9, shifts, 0, 0),          # Cout not a multiple of 8
                 ("ft_conv_rows_gemm", buf, buf, buf, None, 64, 64, 64, 64, 9, None, 0, 0),            # no shift table
                 ("ft_conv3x3_wgrad_splitk", buf, buf, out, 64, 96, 64, 10, 1, 0),                      # Cin not a multiple of 64
                 ("ft_conv3x3_wgrad_splitk", buf, buf, out, 64, 64, 64, 2, 1, 0),                       # row pitch below 3
                 ("ft_conv_wgrad_shift_splitk", buf, buf, out, 64, 64, 64, 0, shifts, 1, 0)):           # B without rows
        with pytest.raises(FerrotorchError, match="invalid argument"):
            _lib.call(*args)
