"""bf16 compute copies of f32 master weights: kept in step by the optimizer, refreshed when the master changes elsewhere, and used by the
master-weight autograd functions (checked here on the host against plain cast-per-step training)."""
import copy

import pytest
import torch

from ferrotorch_b200 import nn, ops, optim
from ferrotorch_b200.nn.compute_copy import compute_copy, optimizer_target


def test_copy_tracks_optimizer_steps_and_outside_changes():
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(8, 4, 3, 3).contiguous(memory_format=torch.channels_last))
    b = torch.nn.Parameter(torch.zeros(8))
    assert nn.attach_compute_copies([w, b]) == 1 and compute_copy(b) is None
    c = compute_copy(w)
    assert c.dtype == torch.bfloat16 and c.stride() == w.stride() and torch.equal(c, w.detach().bfloat16())
    opt = optim.Sgd([w, b], lr=0.1, momentum=0.9, weight_decay=1e-4)
    ref_w = w.detach().clone().contiguous()
    ref = torch.optim.SGD([torch.nn.Parameter(ref_w)], lr=0.1, momentum=0.9, weight_decay=1e-4)
    for step in range(3):
        g = torch.randn(8, 4, 3, 3)                      # contiguous gradient for a channels-last parameter: re-ordered inside the step
        w.grad, b.grad = g.clone(), torch.ones(8)
        ref.param_groups[0]["params"][0].grad = g.clone()
        opt.step()
        ref.step()
        assert torch.allclose(w.detach(), ref.param_groups[0]["params"][0].detach(), atol=1e-6)
        assert torch.equal(optimizer_target(w), w.detach().bfloat16())       # the copy was written in the same pass
    with torch.no_grad():
        w.mul_(2.0)                                       # a change behind the optimizer's back
    assert torch.equal(compute_copy(w), w.detach().bfloat16())
    w.data = w.data.contiguous()                          # re-laid-out: the copy follows
    assert compute_copy(w).stride() == w.stride()
    w.grad = torch.randn(8, 4, 3, 3)
    opt.step()                                            # the momentum buffer is re-ordered to the new layout
    nn.detach_compute_copies([w])
    assert compute_copy(w) is None


def test_linear_master_matches_cast_per_step():
    torch.manual_seed(1)
    x = torch.randn(64, 32).bfloat16()
    w = torch.nn.Parameter(torch.randn(16, 32) * 0.1)
    bias = torch.nn.Parameter(torch.randn(16) * 0.1)
    nn.attach_compute_copies([w])
    y = ops.linear_master(x, w, compute_copy(w), bias.bfloat16())
    y.float().square().mean().backward()
    gw, gb = w.grad.clone(), bias.grad.clone()
    assert gw.dtype == torch.float32 and gw.shape == w.shape
    w.grad = bias.grad = None
    y2 = torch.nn.functional.linear(x.float(), w.bfloat16().float(), bias.bfloat16().float())
    y2.to(torch.bfloat16).float().square().mean().backward()
    assert torch.allclose(gw, w.grad, rtol=2e-2, atol=2e-3) and torch.allclose(gb, bias.grad, rtol=2e-2, atol=2e-3)


def test_conv3x3_master_matches_reference_and_trains():
    torch.manual_seed(2)
    x = torch.randn(2, 64, 8, 8).bfloat16().contiguous(memory_format=torch.channels_last)
    w = torch.nn.Parameter((torch.randn(16, 64, 3, 3) * 0.05).contiguous(memory_format=torch.channels_last))
    nn.attach_compute_copies([w])
    xr = x.clone().requires_grad_(True)
    y = ops.conv.conv3x3_master(xr, w, compute_copy(w))
    assert y.dtype == torch.bfloat16 and y.is_contiguous(memory_format=torch.channels_last)
    y.float().square().mean().backward()
    assert w.grad.dtype == torch.float32 and w.grad.stride() == w.stride()
    w2 = w.detach().clone().requires_grad_(True)
    x2 = x.float().requires_grad_(True)
    y2 = torch.nn.functional.conv2d(x2, w2.bfloat16().float(), padding=1)
    assert torch.allclose(y.float(), y2, rtol=2e-2, atol=2e-2)
    y2.to(torch.bfloat16).float().square().mean().backward()
    assert torch.allclose(w.grad, w2.grad, rtol=3e-2, atol=3e-3)
    assert torch.allclose(xr.grad.float(), x2.grad, rtol=5e-2, atol=5e-3)
    opt = optim.Sgd([w], lr=0.01, momentum=0.9)
    before = w.detach().clone()
    opt.step()
    assert not torch.equal(before, w.detach()) and torch.equal(compute_copy(w), w.detach().bfloat16())


def test_linear_module_uses_the_copy_under_autocast_and_training_follows_the_plain_run():
    """An MLP with f32 masters under bf16 autocast, trained with and without compute copies: same losses up to bf16 rounding of the weight
    gradients, f32 gradients on the masters, copies equal to the rounded masters after every step."""
    def run(copies: bool):
        torch.manual_seed(4)
        m = nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 8))
        if copies:
            assert nn.attach_compute_copies(m) == 2
        opt = optim.Sgd(m.parameters(), lr=0.05, momentum=0.9)
        g = torch.Generator().manual_seed(5)
        x, y = torch.randn(64, 32, generator=g), torch.randint(0, 8, (64,), generator=g)
        losses = []
        for _ in range(5):
            opt.zero_grad()
            with torch.autocast("cpu", dtype=torch.bfloat16):
                loss = torch.nn.functional.cross_entropy(m(x).float(), y)
            loss.backward()
            assert all(p.grad.dtype == torch.float32 for p in m.parameters())
            opt.step()
            losses.append(float(loss.detach()))
            if copies:
                for p in m.parameters():
                    if p.dim() == 2:
                        assert torch.equal(compute_copy(p), p.detach().bfloat16())
        return losses
    plain, shadow = run(False), run(True)
    assert shadow[-1] < shadow[0]
    assert all(abs(a - b) < 0.05 for a, b in zip(plain, shadow)), (plain, shadow)


def test_adamw_keeps_the_copy_in_step_and_matches_torch():
    torch.manual_seed(6)
    w = torch.nn.Parameter(torch.randn(16, 8))
    ref = torch.nn.Parameter(w.detach().clone())
    nn.attach_compute_copies([w])
    a, b = optim.AdamW([w], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1), torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    for _ in range(4):
        g = torch.randn(16, 8)
        w.grad, ref.grad = g.clone(), g.clone()
        a.step()
        b.step()
        assert torch.allclose(w.detach(), ref.detach(), atol=1e-6)
        assert torch.equal(compute_copy(w), w.detach().bfloat16())


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
