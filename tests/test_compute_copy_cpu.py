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
