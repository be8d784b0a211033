"""``interpolate`` / ``affine_grid`` / ``grid_sample`` written out on gather arithmetic (``nn/resample.py``): every mode, size and scale-factor
form, corner alignment, padding mode and the gradients (input and grid) against PyTorch."""
import pytest
import torch

import ferrotorch_b200.nn as nn
from ferrotorch_b200.nn import resample as R

F = torch.nn.functional
D = torch.float64


def close(a, b, tol=1e-9, msg=""):
    assert a.shape == b.shape, (msg, a.shape, b.shape)
    assert torch.allclose(a, b, atol=tol, rtol=tol), (msg, (a - b).abs().max().item())


@pytest.mark.parametrize("shape,modes", [((2, 3, 9), ("nearest", "nearest-exact", "linear", "area")),
                                         ((2, 3, 7, 9), ("nearest", "nearest-exact", "bilinear", "bicubic", "area")),
                                         ((2, 2, 4, 5, 6), ("nearest", "nearest-exact", "trilinear", "area"))])
def test_interpolate_matches_pytorch_for_every_mode_size_and_factor(shape, modes):
    torch.manual_seed(0)
    x = torch.randn(shape, dtype=D)
    nsp = x.dim() - 2
    for mode in modes:
        for ac in ((False, True) if mode in ("linear", "bilinear", "bicubic", "trilinear") else (None,)):
            for size in ([5, 11, 4][:nsp], [13, 3, 9][:nsp], list(x.shape[2:])):
                close(R.interpolate(x, size=size, mode=mode, align_corners=ac), F.interpolate(x, size=size, mode=mode, align_corners=ac), msg=f"{mode} {size} {ac}")
            for sf in (2.0, 0.5, 1.7, [1.5, 2.0, 0.7][:nsp]):
                for rec in (None, True):
                    close(R.interpolate(x, scale_factor=sf, mode=mode, align_corners=ac, recompute_scale_factor=rec),
                          F.interpolate(x, scale_factor=sf, mode=mode, align_corners=ac, recompute_scale_factor=rec), msg=f"{mode} x{sf} {ac} {rec}")


def test_interpolate_gradients_dtypes_module_and_errors():
    torch.manual_seed(1)
    x = torch.randn(2, 3, 7, 9, dtype=D, requires_grad=True)
    w = torch.randn(2, 3, 11, 5, dtype=D)
    for mode, ac in (("bilinear", False), ("bicubic", True), ("nearest", None)):
        ga, = torch.autograd.grad((R.interpolate(x, size=(11, 5), mode=mode, align_corners=ac) * w).sum(), x)
        gb, = torch.autograd.grad((F.interpolate(x, size=(11, 5), mode=mode, align_corners=ac) * w).sum(), x)
        close(ga, gb, msg=mode)
    xf = x.detach().float()
    close(R.interpolate(xf, scale_factor=2, mode="bilinear"), F.interpolate(xf, scale_factor=2, mode="bilinear"), 1e-5)
    xi = torch.randint(0, 9, (1, 1, 4, 4), dtype=torch.uint8)
    assert torch.equal(R.interpolate(xi, scale_factor=2, mode="nearest"), F.interpolate(xi, scale_factor=2, mode="nearest"))
    close(nn.Upsample(scale_factor=2, mode="bilinear", align_corners=False)(xf), torch.nn.Upsample(scale_factor=2, mode="bilinear", align_corners=False)(xf), 1e-5)
    close(nn.functional.interpolate(xf, size=(3, 4), mode=nn.InterpolateMode.Bicubic if hasattr(nn, "InterpolateMode") else "bicubic"),
          F.interpolate(xf, size=(3, 4), mode="bicubic"), 1e-5)
    assert nn.interpolate is R.interpolate and nn.functional.grid_sample is R.grid_sample
    for bad in (lambda: R.interpolate(xf), lambda: R.interpolate(xf, size=4, scale_factor=2), lambda: R.interpolate(xf, size=(4, 4), mode="linear"),
                lambda: R.interpolate(xf, size=(4, 4), mode="nearest", align_corners=True), lambda: R.interpolate(xf, size=(4, 4), mode="cubic"),
                lambda: R.interpolate(torch.randn(3, 4), size=2)):
        with pytest.raises(Exception):
            bad()


def test_affine_grid_and_grid_sample_match_pytorch():
    torch.manual_seed(2)
    for ac in (False, True):
        th = torch.randn(2, 2, 3, dtype=D)
        close(R.affine_grid(th, (2, 3, 5, 7), ac), F.affine_grid(th, (2, 3, 5, 7), ac), 1e-12)
        th3 = torch.randn(2, 3, 4, dtype=D)
        close(R.affine_grid(th3, (2, 3, 4, 5, 6), ac), F.affine_grid(th3, (2, 3, 4, 5, 6), ac), 1e-12)
    img = torch.randn(2, 3, 6, 7, dtype=D)
    grid = torch.rand(2, 5, 4, 2, dtype=D) * 2.8 - 1.4                               # a third of the samples fall outside the image
    grid[0, 0, 0], grid[0, 0, 1], grid[0, 1, 0] = torch.tensor([-1.0, 1.0], dtype=D), torch.tensor([1.0, -1.0], dtype=D), torch.tensor([0.0, 0.0], dtype=D)
    for mode in ("bilinear", "nearest", "bicubic"):
        for pad in ("zeros", "border", "reflection"):
            for ac in (False, True):
                close(R.grid_sample(img, grid, mode, pad, ac), F.grid_sample(img, grid, mode=mode, padding_mode=pad, align_corners=ac), msg=f"{mode} {pad} {ac}")
    gi, gg, wo = img.clone().requires_grad_(), grid.clone().requires_grad_(), torch.randn(2, 3, 5, 4, dtype=D)
    for pad in ("zeros", "border", "reflection"):
        a = torch.autograd.grad((R.grid_sample(gi, gg, "bilinear", pad, False) * wo).sum(), (gi, gg))
        b = torch.autograd.grad((F.grid_sample(gi, gg, mode="bilinear", padding_mode=pad, align_corners=False) * wo).sum(), (gi, gg))
        close(a[0], b[0], msg="input gradient " + pad)
        close(a[1], b[1], 1e-8, "grid gradient " + pad)
    ident = torch.tensor([[[1.0, 0, 0], [0, 1.0, 0]]], dtype=D).expand(2, 2, 3)
    close(R.grid_sample(img, R.affine_grid(ident, img.shape)), img, 1e-12)          # the identity map reproduces the image
    for bad in (lambda: R.affine_grid(torch.randn(2, 3, 3), (2, 1, 4, 4)), lambda: R.grid_sample(img, grid[:1]), lambda: R.grid_sample(img, grid, "linear")):
        with pytest.raises(Exception):
            bad()
