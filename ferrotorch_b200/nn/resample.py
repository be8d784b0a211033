"""Resampling written out on gather / index arithmetic: ``interpolate`` (nearest, nearest-exact, linear, bilinear, bicubic, trilinear, area),
``affine_grid`` and ``grid_sample`` (bilinear, nearest, bicubic; zeros / border / reflection padding). Each output sample is a weighted sum of
gathered input samples, so values and gradients (with respect to the input and, for ``grid_sample``, the grid) come from ordinary tensor
operations on any device.

Reference parity: ferrotorch-nn/src/upsample.rs:140 (interpolate), :672 (Upsample), :757 (grid_sample), :1139 (affine_grid); conventions
(half-pixel centres, ``align_corners``, the A = -0.75 cubic kernel, index clamping) are PyTorch's, against which the tests compare.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from ..errors import InvalidArgument


def _enum_value(m):
    return getattr(m, "value", m)


# ---------------------------------------------------------------------------------------------------------------------
# interpolate
# ---------------------------------------------------------------------------------------------------------------------
def _source_positions(n_in: int, n_out: int, align: bool, scale: Optional[float], device, cubic: bool = False) -> torch.Tensor:
    """Continuous input coordinate of every output sample along one dimension."""
    dst = torch.arange(n_out, dtype=torch.float64, device=device)
    if align:
        return dst * ((n_in - 1) / (n_out - 1) if n_out > 1 else 0.0)
    ratio = (1.0 / scale) if scale else n_in / n_out
    src = (dst + 0.5) * ratio - 0.5
    return src if cubic else src.clamp(min=0.0)


def _linear_taps(n_in, n_out, align, scale, device):
    src = _source_positions(n_in, n_out, align, scale, device)
    i0 = src.floor().clamp(max=n_in - 1).long()
    i1 = (i0 + 1).clamp(max=n_in - 1)
    w1 = (src - i0.to(src.dtype)).clamp(0.0, 1.0)
    return [(i0, 1.0 - w1), (i1, w1)]


def _cubic_weights(t: torch.Tensor, a: float = -0.75) -> List[torch.Tensor]:
    """Weights of the four taps at offsets -1, 0, 1, 2 for the fractional position ``t`` (Keys' kernel)."""
    def near(x):                                     # |x| <= 1
        return ((a + 2.0) * x - (a + 3.0)) * x * x + 1.0

    def far(x):                                      # 1 < |x| < 2
        return ((a * x - 5.0 * a) * x + 8.0 * a) * x - 4.0 * a
    return [far(t + 1.0), near(t), near(1.0 - t), far(2.0 - t)]


def _cubic_taps(n_in, n_out, align, scale, device):
    src = _source_positions(n_in, n_out, align, scale, device, cubic=True)
    base = src.floor()
    ws = _cubic_weights(src - base)
    return [((base.long() + k - 1).clamp(0, n_in - 1), w) for k, w in enumerate(ws)]


def _nearest_taps(n_in, n_out, scale, device, exact: bool):
    dst = torch.arange(n_out, dtype=torch.float64, device=device)
    ratio = (1.0 / scale) if scale else n_in / n_out
    src = ((dst + 0.5) * ratio).floor() if exact else (dst * ratio).floor()
    return [(src.long().clamp(max=n_in - 1), None)]


def _apply_taps(x: torch.Tensor, dim: int, taps) -> torch.Tensor:
    out = None
    shape = [1] * x.dim()
    for idx, w in taps:
        part = x.index_select(dim, idx)
        if w is not None:
            shape[dim] = idx.shape[0]
            part = part * w.to(x.dtype).reshape(shape)
        out = part if out is None else out + part
    return out


def interpolate(x: torch.Tensor, size=None, scale_factor=None, mode="nearest", align_corners: Optional[bool] = None, recompute_scale_factor: Optional[bool] = None,
                antialias: bool = False) -> torch.Tensor:
    """Resizes the spatial dimensions of ``x`` [N, C, *spatial]. One of ``size`` / ``scale_factor`` is given; with ``scale_factor`` the sampling
    positions use the factor itself (not the ratio of the rounded sizes) unless ``recompute_scale_factor``."""
    mode = _enum_value(mode)
    nsp = x.dim() - 2
    if nsp < 1 or nsp > 3:
        raise InvalidArgument("interpolate takes [N, C, L], [N, C, H, W] or [N, C, D, H, W]")
    if antialias:
        return torch.nn.functional.interpolate(x, size=size, scale_factor=scale_factor, mode=mode, align_corners=align_corners,
                                               recompute_scale_factor=recompute_scale_factor, antialias=True)
    if (size is None) == (scale_factor is None):
        raise InvalidArgument("interpolate: give exactly one of size and scale_factor")
    in_sizes = list(x.shape[2:])
    scales: List[Optional[float]] = [None] * nsp
    if size is not None:
        out_sizes = [int(size)] * nsp if isinstance(size, int) else [int(s) for s in size]
    else:
        fs = [float(scale_factor)] * nsp if not isinstance(scale_factor, (tuple, list)) else [float(f) for f in scale_factor]
        if len(fs) != nsp:
            raise InvalidArgument("interpolate: one scale factor per spatial dimension")
        out_sizes = [int(math.floor(n * f)) for n, f in zip(in_sizes, fs)]
        if not recompute_scale_factor:
            scales = fs
    if len(out_sizes) != nsp or any(o < 1 for o in out_sizes):
        raise InvalidArgument("interpolate: one positive output size per spatial dimension")
    linear_modes = {"linear": 1, "bilinear": 2, "trilinear": 3}
    if mode in linear_modes or mode == "bicubic":
        want = linear_modes.get(mode, 2)
        if nsp != want:
            raise InvalidArgument(f"interpolate: mode '{mode}' takes {want} spatial dimension(s), the input has {nsp}")
        align = bool(align_corners)
    elif mode in ("nearest", "nearest-exact", "area"):
        if align_corners is not None:
            raise InvalidArgument(f"interpolate: align_corners does not apply to mode '{mode}'")
        align = False
    else:
        raise InvalidArgument(f"interpolate: unknown mode '{mode}'")
    if mode == "area":
        from . import pooling as _pool
        fn = {1: _pool.adaptive_avg_pool1d, 2: _pool.adaptive_avg_pool2d, 3: _pool.adaptive_avg_pool3d}[nsp]
        return fn(x, out_sizes[0] if nsp == 1 else tuple(out_sizes))
    floating = x.is_floating_point()
    y = x if floating or mode.startswith("nearest") else x.to(torch.get_default_dtype())
    for d in range(nsp):
        n_in, n_out = in_sizes[d], out_sizes[d]
        if mode == "bicubic":
            taps = _cubic_taps(n_in, n_out, align, scales[d], x.device)
        elif mode in linear_modes:
            taps = _linear_taps(n_in, n_out, align, scales[d], x.device)
        else:
            taps = _nearest_taps(n_in, n_out, scales[d], x.device, exact=mode == "nearest-exact")
        y = _apply_taps(y, 2 + d, taps)
    return y


# ---------------------------------------------------------------------------------------------------------------------
# affine_grid / grid_sample
# ---------------------------------------------------------------------------------------------------------------------
def _base_coords(n: int, align: bool, dtype, device) -> torch.Tensor:
    """Normalised pixel-centre coordinates in [-1, 1] of a dimension of ``n`` samples."""
    if n <= 1:
        return torch.zeros(n, dtype=dtype, device=device)
    lin = torch.linspace(-1.0, 1.0, n, dtype=dtype, device=device)
    return lin if align else lin * ((n - 1) / n)


def affine_grid(theta: torch.Tensor, size: Sequence[int], align_corners: bool = False) -> torch.Tensor:
    """Sampling grid [N, H, W, 2] (or [N, D, H, W, 3]) of the affine maps ``theta`` [N, 2, 3] (or [N, 3, 4]) over an output of ``size``."""
    size = tuple(int(s) for s in size)
    if len(size) == 4 and tuple(theta.shape) == (size[0], 2, 3):
        _, _, h, w = size
        xs, ys = _base_coords(w, align_corners, theta.dtype, theta.device), _base_coords(h, align_corners, theta.dtype, theta.device)
        base = torch.stack([xs.expand(h, w), ys.unsqueeze(1).expand(h, w), torch.ones(h, w, dtype=theta.dtype, device=theta.device)], -1)       # [H, W, 3]
        return torch.einsum("hwk,nck->nhwc", base, theta)
    if len(size) == 5 and tuple(theta.shape) == (size[0], 3, 4):
        _, _, d, h, w = size
        xs, ys, zs = (_base_coords(n, align_corners, theta.dtype, theta.device) for n in (w, h, d))
        base = torch.stack([xs.expand(d, h, w), ys.view(1, h, 1).expand(d, h, w), zs.view(d, 1, 1).expand(d, h, w),
                            torch.ones(d, h, w, dtype=theta.dtype, device=theta.device)], -1)
        return torch.einsum("dhwk,nck->ndhwc", base, theta)
    raise InvalidArgument(f"affine_grid: theta {tuple(theta.shape)} does not fit size {size} ([N, 2, 3] with [N, C, H, W] or [N, 3, 4] with [N, C, D, H, W])")


def _unnormalise(g: torch.Tensor, n: int, align: bool) -> torch.Tensor:
    return (g + 1.0) * 0.5 * (n - 1) if align else ((g + 1.0) * n - 1.0) * 0.5


def _reflect(c: torch.Tensor, lo: float, hi: float) -> torch.Tensor:
    """Folds a coordinate into [lo, hi] by reflection at both ends."""
    span = hi - lo
    if span <= 0:
        return torch.zeros_like(c)
    c = (c - lo).abs()
    flips = (c / span).floor()
    extra = c - flips * span
    return torch.where(flips.remainder(2) == 0, extra + lo, span - extra + lo)


def _pad_coords(c: torch.Tensor, n: int, padding: str, align: bool) -> torch.Tensor:
    if padding == "border":
        return c.clamp(0, n - 1)
    if padding == "reflection":
        c = _reflect(c, 0.0, float(n - 1)) if align else _reflect(c, -0.5, n - 0.5)
        return c.clamp(0, n - 1)
    return c


def _gather2d(x: torch.Tensor, iy: torch.Tensor, ix: torch.Tensor, zeros: bool) -> torch.Tensor:
    """x [N, C, H, W] sampled at integer positions iy, ix [N, Ho, Wo]: [N, C, Ho, Wo]; out-of-range taps give 0 (``zeros``) or the clamped pixel."""
    n, c, h, w = x.shape
    inside = (iy >= 0) & (iy < h) & (ix >= 0) & (ix < w)
    flat = (iy.clamp(0, h - 1) * w + ix.clamp(0, w - 1)).view(n, 1, -1).expand(n, c, -1)
    out = x.reshape(n, c, h * w).gather(2, flat).view(n, c, *iy.shape[1:])
    return out * inside.unsqueeze(1).to(x.dtype) if zeros else out


def grid_sample(x: torch.Tensor, grid: torch.Tensor, mode="bilinear", padding_mode="zeros", align_corners: bool = False) -> torch.Tensor:
    """Samples ``x`` [N, C, H, W] at the normalised positions ``grid`` [N, Ho, Wo, 2] (x then y in [-1, 1])."""
    mode, padding = _enum_value(mode), _enum_value(padding_mode)
    if x.dim() != 4 or grid.dim() != 4:
        return torch.nn.functional.grid_sample(x, grid, mode=mode, padding_mode=padding, align_corners=align_corners)       # volumetric inputs: the library
    if grid.shape[0] != x.shape[0] or grid.shape[-1] != 2:
        raise InvalidArgument(f"grid_sample: grid {tuple(grid.shape)} does not fit input {tuple(x.shape)}")
    if mode not in ("bilinear", "nearest", "bicubic") or padding not in ("zeros", "border", "reflection"):
        raise InvalidArgument(f"grid_sample: unknown mode '{mode}' or padding '{padding}'")
    h, w = x.shape[2], x.shape[3]
    gx, gy = _unnormalise(grid[..., 0], w, align_corners), _unnormalise(grid[..., 1], h, align_corners)
    zeros = padding == "zeros"
    if mode == "bicubic":
        fx, fy = gx.floor(), gy.floor()
        wx, wy = _cubic_weights(gx - fx), _cubic_weights(gy - fy)
        out = 0
        for j in range(4):
            for i in range(4):
                cx = _pad_coords(fx + (i - 1), w, padding, align_corners).long()
                cy = _pad_coords(fy + (j - 1), h, padding, align_corners).long()
                out = out + _gather2d(x, cy, cx, zeros) * (wx[i] * wy[j]).unsqueeze(1).to(x.dtype)
        return out
    gx, gy = _pad_coords(gx, w, padding, align_corners), _pad_coords(gy, h, padding, align_corners)
    if mode == "nearest":
        return _gather2d(x, torch.round(gy).long(), torch.round(gx).long(), zeros)
    x0, y0 = gx.floor(), gy.floor()
    tx, ty = (gx - x0).unsqueeze(1).to(x.dtype), (gy - y0).unsqueeze(1).to(x.dtype)
    x0, y0 = x0.long(), y0.long()
    v00, v01 = _gather2d(x, y0, x0, zeros), _gather2d(x, y0, x0 + 1, zeros)
    v10, v11 = _gather2d(x, y0 + 1, x0, zeros), _gather2d(x, y0 + 1, x0 + 1, zeros)
    return (v00 * (1 - tx) + v01 * tx) * (1 - ty) + (v10 * (1 - tx) + v11 * tx) * ty
