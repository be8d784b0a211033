"""Convolution layers (ferrotorch-nn/src/conv.rs:288-3554, lazy_conv.rs, lazy_conv_transpose.rs).

Parameters, initialisation (Kaiming-uniform with the ReLU gain, zero bias: conv.rs:384), padding modes and output-size rules are
stated here. bf16 channels-last CUDA inputs of the two shapes that dominate vision nets run on this package's kernels: 3x3 stride-1
pad-1 on the implicit-GEMM tcgen05 kernel and 1x1 as one GEMM over the pixel rows; the remaining shapes are evaluated by the
library convolution primitive."""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple, Union

import torch
import torch.nn.functional as F

from .. import ops
from ..errors import InvalidArgument, ShapeMismatch
from .module import Module, Parameter

_Size = Union[int, Sequence[int]]


def _tup(v: _Size, n: int, what: str) -> Tuple[int, ...]:
    if isinstance(v, int):
        return (v,) * n
    v = tuple(int(i) for i in v)
    if len(v) != n:
        raise InvalidArgument(f"{what}: expected {n} values, got {len(v)}")
    return v


class _ConvNd(Module):
    _nd = 2
    _transposed = False

    def __init__(self, in_channels: int, out_channels: int, kernel_size: _Size, stride: _Size = 1, padding: Union[_Size, str] = 0,
                 dilation: _Size = 1, groups: int = 1, bias: bool = True, padding_mode: str = "zeros", device=None, dtype=None,
                 output_padding: _Size = 0):
        super().__init__()
        n = self._nd
        if hasattr(padding_mode, "value"):
            padding_mode = {"constant": "zeros"}.get(padding_mode.value, padding_mode.value)
        if groups <= 0 or in_channels % groups or out_channels % groups:
            raise InvalidArgument(f"in_channels {in_channels} and out_channels {out_channels} must be divisible by groups {groups}")
        if padding_mode not in ("zeros", "reflect", "replicate", "circular"):
            raise InvalidArgument(f"unknown padding_mode {padding_mode!r}")
        self.in_channels, self.out_channels, self.groups, self.padding_mode = in_channels, out_channels, groups, padding_mode
        self.kernel_size = _tup(kernel_size, n, "kernel_size")
        self.stride = _tup(stride, n, "stride")
        self.dilation = _tup(dilation, n, "dilation")
        self.output_padding = _tup(output_padding, n, "output_padding")
        self.transposed = self._transposed
        if any(k <= 0 for k in self.kernel_size) or any(s <= 0 for s in self.stride) or any(d <= 0 for d in self.dilation):
            raise InvalidArgument("kernel_size, stride and dilation must be positive")
        if isinstance(padding, str):
            if padding not in ("same", "valid"):
                raise InvalidArgument(f"padding must be 'same', 'valid' or integers, got {padding!r}")
            if self._transposed:
                raise InvalidArgument("string padding is not defined for transposed convolution")
            if padding == "same" and any(s != 1 for s in self.stride):
                raise InvalidArgument("padding='same' needs stride 1")
            self.padding = padding
        else:
            self.padding = _tup(padding, n, "padding")
        if self._transposed:
            if padding_mode != "zeros":
                raise InvalidArgument("transposed convolution supports zero padding only")
            shape = (in_channels, out_channels // groups, *self.kernel_size)
        else:
            shape = (out_channels, in_channels // groups, *self.kernel_size)
        self.weight = Parameter(torch.empty(shape, device=device, dtype=dtype))
        self.bias = Parameter(torch.zeros(out_channels, device=device, dtype=dtype)) if bias else None
        self.reset_parameters()

    def reset_parameters(self) -> None:
        # U(-b, b), b = gain * sqrt(3 / fan_in), gain = sqrt(2); fan_in counts dimension 1 and the window, as for the forward layout
        fan_in = self.weight.shape[1] * math.prod(self.kernel_size)
        bound = math.sqrt(2.0) * math.sqrt(3.0 / max(1, fan_in))
        with torch.no_grad():
            self.weight.uniform_(-bound, bound)
            if self.bias is not None:
                self.bias.zero_()

    def _explicit_pad(self, x: torch.Tensor) -> torch.Tensor:
        """Non-zero padding modes pad the input first; the convolution then runs unpadded."""
        from .padding import pad_nd
        if isinstance(self.padding, str):
            pads = self._same_pads()
        else:
            pads = [(p, p) for p in self.padding]
        return pad_nd(x, pads, self.padding_mode)

    def _same_pads(self):
        out = []
        for k, d in zip(self.kernel_size, self.dilation):
            total = d * (k - 1)
            out.append((total // 2, total - total // 2))
        return out

    def extra_repr(self) -> str:
        s = f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, stride={self.stride}"
        if self.padding != (0,) * self._nd:
            s += f", padding={self.padding}"
        if self.dilation != (1,) * self._nd:
            s += f", dilation={self.dilation}"
        if self.groups != 1:
            s += f", groups={self.groups}"
        if self.bias is None:
            s += ", bias=False"
        return s

    def _check(self, x: torch.Tensor) -> torch.Tensor:
        n = self._nd
        if x.dim() not in (n + 1, n + 2):
            raise ShapeMismatch(f"{type(self).__name__} expects a {n + 1}-D or {n + 2}-D input, got {list(x.shape)}")
        cin = x.shape[-n - 1]
        if cin != self.in_channels:
            raise ShapeMismatch(f"{type(self).__name__}: input has {cin} channels, the layer was built for {self.in_channels}")
        return x

    # forward convolution ------------------------------------------------------------------------------------------------------------
    def _conv(self, x, w, b, padding):
        fn = (F.conv1d, F.conv2d, F.conv3d)[self._nd - 1]
        return fn(x, w, b, self.stride, padding, self.dilation, self.groups)

    def _conv_forward(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
        if self.padding_mode != "zeros":
            return self._conv(self._explicit_pad(x), weight, bias, 0)
        if self.padding == "same":
            pads = self._same_pads()
            if any(a != b_ for a, b_ in pads):                # even window: one more on the right, applied explicitly
                from .padding import pad_nd
                return self._conv(pad_nd(x, pads, "zeros"), weight, bias, 0)
            return self._conv(x, weight, bias, tuple(a for a, _ in pads))
        return self._conv(x, weight, bias, 0 if self.padding == "valid" else self.padding)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._conv_forward(self._check(x), self.weight, self.bias)


class Conv1d(_ConvNd):
    _nd = 1


class Conv3d(_ConvNd):
    _nd = 3


class Conv2d(_ConvNd):
    _nd = 2

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self._check(x)
        w = self.weight
        if x.is_cuda and x.dim() == 4 and self.padding_mode == "zeros" and not isinstance(self.padding, str):
            if torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16:
                x = x.to(torch.bfloat16)
            if x.dtype == torch.bfloat16 and self.bias is None and ops.conv.conv_stem_eligible(x, w, self.stride, self.padding, self.dilation, self.groups):
                return ops.conv.conv_stem(x, w, self.stride, self.padding)              # few input channels: patch matrix + GEMM
            if x.dtype == torch.bfloat16 and x.is_contiguous(memory_format=torch.channels_last):
                if ops.conv.conv3x3_eligible(x, w, self.stride, self.padding, self.dilation, self.groups):
                    y = ops.conv3x3(x, w)
                    return y if self.bias is None else y + self.bias.to(y.dtype).view(1, -1, 1, 1)
                if self.kernel_size == (1, 1) and self.padding == (0, 0) and self.groups == 1 and x.shape[1] % 8 == 0 \
                        and self.out_channels % 8 == 0:
                    if self.stride != (1, 1):
                        x = x[:, :, :: self.stride[0], :: self.stride[1]].contiguous(memory_format=torch.channels_last)
                    N, C, H, W = x.shape
                    rows = x.permute(0, 2, 3, 1).reshape(N * H * W, C)
                    y = ops.linear(rows, w.to(torch.bfloat16).view(self.out_channels, C),
                                   None if self.bias is None else self.bias.to(torch.bfloat16))
                    return y.view(N, H, W, self.out_channels).permute(0, 3, 1, 2)
            if x.dtype != w.dtype:
                return self._conv_forward(x, w.to(x.dtype), None if self.bias is None else self.bias.to(x.dtype))
        return self._conv_forward(x, w, self.bias)


# transposed ----------------------------------------------------------------------------------------------------------------------------
class _ConvTransposeNd(_ConvNd):
    _transposed = True

    def __init__(self, in_channels: int, out_channels: int, kernel_size: _Size, stride: _Size = 1, padding: _Size = 0,
                 output_padding: _Size = 0, groups: int = 1, bias: bool = True, dilation: _Size = 1, padding_mode: str = "zeros",
                 device=None, dtype=None):
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias, padding_mode, device, dtype,
                         output_padding)
        for op, s, d in zip(self.output_padding, self.stride, self.dilation):
            if op >= max(s, d):
                raise InvalidArgument("output_padding must be smaller than stride or dilation")

    def output_size(self, in_size: Sequence[int]) -> Tuple[int, ...]:
        """``(in - 1) * stride - 2 * pad + dilation * (k - 1) + output_padding + 1`` per spatial dimension."""
        return tuple((i - 1) * s - 2 * p + d * (k - 1) + op + 1
                     for i, s, p, d, k, op in zip(in_size, self.stride, self.padding, self.dilation, self.kernel_size, self.output_padding))

    def _output_padding_for(self, x: torch.Tensor, output_size: Optional[Sequence[int]]) -> Tuple[int, ...]:
        if output_size is None:
            return self.output_padding
        want = tuple(output_size)[-self._nd:]
        base = tuple((i - 1) * s - 2 * p + d * (k - 1) + 1
                     for i, s, p, d, k in zip(x.shape[-self._nd:], self.stride, self.padding, self.dilation, self.kernel_size))
        extra = tuple(w - b for w, b in zip(want, base))
        for e, s, d in zip(extra, self.stride, self.dilation):
            if e < 0 or e >= max(s, d):
                raise InvalidArgument(f"requested output size {list(want)} is not reachable from input {list(x.shape[-self._nd:])}")
        return extra

    def forward(self, x: torch.Tensor, output_size: Optional[Sequence[int]] = None) -> torch.Tensor:
        x = self._check(x)
        fn = (F.conv_transpose1d, F.conv_transpose2d, F.conv_transpose3d)[self._nd - 1]
        return fn(x, self.weight, self.bias, self.stride, self.padding, self._output_padding_for(x, output_size), self.groups, self.dilation)


class ConvTranspose1d(_ConvTransposeNd):
    _nd = 1


class ConvTranspose2d(_ConvTransposeNd):
    _nd = 2


class ConvTranspose3d(_ConvTransposeNd):
    _nd = 3


# lazy ----------------------------------------------------------------------------------------------------------------------------------
class _Lazy(Module):
    """Builds the wrapped layer at the first call, reading ``in_channels`` from the input (lazy_conv.rs, lazy_conv_transpose.rs)."""
    _cls = None

    def __init__(self, out_channels: int, kernel_size: _Size, *args, **kwargs):
        super().__init__()
        self.out_channels = out_channels
        self._ctor = (kernel_size, args, kwargs)
        self.inner: Optional[Module] = None

    def is_initialized(self) -> bool:
        return self.inner is not None

    def materialize(self, in_channels: int, device=None, dtype=None) -> Module:
        if self.inner is None:
            k, a, kw = self._ctor
            kw = dict(kw)
            kw.setdefault("device", device)
            kw.setdefault("dtype", dtype)
            self.inner = self._cls(in_channels, self.out_channels, k, *a, **kw)
        return self.inner

    def forward(self, x, *a, **k):
        n = self._cls._nd
        if x.dim() not in (n + 1, n + 2):
            raise ShapeMismatch(f"{type(self).__name__} expects a {n + 1}-D or {n + 2}-D input, got {list(x.shape)}")
        return self.materialize(x.shape[-n - 1], x.device, x.dtype)(x, *a, **k)


class LazyConv1d(_Lazy):
    _cls = Conv1d


class LazyConv2d(_Lazy):
    _cls = Conv2d


class LazyConv3d(_Lazy):
    _cls = Conv3d


class LazyConvTranspose1d(_Lazy):
    _cls = ConvTranspose1d


class LazyConvTranspose2d(_Lazy):
    _cls = ConvTranspose2d


class LazyConvTranspose3d(_Lazy):
    _cls = ConvTranspose3d


__all__ = ["Conv1d", "Conv2d", "Conv3d", "ConvTranspose1d", "ConvTranspose2d", "ConvTranspose3d", "LazyConv1d", "LazyConv2d", "LazyConv3d",
           "LazyConvTranspose1d", "LazyConvTranspose2d", "LazyConvTranspose3d"]
