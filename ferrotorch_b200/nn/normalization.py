"""Batch, group, instance and local-response normalisation (ferrotorch-nn/src/norm.rs:48-2400, lazy_norm.rs).

The statistics, the running-average rule (biased variance to normalise, unbiased into the running buffer, cumulative average when
``momentum`` is None) and the affine step are written here. Channels-last CUDA activations of 2-D batch norm and CUDA group norm run on this
package's fused kernels."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..errors import InvalidArgument, ShapeMismatch
from .module import Module, Parameter


def batch_norm(x, running_mean, running_var, weight=None, bias=None, training: bool = False, momentum: Optional[float] = 0.1, eps: float = 1e-5,
               num_batches_tracked: Optional[torch.Tensor] = None):
    """Normalises over every dimension but 1. While training the batch statistics are used and folded into the running buffers."""
    if x.dim() < 2:
        raise ShapeMismatch(f"batch_norm expects at least 2 dimensions, got {list(x.shape)}")
    C = x.shape[1]
    dims = [d for d in range(x.dim()) if d != 1]
    shape = [1, C] + [1] * (x.dim() - 2)
    use_batch = training or running_mean is None or running_var is None
    if use_batch:
        n = x.numel() // max(1, C)
        if training and n <= 1:
            raise InvalidArgument(f"batch_norm needs more than one value per channel while training, got input {list(x.shape)}")
        xf = x.float() if x.dtype in (torch.bfloat16, torch.float16) else x
        mean = xf.mean(dims)
        var = ((xf - mean.view(shape)) ** 2).mean(dims)
        if training and running_mean is not None and running_var is not None:
            with torch.no_grad():
                if num_batches_tracked is not None:
                    num_batches_tracked.add_(1)
                f = momentum if momentum is not None else 1.0 / float(num_batches_tracked.item() if num_batches_tracked is not None else 1)
                running_mean.mul_(1 - f).add_(mean.detach().to(running_mean.dtype), alpha=f)
                running_var.mul_(1 - f).add_((var.detach() * (n / max(1, n - 1))).to(running_var.dtype), alpha=f)
    else:
        xf = x.float() if x.dtype in (torch.bfloat16, torch.float16) else x
        mean, var = running_mean.to(xf.dtype), running_var.to(xf.dtype)
    y = (xf - mean.view(shape)) * torch.rsqrt(var.view(shape) + eps)
    if weight is not None:
        y = y * weight.to(y.dtype).view(shape)
    if bias is not None:
        y = y + bias.to(y.dtype).view(shape)
    return y.to(x.dtype)


class _BatchNorm(Module):
    _dims = (2, 3)

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: Optional[float] = 0.1, affine: bool = True, track_running_stats: bool = True,
                 device=None, dtype=None):
        super().__init__()
        if num_features <= 0:
            raise InvalidArgument("num_features must be positive")
        self.num_features, self.eps, self.momentum, self.affine, self.track_running_stats = num_features, eps, momentum, affine, track_running_stats
        if affine:
            self.weight = Parameter(torch.ones(num_features, device=device, dtype=dtype))
            self.bias = Parameter(torch.zeros(num_features, device=device, dtype=dtype))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)
        if track_running_stats:
            self.register_buffer("running_mean", torch.zeros(num_features, device=device, dtype=dtype))
            self.register_buffer("running_var", torch.ones(num_features, device=device, dtype=dtype))
            self.register_buffer("num_batches_tracked", torch.zeros((), dtype=torch.long, device=device))
        else:
            self.register_buffer("running_mean", None)
            self.register_buffer("running_var", None)
            self.register_buffer("num_batches_tracked", None)

    def reset_running_stats(self) -> None:
        if self.track_running_stats:
            self.running_mean.zero_()
            self.running_var.fill_(1)
            self.num_batches_tracked.zero_()

    def reset_parameters(self) -> None:
        self.reset_running_stats()
        if self.affine:
            with torch.no_grad():
                self.weight.fill_(1)
                self.bias.zero_()

    def _check(self, x):
        if x.dim() not in self._dims:
            raise ShapeMismatch(f"{type(self).__name__} expects {' or '.join(str(d) + '-D' for d in self._dims)} input, got {list(x.shape)}")
        if x.shape[1] != self.num_features:
            raise ShapeMismatch(f"{type(self).__name__}: input has {x.shape[1]} channels, the layer was built for {self.num_features}")

    def forward(self, x):
        self._check(x)
        return batch_norm(x, self.running_mean, self.running_var, self.weight, self.bias, self.training or not self.track_running_stats,
                          self.momentum, self.eps, self.num_batches_tracked)

    def extra_repr(self):
        return f"{self.num_features}, eps={self.eps}, momentum={self.momentum}, affine={self.affine}, track_running_stats={self.track_running_stats}"

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        key = prefix + "num_batches_tracked"
        if self.track_running_stats and key not in state_dict:          # checkpoints written before the counter existed
            state_dict[key] = torch.zeros((), dtype=torch.long)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)


class BatchNorm1d(_BatchNorm):
    _dims = (2, 3)


class BatchNorm3d(_BatchNorm):
    _dims = (5,)


class BatchNorm2d(_BatchNorm):
    _dims = (4,)

    def forward(self, x):
        self._check(x)
        if (x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and x.shape[1] % 8 == 0 and self.affine and self.track_running_stats
                and self.momentum is not None and x.is_contiguous(memory_format=torch.channels_last) and self.weight.dtype == torch.float32):
            if self.training:
                self.num_batches_tracked.add_(1)
            return ops.nn_ops.batch_norm_nhwc(x, self.weight, self.bias, self.running_mean, self.running_var, training=self.training,
                                              momentum=self.momentum, eps=self.eps)
        return super().forward(x)


class _LazyBatchNorm(Module):
    """Batch norm whose channel count is read from the first input (lazy_norm.rs)."""
    _cls = BatchNorm2d

    def __init__(self, eps: float = 1e-5, momentum: Optional[float] = 0.1, affine: bool = True, track_running_stats: bool = True, device=None, dtype=None):
        super().__init__()
        self._kw = dict(eps=eps, momentum=momentum, affine=affine, track_running_stats=track_running_stats, device=device, dtype=dtype)
        self.inner: Optional[Module] = None

    def is_initialized(self) -> bool:
        return self.inner is not None

    def forward(self, x):
        if self.inner is None:
            if x.dim() < 2:
                raise ShapeMismatch(f"{type(self).__name__} expects at least 2 dimensions")
            kw = dict(self._kw)
            kw["device"] = kw["device"] or x.device
            self.inner = self._cls(x.shape[1], **kw)
            self.inner.train(self.training)
        return self.inner(x)


class LazyBatchNorm1d(_LazyBatchNorm):
    _cls = BatchNorm1d


class LazyBatchNorm2d(_LazyBatchNorm):
    _cls = BatchNorm2d


class LazyBatchNorm3d(_LazyBatchNorm):
    _cls = BatchNorm3d


def group_norm(x, num_groups: int, weight=None, bias=None, eps: float = 1e-5):
    if x.dim() < 2:
        raise ShapeMismatch(f"group_norm expects at least 2 dimensions, got {list(x.shape)}")
    N, C = x.shape[:2]
    if num_groups <= 0 or C % num_groups:
        raise InvalidArgument(f"channels {C} must be divisible by num_groups {num_groups}")
    if x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and x.is_contiguous() and x.numel() > 0:
        return ops.nn_ops.group_norm(x, num_groups, weight, bias, eps)
    xf = x.float() if x.dtype in (torch.bfloat16, torch.float16) else x
    g = xf.reshape(N, num_groups, -1)
    mean = g.mean(-1, keepdim=True)
    var = ((g - mean) ** 2).mean(-1, keepdim=True)
    y = ((g - mean) * torch.rsqrt(var + eps)).reshape(x.shape)
    shape = [1, C] + [1] * (x.dim() - 2)
    if weight is not None:
        y = y * weight.to(y.dtype).view(shape)
    if bias is not None:
        y = y + bias.to(y.dtype).view(shape)
    return y.to(x.dtype)


class GroupNorm(Module):
    def __init__(self, num_groups: int, num_channels: int, eps: float = 1e-5, affine: bool = True, device=None, dtype=None):
        super().__init__()
        if num_groups <= 0 or num_channels % num_groups:
            raise InvalidArgument(f"num_channels {num_channels} must be divisible by num_groups {num_groups}")
        self.num_groups, self.num_channels, self.eps, self.affine = num_groups, num_channels, eps, affine
        if affine:
            self.weight = Parameter(torch.ones(num_channels, device=device, dtype=dtype))
            self.bias = Parameter(torch.zeros(num_channels, device=device, dtype=dtype))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)

    def forward(self, x):
        if x.dim() < 2 or x.shape[1] != self.num_channels:
            raise ShapeMismatch(f"GroupNorm: expected {self.num_channels} channels, got input {list(x.shape)}")
        return group_norm(x, self.num_groups, self.weight, self.bias, self.eps)

    def extra_repr(self):
        return f"{self.num_groups}, {self.num_channels}, eps={self.eps}, affine={self.affine}"


def instance_norm(x, running_mean=None, running_var=None, weight=None, bias=None, use_input_stats: bool = True, momentum: float = 0.1,
                  eps: float = 1e-5):
    """Per-sample, per-channel statistics over the spatial dimensions. Running buffers, when given, average the per-sample statistics."""
    if x.dim() < 3:
        raise ShapeMismatch(f"instance_norm expects [N, C, *spatial], got {list(x.shape)}")
    N, C = x.shape[:2]
    shape = [1, C] + [1] * (x.dim() - 2)
    xf = x.float() if x.dtype in (torch.bfloat16, torch.float16) else x
    if use_input_stats:
        flat = xf.reshape(N, C, -1)
        n = flat.shape[-1]
        if n <= 1:
            raise InvalidArgument("instance_norm needs more than one spatial element per channel")
        mean = flat.mean(-1)
        var = ((flat - mean.unsqueeze(-1)) ** 2).mean(-1)
        if running_mean is not None and running_var is not None:
            with torch.no_grad():
                running_mean.mul_(1 - momentum).add_(mean.detach().mean(0).to(running_mean.dtype), alpha=momentum)
                running_var.mul_(1 - momentum).add_((var.detach() * (n / (n - 1))).mean(0).to(running_var.dtype), alpha=momentum)
        st = [N, C] + [1] * (x.dim() - 2)
        y = (xf - mean.view(st)) * torch.rsqrt(var.view(st) + eps)
    else:
        y = (xf - running_mean.to(xf.dtype).view(shape)) * torch.rsqrt(running_var.to(xf.dtype).view(shape) + eps)
    if weight is not None:
        y = y * weight.to(y.dtype).view(shape)
    if bias is not None:
        y = y + bias.to(y.dtype).view(shape)
    return y.to(x.dtype)


class _InstanceNorm(Module):
    _nd = 2

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1, affine: bool = False, track_running_stats: bool = False,
                 device=None, dtype=None):
        super().__init__()
        self.num_features, self.eps, self.momentum, self.affine, self.track_running_stats = num_features, eps, momentum, affine, track_running_stats
        if affine:
            self.weight = Parameter(torch.ones(num_features, device=device, dtype=dtype))
            self.bias = Parameter(torch.zeros(num_features, device=device, dtype=dtype))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)
        if track_running_stats:
            self.register_buffer("running_mean", torch.zeros(num_features, device=device, dtype=dtype))
            self.register_buffer("running_var", torch.ones(num_features, device=device, dtype=dtype))
            self.register_buffer("num_batches_tracked", torch.zeros((), dtype=torch.long, device=device))
        else:
            self.register_buffer("running_mean", None)
            self.register_buffer("running_var", None)
            self.register_buffer("num_batches_tracked", None)

    def forward(self, x):
        unbatched = x.dim() == self._nd + 1
        if x.dim() not in (self._nd + 1, self._nd + 2):
            raise ShapeMismatch(f"{type(self).__name__} expects a {self._nd + 1}-D or {self._nd + 2}-D input, got {list(x.shape)}")
        if unbatched:
            x = x.unsqueeze(0)
        if x.shape[1] != self.num_features and (self.affine or self.track_running_stats):
            raise ShapeMismatch(f"{type(self).__name__}: input has {x.shape[1]} channels, the layer was built for {self.num_features}")
        use_input = self.training or not self.track_running_stats
        y = instance_norm(x, self.running_mean if self.track_running_stats else None, self.running_var if self.track_running_stats else None,
                          self.weight, self.bias, use_input, self.momentum, self.eps)
        return y.squeeze(0) if unbatched else y


class InstanceNorm1d(_InstanceNorm):
    _nd = 1


class InstanceNorm2d(_InstanceNorm):
    _nd = 2


class InstanceNorm3d(_InstanceNorm):
    _nd = 3


def local_response_norm(x, size: int, alpha: float = 1e-4, beta: float = 0.75, k: float = 1.0):
    """``x / (k + alpha / size * sum_{neighbouring channels} x^2) ** beta`` with ``size // 2`` channels before and ``(size - 1) // 2`` after."""
    if x.dim() < 3:
        raise ShapeMismatch(f"local_response_norm expects at least 3 dimensions, got {list(x.shape)}")
    if size <= 0:
        raise InvalidArgument("size must be positive")
    sq = (x * x).transpose(1, -1)                                        # channels last for the window view
    from .padding import pad_nd
    win = pad_nd(sq, [(size // 2, (size - 1) // 2)], "constant", 0.0).unfold(-1, size, 1).sum(-1)
    div = (win.transpose(1, -1) * (alpha / size) + k) ** beta
    return x / div


class LocalResponseNorm(Module):
    def __init__(self, size: int, alpha: float = 1e-4, beta: float = 0.75, k: float = 1.0):
        super().__init__()
        self.size, self.alpha, self.beta, self.k = size, alpha, beta, k

    def forward(self, x):
        return local_response_norm(x, self.size, self.alpha, self.beta, self.k)


__all__ = ["batch_norm", "group_norm", "instance_norm", "local_response_norm", "BatchNorm1d", "BatchNorm2d", "BatchNorm3d", "LazyBatchNorm1d",
           "LazyBatchNorm2d", "LazyBatchNorm3d", "GroupNorm", "InstanceNorm1d", "InstanceNorm2d", "InstanceNorm3d", "LocalResponseNorm"]
