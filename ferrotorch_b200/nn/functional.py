"""Functional forms (ferrotorch-nn/src/functional.rs: linear ... scaled_dot_product_attention).

The hot ones dispatch to the sm_100a kernels; the rest are written out in the sibling modules of this package."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as _F

from .. import ops
from .layers import flash_attention, standard_attention, repeat_kv

linear = ops.linear
rms_norm = ops.rms_norm
cross_entropy = ops.cross_entropy
swiglu = ops.swiglu
embedding_fast = ops.embedding


def layer_norm(x, normalized_shape, weight=None, bias=None, eps=1e-5):
    if weight is not None and len(tuple(normalized_shape)) == 1:
        return ops.layer_norm(x, weight, bias, eps)
    dims = tuple(range(-len(tuple(normalized_shape)), 0))
    mean = x.mean(dims, keepdim=True)
    y = (x - mean) * torch.rsqrt(((x - mean) ** 2).mean(dims, keepdim=True) + eps)
    if weight is not None:
        y = y * weight
    return y if bias is None else y + bias


def scaled_dot_product_attention(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None):
    """``softmax(q k^T * scale + mask) v`` on ``[B, H, S, D]``. Without a mask or dropout this is :func:`flash_attention` (the tcgen05
    kernels for bf16 CUDA operands with ``D <= 128``); masked CUDA calls go to the library's fused attention, and CPU calls to the
    materialised-score form."""
    if attn_mask is None and dropout_p == 0.0:
        return flash_attention(q, k, v, is_causal, scale)
    if q.is_cuda:
        return _F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal, scale=scale,
                                               enable_gqa=q.shape[1] != k.shape[1])
    rep = q.shape[1] // k.shape[1]
    o = standard_attention(q, repeat_kv(k, rep), repeat_kv(v, rep), is_causal, scale,
                           attn_mask if attn_mask is None or attn_mask.is_floating_point() else attn_mask)
    return o if dropout_p == 0.0 else dropout(o, dropout_p, True)


# -- the forms written out in this package ---------------------------------------------------------------------------------------------------
from .activation import (relu, silu, sigmoid, tanh, softmax, log_softmax, leaky_relu, elu, mish, celu, selu, hardsigmoid, hardswish,  # noqa: E402,F401
                         softplus, glu, relu6, hardtanh, logsigmoid, softmin, threshold, softshrink, hardshrink, tanhshrink, softsign, rrelu)
from .activation import prelu as _prelu  # noqa: E402
from .misc import dropout, alpha_dropout, embedding_bag  # noqa: E402,F401
from .pooling import (max_pool1d, max_pool2d, max_pool3d, avg_pool1d, avg_pool2d, avg_pool3d, adaptive_avg_pool1d, adaptive_avg_pool2d,  # noqa: E402,F401
                      adaptive_avg_pool3d, adaptive_max_pool1d, adaptive_max_pool2d, adaptive_max_pool3d, lp_pool1d, lp_pool2d, max_unpool2d,
                      fractional_max_pool2d, pixel_shuffle, pixel_unshuffle, unfold, fold)
from .normalization import batch_norm, group_norm, instance_norm, local_response_norm  # noqa: E402,F401
from .padding import pad  # noqa: E402,F401
from .loss import (mse_loss, l1_loss, smooth_l1_loss, huber_loss, nll_loss, binary_cross_entropy, binary_cross_entropy_with_logits, kl_div,  # noqa: E402,F401
                   cosine_embedding_loss, margin_ranking_loss, triplet_margin_loss, hinge_embedding_loss, poisson_nll_loss, gaussian_nll_loss,
                   multi_margin_loss, multilabel_soft_margin_loss, ctc_loss, cosine_similarity, pairwise_distance)
from .extras import interpolate, grid_sample, affine_grid  # noqa: E402,F401

# convolution primitives: the library's (the layers in ``nn.conv`` route the hot shapes to this package's kernels)
for _n in ["conv1d", "conv2d", "conv3d", "conv_transpose1d", "conv_transpose2d", "conv_transpose3d"]:
    globals()[_n] = getattr(_F, _n)


def embedding(ids, weight, padding_idx=None):
    """Row lookup; ``padding_idx`` only matters for the gradient (that row receives none)."""
    if weight.is_cuda and weight.dtype == torch.bfloat16 and padding_idx is None:
        return ops.embedding(ids, weight)
    if padding_idx is not None:
        keep = (torch.arange(weight.shape[0], device=weight.device) != padding_idx).to(weight.dtype).unsqueeze(-1)
        weight = weight * keep + (weight * (1 - keep)).detach()
    return weight.index_select(0, ids.reshape(-1)).view(*ids.shape, weight.shape[1])


def one_hot(ids, num_classes: int = -1):
    if ids.is_floating_point():
        from ..errors import InvalidArgument
        raise InvalidArgument("one_hot takes integer class indices")
    n = int(ids.max()) + 1 if num_classes < 0 else num_classes
    return torch.zeros(*ids.shape, n, dtype=torch.long, device=ids.device).scatter_(-1, ids.unsqueeze(-1).long(), 1)


def normalize(x, p: float = 2.0, dim: int = 1, eps: float = 1e-12):
    """``x / max(||x||_p, eps)`` along ``dim``."""
    if p == 2:
        n = torch.sqrt((x * x).sum(dim, keepdim=True))
    elif p == 1:
        n = torch.abs(x).sum(dim, keepdim=True)
    elif p == float("inf"):
        n = torch.abs(x).amax(dim, keepdim=True)
    else:
        n = torch.abs(x).pow(p).sum(dim, keepdim=True).pow(1.0 / p)
    return x / torch.clamp_min(n, eps)


# -- parameterised forms (ferrotorch-nn/src/functional.rs:158-880) ------------------------------------------------------------------------
from .extras import gelu, gelu_with  # noqa: E402,F401  (``gelu(x, approximate)`` with the none / tanh / sigmoid forms)


def sum(x):  # noqa: A001
    """Sum of all elements (a 0-D tensor)."""
    return x.sum()


def mean(x):
    return x.mean()


def hardtanh_with(x, min_val: float, max_val: float):
    if min_val > max_val:
        from ..errors import InvalidArgument
        raise InvalidArgument(f"hardtanh: min_val {min_val} > max_val {max_val}")
    return hardtanh(x, min_val, max_val)


def log_sigmoid(x):
    return logsigmoid(x)


def softplus_with(x, beta: float = 1.0, threshold: float = 20.0):
    if beta <= 0:
        from ..errors import InvalidArgument
        raise InvalidArgument(f"softplus: beta must be > 0, got {beta}")
    return softplus(x, beta, threshold)


def elu_with(x, alpha: float = 1.0):
    return elu(x, alpha)


def prelu(x, alpha):
    """``max(0, x) + alpha * min(0, x)`` with one ``alpha`` or one per channel (dimension 1)."""
    a = torch.as_tensor(alpha, dtype=x.dtype, device=x.device).reshape(-1)
    if a.numel() not in (1, x.shape[1] if x.dim() > 1 else 1):
        from ..errors import ShapeMismatch
        raise ShapeMismatch(f"prelu: {a.numel()} slopes for input shape {list(x.shape)}")
    return _prelu(x, a)
