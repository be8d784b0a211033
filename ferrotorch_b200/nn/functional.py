"""Functional forms (ferrotorch-nn/src/functional.rs: linear ... scaled_dot_product_attention).

The hot ones dispatch to the sm_100a kernels; everything else carries PyTorch's reference semantics."""
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
    return _F.layer_norm(x, normalized_shape, weight, bias, eps)


def scaled_dot_product_attention(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None):
    if attn_mask is None and dropout_p == 0.0:
        return flash_attention(q, k, v, is_causal, scale)
    rep = q.shape[1] // k.shape[1]
    return standard_attention(q, repeat_kv(k, rep), repeat_kv(v, rep), is_causal, scale, attn_mask)


# PyTorch-semantics forms re-exported under the same names
for _n in ["relu", "gelu", "silu", "sigmoid", "tanh", "softmax", "log_softmax", "leaky_relu", "elu", "mish", "celu", "selu", "hardsigmoid",
           "hardswish", "softplus", "glu", "relu6", "hardtanh", "logsigmoid", "softmin", "threshold", "softshrink", "hardshrink",
           "tanhshrink", "softsign", "dropout", "conv1d", "conv2d", "conv3d", "conv_transpose1d", "conv_transpose2d", "conv_transpose3d",
           "max_pool1d", "max_pool2d", "max_pool3d", "avg_pool1d", "avg_pool2d", "avg_pool3d", "adaptive_avg_pool1d", "adaptive_avg_pool2d",
           "adaptive_avg_pool3d", "adaptive_max_pool1d", "adaptive_max_pool2d", "lp_pool1d", "lp_pool2d", "batch_norm", "group_norm",
           "instance_norm", "local_response_norm", "embedding", "embedding_bag", "one_hot", "pad", "interpolate", "grid_sample",
           "affine_grid", "pixel_shuffle", "pixel_unshuffle", "unfold", "fold", "mse_loss", "l1_loss", "smooth_l1_loss", "huber_loss",
           "nll_loss", "binary_cross_entropy", "binary_cross_entropy_with_logits", "kl_div", "cosine_embedding_loss", "margin_ranking_loss",
           "triplet_margin_loss", "hinge_embedding_loss", "poisson_nll_loss", "gaussian_nll_loss", "multi_margin_loss",
           "multilabel_soft_margin_loss", "ctc_loss", "cosine_similarity", "pairwise_distance", "normalize"]:
    globals()[_n] = getattr(_F, _n)


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
    return _F.hardtanh(x, min_val, max_val)


def log_sigmoid(x):
    return _F.logsigmoid(x)


def softplus_with(x, beta: float = 1.0, threshold: float = 20.0):
    if beta <= 0:
        from ..errors import InvalidArgument
        raise InvalidArgument(f"softplus: beta must be > 0, got {beta}")
    return _F.softplus(x, beta, threshold)


def elu_with(x, alpha: float = 1.0):
    return _F.elu(x, alpha)


def prelu(x, alpha):
    """``max(0, x) + alpha * min(0, x)`` with one ``alpha`` or one per channel (dimension 1)."""
    a = torch.as_tensor(alpha, dtype=x.dtype, device=x.device).reshape(-1)
    if a.numel() not in (1, x.shape[1] if x.dim() > 1 else 1):
        from ..errors import ShapeMismatch
        raise ShapeMismatch(f"prelu: {a.numel()} slopes for input shape {list(x.shape)}")
    return _F.prelu(x, a)
