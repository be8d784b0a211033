"""Layers. Hot layers (Linear, RMSNorm, LayerNorm, Embedding, SwiGLU, rotary embedding, attention, cross-entropy) run on the
hand-written sm_100a kernels for bf16 CUDA tensors; the long tail (activations, losses, convolutions, normalisation, pooling,
padding, recurrent and transformer stacks) lives in the sibling modules of this package and is re-exported here.

Reference parity: ferrotorch-nn/src/{activation,linear,lazy_linear,lora,se,conv,lazy_conv,lazy_conv_transpose,lazy_norm,norm,
pooling,dropout,embedding,identity,padding,rnn,rnn_utils,attention,transformer,loss,upsample}.rs.
"""
from __future__ import annotations

import enum
import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from .. import ops
from ..errors import InvalidArgument, ShapeMismatch
from .module import Module, Parameter, Buffer, Sequential, ModuleList

# -- the long tail: every layer below is implemented in its own module of this package ------------------------------------------------------
from .activation import *  # noqa: F401,F403,E402
from .activation import relu, sigmoid  # noqa: E402
from .loss import *  # noqa: F401,F403,E402
from .conv import *  # noqa: F401,F403,E402
from .normalization import (BatchNorm1d, BatchNorm2d, BatchNorm3d, LazyBatchNorm1d, LazyBatchNorm2d, LazyBatchNorm3d, GroupNorm,  # noqa: F401,E402
                            InstanceNorm1d, InstanceNorm2d, InstanceNorm3d, LocalResponseNorm)
from .pooling import (MaxPool1d, MaxPool2d, MaxPool3d, AvgPool1d, AvgPool2d, AvgPool3d, AdaptiveAvgPool1d, AdaptiveAvgPool2d,  # noqa: F401,E402
                      AdaptiveAvgPool3d, AdaptiveMaxPool1d, AdaptiveMaxPool2d, AdaptiveMaxPool3d, LPPool1d, LPPool2d, MaxUnpool2d,
                      FractionalMaxPool2d, PixelShuffle, PixelUnshuffle, Unfold, Fold)
from .padding import (ConstantPad1d, ConstantPad2d, ConstantPad3d, ZeroPad1d, ZeroPad2d, ZeroPad3d, ReflectionPad1d, ReflectionPad2d,  # noqa: F401,E402
                      ReflectionPad3d, ReplicationPad1d, ReplicationPad2d, ReplicationPad3d, CircularPad1d, CircularPad2d, CircularPad3d)
from .misc import (Dropout, Dropout1d, Dropout2d, Dropout3d, AlphaDropout, Identity, Flatten, Unflatten, ChannelShuffle, EmbeddingBag,  # noqa: F401,E402
                   Upsample)
from .rnn import RNN, LSTM, GRU, RNNCell, LSTMCell, GRUCell  # noqa: F401,E402


class PaddingMode(enum.Enum):
    Constant = "constant"
    Zeros = "constant"
    Reflect = "reflect"
    Replicate = "replicate"
    Circular = "circular"


class RNNNonlinearity(enum.Enum):
    Tanh = "tanh"
    ReLU = "relu"


class EmbeddingBagMode(enum.Enum):
    Sum = "sum"
    Mean = "mean"
    Max = "max"


# -- Linear family ---------------------------------------------------------------------------------------------------------------
class Linear(Module):
    """``y = x W^T + b`` with ``W`` of shape ``[out, in]``. Weight init is Kaiming-uniform with the ReLU gain and the bias
    starts at zero, as in the reference (ferrotorch-nn/src/linear.rs:82-92; PyTorch's default uses ``a=sqrt(5)`` instead)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.bias = Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        self.reset_parameters()

    def reset_parameters(self) -> None:
        torch.nn.init.kaiming_uniform_(self.weight, nonlinearity="relu")
        if self.bias is not None:
            torch.nn.init.zeros_(self.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self.weight
        if w.dtype == torch.float32 and x.dim() >= 2 and self.in_features % 8 == 0 and self.out_features % 8 == 0 \
                and torch.is_autocast_enabled(x.device.type) and torch.get_autocast_dtype(x.device.type) == torch.bfloat16:
            from .compute_copy import compute_copy
            wc = compute_copy(w)
            if wc is not None and wc.dtype == torch.bfloat16:
                # f32 master with an optimizer-maintained bf16 copy: no cast launch, f32 weight gradient straight from the GEMM
                b = None if self.bias is None else self.bias.to(torch.bfloat16)
                return ops.linear_master(x.to(torch.bfloat16), w, wc, b)
            if x.is_cuda:
                # f32 master without a maintained copy: cast once here, run this package's GEMM, f32 weight gradient straight from its split-K form
                b = None if self.bias is None else self.bias.to(torch.bfloat16)
                return ops.linear_master(x.to(torch.bfloat16), w, w.detach().to(torch.bfloat16), b)
        return ops.linear(x, w, self.bias)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


class LazyLinear(Module):
    """Linear whose ``in_features`` is inferred from the first input (ferrotorch-nn/src/lazy_linear.rs:55)."""

    def __init__(self, out_features: int, bias: bool = True, device=None, dtype=None):
        super().__init__()
        self.out_features, self._bias, self._dev, self._dt = out_features, bias, device, dtype
        self.inner: Optional[Linear] = None

    def forward(self, x):
        if self.inner is None:
            self.inner = Linear(x.shape[-1], self.out_features, self._bias, self._dev or x.device, self._dt or x.dtype)
        return self.inner(x)


class LoRALinear(Module):
    """Frozen base Linear plus a trainable low-rank update ``(alpha/r) * B A`` (ferrotorch-nn/src/lora.rs:62)."""

    def __init__(self, base: Linear, rank: int = 8, alpha: float = 16.0, dropout: float = 0.0):
        super().__init__()
        self.base, self.rank, self.scaling = base, rank, alpha / rank
        for p in self.base.parameters():
            p.requires_grad_(False)
        dev, dt = base.weight.device, base.weight.dtype
        self.lora_a = Parameter(torch.empty(rank, base.in_features, device=dev, dtype=dt))
        self.lora_b = Parameter(torch.zeros(base.out_features, rank, device=dev, dtype=dt))
        torch.nn.init.kaiming_uniform_(self.lora_a, a=math.sqrt(5))
        self.drop = Dropout(dropout) if dropout > 0 else None
        self.merged = False

    def forward(self, x):
        y = self.base(x)
        if self.merged:
            return y
        h = self.drop(x) if self.drop is not None else x
        return y + ops.linear(ops.linear(h, self.lora_a), self.lora_b) * self.scaling

    def merge(self) -> None:
        if not self.merged:
            with torch.no_grad():
                self.base.weight += (self.lora_b.float() @ self.lora_a.float()).to(self.base.weight.dtype) * self.scaling
            self.merged = True

    def unmerge(self) -> None:
        if self.merged:
            with torch.no_grad():
                self.base.weight -= (self.lora_b.float() @ self.lora_a.float()).to(self.base.weight.dtype) * self.scaling
            self.merged = False


class SqueezeExcitation(Module):
    """Channel attention: global average pool -> FC -> activation -> FC -> gate (ferrotorch-nn/src/se.rs:64). The two FC layers are 1x1
    convolutions; ``activation`` (default ReLU) follows the first and ``scale_activation`` (default sigmoid) produces the gate."""

    def __init__(self, channels: int, squeeze_channels: int, activation=None, scale_activation=None):
        super().__init__()
        self.fc1 = Conv2d(channels, squeeze_channels, 1)
        self.fc2 = Conv2d(squeeze_channels, channels, 1)
        self._act = activation or relu
        self._gate = scale_activation or sigmoid

    def forward(self, x):
        s = x.mean((-2, -1), keepdim=True)
        return x * self._gate(self.fc2(self._act(self.fc1(s))))


# -- normalisation on our kernels -----------------------------------------------------------------------------------------------------
class RMSNorm(Module):
    def __init__(self, dim: int, eps: float = 1e-6, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = Parameter(torch.ones(dim, device=device, dtype=dtype))

    def forward(self, x):
        return ops.rms_norm(x, self.weight, self.eps)


class LayerNorm(Module):
    def __init__(self, normalized_shape, eps: float = 1e-5, elementwise_affine: bool = True, bias: bool = True, device=None, dtype=None):
        super().__init__()
        self.normalized_shape = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
        self.eps = eps
        self.weight = Parameter(torch.ones(self.normalized_shape, device=device, dtype=dtype)) if elementwise_affine else None
        self.bias = Parameter(torch.zeros(self.normalized_shape, device=device, dtype=dtype)) if (elementwise_affine and bias) else None

    def forward(self, x):
        if len(self.normalized_shape) == 1 and self.weight is not None:
            return ops.layer_norm(x, self.weight, self.bias, self.eps)
        return F.layer_norm(x, self.normalized_shape, self.weight, self.bias, self.eps)


class Embedding(Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: Optional[int] = None, device=None, dtype=None):
        super().__init__()
        self.num_embeddings, self.embedding_dim, self.padding_idx = num_embeddings, embedding_dim, padding_idx
        self.weight = Parameter(torch.randn(num_embeddings, embedding_dim, device=device, dtype=dtype))
        if padding_idx is not None:
            with torch.no_grad():
                self.weight[padding_idx].zero_()

    def forward(self, ids):
        if self.weight.is_cuda and self.weight.dtype == torch.bfloat16 and self.padding_idx is None:
            return ops.embedding(ids, self.weight)
        return F.embedding(ids, self.weight, self.padding_idx)


# -- transformer pieces (ferrotorch-nn/src/transformer.rs:49-1030) ------------------------------------------------------------------
class RoPEConvention(enum.Enum):
    Interleaved = "interleaved"      # pairs (2i, 2i+1)
    HalfRotation = "half_rotation"   # pairs (i, i + D/2) - the Llama/HF convention


class RoPEScaling:
    """``none`` | ``linear(factor)`` | ``ntk(factor)`` | ``yarn(factor, original_max_position, beta_fast, beta_slow)``."""

    def __init__(self, kind: str = "none", **kw):
        self.kind, self.kw = kind, kw

    @staticmethod
    def none():
        return RoPEScaling("none")

    @staticmethod
    def linear(factor: float):
        return RoPEScaling("linear", factor=factor)

    @staticmethod
    def ntk_aware(factor: float):
        return RoPEScaling("ntk", factor=factor)

    @staticmethod
    def yarn(factor: float, original_max_position: int, beta_fast: float = 32.0, beta_slow: float = 1.0):
        return RoPEScaling("yarn", factor=factor, original_max_position=original_max_position, beta_fast=beta_fast, beta_slow=beta_slow)

    def as_dict(self):
        return None if self.kind == "none" else {"type": self.kind, **self.kw}


class RotaryPositionEmbedding(Module):
    def __init__(self, head_dim: int, max_position: int = 8192, theta: float = 10000.0, convention: RoPEConvention = RoPEConvention.HalfRotation,
                 scaling: Optional[RoPEScaling] = None, device="cpu"):
        super().__init__()
        self.head_dim, self.convention = head_dim, convention
        cos, sin = ops.rope_tables(max_position, head_dim, theta, device, scaling.as_dict() if scaling else None)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    def apply(self, x: torch.Tensor, positions: Optional[torch.Tensor] = None, offset: int = 0) -> torch.Tensor:  # noqa: A003
        """``x``: ``[B, S, H, D]``. ``offset`` shifts positions (decoding with a KV cache)."""
        B, S, H, D = x.shape
        if self.convention == RoPEConvention.HalfRotation and x.is_cuda and x.dtype == torch.bfloat16 and D % 16 == 0:
            if offset and positions is None:
                positions = (torch.arange(S, device=x.device, dtype=torch.int32) + offset).repeat(B)
            return ops.apply_rope(x, self.cos, self.sin, positions)
        pos = (torch.arange(S, device=x.device) + offset) if positions is None else positions.reshape(B, S)
        c, s = self.cos[pos], self.sin[pos]
        c, s = (c.view(1, S, 1, -1), s.view(1, S, 1, -1)) if positions is None else (c.view(B, S, 1, -1), s.view(B, S, 1, -1))
        xf = x.float()
        if self.convention == RoPEConvention.HalfRotation:
            a, b = xf[..., : D // 2], xf[..., D // 2:]
            return torch.cat([a * c - b * s, b * c + a * s], -1).to(x.dtype)
        a, b = xf[..., 0::2], xf[..., 1::2]
        return torch.stack([a * c - b * s, b * c + a * s], -1).flatten(-2).to(x.dtype)

    forward = apply


class SwiGLU(Module):
    """``down(silu(gate(x)) * up(x))`` with gate and up fused into one ``[2F, d]`` GEMM and one fused activation kernel."""

    def __init__(self, dim: int, hidden: int, bias: bool = False, device=None, dtype=None):
        super().__init__()
        self.gate_up = Linear(dim, 2 * hidden, bias, device, dtype)
        self.down = Linear(hidden, dim, bias, device, dtype)

    def forward(self, x):
        gu = self.gate_up(x)
        if gu.is_cuda and gu.dtype == torch.bfloat16:
            return self.down(ops.swiglu(gu))
        F_ = gu.shape[-1] // 2
        return self.down(F.silu(gu[..., :F_]) * gu[..., F_:])


class KVCache:
    """Pre-allocated key/value cache ``[B, H_kv, max_len, D]`` with in-place append (ferrotorch-nn/src/transformer.rs:848-1030)."""

    def __init__(self, batch: int, kv_heads: int, max_len: int, head_dim: int, device="cpu", dtype=torch.float32):
        self.k = torch.zeros(batch, kv_heads, max_len, head_dim, device=device, dtype=dtype)
        self.v = torch.zeros_like(self.k)
        self.len = 0
        self.max_len = max_len

    def update(self, k_new: torch.Tensor, v_new: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        n = k_new.shape[2]
        if self.len + n > self.max_len:
            raise InvalidArgument(f"KV cache overflow: {self.len}+{n} > {self.max_len}")
        self.k[:, :, self.len: self.len + n] = k_new
        self.v[:, :, self.len: self.len + n] = v_new
        self.len += n
        return self.k[:, :, : self.len], self.v[:, :, : self.len]

    def reset(self) -> None:
        self.len = 0


# -- attention (ferrotorch-nn/src/attention.rs:47-665, flash_attention.rs:45-633) ----------------------------------------------------
def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """``[B, H_kv, S, D] -> [B, H_kv*n_rep, S, D]``."""
    return x if n_rep == 1 else x.repeat_interleave(n_rep, 1)


def reshape_to_heads(x: torch.Tensor, heads: int) -> torch.Tensor:
    B, S, E = x.shape
    return x.view(B, S, heads, E // heads).transpose(1, 2)


def transpose_heads_to_2d(x: torch.Tensor) -> torch.Tensor:
    B, H, S, D = x.shape
    return x.transpose(1, 2).reshape(B, S, H * D)


def standard_attention(q, k, v, causal: bool = False, scale: Optional[float] = None, mask: Optional[torch.Tensor] = None):
    """Materialised-score attention on ``[B, H, S, D]`` tensors (the oracle for the flash kernels)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    if causal:
        Sq, Sk = s.shape[-2:]
        s = s.masked_fill(torch.ones(Sq, Sk, dtype=torch.bool, device=s.device).triu(Sk - Sq + 1), float("-inf"))
    if mask is not None:
        s = s + mask if mask.is_floating_point() else s.masked_fill(~mask, float("-inf"))
    return torch.matmul(torch.softmax(s, -1), v.float()).to(q.dtype)


def flash_attention(q, k, v, causal: bool = False, scale: Optional[float] = None):
    """Tiled online-softmax attention on ``[B, H, S, D]`` (GQA when ``k``/``v`` have fewer heads).

    bf16 CUDA inputs with equal query/key lengths and a head dimension up to 128 (a multiple of 8) run on the tcgen05 kernels. The
    kernels are built for ``D = 128``: smaller heads are zero-padded to 128, which changes neither the scores (the padded products are
    zero) nor the first ``D`` output columns, at the cost of the padded FLOPs. Anything else evaluates the same math through
    :func:`standard_attention`."""
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    if (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == v.dtype == torch.bfloat16 and D <= 128 and D % 8 == 0 and k.shape[2] == S
            and v.shape[-1] == D and Hq % Hkv == 0 and ops.attention.backend() == "tcgen05"):
        pad = 128 - D

        def rows(t, H):
            t = t.transpose(1, 2)                                           # [B, S, H, D]
            if pad:
                t = torch.cat([t, t.new_zeros(B, S, H, pad)], -1)
            return t.reshape(B * S, H * 128)

        packed = torch.cat([rows(q, Hq), rows(k, Hkv), rows(v, Hkv)], 1)
        o = ops.attention_packed(packed, B, S, Hq, Hkv, 128, causal, scale if scale is not None else 1.0 / math.sqrt(D))
        return o.view(B, S, Hq, 128)[..., :D].transpose(1, 2)
    return standard_attention(q, repeat_kv(k, Hq // Hkv), repeat_kv(v, Hq // Hkv), causal, scale)


def attention_backend(q: torch.Tensor, k: Optional[torch.Tensor] = None) -> str:
    """Which implementation :func:`flash_attention` takes for these operands: ``"tcgen05"`` or ``"standard"``."""
    k = q if k is None else k
    D = q.shape[-1]
    ok = (q.is_cuda and q.dtype == torch.bfloat16 and D <= 128 and D % 8 == 0 and k.shape[2] == q.shape[2] and ops.attention.backend() == "tcgen05")
    return "tcgen05" if ok else "standard"


class MultiheadAttention(Module):
    """Multi-head attention with optional grouped-query KV heads (``with_gqa``), batch-first ``[B, S, E]``."""

    def __init__(self, embed_dim: int, num_heads: int, num_kv_heads: Optional[int] = None, bias: bool = True, device=None, dtype=None):
        super().__init__()
        self.embed_dim, self.num_heads = embed_dim, num_heads
        self.num_kv_heads = num_kv_heads or num_heads
        if embed_dim % num_heads or num_heads % self.num_kv_heads:
            raise InvalidArgument("embed_dim % num_heads and num_heads % num_kv_heads must be 0")
        self.head_dim = embed_dim // num_heads
        kv = self.num_kv_heads * self.head_dim
        self.q_proj = Linear(embed_dim, embed_dim, bias, device, dtype)
        self.k_proj = Linear(embed_dim, kv, bias, device, dtype)
        self.v_proj = Linear(embed_dim, kv, bias, device, dtype)
        self.out_proj = Linear(embed_dim, embed_dim, bias, device, dtype)
        self._register_load_state_dict_pre_hook(self._split_packed_projection)

    def _split_packed_projection(self, state_dict, prefix, *_):
        """A checkpoint written by ``torch.nn.MultiheadAttention`` stores the three input projections as one ``in_proj_weight`` /
        ``in_proj_bias``; cut them into this layer's q, k and v entries (rows in that order) before the keys are matched."""
        kv = self.num_kv_heads * self.head_dim
        for packed, leaf in (("in_proj_weight", "weight"), ("in_proj_bias", "bias")):
            t = state_dict.pop(prefix + packed, None)
            if t is None:
                continue
            if t.shape[0] != self.embed_dim + 2 * kv:
                raise ShapeMismatch(f"{prefix}{packed}: {t.shape[0]} rows, expected {self.embed_dim + 2 * kv}")
            q, k, v = t.split([self.embed_dim, kv, kv], 0)
            state_dict[f"{prefix}q_proj.{leaf}"], state_dict[f"{prefix}k_proj.{leaf}"], state_dict[f"{prefix}v_proj.{leaf}"] = q, k, v

    @classmethod
    def with_gqa(cls, embed_dim: int, num_heads: int, num_kv_heads: int, **kw) -> "MultiheadAttention":
        return cls(embed_dim, num_heads, num_kv_heads, **kw)

    def forward_qkv(self, query, key, value, causal: bool = False, mask: Optional[torch.Tensor] = None):
        q = reshape_to_heads(self.q_proj(query), self.num_heads)
        k = reshape_to_heads(self.k_proj(key), self.num_kv_heads)
        v = reshape_to_heads(self.v_proj(value), self.num_kv_heads)
        if mask is None:
            o = flash_attention(q, k, v, causal)
        else:
            rep = self.num_heads // self.num_kv_heads
            o = standard_attention(q, repeat_kv(k, rep), repeat_kv(v, rep), causal, None, mask)
        return self.out_proj(transpose_heads_to_2d(o))

    def forward(self, x, causal: bool = False, mask: Optional[torch.Tensor] = None):
        return self.forward_qkv(x, x, x, causal, mask)

    def forward_2d(self, x2d: torch.Tensor, causal: bool = False):
        return self.forward(x2d.unsqueeze(0), causal).squeeze(0)


# -- loss on our kernel ----------------------------------------------------------------------------------------------------------------
class CrossEntropyLoss(Module):
    """Mean/sum/none cross-entropy on ``[N, C]`` logits. Targets may be integer class indices or, as in the reference
    (ferrotorch-nn/src/loss.rs:187-215), a float tensor holding class indices."""

    def __init__(self, reduction: str = "mean", ignore_index: int = -100, label_smoothing: float = 0.0, weight: Optional[torch.Tensor] = None):
        super().__init__()
        self.reduction, self.ignore_index, self.label_smoothing = reduction, ignore_index, label_smoothing
        self.weight = weight          # per-class weights; the weighted form runs outside the fused kernel

    def forward(self, logits, target):
        if target.is_floating_point() and target.dim() == logits.dim() - 1:
            target = target.long()
        if self.weight is None and self.reduction == "mean" and target.dtype == torch.long and logits.is_cuda and logits.dim() == 2:
            return ops.cross_entropy(logits, target, self.ignore_index, self.label_smoothing)
        w = None if self.weight is None else self.weight.to(device=logits.device, dtype=logits.dtype)
        return F.cross_entropy(logits, target, weight=w, reduction=self.reduction, ignore_index=self.ignore_index, label_smoothing=self.label_smoothing)


from .transformer import (TransformerEncoderLayer, TransformerDecoderLayer, TransformerEncoder, TransformerDecoder, Transformer)  # noqa: F401,E402
