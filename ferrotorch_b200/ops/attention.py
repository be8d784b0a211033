"""Attention front-end: causal GQA FlashAttention forward/backward on packed QKV.

The packed layout is the QKV GEMM's own output: ``qkv[T, (Hq + 2*Hkv) * D]`` with
the query heads first, then the key heads, then the value heads, so no
transpose / repeat_kv copies are made (the reference's GPU path materialises
``[H,S,S]`` scores and repeats KV heads: ferrotorch-llama/src/gpu.rs:609-628,
ferrotorch-gpu/src/bf16.rs:1987).

``flash_fwd`` / ``flash_bwd`` dispatch to the tcgen05 kernels when the native
library exports them for the shape (D = 128, bf16); otherwise they evaluate the
same math with torch's scaled_dot_product_attention, which the GPU tests also
use as the oracle. ``backend()`` reports which one runs.
"""
from __future__ import annotations

import math
import os

import torch

from .. import _lib
from ._workspace import workspace

_native_ok: bool | None = None


def _native_available() -> bool:
    global _native_ok
    if _native_ok is None:
        ok = False
        if os.environ.get("FT_ATTN_BACKEND", "") != "sdpa":
            try:
                ok = hasattr(_lib.kernels(), "ft_flash_fwd")
            except Exception:
                ok = False
        _native_ok = ok
    return _native_ok


def _bwd_native() -> bool:
    return os.environ.get("FT_ATTN_BWD", "") != "sdpa" and hasattr(_lib.kernels(), "ft_flash_bwd_ws")


def backend(D: int = 128, dtype=torch.bfloat16, device_is_cuda: bool = True) -> str:
    return "tcgen05" if (device_is_cuda and _native_available() and D == 128 and dtype == torch.bfloat16) else "sdpa"


def _split(qkv2, B, S, Hq, Hkv, D):
    q = qkv2[:, : Hq * D].reshape(B, S, Hq, D).transpose(1, 2)
    k = qkv2[:, Hq * D: (Hq + Hkv) * D].reshape(B, S, Hkv, D).transpose(1, 2)
    v = qkv2[:, (Hq + Hkv) * D:].reshape(B, S, Hkv, D).transpose(1, 2)
    return q, k, v


def _sdpa(q, k, v, causal, scale):
    if q.is_cuda:
        return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=scale, enable_gqa=True)
    rep = q.shape[1] // k.shape[1]
    k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    if causal:
        Sq, Sk = s.shape[-2:]
        s = s.masked_fill(torch.ones(Sq, Sk, dtype=torch.bool, device=s.device).triu(Sk - Sq + 1), float("-inf"))
    return torch.matmul(torch.softmax(s, -1), v.float()).to(q.dtype)


def flash_fwd(qkv2: torch.Tensor, B: int, S: int, Hq: int, Hkv: int, D: int, causal: bool = True, scale: float | None = None):
    """Returns (out ``[T, Hq*D]``, lse ``[B, Hq, S]`` f32 or None for the sdpa path)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if backend(D, qkv2.dtype, qkv2.is_cuda) == "tcgen05":
        out = torch.empty((B * S, Hq * D), device=qkv2.device, dtype=qkv2.dtype)
        lse = torch.empty((B, Hq, S), device=qkv2.device, dtype=torch.float32)
        _lib.call("ft_flash_fwd", qkv2, out, lse, B, S, Hq, Hkv, D, qkv2.stride(0), int(causal), float(scale), _lib.S())
        return out, lse
    q, k, v = _split(qkv2, B, S, Hq, Hkv, D)
    o = _sdpa(q, k, v, causal, scale)
    return o.transpose(1, 2).reshape(B * S, Hq * D).contiguous(), None


def flash_bwd(qkv2, out2, lse, dout2, B, S, Hq, Hkv, D, causal: bool = True, scale: float | None = None) -> torch.Tensor:
    """Returns dqkv ``[T, (Hq+2Hkv)*D]`` in the packed layout."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if lse is not None and backend(D, qkv2.dtype, qkv2.is_cuda) == "tcgen05" and _bwd_native():
        dqkv = torch.empty_like(qkv2)
        delta = workspace(qkv2.device, "flash_delta", B * Hq * S * 4)
        if not dout2.is_contiguous():
            dout2 = dout2.contiguous()
        _lib.call("ft_flash_bwd_ws", qkv2, out2, lse, dout2, dqkv, delta, B, S, Hq, Hkv, D, qkv2.stride(0), int(causal), float(scale),
                  _lib.S())
        return dqkv
    with torch.enable_grad():
        leaf = qkv2.detach().requires_grad_(True)
        q, k, v = _split(leaf, B, S, Hq, Hkv, D)
        o = _sdpa(q, k, v, causal, scale).transpose(1, 2).reshape(B * S, Hq * D)
        (dqkv,) = torch.autograd.grad(o, leaf, dout2)
    return dqkv


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv2, B, S, Hq, Hkv, D, causal, scale):
        out, lse = flash_fwd(qkv2, B, S, Hq, Hkv, D, causal, scale)
        ctx.save_for_backward(qkv2, out, lse if lse is not None else torch.empty(0))
        ctx.meta = (B, S, Hq, Hkv, D, causal, scale, lse is not None)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv2, out, lse = ctx.saved_tensors
        B, S, Hq, Hkv, D, causal, scale, has = ctx.meta
        return flash_bwd(qkv2, out, lse if has else None, dout.contiguous(), B, S, Hq, Hkv, D, causal, scale), *([None] * 7)


def attention_packed(qkv2, B, S, Hq, Hkv, D, causal=True, scale=None):
    """Differentiable attention on the packed QKV buffer."""
    return _AttnFn.apply(qkv2, B, S, Hq, Hkv, D, causal, scale)
