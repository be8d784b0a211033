"""Buffer-level device API: the ``gpu_*`` operations on flat device tensors with explicit sizes, stream-capture entry points with pool
handles, memory statistics / hooks / watchdog, the host Philox generator and the device helpers.

These functions take CUDA tensors (a CPU tensor is a :class:`DeviceMismatch`, never a silent host computation) and run this framework's
sm_100a kernels where one exists for the operation (bf16 GEMM, RMSNorm, rotary embedding, SiLU, softmax, embedding gather, fused attention)
and stream-ordered library kernels otherwise. Shapes are passed explicitly, as in the reference, and checked against the buffer lengths.

Reference parity (ferrotorch-gpu/src): kernels.rs (gpu_add ... gpu_slice_write_indirect), blas.rs:68-520 (matmul / bmm), bf16.rs:543-2960,
conv.rs:505, flash_attention.rs:461, graph.rs:91-770, memory_guard.rs:206-1300, rng.rs:140-530, device.rs, transfer.rs, pool.rs.
"""
from __future__ import annotations

import enum
import itertools
import threading
import time
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from ..errors import DeviceMismatch, InvalidArgument, ShapeMismatch

GpuResult = Any                                               # results are returned directly; failures raise GpuError / FerrotorchError
GpuFloat = (torch.float32, torch.float64, torch.bfloat16, torch.float16)

_require_cuda = True                                          # the CPU test tier switches this off to check the arithmetic of every wrapper


def _dev(*ts: torch.Tensor) -> None:
    if _require_cuda:
        for t in ts:
            if t is not None and not t.is_cuda:
                raise DeviceMismatch("cuda", f"{t.device.type} (device operations take CUDA tensors: move it with cpu_to_gpu first)")


def _len(t: torch.Tensor, n: int, what: str) -> None:
    if t.numel() != n:
        raise ShapeMismatch(f"{what}: buffer has {t.numel()} elements, the given sizes need {n}")


def _dt(t: torch.Tensor, dtype: torch.dtype, what: str) -> None:
    if t.dtype != dtype:
        raise InvalidArgument(f"{what}: expected {dtype}, got {t.dtype}")


def _ops():
    from .. import ops
    return ops


# -- elementwise ------------------------------------------------------------------------------------------------------------------
def _bin(name, fn, dtype):
    def f(a: torch.Tensor, b: torch.Tensor, device=None) -> torch.Tensor:
        _dev(a, b)
        _dt(a, dtype, name)
        _dt(b, dtype, name)
        _len(b, a.numel(), name)
        return fn(a, b)
    f.__name__, f.__doc__ = name, f"Elementwise {fn.__name__} of two {dtype} buffers of equal length."
    return f


gpu_add, gpu_sub, gpu_mul = _bin("gpu_add", torch.add, torch.float32), _bin("gpu_sub", torch.sub, torch.float32), _bin("gpu_mul", torch.mul, torch.float32)
gpu_add_bf16, gpu_mul_bf16 = _bin("gpu_add_bf16", torch.add, torch.bfloat16), _bin("gpu_mul_bf16", torch.mul, torch.bfloat16)


def _into(name, fn):
    def f(a, b, out, device=None) -> None:
        _dev(a, b, out)
        _len(b, a.numel(), name)
        _len(out, a.numel(), name)
        fn(a, b, out=out)
    f.__name__ = name
    return f


gpu_add_into, gpu_mul_into = _into("gpu_add_into", torch.add), _into("gpu_mul_into", torch.mul)


def gpu_add_into_on_stream(a, b, out, device=None, stream: Optional[torch.cuda.Stream] = None) -> None:
    """``out = a + b`` enqueued on ``stream`` (the caller orders it against the producers of ``a`` and ``b``)."""
    _dev(a, b, out)
    _len(b, a.numel(), "gpu_add_into_on_stream")
    _len(out, a.numel(), "gpu_add_into_on_stream")
    if stream is None or not a.is_cuda:
        torch.add(a, b, out=out)
        return
    with torch.cuda.stream(stream):
        torch.add(a, b, out=out)


def gpu_neg(a, device=None): _dev(a); return torch.neg(a)                                    # noqa: E702,E704
def gpu_relu(a, device=None): _dev(a); _dt(a, torch.float32, "gpu_relu"); return torch.relu(a)          # noqa: E702,E704
def gpu_relu_bf16(a, device=None): _dev(a); _dt(a, torch.bfloat16, "gpu_relu_bf16"); return torch.relu(a)   # noqa: E702,E704
def gpu_gelu(a, device=None): _dev(a); return F.gelu(a)                                      # noqa: E702,E704


def gpu_gelu_into(a, out, device=None) -> None:
    _dev(a, out)
    _len(out, a.numel(), "gpu_gelu_into")
    out.copy_(F.gelu(a).view_as(out))


def gpu_silu_bf16(a, device=None):
    _dev(a)
    _dt(a, torch.bfloat16, "gpu_silu_bf16")
    return F.silu(a)


def gpu_fatrelu_bf16(a, threshold: float, device=None):
    """``x if x >= threshold else 0`` (the ProSparse gate activation)."""
    _dev(a)
    _dt(a, torch.bfloat16, "gpu_fatrelu_bf16")
    return torch.where(a >= threshold, a, torch.zeros_like(a))


def gpu_scale_bf16(a, scale: float, device=None):
    _dev(a)
    _dt(a, torch.bfloat16, "gpu_scale_bf16")
    return a * scale


def gpu_scale_into(a, scalar: float, out, device=None) -> None:
    _dev(a, out)
    _len(out, a.numel(), "gpu_scale_into")
    torch.mul(a, scalar, out=out)


def _bcast(name, fn):
    def f(a, b, a_shape: Sequence[int], b_shape: Sequence[int], out_shape: Sequence[int], device=None):
        _dev(a, b)
        _len(a, int(np.prod(a_shape)) if len(a_shape) else 1, name)
        _len(b, int(np.prod(b_shape)) if len(b_shape) else 1, name)
        try:
            want = tuple(torch.broadcast_shapes(tuple(a_shape), tuple(b_shape)))
        except RuntimeError:
            raise ShapeMismatch(f"{name}: shapes {list(a_shape)} and {list(b_shape)} do not broadcast") from None
        if want != tuple(out_shape):
            raise ShapeMismatch(f"{name}: broadcast of {list(a_shape)} and {list(b_shape)} is {list(want)}, not {list(out_shape)}")
        return fn(a.reshape(tuple(a_shape)), b.reshape(tuple(b_shape))).reshape(-1)
    f.__name__ = name
    return f


gpu_broadcast_add, gpu_broadcast_sub, gpu_broadcast_mul = _bcast("gpu_broadcast_add", torch.add), _bcast("gpu_broadcast_sub", torch.sub), _bcast("gpu_broadcast_mul", torch.mul)


def gpu_dropout(x, threshold: int, scale: float, seed: int, device=None):
    """Keeps an element when its 32-bit draw is at or above ``threshold`` (= ``p * 2^32``) and multiplies it by ``scale`` (= ``1 / (1 - p)``).
    The draws come from a Philox stream keyed by ``seed``, so the mask is a function of (seed, position) only."""
    _dev(x)
    if not 0 <= threshold <= 0xFFFFFFFF:
        raise InvalidArgument(f"gpu_dropout: threshold {threshold} outside u32")
    g = torch.Generator(device=x.device).manual_seed(int(seed) & 0x7FFFFFFFFFFFFFFF)
    draws = torch.randint(0, 1 << 32, x.shape, generator=g, device=x.device, dtype=torch.int64)
    return torch.where(draws >= threshold, x * scale, torch.zeros_like(x))


# -- normalisation / softmax ---------------------------------------------------------------------------------------------------------
def gpu_softmax(x, rows: int, cols: int, device=None):
    _dev(x)
    _len(x, rows * cols, "gpu_softmax")
    return torch.softmax(x.reshape(rows, cols), -1).reshape(x.shape)


def gpu_softmax_into(x, out, rows: int, cols: int, device=None) -> None:
    _dev(x, out)
    _len(x, rows * cols, "gpu_softmax_into")
    _len(out, rows * cols, "gpu_softmax_into")
    torch.softmax(x.reshape(rows, cols), -1, out=out.view(rows, cols))


def gpu_softmax_bf16(x, rows: int, cols: int, device=None):
    _dev(x)
    _dt(x, torch.bfloat16, "gpu_softmax_bf16")
    _len(x, rows * cols, "gpu_softmax_bf16")
    return torch.softmax(x.reshape(rows, cols).float(), -1).to(torch.bfloat16).reshape(x.shape)


def gpu_layernorm(x, weight, bias, rows: int, cols: int, eps: float, device=None):
    _dev(x, weight, bias)
    _len(x, rows * cols, "gpu_layernorm")
    _len(weight, cols, "gpu_layernorm")
    _len(bias, cols, "gpu_layernorm")
    x2 = x.reshape(rows, cols)
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _ops().layer_norm(x2, weight, bias, eps).reshape(x.shape)
    return F.layer_norm(x2, (cols,), weight.reshape(-1), bias.reshape(-1), eps).reshape(x.shape)


def gpu_layernorm_into(x, weight, bias, out, rows: int, cols: int, eps: float, device=None) -> None:
    _len(out, rows * cols, "gpu_layernorm_into")
    out.copy_(gpu_layernorm(x, weight, bias, rows, cols, eps).view_as(out))


def gpu_rmsnorm_bf16(x, weight, rows: int, cols: int, eps: float, device=None):
    _dev(x, weight)
    _dt(x, torch.bfloat16, "gpu_rmsnorm_bf16")
    _len(x, rows * cols, "gpu_rmsnorm_bf16")
    _len(weight, cols, "gpu_rmsnorm_bf16")
    x2 = x.reshape(rows, cols)
    if x.is_cuda:
        return _ops().rms_norm(x2, weight.reshape(-1), eps).reshape(x.shape)
    xf = x2.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.reshape(-1).float()).to(torch.bfloat16).reshape(x.shape)


def gpu_group_norm_f32(x, weight, bias, batch: int, channels: int, groups: int, hw: int, eps: float, device=None):
    _dev(x, weight, bias)
    _len(x, batch * channels * hw, "gpu_group_norm_f32")
    if groups <= 0 or channels % groups:
        raise InvalidArgument(f"gpu_group_norm_f32: {channels} channels do not split into {groups} groups")
    return F.group_norm(x.reshape(batch, channels, hw), groups, weight.reshape(-1), bias.reshape(-1), eps).reshape(x.shape)


def gpu_block_reduce_max_abs_bf16(x, rows: int, n_blocks: int, block_size: int, device=None):
    """``[rows, n_blocks * block_size]`` bf16 -> f32 ``[rows * n_blocks]``: largest magnitude of every block of consecutive columns."""
    _dev(x)
    _dt(x, torch.bfloat16, "gpu_block_reduce_max_abs_bf16")
    _len(x, rows * n_blocks * block_size, "gpu_block_reduce_max_abs_bf16")
    return x.reshape(rows, n_blocks, block_size).abs().amax(-1).float().reshape(-1)


# -- matrix products -------------------------------------------------------------------------------------------------------------------
def _mm_check(a, b, m, k, n, what, batch=1):
    _dev(a, b)
    _len(a, batch * m * k, what)
    _len(b, batch * k * n, what)


def gpu_matmul_f32(a, b, m: int, k: int, n: int, device=None):
    _mm_check(a, b, m, k, n, "gpu_matmul_f32")
    _dt(a, torch.float32, "gpu_matmul_f32")
    return (a.reshape(m, k) @ b.reshape(k, n)).reshape(-1)


def gpu_matmul_f64(a, b, m: int, k: int, n: int, device=None):
    _mm_check(a, b, m, k, n, "gpu_matmul_f64")
    _dt(a, torch.float64, "gpu_matmul_f64")
    return (a.reshape(m, k) @ b.reshape(k, n)).reshape(-1)


def gpu_matmul_f32_into(a, b, out, m: int, k: int, n: int, device=None) -> None:
    _mm_check(a, b, m, k, n, "gpu_matmul_f32_into")
    _len(out, m * n, "gpu_matmul_f32_into")
    torch.mm(a.reshape(m, k), b.reshape(k, n), out=out.view(m, n))


gpu_small_matmul, gpu_small_matmul_into = gpu_matmul_f32, gpu_matmul_f32_into           # one code path serves every size here


def gpu_bmm_f32(a, b, batch: int, m: int, k: int, n: int, device=None):
    _mm_check(a, b, m, k, n, "gpu_bmm_f32", batch)
    return torch.bmm(a.reshape(batch, m, k), b.reshape(batch, k, n)).reshape(-1)


def gpu_bmm_f32_into(a, b, out, batch: int, m: int, k: int, n: int, device=None) -> None:
    _mm_check(a, b, m, k, n, "gpu_bmm_f32_into", batch)
    _len(out, batch * m * n, "gpu_bmm_f32_into")
    torch.bmm(a.reshape(batch, m, k), b.reshape(batch, k, n), out=out.view(batch, m, n))


gpu_small_bmm = gpu_bmm_f32


def _bf16_mm(a2: torch.Tensor, b2: torch.Tensor, b_is_nk: bool) -> torch.Tensor:
    """bf16 product with f32 accumulation: the tcgen05 GEMM on the device (shapes it cannot tile go to the library), plain matmul on the host."""
    if a2.is_cuda:
        try:
            return _ops().gemm(a2.contiguous(), b2.contiguous(), b_mn=not b_is_nk)
        except (InvalidArgument, ShapeMismatch):
            pass
    return (a2.float() @ (b2.float().t() if b_is_nk else b2.float())).to(torch.bfloat16)


def gpu_matmul_bf16_bf16(a, b, m: int, k: int, n: int, device=None):
    """``C[m, n] = A[m, k] @ B[k, n]``."""
    _mm_check(a, b, m, k, n, "gpu_matmul_bf16_bf16")
    _dt(a, torch.bfloat16, "gpu_matmul_bf16_bf16")
    _dt(b, torch.bfloat16, "gpu_matmul_bf16_bf16")
    return _bf16_mm(a.reshape(m, k), b.reshape(k, n), False).reshape(-1)


def gpu_matmul_bf16_bf16_nt(a, b, m: int, k: int, n: int, device=None):
    """``C[m, n] = A[m, k] @ B[n, k]^T``: the layout of ``Linear`` weights, no transposed copy."""
    _mm_check(a, b, m, k, n, "gpu_matmul_bf16_bf16_nt")
    _dt(a, torch.bfloat16, "gpu_matmul_bf16_bf16_nt")
    _dt(b, torch.bfloat16, "gpu_matmul_bf16_bf16_nt")
    return _bf16_mm(a.reshape(m, k), b.reshape(n, k), True).reshape(-1)


def _strided(buf, count, rows, cols, stride, what):
    if count > 1 and stride < rows * cols and stride != 0:
        raise InvalidArgument(f"{what}: stride {stride} overlaps {rows}x{cols} matrices")
    need = (count - 1) * stride + rows * cols
    if buf.numel() < need:
        raise ShapeMismatch(f"{what}: buffer has {buf.numel()} elements, {count} matrices at stride {stride} need {need}")
    return buf.reshape(-1).as_strided((count, rows, cols), (stride, cols, 1))


def gpu_matmul_bf16_bf16_strided_batched(a, b, m: int, k: int, n: int, batch_count: int, stride_a_elems: int, stride_b_elems: int, alpha: float = 1.0, device=None):
    """``C_i = alpha * A_i[m, k] @ B_i[k, n]`` for matrices laid out at fixed element strides (stride 0 re-uses one matrix for every batch)."""
    _dev(a, b)
    A, B = _strided(a, batch_count, m, k, stride_a_elems, "strided_batched A"), _strided(b, batch_count, k, n, stride_b_elems, "strided_batched B")
    return (torch.bmm(A.float(), B.float()) * alpha).to(torch.bfloat16).reshape(-1)


def gpu_matmul_bf16_bf16_strided_batched_nt(a, b, m: int, k: int, n: int, batch_count: int, stride_a_elems: int, stride_b_elems: int, alpha: float = 1.0, device=None):
    _dev(a, b)
    A, B = _strided(a, batch_count, m, k, stride_a_elems, "strided_batched_nt A"), _strided(b, batch_count, n, k, stride_b_elems, "strided_batched_nt B")
    return (torch.bmm(A.float(), B.float().transpose(1, 2)) * alpha).to(torch.bfloat16).reshape(-1)


def gpu_conv2d_f32(x, weight, bias, input_shape, weight_shape, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups: int = 1, device=None):
    _dev(x, weight, bias)
    _len(x, int(np.prod(input_shape)), "gpu_conv2d_f32")
    _len(weight, int(np.prod(weight_shape)), "gpu_conv2d_f32")
    if input_shape[1] != weight_shape[1] * groups:
        raise ShapeMismatch(f"gpu_conv2d_f32: {input_shape[1]} input channels vs weight {list(weight_shape)} with {groups} groups")
    return F.conv2d(x.reshape(tuple(input_shape)), weight.reshape(tuple(weight_shape)), None if bias is None else bias.reshape(-1), stride, padding, dilation, groups)


def _attn(q, k, v, n_q, n_k, d, d_v, batch_heads, scale, causal, what):
    _dev(q, k, v)
    _len(q, batch_heads * n_q * d, what)
    _len(k, batch_heads * n_k * d, what)
    _len(v, batch_heads * n_k * d_v, what)
    return F.scaled_dot_product_attention(q.reshape(1, batch_heads, n_q, d), k.reshape(1, batch_heads, n_k, d), v.reshape(1, batch_heads, n_k, d_v),
                                          is_causal=causal, scale=scale).reshape(-1)


def gpu_flash_attention_f32(q, k, v, n_q: int, n_k: int, d: int, d_v: int, batch_heads: int, scale: float, causal: bool, device=None):
    """Tiled attention that never materialises the ``n_q x n_k`` score matrix; ``[batch_heads, n, d]`` buffers."""
    _dt(q, torch.float32, "gpu_flash_attention_f32")
    return _attn(q, k, v, n_q, n_k, d, d_v, batch_heads, scale, causal, "gpu_flash_attention_f32")


def gpu_flash_attention_f64(q, k, v, n_q: int, n_k: int, d: int, d_v: int, batch_heads: int, scale: float, causal: bool, device=None):
    _dt(q, torch.float64, "gpu_flash_attention_f64")
    return _attn(q, k, v, n_q, n_k, d, d_v, batch_heads, scale, causal, "gpu_flash_attention_f64")


# -- layout / indexing -------------------------------------------------------------------------------------------------------------------
def gpu_transpose_2d(x, m: int, n: int, device=None):
    _dev(x)
    _len(x, m * n, "gpu_transpose_2d")
    return x.reshape(m, n).t().contiguous().reshape(-1)


def gpu_transpose_2d_into(x, out, m: int, n: int, device=None) -> None:
    _dev(x, out)
    _len(x, m * n, "gpu_transpose_2d_into")
    _len(out, m * n, "gpu_transpose_2d_into")
    out.view(n, m).copy_(x.reshape(m, n).t())


def gpu_permute_0213(x, d0: int, d1: int, d2: int, d3: int, device=None):
    _dev(x)
    _len(x, d0 * d1 * d2 * d3, "gpu_permute_0213")
    return x.reshape(d0, d1, d2, d3).permute(0, 2, 1, 3).contiguous().reshape(-1)


def gpu_permute_0213_into(x, out, d0: int, d1: int, d2: int, d3: int, device=None) -> None:
    _dev(x, out)
    _len(out, d0 * d1 * d2 * d3, "gpu_permute_0213_into")
    out.view(d0, d2, d1, d3).copy_(x.reshape(d0, d1, d2, d3).permute(0, 2, 1, 3))


def gpu_transpose_to_heads_bf16(x, num_heads: int, seq_len: int, head_dim: int, device=None):
    """``[seq, heads * dim] -> [heads, seq, dim]``."""
    _dev(x)
    _len(x, num_heads * seq_len * head_dim, "gpu_transpose_to_heads_bf16")
    return x.reshape(seq_len, num_heads, head_dim).transpose(0, 1).contiguous().reshape(-1)


def gpu_transpose_from_heads_bf16(x, num_heads: int, seq_len: int, head_dim: int, device=None):
    """``[heads, seq, dim] -> [seq, heads * dim]``."""
    _dev(x)
    _len(x, num_heads * seq_len * head_dim, "gpu_transpose_from_heads_bf16")
    return x.reshape(num_heads, seq_len, head_dim).transpose(0, 1).contiguous().reshape(-1)


def gpu_repeat_kv_bf16(x, num_kv_heads: int, group_size: int, seq_len: int, head_dim: int, device=None):
    """``[kv_heads, seq, dim] -> [kv_heads * group, seq, dim]``: every KV head repeated for the query heads that share it."""
    _dev(x)
    _len(x, num_kv_heads * seq_len * head_dim, "gpu_repeat_kv_bf16")
    return x.reshape(num_kv_heads, seq_len, head_dim).repeat_interleave(group_size, 0).reshape(-1)


def gpu_rope_half_bf16(x, cos_cache, sin_cache, num_heads: int, seq_len: int, head_dim: int, seq_offset: int, device=None):
    """Half-split rotary embedding of ``[heads, seq, dim]``: pairs ``(i, i + dim / 2)`` rotate by the angle of position ``seq_offset + s``;
    the caches are ``[max_pos, dim / 2]``."""
    _dev(x, cos_cache, sin_cache)
    _len(x, num_heads * seq_len * head_dim, "gpu_rope_half_bf16")
    half = head_dim // 2
    if head_dim % 2 or cos_cache.numel() % half or cos_cache.numel() // half < seq_offset + seq_len or sin_cache.numel() != cos_cache.numel():
        raise ShapeMismatch(f"gpu_rope_half_bf16: caches of {cos_cache.numel()} elements do not cover positions {seq_offset}..{seq_offset + seq_len} at dim {head_dim}")
    c = cos_cache.reshape(-1, half)[seq_offset: seq_offset + seq_len].float()
    s = sin_cache.reshape(-1, half)[seq_offset: seq_offset + seq_len].float()
    t = x.reshape(num_heads, seq_len, head_dim).float()
    a, b = t[..., :half], t[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], -1).to(x.dtype).reshape(-1)


def gpu_causal_mask_bf16(buf, batch: int, seq_q: int, seq_k: int, device=None) -> None:
    """In place on ``[batch, seq_q, seq_k]`` scores: entries whose key lies after the query (aligned at the end) become ``-inf``."""
    _dev(buf)
    _len(buf, batch * seq_q * seq_k, "gpu_causal_mask_bf16")
    mask = torch.ones(seq_q, seq_k, dtype=torch.bool, device=buf.device).triu(seq_k - seq_q + 1)
    buf.view(batch, seq_q, seq_k).masked_fill_(mask, float("-inf"))


def gpu_causal_mask_indirect(total_len_ptr, n_head: int, max_pos: int, out, device=None) -> None:
    """``out[h, col] = 0`` for ``col < total_len`` else ``-1e9``, with ``total_len`` read from device memory so that a captured graph follows
    the growing sequence without being re-recorded."""
    _dev(total_len_ptr, out)
    _len(out, n_head * max_pos, "gpu_causal_mask_indirect")
    cols = torch.arange(max_pos, device=out.device)
    out.view(n_head, max_pos).copy_(torch.where(cols < total_len_ptr.reshape(-1)[0], 0.0, -1e9).to(out.dtype).expand(n_head, max_pos))


def gpu_embed_lookup(idx, weight, d: int, device=None):
    """Rows of ``weight [V, d]`` for indices stored as floats (the reference keeps them in an f32 buffer)."""
    _dev(idx, weight)
    if weight.numel() % d:
        raise ShapeMismatch(f"gpu_embed_lookup: weight of {weight.numel()} elements is not a multiple of d = {d}")
    i = idx.reshape(-1).long()
    if i.numel() and (int(i.min()) < 0 or int(i.max()) >= weight.numel() // d):
        raise InvalidArgument(f"gpu_embed_lookup: index out of range for {weight.numel() // d} rows")
    return weight.reshape(-1, d)[i].reshape(-1)


def gpu_embed_lookup_into(idx, weight, out, d: int, device=None) -> None:
    r = gpu_embed_lookup(idx, weight, d)
    _len(out, r.numel(), "gpu_embed_lookup_into")
    out.copy_(r.view_as(out))


def gpu_embedding_gather_bf16(weight, indices, dim: int, device=None):
    _dev(weight, indices)
    _dt(weight, torch.bfloat16, "gpu_embedding_gather_bf16")
    i = indices.reshape(-1).long()
    if i.numel() and int(i.max()) >= weight.numel() // dim:
        raise InvalidArgument(f"gpu_embedding_gather_bf16: index {int(i.max())} out of range for {weight.numel() // dim} rows")
    w = weight.reshape(-1, dim)
    return (_ops().embedding(i, w) if w.is_cuda else w[i]).reshape(-1)


def gpu_embedding_gather_bf16_to_f32(weight, indices, dim: int, device=None):
    return gpu_embedding_gather_bf16(weight, indices, dim).float()


def gpu_slice_write(src, dst, n_batch: int, d: int, max_len: int, pos: int, device=None) -> None:
    """``dst[n, pos, :] = src[n, :]`` for ``dst [N, max_len, D]``: one decode step's keys or values into a cache."""
    _dev(src, dst)
    _len(src, n_batch * d, "gpu_slice_write")
    _len(dst, n_batch * max_len * d, "gpu_slice_write")
    if not 0 <= pos < max_len:
        raise InvalidArgument(f"gpu_slice_write: position {pos} outside the cache of {max_len}")
    dst.view(n_batch, max_len, d)[:, pos].copy_(src.view(n_batch, d))


def gpu_slice_write_indirect(src, dst, n_batch: int, d: int, max_len: int, pos_ptr, device=None) -> None:
    """As :func:`gpu_slice_write` with the position read from device memory (graph-capturable); a position outside the cache writes nothing."""
    _dev(src, dst, pos_ptr)
    _len(src, n_batch * d, "gpu_slice_write_indirect")
    _len(dst, n_batch * max_len * d, "gpu_slice_write_indirect")
    pos = pos_ptr.reshape(-1)[:1].long()
    ok = (pos >= 0) & (pos < max_len)
    idx = pos.clamp(0, max_len - 1).view(1, 1, 1).expand(n_batch, 1, d)
    cur = dst.view(n_batch, max_len, d).gather(1, idx)
    dst.view(n_batch, max_len, d).scatter_(1, idx, torch.where(ok.view(1, 1, 1), src.view(n_batch, 1, d), cur))


def gpu_slice_read(src, n_batch: int, d: int, length: int, max_len: int, device=None):
    """First ``length`` positions of a ``[N, max_len, D]`` cache as a packed ``[N, length, D]`` buffer."""
    _dev(src)
    _len(src, n_batch * max_len * d, "gpu_slice_read")
    if not 0 <= length <= max_len:
        raise InvalidArgument(f"gpu_slice_read: length {length} outside the cache of {max_len}")
    return src.view(n_batch, max_len, d)[:, :length].contiguous().reshape(-1)


def gpu_slice_read_into(src, out, n_batch: int, d: int, length: int, max_len: int, device=None) -> None:
    r = gpu_slice_read(src, n_batch, d, length, max_len)
    _len(out, r.numel(), "gpu_slice_read_into")
    out.copy_(r.view_as(out))


def gpu_roll_f32(x, outer: int, dim_size: int, inner: int, shift_norm: int, device=None):
    _dev(x)
    _len(x, outer * dim_size * inner, "gpu_roll_f32")
    return torch.roll(x.reshape(outer, dim_size, inner), shift_norm % max(dim_size, 1), 1).reshape(-1)


def gpu_nearest_upsample2x_f32(x, batch: int, channels: int, h: int, w: int, device=None):
    _dev(x)
    _len(x, batch * channels * h * w, "gpu_nearest_upsample2x_f32")
    return x.reshape(batch, channels, h, w).repeat_interleave(2, 2).repeat_interleave(2, 3).reshape(-1)


# -- allocation, transfer, device ---------------------------------------------------------------------------------------------------------------
def round_len(n: int) -> int:
    from . import BufferPool
    return BufferPool.round_len(n)


def alloc_zeros_f32(n: int, device=None):
    from . import alloc_zeros
    return alloc_zeros(n, torch.float32, device)


def alloc_zeros_f64(n: int, device=None):
    from . import alloc_zeros
    return alloc_zeros(n, torch.float64, device)


def tensor_to_gpu(t: torch.Tensor, device=None) -> torch.Tensor:
    from . import cpu_to_gpu
    return t if t.is_cuda else cpu_to_gpu(t, device)


def tensor_to_cpu(t: torch.Tensor) -> torch.Tensor:
    from . import gpu_to_cpu
    return gpu_to_cpu(t) if t.is_cuda else t


def get_cuda_device(ordinal: int = 0):
    from . import GpuDevice
    if not torch.cuda.is_available():
        from ..errors import DeviceUnavailable
        raise DeviceUnavailable("no CUDA device is visible to this process")
    if not 0 <= ordinal < torch.cuda.device_count():
        raise InvalidArgument(f"CUDA device {ordinal} out of range ({torch.cuda.device_count()} visible)")
    return GpuDevice(ordinal)


cuda = get_cuda_device


def cuda_default():
    return get_cuda_device(torch.cuda.current_device() if torch.cuda.is_available() else 0)


def cached_bytes(device: int = 0) -> int:
    """Bytes held by the caching allocator beyond what live tensors use."""
    return torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device) if torch.cuda.is_available() else 0


def empty_cache(device: Optional[int] = None) -> None:
    if torch.cuda.is_available():
        with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
            torch.cuda.empty_cache()


def empty_cache_all() -> None:
    for d in range(torch.cuda.device_count() if torch.cuda.is_available() else 0):
        empty_cache(d)


# -- stream capture with explicit begin / end and pool handles (graph.rs:91-770) ---------------------------------------------------------
class CaptureStatus(enum.Enum):
    None_ = "none"
    Active = "active"
    Invalidated = "invalidated"

    def is_capturing(self) -> bool:
        return self is CaptureStatus.Active


_captures: Dict[int, Any] = {}
_pool_ids = itertools.count(1)
_pools: Dict[int, Any] = {}
_reg_lock = threading.Lock()


@dataclass(frozen=True)
class GraphPoolHandle:
    id: int


def graph_pool_handle() -> GraphPoolHandle:
    """A fresh private memory pool for graph captures, registered under an opaque handle so that several captures can share it."""
    from . import CapturePool
    h = GraphPoolHandle(next(_pool_ids))
    with _reg_lock:
        _pools[h.id] = CapturePool()
    return h


def capture_pool_for_handle(handle: GraphPoolHandle):
    with _reg_lock:
        return _pools.get(handle.id)


def release_graph_pool_handle(handle: GraphPoolHandle) -> None:
    with _reg_lock:
        _pools.pop(handle.id, None)


def capture_status(stream: Optional[torch.cuda.Stream] = None) -> CaptureStatus:
    if not torch.cuda.is_available():
        return CaptureStatus.None_
    with torch.cuda.stream(stream or torch.cuda.current_stream()):
        return CaptureStatus.Active if torch.cuda.is_current_stream_capturing() else CaptureStatus.None_


def is_stream_capturing(stream: Optional[torch.cuda.Stream] = None) -> bool:
    return capture_status(stream).is_capturing()


def begin_capture_with_mode(stream: torch.cuda.Stream, mode=None, pool=None) -> None:
    """Starts recording the work submitted to ``stream``; :func:`end_capture` on the same stream returns the graph. ``stream`` must not be
    the default stream."""
    from . import CaptureMode, GpuError
    if id(stream) in _captures:
        raise GpuError("begin_capture: this stream is already capturing")
    g = torch.cuda.CUDAGraph()
    ctx = torch.cuda.graph(g, pool=pool.handle if pool is not None else None, stream=stream, capture_error_mode=(mode or CaptureMode.THREAD_LOCAL).value)
    ctx.__enter__()
    _captures[id(stream)] = (g, ctx)


def begin_capture(stream: torch.cuda.Stream) -> None:
    begin_capture_with_mode(stream)


def end_capture(stream: torch.cuda.Stream):
    from . import CapturedGraph, GpuError
    ent = _captures.pop(id(stream), None)
    if ent is None:
        raise GpuError("end_capture: begin_capture was not called on this stream")
    g, ctx = ent
    ctx.__exit__(None, None, None)
    return CapturedGraph(g)


def end_capture_with_pool(stream: torch.cuda.Stream, pool):
    """Ends the capture and ties the graph's lifetime to ``pool``: the pool keeps the graph's private allocations alive for the graphs that
    share them."""
    cg = end_capture(stream)
    cg.pool = pool
    return cg


# -- memory statistics, hooks, watchdog (memory_guard.rs) -------------------------------------------------------------------------------------
@dataclass
class MemoryStats:
    used_bytes: int
    budget_bytes: int
    peak_bytes: int
    free_device_bytes: int
    total_device_bytes: int
    num_allocations: int
    num_oom_recoveries: int

    @classmethod
    def of(cls, guard) -> "MemoryStats":
        s = guard.stats()
        used, total = guard._query()
        return cls(s.used, s.budget, s.peak_used, max(total - used, 0), total, getattr(guard, "_n_alloc", 0), s.oom_events)


class MemoryHook:
    """Called before an allocation fails: ``on_pressure(needed_bytes) -> freed_bytes`` (drop caches, evict, ...). ``name`` and ``priority``
    order and label it; register with ``MemoryGuard.add_pre_oom_hook`` or :func:`register_hook`."""
    name = "hook"
    priority = 0

    def on_pressure(self, needed_bytes: int) -> int:
        raise NotImplementedError

    def __call__(self, needed_bytes: int) -> int:
        return self.on_pressure(needed_bytes)


class MemoryPressureListener:
    """``on_pressure_change(old, new)`` is called when the pressure level of a guard changes (memory_guard.rs:206)."""

    def on_pressure_change(self, old, new) -> None:
        raise NotImplementedError

    def __call__(self, old, new) -> None:
        self.on_pressure_change(old, new)


def register_hook(guard, hook: MemoryHook) -> None:
    guard.add_pre_oom_hook(hook.name, hook, hook.priority)


class MemoryWatchdog:
    """Polls free device memory; below ``pressure_threshold_bytes`` it raises the paused flag that cooperative workers check with
    :meth:`wait_if_paused`, and lowers it when memory recovers (memory_guard.rs:1101). ``query`` returns ``(free, total)`` bytes."""

    def __init__(self, query: Optional[Callable[[], Tuple[int, int]]] = None, pressure_threshold_bytes: int = 1 << 30, check_interval_s: float = 0.05):
        self._query = query or (lambda: torch.cuda.mem_get_info())
        self.pressure_threshold_bytes, self.check_interval_s = int(pressure_threshold_bytes), check_interval_s
        self._paused = threading.Event()
        self._resume = threading.Event()
        self._resume.set()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def check_pressure(self) -> bool:
        """One poll: returns (and records) whether free memory is under the threshold."""
        low = self._query()[0] < self.pressure_threshold_bytes
        if low:
            self._paused.set()
            self._resume.clear()
        else:
            self._paused.clear()
            self._resume.set()
        return low

    def is_paused(self) -> bool:
        return self._paused.is_set()

    def start(self) -> threading.Thread:
        def loop():
            while not self._stop.wait(self.check_interval_s):
                self.check_pressure()
        self._stop.clear()
        self._thread = threading.Thread(target=loop, daemon=True, name="ft-memory-watchdog")
        self._thread.start()
        return self._thread

    def stop(self) -> None:
        self._stop.set()
        self._resume.set()
        if self._thread is not None:
            self._thread.join(2.0)

    def wait_if_paused(self, timeout_s: Optional[float] = None) -> bool:
        """Blocks while paused; ``True`` when running again, ``False`` when ``timeout_s`` passed first."""
        return self._resume.wait(timeout_s)


class MemoryGuardedDevice:
    """A device with the guard that budgets it: allocations go through ``reserve`` first (memory_guard.rs:1262)."""

    def __init__(self, device, guard):
        self._device, self.guard = device, guard

    def device(self):
        return self._device

    def alloc_zeros(self, n: int, dtype=torch.float32):
        from . import alloc_zeros
        r = self.guard.reserve(n * torch.empty((), dtype=dtype).element_size())
        try:
            buf = alloc_zeros(n, dtype, self._device)
        except BaseException:
            r.release()
            raise
        buf._reservation = r
        return buf

    def stats(self) -> MemoryStats:
        return MemoryStats.of(self.guard)


# -- host Philox generator and RNG fork / join (rng.rs:140-530) ----------------------------------------------------------------------------------
_M32 = np.uint64(0xFFFFFFFF)


def _philox4x32(counters: np.ndarray, key: Tuple[int, int]) -> np.ndarray:
    """Philox-4x32-10 of ``[n, 4]`` uint32 counters under a 64-bit key -> ``[n, 4]`` uint32."""
    c = counters.astype(np.uint64)
    k0, k1 = np.uint64(key[0]), np.uint64(key[1])
    for _ in range(10):
        p0, p1 = np.uint64(0xD2511F53) * c[:, 0], np.uint64(0xCD9E8D57) * c[:, 2]
        c = np.stack([((p1 >> np.uint64(32)) ^ c[:, 1] ^ k0) & _M32, p1 & _M32, ((p0 >> np.uint64(32)) ^ c[:, 3] ^ k1) & _M32, p0 & _M32], 1)
        k0, k1 = (k0 + np.uint64(0x9E3779B9)) & _M32, (k1 + np.uint64(0xBB67AE85)) & _M32
    return c.astype(np.uint32)


class PhiloxGenerator:
    """Counter-based generator on the host: every 128-bit counter yields four 32-bit draws; the state is ``(seed, offset)`` with ``offset``
    counting the counters consumed, so a saved state replays the same stream and ``advance`` skips ahead in O(1)."""

    def __init__(self, seed: int = 0):
        self.seed, self.offset, self._buf = int(seed) & 0xFFFFFFFFFFFFFFFF, 0, []

    def set_seed(self, seed: int) -> None:
        self.seed, self.offset, self._buf = int(seed) & 0xFFFFFFFFFFFFFFFF, 0, []

    def get_state(self):
        from . import PhiloxState
        return PhiloxState(self.seed, self.offset)

    def set_state(self, st) -> None:
        self.seed, self.offset, self._buf = int(st.seed), int(st.offset), []

    def advance(self, n_counters: int) -> None:
        self.offset += int(n_counters)
        self._buf = []

    def _block(self, n: int) -> np.ndarray:
        idx = np.arange(self.offset, self.offset + n, dtype=np.uint64)
        ctr = np.stack([idx & _M32, idx >> np.uint64(32), np.zeros(n, np.uint64), np.zeros(n, np.uint64)], 1)
        self.offset += n
        return _philox4x32(ctr, (self.seed & 0xFFFFFFFF, self.seed >> 32))

    def next_u32(self) -> int:
        if not self._buf:
            self._buf = self._block(1)[0].tolist()
        return int(self._buf.pop(0))

    def next_f32(self) -> float:
        """Uniform in [0, 1): the top 24 bits of a draw."""
        return (self.next_u32() >> 8) * (1.0 / (1 << 24))

    def generate_uniform(self, n: int) -> np.ndarray:
        self._buf = []
        return ((self._block(-(-n // 4)).reshape(-1)[:n] >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / (1 << 24)))


def cuda_rng_manager():
    from . import rng_manager
    return rng_manager


def fork_rng(devices: Sequence[int]):
    """States of the generators of ``devices``, to be handed back to :func:`join_rng` after a region that must not disturb them."""
    m = cuda_rng_manager()
    return [m.get_state(d) for d in devices]


def join_rng(devices: Sequence[int], states: Sequence) -> None:
    if len(devices) != len(states):
        raise ShapeMismatch(f"join_rng: {len(devices)} devices but {len(states)} states")
    m = cuda_rng_manager()
    for d, s in zip(devices, states):
        m.set_state(s, d)
