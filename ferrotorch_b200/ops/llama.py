"""RoPE, SwiGLU, embedding and residual-add on the hand-written kernels, with autograd.

Reference parity: half-rotation RoPE (ferrotorch-gpu/src/bf16.rs:1438, ferrotorch-nn/src/transformer.rs:49,503),
SwiGLU (ferrotorch-nn/src/transformer.rs:677), Embedding (ferrotorch-nn/src/embedding.rs:66,195).
"""
from __future__ import annotations

import math

import torch

from ..errors import InvalidArgument

from .. import _lib


def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None = None, seq_len: int | None = None):
    """Inverse frequencies ``[head_dim / 2]`` (f64) and the factor that multiplies the cos / sin tables, for a rope-scaling description.

    ``scaling`` is either this framework's form ``{"type": "linear" | "ntk" | "yarn", "factor": f, ...}`` (the variants of
    ferrotorch-nn/src/transformer.rs:210-266: linear position interpolation, static NTK-aware base scaling, YaRN) or a HF ``rope_scaling``
    dict ``{"rope_type": "default" | "linear" | "dynamic" | "llama3" | "yarn", ...}`` as found in ``config.json`` (``llama3``: the
    frequency-dependent scaling of Llama 3.1 and later; ``dynamic``: NTK base scaling that grows with ``seq_len`` beyond
    ``original_max_position_embeddings``; the reference ignores ``rope_scaling`` altogether). HF YaRN dicts also scale the tables by
    ``0.1 ln(factor) + 1`` (or their ``attention_factor``), as the HF implementation does. Unknown types are refused, not ignored."""
    half = head_dim // 2
    base = float(theta)
    # older HF configs spell the key "type"; what tells them from this framework's own dicts is the HF name of the original-length field
    hf = bool(scaling) and ("rope_type" in scaling or "original_max_position_embeddings" in scaling)
    kind = (scaling.get("rope_type") or scaling.get("type") or "none") if scaling else "none"
    att = 1.0
    if kind in ("none", "default"):
        return 1.0 / (base ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / head_dim)), att
    factor = float(scaling.get("factor", 1.0))
    if kind == "ntk":
        base = base * factor ** (head_dim / (head_dim - 2))
    inv = 1.0 / (base ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / head_dim))
    if kind == "ntk":
        return inv, att
    if kind == "linear":
        return inv / factor, att
    if kind == "dynamic":
        orig = scaling.get("original_max_position_embeddings", scaling.get("max_position_embeddings"))
        if orig is None:
            raise InvalidArgument("dynamic rope scaling needs original_max_position_embeddings")
        n = max(int(seq_len or orig), int(orig))
        b = base * ((factor * n / orig) - (factor - 1)) ** (head_dim / (head_dim - 2))
        return 1.0 / (b ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / head_dim)), att
    if kind == "llama3":
        lo_f, hi_f = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        old = float(scaling.get("original_max_position_embeddings", 8192))
        wavelen = 2 * math.pi / inv
        inv_l = torch.where(wavelen > old / lo_f, inv / factor, inv)
        smooth = (old / wavelen - lo_f) / (hi_f - lo_f)
        smoothed = (1 - smooth) * inv_l / factor + smooth * inv_l
        medium = ~(wavelen < old / hi_f) & ~(wavelen > old / lo_f)
        return torch.where(medium, smoothed, inv_l), att
    if kind == "yarn":
        orig = scaling.get("original_max_position", scaling.get("original_max_position_embeddings"))
        if orig is None:
            raise InvalidArgument("yarn rope scaling needs the original maximum position")
        beta_fast, beta_slow = float(scaling.get("beta_fast", 32.0)), float(scaling.get("beta_slow", 1.0))

        def corr(n):
            return head_dim * math.log(orig / (n * 2 * math.pi)) / (2 * math.log(base))
        lo, hi = max(math.floor(corr(beta_fast)), 0), min(math.ceil(corr(beta_slow)), head_dim - 1)
        ramp = ((torch.arange(half, dtype=torch.float64) - lo) / (hi - lo if hi != lo else 1e-3)).clamp(0, 1)
        if hf or "attention_factor" in scaling:
            att = float(scaling.get("attention_factor") or (0.1 * math.log(factor) + 1.0 if factor > 1 else 1.0))
        return inv / factor * ramp + inv * (1 - ramp), att
    raise InvalidArgument(f"unknown rope scaling type {kind!r} (none, default, linear, ntk, dynamic, llama3, yarn)")


def rope_tables(max_pos: int, head_dim: int, theta: float, device, scaling: dict | None = None):
    """cos/sin tables ``[max_pos, head_dim/2]`` in f32 for the scaling description of :func:`rope_inv_freq`."""
    inv, att = rope_inv_freq(head_dim, theta, scaling, seq_len=max_pos)
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float64), inv)
    return (ang.cos() * att).float().to(device).contiguous(), (ang.sin() * att).float().to(device).contiguous()


def rope_inplace(x2: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq_len: int, head0: int, nheads: int, head_dim: int,
                 inverse: bool = False, positions: torch.Tensor | None = None) -> torch.Tensor:
    """Rotate heads ``[head0, head0+nheads)`` of the packed ``[tokens, row]`` buffer in place."""
    tokens = x2.shape[0]
    if x2.is_cuda:
        _lib.call("ft_rope_inplace", x2, cos, sin, positions, tokens, seq_len, x2.stride(0), head0, nheads, head_dim, int(inverse),
                  _lib.S())
        return x2
    pos = positions.long() if positions is not None else (torch.arange(tokens, device=x2.device) % seq_len)
    c, s = cos[pos].unsqueeze(1), sin[pos].unsqueeze(1)
    if inverse:
        s = -s
    v = x2[:, head0 * head_dim:(head0 + nheads) * head_dim].reshape(tokens, nheads, head_dim).float()
    a, b = v[..., : head_dim // 2], v[..., head_dim // 2:]
    out = torch.cat([a * c - b * s, b * c + a * s], -1).to(x2.dtype)
    x2[:, head0 * head_dim:(head0 + nheads) * head_dim] = out.reshape(tokens, nheads * head_dim)
    return x2


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, positions):
        # x: [B, S, H, D]
        B, S, H, D = x.shape
        y = x.contiguous().clone().reshape(B * S, H * D)
        rope_inplace(y, cos, sin, S, 0, H, D, False, positions)
        ctx.save_for_backward(cos, sin, positions if positions is not None else torch.empty(0))
        ctx.meta = (B, S, H, D, positions is not None)
        return y.reshape(B, S, H, D)

    @staticmethod
    def backward(ctx, dy):
        cos, sin, pos = ctx.saved_tensors
        B, S, H, D, has_pos = ctx.meta
        g = dy.contiguous().clone().reshape(B * S, H * D)
        rope_inplace(g, cos, sin, S, 0, H, D, True, pos if has_pos else None)
        return g.reshape(B, S, H, D), None, None, None


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor | None = None) -> torch.Tensor:
    """Half-rotation RoPE on ``x`` of shape ``[B, S, H, D]`` (differentiable)."""
    return _RopeFn.apply(x, cos, sin, positions)


def swiglu_fwd(gu2: torch.Tensor) -> torch.Tensor:
    rows, F2 = gu2.shape
    F = F2 // 2
    if gu2.is_cuda:
        out = torch.empty((rows, F), device=gu2.device, dtype=gu2.dtype)
        _lib.call("ft_swiglu_fwd", gu2, out, rows, F, _lib.S())
        return out
    g, u = gu2[:, :F].float(), gu2[:, F:].float()
    return (torch.nn.functional.silu(g) * u).to(gu2.dtype)


def swiglu_bwd(gu2: torch.Tensor, dout2: torch.Tensor, inplace: bool = False) -> torch.Tensor:
    rows, F2 = gu2.shape
    F = F2 // 2
    if gu2.is_cuda:
        dgu = gu2 if inplace else torch.empty_like(gu2)
        _lib.call("ft_swiglu_bwd", gu2, dout2, dgu, rows, F, _lib.S())
        return dgu
    g, u, d = gu2[:, :F].float(), gu2[:, F:].float(), dout2.float()
    sg = torch.sigmoid(g)
    silu = g * sg
    return torch.cat([d * u * (sg + silu * (1 - sg)), d * silu], 1).to(gu2.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        shp = gu.shape
        gu2 = gu.reshape(-1, shp[-1]).contiguous()
        ctx.save_for_backward(gu2)
        ctx.shp = shp
        return swiglu_fwd(gu2).reshape(*shp[:-1], shp[-1] // 2)

    @staticmethod
    def backward(ctx, dout):
        (gu2,) = ctx.saved_tensors
        return swiglu_bwd(gu2, dout.reshape(gu2.shape[0], -1).contiguous()).reshape(ctx.shp)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up = [..., gate | up]`` (differentiable, one fused kernel each way)."""
    return _SwiGLUFn.apply(gate_up)


def embedding_fwd(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    flat = ids.reshape(-1).contiguous()
    if table.is_cuda and table.dtype == torch.bfloat16 and table.shape[1] % 8 == 0:
        out = torch.empty((flat.numel(), table.shape[1]), device=table.device, dtype=table.dtype)
        _lib.call("ft_embedding_fwd", flat, table, out, flat.numel(), table.shape[1], table.shape[0], None, _lib.S())
        return out.reshape(*ids.shape, table.shape[1])
    return table[flat].reshape(*ids.shape, table.shape[1])


def embedding_bwd(ids: torch.Tensor, dout2: torch.Tensor, dtable: torch.Tensor, deterministic: bool = True) -> torch.Tensor:
    """``dtable[ids] += dout`` (dtable bf16 or f32, already zeroed or holding a running sum). The default groups the token rows by id (stable
    sort) and sums each table row in token order in f32 without atomics, so repeated runs give identical bits; ``deterministic=False`` is the
    atomic scatter (a little faster, order of the additions left to the hardware)."""
    flat = ids.reshape(-1).contiguous()
    if dtable.is_cuda and dout2.dtype == torch.bfloat16:
        d = dtable.shape[1]
        if deterministic and d % 8 == 0:
            sorted_ids, perm = torch.sort(flat, stable=True)
            uniq, counts = torch.unique_consecutive(sorted_ids, return_counts=True)
            seg_end = torch.cumsum(counts, 0)
            _lib.call("ft_embedding_bwd_sorted", uniq, seg_end, perm, dout2, dtable, uniq.numel(), d, dtable.shape[0],
                      int(dtable.dtype == torch.float32), _lib.S())
            return dtable
        _lib.call("ft_embedding_bwd", flat, dout2, dtable, flat.numel(), d, dtable.shape[0],
                  int(dtable.dtype == torch.float32), _lib.S())
        return dtable
    dtable.index_add_(0, flat, dout2.to(dtable.dtype))
    return dtable


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        ctx.save_for_backward(ids)
        ctx.tshape = table.shape
        return embedding_fwd(ids, table)

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        dt = torch.zeros(ctx.tshape, device=dout.device, dtype=dout.dtype)
        embedding_bwd(ids, dout.reshape(-1, ctx.tshape[1]).contiguous(), dt)
        return None, dt


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    return _EmbeddingFn.apply(ids, table)


def add_(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out = a + b`` for contiguous bf16 tensors (``out`` may alias ``a``)."""
    out = a if out is None else out
    if a.is_cuda and a.dtype == torch.bfloat16 and a.numel() % 8 == 0 and a.is_contiguous() and b.is_contiguous():
        _lib.call("ft_add_bf16", a, b, out, a.numel(), _lib.S())
        return out
    return torch.add(a, b, out=out)
