"""Python surface of the generic device kernels: elementwise (unary / backward / binary / where / cast / fill), strided copies, reductions,
scans, index ops, Philox random numbers and dropout, multi-tensor unscale, GGUF block dequantisation and vocabulary masks.

Each function checks its operands, allocates the result and calls one exported launcher of the kernels library on the current stream.
CPU tensors (and dtypes the kernels do not cover) take the equivalent torch expression, so the module is usable everywhere; on a CUDA
device the native path is the one that runs.

Reference parity: ferrotorch-gpu/src/kernels.rs:13031-26770 (free ``gpu_*`` functions), ferrotorch-gpu/src/rng.rs, ferrotorch-cubecl/src/quant.rs.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import torch

from .. import _lib
from ..errors import InvalidArgument

_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2, torch.float64: 3}
UNARY = {n: i for i, n in enumerate(
    ["neg", "abs", "exp", "log", "sqrt", "rsqrt", "reciprocal", "sin", "cos", "tanh", "sigmoid", "relu", "gelu", "gelu_tanh", "silu", "elu", "mish",
     "erf", "floor", "ceil", "round", "sign", "square", "softplus", "scale", "add_scalar", "pow_scalar", "clamp", "leaky_relu", "hardswish",
     "hardsigmoid", "exp2", "log2", "log1p", "expm1", "copy", "fatrelu"])}
UNARY_BWD = {n: i for i, n in enumerate(
    ["relu", "abs", "sigmoid_y", "tanh_y", "gelu", "gelu_tanh", "silu", "elu", "mish", "clamp", "leaky_relu", "exp_y", "log", "sqrt_y", "softplus",
     "hardswish", "hardtanh"])}
BINARY = {n: i for i, n in enumerate(["add", "sub", "mul", "div", "pow", "maximum", "minimum", "eq", "ne", "lt", "le", "gt", "ge", "atan2", "fmod"])}
REDUCE = {n: i for i, n in enumerate(["sum", "prod", "min", "max", "mean", "sumsq", "absmax", "logsumexp"])}
SCAN = {n: i for i, n in enumerate(["cumsum", "cumprod", "cummax", "cummin", "logcumsumexp"])}
GGUF_TYPES = {"q4_0": 2, "q4_1": 3, "q5_0": 6, "q5_1": 7, "q8_0": 8, "q8_1": 9}
GGUF_BLOCK_BYTES = {"q4_0": 18, "q4_1": 20, "q5_0": 22, "q5_1": 24, "q8_0": 34, "q8_1": 36}


def _native(*ts: torch.Tensor) -> bool:
    return all(t.is_cuda and t.dtype in _DT for t in ts)


def _i64(vals: Sequence[int]):
    return (ctypes.c_int64 * len(vals))(*vals)


def unary(op: str, x: torch.Tensor, a: float = 0.0, b: float = 0.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out = op(x)``; ``a``/``b`` are the op's parameters (ELU alpha, clamp bounds, ``scale``: x*a+b, softplus beta/threshold ...)."""
    if op not in UNARY:
        raise InvalidArgument(f"unknown unary op {op}")
    if not _native(x):
        return _unary_torch(op, x, a, b)
    if out is None:
        out = torch.empty(x.shape, device=x.device, dtype=x.dtype)
    if x.is_contiguous() and out.is_contiguous():
        _lib.call("ft_ew_unary", _DT[x.dtype], UNARY[op], x, out, x.numel(), float(a), float(b), _lib.S())
    else:
        if x.dim() > 6 or not out.is_contiguous():
            return unary(op, x.contiguous(), a, b)
        shp = list(x.shape) or [1]
        _lib.call("ft_ew_unary_strided", _DT[x.dtype], UNARY[op], x, out, len(shp), _i64(shp), _i64(list(x.stride()) or [1]), float(a), float(b), _lib.S())
    return out


def _unary_torch(op, x, a, b):
    F = torch.nn.functional
    table = {"neg": torch.neg, "abs": torch.abs, "exp": torch.exp, "log": torch.log, "sqrt": torch.sqrt, "rsqrt": torch.rsqrt, "reciprocal": torch.reciprocal,
             "sin": torch.sin, "cos": torch.cos, "tanh": torch.tanh, "sigmoid": torch.sigmoid, "relu": torch.relu, "gelu": F.gelu,
             "gelu_tanh": lambda t: F.gelu(t, approximate="tanh"), "silu": F.silu, "elu": lambda t: F.elu(t, a), "mish": F.mish, "erf": torch.erf,
             "floor": torch.floor, "ceil": torch.ceil, "round": torch.round, "sign": torch.sign, "square": torch.square,
             "softplus": lambda t: F.softplus(t, a or 1.0, b or 20.0), "scale": lambda t: t * a + b, "add_scalar": lambda t: t + a,
             "pow_scalar": lambda t: t.pow(a), "clamp": lambda t: t.clamp(a, b), "leaky_relu": lambda t: F.leaky_relu(t, a), "hardswish": F.hardswish,
             "hardsigmoid": F.hardsigmoid, "exp2": torch.exp2, "log2": torch.log2, "log1p": torch.log1p, "expm1": torch.expm1, "copy": lambda t: t.clone(),
             "fatrelu": lambda t: torch.where(t > a, t, torch.zeros_like(t))}
    return table[op](x)


def unary_backward(op: str, grad: torch.Tensor, saved: torch.Tensor, a: float = 0.0, b: float = 0.0) -> torch.Tensor:
    """``grad_in = grad * f'``; ``saved`` is the forward input, or the forward output for the ``*_y`` codes."""
    if op not in UNARY_BWD:
        raise InvalidArgument(f"unknown unary backward op {op}")
    if grad.shape != saved.shape or grad.dtype != saved.dtype:
        raise InvalidArgument("grad and saved tensor must match in shape and dtype")
    if not _native(grad, saved):
        raise InvalidArgument("unary_backward runs on CUDA float tensors")
    g, s = grad.contiguous(), saved.contiguous()
    out = torch.empty_like(g)
    _lib.call("ft_ew_unary_bwd", _DT[g.dtype], UNARY_BWD[op], g, s, out, g.numel(), float(a), float(b), _lib.S())
    return out


def binary(op: str, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """Broadcasting binary op; comparisons return 0/1 in the operand dtype."""
    if op not in BINARY:
        raise InvalidArgument(f"unknown binary op {op}")
    if not _native(x, y) or x.dtype != y.dtype:
        return getattr(torch, op)(x, y)
    shape = torch.broadcast_shapes(x.shape, y.shape)
    out = torch.empty(shape, device=x.device, dtype=x.dtype)
    if tuple(x.shape) == tuple(shape) == tuple(y.shape) and x.is_contiguous() and y.is_contiguous():
        _lib.call("ft_ew_binary", _DT[x.dtype], BINARY[op], x, y, out, out.numel(), _lib.S())
        return out
    if len(shape) > 6:
        return binary(op, x.expand(shape).contiguous(), y.expand(shape).contiguous())
    shp = list(shape) or [1]
    xe, ye = x.expand(shape), y.expand(shape)
    _lib.call("ft_ew_binary_strided", _DT[x.dtype], BINARY[op], xe, ye, out, len(shp), _i64(shp), _i64(list(xe.stride()) or [0]), _i64(list(ye.stride()) or [0]), _lib.S())
    return out


def where(cond: torch.Tensor, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    if not _native(x, y) or x.dtype != y.dtype or not cond.is_cuda:
        return torch.where(cond, x, y)
    shape = torch.broadcast_shapes(cond.shape, x.shape, y.shape)
    if len(shape) > 6:
        return torch.where(cond, x, y)
    c = cond.to(torch.uint8) if cond.dtype != torch.uint8 else cond
    ce, xe, ye = c.expand(shape), x.expand(shape), y.expand(shape)
    out = torch.empty(shape, device=x.device, dtype=x.dtype)
    shp = list(shape) or [1]
    _lib.call("ft_ew_where", _DT[x.dtype], ce, xe, ye, out, len(shp), _i64(shp), _i64(list(ce.stride()) or [0]), _i64(list(xe.stride()) or [0]),
              _i64(list(ye.stride()) or [0]), _lib.S())
    return out


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if x.dtype == dtype:
        return x
    if not (_native(x) and dtype in _DT) or {x.dtype, dtype} == {torch.float64, torch.bfloat16} or {x.dtype, dtype} == {torch.float64, torch.float16}:
        return x.to(dtype)
    xc = x.contiguous()
    out = torch.empty(x.shape, device=x.device, dtype=dtype)
    _lib.call("ft_ew_cast", _DT[x.dtype], _DT[dtype], xc, out, xc.numel(), _lib.S())
    return out


def fill_(x: torch.Tensor, value: float) -> torch.Tensor:
    if not _native(x) or not x.is_contiguous():
        return x.fill_(value)
    _lib.call("ft_ew_fill", _DT[x.dtype], x, x.numel(), float(value), _lib.S())
    return x


def masked_fill_(x: torch.Tensor, mask: torch.Tensor, value: float) -> torch.Tensor:
    if not _native(x) or not x.is_contiguous() or mask.shape != x.shape:
        return x.masked_fill_(mask, value)
    m = mask.to(torch.uint8).contiguous()
    _lib.call("ft_ew_masked_fill", _DT[x.dtype], x, m, x.numel(), float(value), _lib.S())
    return x


def contiguous(x: torch.Tensor) -> torch.Tensor:
    """Materialises any strided view (transpose, permute, expand, slice) with the strided-gather kernel."""
    if x.is_contiguous():
        return x
    return unary("copy", x)


def slice_write_(dst_view: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """Writes dense ``src`` into the strided view ``dst_view`` (slice assignment / concatenation building block)."""
    if not (dst_view.is_cuda and src.is_cuda) or dst_view.shape != src.shape or dst_view.dtype != src.dtype or dst_view.dim() > 6:
        dst_view.copy_(src)
        return dst_view
    s = src.contiguous()
    shp = list(s.shape) or [1]
    _lib.call("ft_ew_scatter_copy", s.element_size(), s, dst_view, len(shp), _i64(shp), _i64(list(dst_view.stride()) or [1]), _lib.S())
    return dst_view


def cat(tensors: Sequence[torch.Tensor], dim: int = 0) -> torch.Tensor:
    t0 = tensors[0]
    dim %= t0.dim()
    shape = list(t0.shape)
    shape[dim] = sum(t.shape[dim] for t in tensors)
    out = torch.empty(shape, device=t0.device, dtype=t0.dtype)
    pos = 0
    for t in tensors:
        slice_write_(out.narrow(dim, pos, t.shape[dim]), t)
        pos += t.shape[dim]
    return out


# ----------------------------------------------------------------------------------------------------------------------
_scratch = {}


def _split3(shape: Sequence[int], dim: int) -> Tuple[int, int, int]:
    outer = 1
    for s in shape[:dim]:
        outer *= s
    inner = 1
    for s in shape[dim + 1:]:
        inner *= s
    return outer, shape[dim], inner


def reduce(op: str, x: torch.Tensor, dim: Optional[int] = None, keepdim: bool = False) -> torch.Tensor:
    """sum / prod / min / max / mean / sumsq / absmax / logsumexp along one dim, or over everything when ``dim`` is None."""
    if op not in REDUCE:
        raise InvalidArgument(f"unknown reduction {op}")
    if not _native(x) or x.numel() == 0:
        return _reduce_torch(op, x, dim, keepdim)
    xc = x.contiguous()
    if dim is None:
        outer, ln, inner = 1, xc.numel(), 1
        oshape = [1] * x.dim() if keepdim else []
    else:
        dim %= x.dim()
        outer, ln, inner = _split3(xc.shape, dim)
        oshape = list(xc.shape)
        if keepdim:
            oshape[dim] = 1
        else:
            del oshape[dim]
    if inner > 1 and outer > 65535:
        return _reduce_torch(op, x, dim, keepdim)
    out = torch.empty(oshape, device=x.device, dtype=x.dtype)
    sc = _scratch.get(x.device)
    if sc is None:
        sc = _scratch[x.device] = torch.empty(148 * 4 * 8, device=x.device, dtype=torch.uint8)
    _lib.call("ft_reduce", _DT[x.dtype], REDUCE[op], xc, out, outer, ln, inner, sc, sc.numel(), _lib.S())
    return out


def _reduce_torch(op, x, dim, keepdim):
    if op == "sumsq":
        return (x * x).sum() if dim is None else (x * x).sum(dim, keepdim)
    if op == "absmax":
        return x.abs().amax() if dim is None else x.abs().amax(dim, keepdim)
    name = {"min": "amin", "max": "amax"}.get(op, op)
    if dim is None:
        return getattr(torch, name)(x, tuple(range(x.dim()))) if op == "logsumexp" else getattr(x, name)()
    return getattr(torch, name)(x, dim, keepdim)


def scan(op: str, x: torch.Tensor, dim: int, reverse: bool = False) -> torch.Tensor:
    if op not in SCAN:
        raise InvalidArgument(f"unknown scan {op}")
    dim %= x.dim()
    if not _native(x):
        f = {"cumsum": torch.cumsum, "cumprod": torch.cumprod, "cummax": lambda t, d: torch.cummax(t, d).values, "cummin": lambda t, d: torch.cummin(t, d).values,
             "logcumsumexp": torch.logcumsumexp}[op]
        return f(x.flip(dim), dim).flip(dim) if reverse else f(x, dim)
    xc = x.contiguous()
    outer, ln, inner = _split3(xc.shape, dim)
    out = torch.empty_like(xc)
    _lib.call("ft_scan", _DT[x.dtype], SCAN[op], xc, out, outer, ln, inner, int(reverse), _lib.S())
    return out


def index_select(x: torch.Tensor, dim: int, index: torch.Tensor) -> torch.Tensor:
    dim %= x.dim()
    if not x.is_cuda or x.element_size() not in (2, 4, 8):
        return x.index_select(dim, index)
    xc, idx = x.contiguous(), index.to(torch.int64).contiguous()
    outer, ln, inner = _split3(xc.shape, dim)
    shape = list(xc.shape)
    shape[dim] = idx.numel()
    out = torch.empty(shape, device=x.device, dtype=x.dtype)
    _lib.call("ft_index_select", x.element_size(), xc, idx, out, outer, ln, idx.numel(), inner, _lib.S())
    return out


def index_add_(dst: torch.Tensor, dim: int, index: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    dim %= dst.dim()
    if not (dst.is_cuda and dst.dtype == torch.float32 and dst.is_contiguous() and src.dtype == torch.float32):
        return dst.index_add_(dim, index, src)
    outer, ln, inner = _split3(dst.shape, dim)
    _lib.call("ft_index_add_f32", dst, index.to(torch.int64).contiguous(), src.contiguous(), outer, ln, index.numel(), inner, _lib.S())
    return dst


def gather(x: torch.Tensor, dim: int, index: torch.Tensor) -> torch.Tensor:
    dim %= x.dim()
    same = all(index.shape[d] == x.shape[d] for d in range(x.dim()) if d != dim)
    if not x.is_cuda or x.element_size() not in (2, 4, 8) or not same:
        return x.gather(dim, index)
    xc, idx = x.contiguous(), index.to(torch.int64).contiguous()
    outer, ln, inner = _split3(xc.shape, dim)
    out = torch.empty(idx.shape, device=x.device, dtype=x.dtype)
    _lib.call("ft_gather", x.element_size(), xc, idx, out, outer, ln, idx.shape[dim], inner, _lib.S())
    return out


def scatter_add_(dst: torch.Tensor, dim: int, index: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    dim %= dst.dim()
    same = all(index.shape[d] == dst.shape[d] for d in range(dst.dim()) if d != dim) and index.shape == src.shape
    if not (dst.is_cuda and dst.dtype == torch.float32 and dst.is_contiguous() and src.dtype == torch.float32 and same):
        return dst.scatter_add_(dim, index, src)
    outer, ln, inner = _split3(dst.shape, dim)
    _lib.call("ft_scatter_add_f32", dst, index.to(torch.int64).contiguous(), src.contiguous(), outer, ln, index.shape[dim], inner, _lib.S())
    return dst


# ----------------------------------------------------------------------------------------------------------------------
class PhiloxGenerator:
    """Counter-based generator: (seed, offset) fully determine every draw, so restoring the two integers from a checkpoint replays the stream.
    Reference: ferrotorch-gpu/src/rng.rs (Philox4x32-10, ``PhiloxState``)."""

    def __init__(self, seed: int = 0, offset: int = 0):
        self.seed, self.offset = int(seed), int(offset)

    def state(self) -> Tuple[int, int]:
        return self.seed, self.offset

    def set_state(self, st: Tuple[int, int]) -> None:
        self.seed, self.offset = int(st[0]), int(st[1])

    def _advance(self, n: int) -> int:
        o = self.offset
        self.offset += (n + 3) // 4
        return o

    def uniform_(self, x: torch.Tensor, lo: float = 0.0, hi: float = 1.0) -> torch.Tensor:
        _check_rng(x)
        _lib.call("ft_philox_fill", _DT[x.dtype], 0, x, x.numel(), self.seed, self._advance(x.numel()), float(lo), float(hi), _lib.S())
        return x

    def normal_(self, x: torch.Tensor, mean: float = 0.0, std: float = 1.0) -> torch.Tensor:
        _check_rng(x)
        _lib.call("ft_philox_fill", _DT[x.dtype], 1, x, x.numel(), self.seed, self._advance(x.numel()), float(mean), float(std), _lib.S())
        return x

    def dropout(self, x: torch.Tensor, p: float, return_mask: bool = False):
        _check_rng(x)
        xc = x.contiguous()
        out = torch.empty_like(xc)
        mask = torch.empty(xc.shape, device=x.device, dtype=torch.uint8) if return_mask else None
        _lib.call("ft_philox_dropout", _DT[x.dtype], xc, out, mask, xc.numel(), float(p), self.seed, self._advance(xc.numel()), _lib.S())
        return (out, mask) if return_mask else out


def _check_rng(x):
    if not (x.is_cuda and x.dtype in (torch.float32, torch.bfloat16, torch.float16) and x.is_contiguous()):
        raise InvalidArgument("Philox kernels take contiguous CUDA f32/bf16/f16 tensors")


def philox_reference(seed: int, offset: int, n: int) -> torch.Tensor:
    """Host restatement of the uniform stream (for tests): returns ``n`` floats in (0, 1)."""
    import numpy as np
    groups = (n + 3) // 4
    ctr = np.arange(offset, offset + groups, dtype=np.uint64)
    c = [(ctr & 0xFFFFFFFF).astype(np.uint64), (ctr >> np.uint64(32)).astype(np.uint64), np.zeros(groups, np.uint64), np.zeros(groups, np.uint64)]
    k0, k1 = np.uint64(seed & 0xFFFFFFFF), np.uint64((seed >> 32) & 0xFFFFFFFF)
    M0, M1, mask = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57), np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        h0, l0, h1, l1 = p0 >> np.uint64(32), p0 & mask, p1 >> np.uint64(32), p1 & mask
        c = [h1 ^ c[1] ^ k0, l1, h0 ^ c[3] ^ k1, l0]
        k0, k1 = (k0 + np.uint64(0x9E3779B9)) & mask, (k1 + np.uint64(0xBB67AE85)) & mask
    r = np.stack(c, 1).reshape(-1)[:n]
    return torch.from_numpy((((r >> np.uint64(8)).astype(np.float32) + 0.5) * np.float32(1.0 / 16777216.0)))


def multi_unscale_(grads: Sequence[torch.Tensor], inv_scale: float, found_inf: torch.Tensor, sqnorm: Optional[torch.Tensor] = None) -> None:
    """One launch per 96 tensors: every f32 gradient is multiplied by ``inv_scale`` in place; ``found_inf`` (f32 scalar on the device) is set
    to 1 if any value is non-finite; ``sqnorm`` accumulates the squared L2 norm. No host synchronisation."""
    gs = [g for g in grads if g is not None]
    for i in range(0, len(gs), 96):
        chunk = gs[i: i + 96]
        for g in chunk:
            if not (g.is_cuda and g.dtype == torch.float32 and g.is_contiguous()):
                raise InvalidArgument("multi_unscale_ takes contiguous CUDA f32 tensors")
        ptrs = (ctypes.c_void_p * len(chunk))(*[g.data_ptr() for g in chunk])
        _lib.call("ft_multi_unscale", ptrs, _i64([g.numel() for g in chunk]), len(chunk), float(inv_scale), found_inf, sqnorm, _lib.S())


def gguf_dequantize(blocks: torch.Tensor, qtype: str, numel: int) -> torch.Tensor:
    """uint8 tensor of packed blocks -> f32 weights (q4_0, q4_1, q5_0, q5_1, q8_0, q8_1; 32 weights per block)."""
    if qtype not in GGUF_TYPES or numel % 32:
        raise InvalidArgument(f"unsupported GGUF type {qtype} or numel {numel} not a multiple of 32")
    nb = numel // 32
    if blocks.numel() != nb * GGUF_BLOCK_BYTES[qtype]:
        raise InvalidArgument("block buffer size does not match numel")
    if not blocks.is_cuda:
        from ..serialize import formats
        return formats.dequantize_gguf_blocks(blocks, qtype, numel) if hasattr(formats, "dequantize_gguf_blocks") else _gguf_host(blocks, qtype, numel)
    out = torch.empty(numel, device=blocks.device, dtype=torch.float32)
    _lib.call("ft_gguf_dequant", GGUF_TYPES[qtype], blocks.contiguous(), out, nb, _lib.S())
    return out


def _gguf_host(blocks: torch.Tensor, qtype: str, numel: int) -> torch.Tensor:
    import numpy as np
    b = blocks.cpu().numpy().reshape(numel // 32, GGUF_BLOCK_BYTES[qtype])
    d = b[:, :2].copy().view(np.float16).astype(np.float32)
    if qtype == "q8_0":
        return torch.from_numpy((b[:, 2:].view(np.int8).astype(np.float32) * d).reshape(-1))
    if qtype == "q8_1":
        return torch.from_numpy((b[:, 4:].view(np.int8).astype(np.float32) * d).reshape(-1))
    if qtype in ("q4_0", "q4_1"):
        off = 2 if qtype == "q4_0" else 4
        q = b[:, off:]
        lo, hi = (q & 0xF).astype(np.float32), (q >> 4).astype(np.float32)
        v = np.concatenate([lo, hi], 1)
        if qtype == "q4_0":
            return torch.from_numpy(((v - 8) * d).reshape(-1))
        m = b[:, 2:4].copy().view(np.float16).astype(np.float32)
        return torch.from_numpy((v * d + m).reshape(-1))
    off = 2 if qtype == "q5_0" else 4
    qh = b[:, off: off + 4].copy().view(np.uint32)
    q = b[:, off + 4:]
    j = np.arange(16, dtype=np.uint32)
    lo = (q & 0xF) | (((qh >> j) & 1) << 4).astype(np.uint8)
    hi = (q >> 4) | (((qh >> (j + 16)) & 1) << 4).astype(np.uint8)
    v = np.concatenate([lo, hi], 1).astype(np.float32)
    if qtype == "q5_0":
        return torch.from_numpy(((v - 16) * d).reshape(-1))
    m = b[:, 2:4].copy().view(np.float16).astype(np.float32)
    return torch.from_numpy((v * d + m).reshape(-1))


def token_mask_(logits: torch.Tensor, allow_words: torch.Tensor) -> torch.Tensor:
    """Sets ``logits[r, v] = -inf`` wherever bit ``v`` of the allow mask is clear. ``allow_words``: int32 ``[ceil(V/32)]`` (shared) or ``[rows, ceil(V/32)]``."""
    V = logits.shape[-1]
    rows = logits.numel() // V
    words = (V + 31) // 32
    mrows = 1 if allow_words.dim() == 1 else allow_words.shape[0]
    if allow_words.shape[-1] != words or mrows not in (1, rows):
        raise InvalidArgument("allow mask has the wrong shape")
    if not (_native(logits) and logits.dtype != torch.float64 and logits.is_contiguous() and allow_words.is_cuda):
        bits = (allow_words.to(torch.int64).reshape(mrows, words, 1) >> torch.arange(32, device=allow_words.device)) & 1
        allow = bits.reshape(mrows, words * 32)[:, :V].bool()
        return logits.masked_fill_(~allow.expand(rows, V).reshape(logits.shape), float("-inf"))
    _lib.call("ft_token_mask", _DT[logits.dtype], logits, allow_words.contiguous(), rows, V, mrows, _lib.S())
    return logits
