"""bf16 GEMM on the tcgen05 kernel, and the differentiable ``linear`` built on it.

``gemm(a, b, a_mn=, b_mn=)`` computes ``D[M,N] = A (x) B`` where the flags say
which dimension of each operand is contiguous in memory:

* ``a_mn=False``: ``a`` is ``[M,K]``;  ``a_mn=True``: ``a`` is ``[K,M]`` (used transposed)
* ``b_mn=False``: ``b`` is ``[N,K]``;  ``b_mn=True``: ``b`` is ``[K,N]``

so ``(False, False)`` is ``x @ w.T`` (Linear forward), ``(False, True)`` is
``dy @ w`` (dgrad) and ``(True, True)`` is ``dy.T @ x`` (wgrad). No operand is
ever transposed in memory: the layout goes into the TMA/UMMA descriptors.

On CPU tensors the same function evaluates the product with ``torch.matmul``
in f32 (the oracle the GPU tests compare against).

Reference parity: cuBLAS wrappers ferrotorch-gpu/src/blas.rs:1964-2922 and
``linear_fused`` ferrotorch-core/src/grad_fns/linalg.rs:1214-1262.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import _lib
from ..errors import InvalidArgument

_FORCE_LIBRARY = os.environ.get("FT_GEMM_BACKEND", "") == "cublas"  # A/B switch for the library baseline


def _as_2d_rowmajor(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        raise InvalidArgument(f"gemm operands must be 2-D, got {tuple(t.shape)}")
    if t.stride(1) != 1 or (t.stride(0) % 8) or (t.data_ptr() % 16):
        t = t.contiguous()
    return t


_ACT = {None: 0, "none": 0, "relu": 1, "gelu": 2, "gelu_tanh": 3, "silu": 4}


def _act_torch(r: torch.Tensor, act) -> torch.Tensor:
    F = torch.nn.functional
    return {0: lambda t: t, 1: F.relu, 2: F.gelu, 3: lambda t: F.gelu(t, approximate="tanh"), 4: F.silu}[_ACT[act]](r)


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, bias: torch.Tensor | None = None,
         out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None, act: str | None = None,
         residual: torch.Tensor | None = None, gate=None) -> torch.Tensor:
    """``D = act(A (x) B + bias) + residual``. Operands bf16 or fp16 (both the same); output in the operand dtype or f32. The epilogue order is
    bias, activation (``relu`` / ``gelu`` / ``gelu_tanh`` / ``silu``), residual add (``residual`` is ``[M, N]`` in the output dtype).

    ``gate`` (a :class:`ferrotorch_b200.parallel.gather.GatherGate`): ``b`` is a weight inside a gather slot that peers may still be filling;
    the kernel waits for the pieces under each tile of ``b`` inside its TMA producer (or, for forms the gated kernel does not cover, a gate
    kernel waits for all of ``b`` first)."""
    if act not in _ACT:
        raise InvalidArgument(f"unknown epilogue activation {act!r}")
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else (a.dtype if a.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16)
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise InvalidArgument(f"gemm inner dimensions differ: {K} vs {Kb}")
    if not a.is_cuda or _FORCE_LIBRARY:
        A = a.t() if a_mn else a
        B = b if b_mn else b.t()
        r = torch.matmul(A, B).float() if a.is_cuda else torch.matmul(A.float(), B.float())
        if bias is not None:
            r = r + bias.float()
        r = _act_torch(r, act)
        if residual is not None:
            r = r + residual.float()
        r = r.to(out_dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    if a.dtype not in (torch.bfloat16, torch.float16) or b.dtype != a.dtype:
        raise InvalidArgument("gemm expects bf16 or fp16 operands of one dtype on CUDA")
    in_f16 = a.dtype == torch.float16
    a = _as_2d_rowmajor(a)
    b = _as_2d_rowmajor(b)
    if out is None:
        ldd_align = 4 if out_dtype == torch.float32 else 8
        if N % ldd_align == 0:
            out = torch.empty((M, N), device=a.device, dtype=out_dtype)
        else:  # pad the leading dimension so each output row starts on a 16-byte boundary
            Np = (N + ldd_align - 1) // ldd_align * ldd_align
            out = torch.empty((M, Np), device=a.device, dtype=out_dtype)[:, :N]
    else:
        out_dtype = out.dtype
        if out.stride(1) != 1:
            raise InvalidArgument("gemm out must be row-major")
    if out_dtype not in (a.dtype, torch.float32):
        raise InvalidArgument("gemm output must have the operand dtype or be f32")
    if bias is not None:
        bias = bias.to(a.dtype).contiguous()
    if residual is not None:
        if residual.shape != (M, N) or residual.dtype != out_dtype or residual.stride(1) != 1:
            raise InvalidArgument("residual must be a row-major [M, N] tensor in the output dtype")
    gated = False
    if gate is not None and not gate.covered(b):
        gated = not in_f16 and bias is None and not (act is not None and _ACT[act]) and residual is None and _auto_splits(M, N, K) == 1
        if not gated:
            gate.wait(b)
    if gated:
        with torch.cuda.device(a.device):
            _lib.call("ft_gemm_gated", _lib.P(a), _lib.P(b), _lib.P(out), M, N, K, ctypes.c_int64(a.stride(0)), ctypes.c_int64(b.stride(0)),
                      ctypes.c_int64(out.stride(0)), int(a_mn), int(b_mn), int(out_dtype == torch.float32), ctypes.c_void_p(gate.counters_ptr),
                      gate.expected, ctypes.c_void_p(gate.slot_ptr), ctypes.c_int64(gate.piece_bytes), _lib.S())
        gate.mark(b)
        return out
    if in_f16 or act is not None and _ACT[act] or residual is not None:
        with torch.cuda.device(a.device):
            _lib.call("ft_gemm_ex", _lib.P(a), _lib.P(b), _lib.P(out), _lib.P(bias), _lib.P(residual), M, N, K, ctypes.c_int64(a.stride(0)), ctypes.c_int64(b.stride(0)),
                      ctypes.c_int64(out.stride(0)), ctypes.c_int64(residual.stride(0) if residual is not None else 0), int(a_mn), int(b_mn),
                      int(out_dtype == torch.float32), int(in_f16), _ACT[act], _lib.S())
        return out
    splits = _auto_splits(M, N, K)
    if splits > 1:
        # few output tiles and a long K (weight gradients of 1x1 convolutions, decode): spread K over the SMs as f32 planes, then sum
        planes = _plane_cache(a.device, splits * M * N)[: splits * M * N].view(splits, M, N)
        with torch.cuda.device(a.device):
            _lib.call("ft_gemm_bf16_splitk", _lib.P(a), _lib.P(b), _lib.P(planes), M, N, K, ctypes.c_int64(a.stride(0)), ctypes.c_int64(b.stride(0)),
                      ctypes.c_int64(N), int(a_mn), int(b_mn), splits, _lib.S())
            _lib.call("ft_splitk_reduce", _lib.P(planes), splits, M, N, ctypes.c_int64(N), ctypes.c_int64(M * N), _lib.P(bias), _lib.P(out),
                      ctypes.c_int64(out.stride(0)), int(out_dtype == torch.float32), _lib.S())
        return out
    with torch.cuda.device(a.device):
        _lib.call("ft_gemm_bf16", _lib.P(a), _lib.P(b), _lib.P(out), _lib.P(bias), M, N, K, ctypes.c_int64(a.stride(0)),
                  ctypes.c_int64(b.stride(0)), ctypes.c_int64(out.stride(0)), int(a_mn), int(b_mn),
                  int(out_dtype == torch.float32), _lib.S())
    return out


_planes: dict = {}


def _plane_cache(device: torch.device, numel: int) -> torch.Tensor:
    buf = _planes.get(device)
    if buf is None or buf.numel() < numel:
        buf = _planes[device] = torch.empty(max(numel, 1 << 22), device=device, dtype=torch.float32)
    return buf


def _auto_splits(M: int, N: int, K: int) -> int:
    """Number of K slices: 1 unless the 128x256 output tiles cover less than half of the 148 SMs and K is long enough that every
    slice still runs at least eight 64-wide K steps. N must be a multiple of 4 (f32 plane rows start on 16-byte boundaries)."""
    tiles = -(-M // 128) * -(-N // 256)
    if tiles * 2 > 148 or N % 4 or K < 2048:
        return 1
    splits = min(148 // tiles, K // 512)
    num_kb = -(-K // 64)
    while splits > 1 and -(-num_kb // splits) * (splits - 1) >= num_kb:               # no empty trailing slice
        splits -= 1
    return max(splits, 1)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        y = gemm(x2, w, bias=bias)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.shp = shp
        return y.reshape(*shp[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).reshape(ctx.shp)
        if ctx.needs_input_grad[1]:
            dw = gemm(dy2, x2, a_mn=True, b_mn=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy2.dtype)
        return dx, dw, db


class _MasterLinearFn(torch.autograd.Function):
    """``x @ w_compute.T`` where ``w_compute`` is the low-precision copy of the f32 master ``w_master``: the master receives its gradient in
    f32 straight from the weight-gradient GEMM (no bf16 round trip, no cast launches)."""

    @staticmethod
    def forward(ctx, x, w_master, w_compute, bias):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        w2 = w_compute.reshape(w_compute.shape[0], -1)
        y = gemm(x2, w2, bias=bias)
        ctx.save_for_backward(x2, w2)
        ctx.has_bias = bias is not None
        ctx.shp, ctx.wshape = shp, w_master.shape
        return y.reshape(*shp[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w2 = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w2, b_mn=True).reshape(ctx.shp)
        if ctx.needs_input_grad[1]:
            dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32).reshape(ctx.wshape)
        if ctx.has_bias and ctx.needs_input_grad[3]:
            db = dy2.float().sum(0)
        return dx, dw, None, db


def linear_master(x: torch.Tensor, w_master: torch.Tensor, w_compute: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ w.T + bias`` computed with ``w_compute`` (the bf16 copy of the f32 ``w_master``, same shape); gradients flow to ``w_master``
    (f32) and to ``bias`` (f32 sum, cast by autograd to the bias dtype if needed). ``x`` must have ``w_compute``'s dtype."""
    if x.dtype != w_compute.dtype or w_master.shape != w_compute.shape:
        raise InvalidArgument("linear_master: x and the compute copy must share a dtype, master and copy a shape")
    return _MasterLinearFn.apply(x, w_master, w_compute, bias)


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ w.T + bias`` for ``w`` of shape ``[out, in]`` with autograd; bf16 CUDA tensors run on the tcgen05 GEMM."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        return _LinearFn.apply(x, w, bias)
    return torch.nn.functional.linear(x, w, bias)


def matmul_exact(a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0, beta: float = 0.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """f32 / f64 matrix product without operand rounding, on the FMA pipes: ``[.., M, K] @ [.., K, N]`` with one shared batch shape (or an
    unbatched operand broadcast over the batch), either operand possibly a transposed view. ``out = alpha * a @ b + beta * out``."""
    if a.dtype != b.dtype or a.dtype not in (torch.float32, torch.float64):
        raise InvalidArgument("matmul_exact takes two f32 or two f64 tensors")
    if not a.is_cuda:
        r = torch.matmul(a, b) * alpha
        return r if out is None else out.mul_(beta).add_(r)
    if a.dim() < 2 or b.dim() < 2 or a.shape[-1] != b.shape[-2]:
        raise InvalidArgument(f"matmul_exact shapes {tuple(a.shape)} x {tuple(b.shape)}")
    batch_shape = torch.broadcast_shapes(a.shape[:-2], b.shape[:-2])
    nb = 1
    for s in batch_shape:
        nb *= s

    def prep(t):
        m = t.reshape(-1, *t.shape[-2:]) if t.dim() > 2 else t[None]
        if m.shape[0] not in (1, nb):
            m = t.expand(*batch_shape, *t.shape[-2:]).reshape(nb, *t.shape[-2:])
        trans = m.stride(-1) != 1 and m.stride(-2) == 1
        if not trans and m.stride(-1) != 1:
            m = m.contiguous()
        return m, int(trans), (m.stride(-1) if trans else m.stride(-2)), (0 if m.shape[0] == 1 else m.stride(0))
    am, ta, lda, sa = prep(a)
    bm, tb_, ldb, sb = prep(b)
    M, K, N = a.shape[-2], a.shape[-1], b.shape[-1]
    if out is None:
        out = torch.empty(*batch_shape, M, N, device=a.device, dtype=a.dtype)
        beta = 0.0
    _lib.call("ft_gemm_simt", 0 if a.dtype == torch.float32 else 3, am, bm, out, nb, M, N, K, ctypes.c_int64(max(lda, 1)), ctypes.c_int64(max(ldb, 1)),
              ctypes.c_int64(N), ctypes.c_int64(sa), ctypes.c_int64(sb), ctypes.c_int64(M * N), ta, tb_, float(alpha), float(beta), _lib.S())
    return out


def mv(a: torch.Tensor, x: torch.Tensor, trans: bool = False) -> torch.Tensor:
    """``a @ x`` (or ``a.T @ x`` with ``trans``) for a row-major f32 / f64 matrix."""
    if not a.is_cuda or a.dtype not in (torch.float32, torch.float64):
        return (a.t() if trans else a) @ x
    a = a if a.stride(1) == 1 else a.contiguous()
    y = torch.empty(a.shape[1] if trans else a.shape[0], device=a.device, dtype=a.dtype)
    _lib.call("ft_gemv", 0 if a.dtype == torch.float32 else 3, a, x.contiguous(), y, a.shape[0], a.shape[1], ctypes.c_int64(a.stride(0)), int(trans), 1.0, 0.0, _lib.S())
    return y


def dot(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    return mv(x.reshape(1, -1), y.reshape(-1))[0] if x.is_cuda and x.dtype in (torch.float32, torch.float64) else torch.dot(x, y)


def bmm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Batched product: bf16 / fp16 batches run the tcgen05 GEMM per batch entry; f32 / f64 the exact strided-batched kernel."""
    if a.dtype in (torch.float32, torch.float64) or not a.is_cuda:
        return matmul_exact(a, b) if a.is_cuda else torch.bmm(a, b)
    out = torch.empty(a.shape[0], a.shape[1], b.shape[2], device=a.device, dtype=a.dtype)
    for i in range(a.shape[0]):
        gemm(a[i], b[i], b_mn=True, out=out[i])
    return out
