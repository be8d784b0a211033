"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory where they call a kernel (a serving loop that must not
trigger cudaMalloc's implicit synchronisation, a plug-in working inside buffers its host handed over). For them
``ft_rmsnorm_bwd_noalloc`` keeps the scratch for the weight-gradient partial sums in a fixed array inside the
library. This test checks that it computes what the ordinary launcher (caller-provided scratch) computes, on two
calls in a row with different data - the second call sees the first call's leftovers in the shared scratch -
and that a hidden size beyond the built-in maximum is refused.
"""
import ctypes

import pytest
import torch

from ferrotorch_b200 import _lib, ops

pytestmark = pytest.mark.gpu


def _sym():
    lib = _lib.kernels()
    fn = lib.ft_rmsnorm_bwd_noalloc
    vp, ci = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, vp]
    fn.restype = ci
    return fn


def _case(rows, d, seed, with_res):
    torch.manual_seed(seed)
    x = torch.randn(rows, d, device="cuda").to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16)
    dy = torch.randn(rows, d, device="cuda").to(torch.bfloat16)
    dres = torch.randn(rows, d, device="cuda").to(torch.bfloat16) if with_res else None
    _, rstd, _ = ops.rmsnorm_fwd(x, w, 1e-5)
    return x, w, dy, rstd, dres


def test_noalloc_matches_regular_entry_point_twice():
    fn = _sym()
    for rows, d, seed, with_res in ((515, 4096, 11, True), (97, 8192, 12, False)):
        x, w, dy, rstd, dres = _case(rows, d, seed, with_res)
        ref_dx, ref_dw = ops.rmsnorm_bwd(x, w, dy, rstd, dres=dres)
        dx = torch.empty_like(x)
        dw = torch.empty(d, device="cuda", dtype=torch.bfloat16)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = fn(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), dres.data_ptr() if dres is not None else None,
                dx.data_ptr(), dw.data_ptr(), None, 0, rows, d, torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before          # nothing was taken from torch's allocator either
        assert torch.allclose(dx.float(), ref_dx.float(), rtol=2e-2, atol=2e-2)
        rel = (dw.float() - ref_dw.float()).norm() / ref_dw.float().norm()
        assert rel.item() < 2e-2, rel.item()


def test_noalloc_accumulates_into_f32_and_bf16_outputs():
    """``accumulate = 1`` adds the weight gradient to what the two optional outputs already hold (the f32 one exactly, the bf16 one rounded)."""
    fn = _sym()
    rows, d = 300, 2048
    x, w, dy, rstd, _ = _case(rows, d, 21, False)
    _, ref_dw = ops.rmsnorm_bwd(x, w, dy, rstd)
    dx = torch.empty_like(x)
    base32 = torch.randn(d, device="cuda")
    base16 = torch.randn(d, device="cuda").to(torch.bfloat16)
    dw32, dw16 = base32.clone(), base16.clone()
    st = torch.cuda.current_stream().cuda_stream
    assert fn(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), dw16.data_ptr(), dw32.data_ptr(), 1, rows, d, st) == 0
    plain32 = torch.empty(d, device="cuda")
    assert fn(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), None, plain32.data_ptr(), 0, rows, d, st) == 0
    torch.cuda.synchronize()
    assert torch.allclose(dw32, base32 + plain32, rtol=1e-5, atol=1e-4)
    assert ((plain32 - ref_dw.float()).norm() / ref_dw.float().norm()).item() < 2e-2
    assert torch.allclose(dw16.float(), base16.float() + plain32, rtol=2e-2, atol=5e-2)


def test_noalloc_rejects_oversize():
    fn = _sym()
    max_d = _lib.kernels().ft_rmsnorm_bwd_noalloc_max_d()
    d = max_d + 8
    x = torch.zeros(2, d, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(d, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(2, device="cuda")
    dw = torch.empty(d, device="cuda", dtype=torch.bfloat16)
    rc = fn(x.data_ptr(), w.data_ptr(), x.data_ptr(), rstd.data_ptr(), None, x.data_ptr(), dw.data_ptr(), None, 0, 2, d,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -4
