"""Run-twice bit-comparison of the hot kernels: a data race or an unordered reduction shows up as differing bits (the stand-in for a race detector on this
hardware). Atomics-based kernels (index_add, scatter_add, embedding backward) are excluded by design and listed here for that reason."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _twice(fn):
    a = fn()
    torch.cuda.synchronize()
    b = fn()
    torch.cuda.synchronize()
    a, b = (a if isinstance(a, (tuple, list)) else [a]), (b if isinstance(b, (tuple, list)) else [b])
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_gemm_attention_norm_conv_are_bit_stable():
    from ferrotorch_b200 import ops
    from ferrotorch_b200.ops import nn_ops, tensor_ops
    g = torch.Generator(device="cuda").manual_seed(0)
    a, b = torch.randn(1000, 520, device="cuda", generator=g).bfloat16(), torch.randn(776, 520, device="cuda", generator=g).bfloat16()
    _twice(lambda: ops.gemm(a, b))
    dy, x = torch.randn(50_000, 64, device="cuda", generator=g).bfloat16(), torch.randn(50_000, 128, device="cuda", generator=g).bfloat16()
    _twice(lambda: ops.gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32))          # split-K planes + fixed-order reduce
    B, S, Hq, Hkv, D = 2, 512, 8, 2, 128
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, device="cuda", generator=g).bfloat16()
    do = torch.randn(B * S, Hq * D, device="cuda", generator=g).bfloat16()

    def attn():
        out, lse = ops.flash_fwd(qkv, B, S, Hq, Hkv, D, True)
        return out, ops.flash_bwd(qkv, out, lse, do, B, S, Hq, Hkv, D, True)
    _twice(attn)
    xb = torch.randn(16, 64, 28, 28, device="cuda", generator=g).bfloat16().contiguous(memory_format=torch.channels_last)
    gam, bet = torch.ones(64, device="cuda"), torch.zeros(64, device="cuda")
    dyb = torch.randn_like(xb)

    def bn():
        xi = xb.clone().requires_grad_()
        y = nn_ops.batch_norm_nhwc(xi, gam.clone().requires_grad_(), bet.clone().requires_grad_(), torch.zeros(64, device="cuda"), torch.ones(64, device="cuda"), relu=True)
        y.backward(dyb)
        return y.detach(), xi.grad
    _twice(bn)
    w = torch.randn(128, 64, 3, 3, device="cuda", generator=g) * 0.05
    _twice(lambda: ops.conv3x3(xb, w))
    big = torch.randn(3_000_001, device="cuda", generator=g)
    _twice(lambda: tensor_ops.reduce("sum", big))
    _twice(lambda: tensor_ops.scan("cumsum", big.view(-1, 1)[:4096 * 64].view(64, 4096), 1))
    h = torch.randn(333, 4096, device="cuda", generator=g).bfloat16()
    wn = torch.ones(4096, device="cuda").bfloat16()
    _twice(lambda: ops.rms_norm(h, wn, 1e-5))
    logits = torch.randn(512, 32003, device="cuda", generator=g).bfloat16()
    tgt = torch.randint(0, 32003, (512,), device="cuda", generator=g)
    _twice(lambda: ops.cross_entropy_fwd_bwd(logits.clone(), tgt))
