"""Run-twice bit-comparison of the hot kernels: a data race or an unordered reduction shows up as differing bits (the stand-in for a race detector on this
hardware). Atomics-based kernels (index_add, scatter_add, the atomic form of the embedding backward) are excluded by design and listed here for that
reason; the default embedding backward sorts by id and sums in token order, and is checked."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _twice(fn, what):
    a = fn()
    torch.cuda.synchronize()
    b = fn()
    torch.cuda.synchronize()
    a, b = (a if isinstance(a, (tuple, list)) else [a]), (b if isinstance(b, (tuple, list)) else [b])
    for i, (x, y) in enumerate(zip(a, b)):
        if isinstance(x, torch.Tensor):
            assert torch.equal(x, y), f"{what}: output {i} differs between two runs (max abs diff {float((x.float() - y.float()).abs().max())})"


def test_gemm_attention_norm_conv_are_bit_stable():
    from ferrotorch_b200 import ops
    from ferrotorch_b200.ops import nn_ops, tensor_ops
    g = torch.Generator(device="cuda").manual_seed(0)
    a, b = torch.randn(1000, 520, device="cuda", generator=g).bfloat16(), torch.randn(776, 520, device="cuda", generator=g).bfloat16()
    _twice(lambda: ops.gemm(a, b), "gemm")
    dy, x = torch.randn(50_000, 64, device="cuda", generator=g).bfloat16(), torch.randn(50_000, 128, device="cuda", generator=g).bfloat16()
    _twice(lambda: ops.gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32), "split-K gemm")          # split-K planes + fixed-order reduce
    B, S, Hq, Hkv, D = 2, 512, 8, 2, 128
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, device="cuda", generator=g).bfloat16()
    do = torch.randn(B * S, Hq * D, device="cuda", generator=g).bfloat16()

    def attn():
        out, lse = ops.flash_fwd(qkv, B, S, Hq, Hkv, D, True)
        return out, ops.flash_bwd(qkv, out, lse, do, B, S, Hq, Hkv, D, True)
    _twice(attn, "attention fwd+bwd")
    xb = torch.randn(16, 64, 28, 28, device="cuda", generator=g).bfloat16().contiguous(memory_format=torch.channels_last)
    gam, bet = torch.ones(64, device="cuda"), torch.zeros(64, device="cuda")
    dyb = torch.randn_like(xb)

    def bn():
        xi = xb.clone().requires_grad_()
        y = nn_ops.batch_norm_nhwc(xi, gam.clone().requires_grad_(), bet.clone().requires_grad_(), torch.zeros(64, device="cuda"), torch.ones(64, device="cuda"), relu=True)
        y.backward(dyb)
        return y.detach(), xi.grad
    _twice(bn, "batch norm fwd+bwd")
    w = torch.randn(128, 64, 3, 3, device="cuda", generator=g) * 0.05
    _twice(lambda: ops.conv3x3(xb, w), "conv3x3")
    big = torch.randn(3_000_001, device="cuda", generator=g)
    _twice(lambda: tensor_ops.reduce("sum", big), "full sum")
    _twice(lambda: tensor_ops.scan("cumsum", big.view(-1, 1)[:4096 * 64].view(64, 4096), 1), "cumsum")
    h = torch.randn(333, 4096, device="cuda", generator=g).bfloat16()
    wn = torch.ones(4096, device="cuda").bfloat16()
    _twice(lambda: ops.rms_norm(h, wn, 1e-5), "rms norm")
    logits = torch.randn(512, 32000, device="cuda", generator=g).bfloat16()
    tgt = torch.randint(0, 32000, (512,), device="cuda", generator=g)
    _twice(lambda: ops.cross_entropy_fwd_bwd(logits.clone(), tgt), "cross entropy")
    # embedding backward with many repeated ids (every id about 60 times): bf16 accumulation in an order left to the hardware would differ run to run
    ids = torch.randint(0, 70, (4096,), device="cuda", generator=g)
    dout = torch.randn(4096, 512, device="cuda", generator=g).bfloat16()
    _twice(lambda: ops.embedding_bwd(ids, dout, torch.zeros(70, 512, device="cuda", dtype=torch.bfloat16)), "embedding backward")
