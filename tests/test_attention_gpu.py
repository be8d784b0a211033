"""tcgen05 FlashAttention forward/backward against an f32 PyTorch evaluation of the same attention."""
import math

import pytest
import torch

from ferrotorch_b200 import ops

pytestmark = pytest.mark.gpu


def _ref(qkv, B, S, Hq, Hkv, D, causal):
    x = qkv.float()
    q = x[:, : Hq * D].reshape(B, S, Hq, D).transpose(1, 2)
    k = x[:, Hq * D: (Hq + Hkv) * D].reshape(B, S, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, 1)
    v = x[:, (Hq + Hkv) * D:].reshape(B, S, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, 1)
    s = q @ k.transpose(-1, -2) / math.sqrt(D)
    if causal:
        s = s.masked_fill(torch.ones(S, S, dtype=torch.bool, device=x.device).triu(1), float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.softmax(s, -1) @ v
    return o.transpose(1, 2).reshape(B * S, Hq * D), lse


needs_native = pytest.mark.skipif(ops.attention.backend() != "tcgen05", reason="native attention kernels not built")


@needs_native
@pytest.mark.parametrize("B,S,Hq,Hkv,causal", [(1, 128, 1, 1, True), (2, 256, 4, 2, True), (1, 200, 2, 1, True), (1, 320, 2, 2, False),
                                               (1, 1024, 8, 2, True)])
def test_flash_fwd(B, S, Hq, Hkv, causal):
    torch.manual_seed(S + Hq)
    D = 128
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
    out, lse = ops.flash_fwd(qkv, B, S, Hq, Hkv, D, causal)
    ro, rl = _ref(qkv, B, S, Hq, Hkv, D, causal)
    assert (out.float() - ro).abs().max().item() < 2e-2
    assert (lse - rl).abs().max().item() < 2e-2


@needs_native
@pytest.mark.parametrize("B,S,Hq,Hkv,causal", [(1, 128, 1, 1, True), (2, 256, 4, 2, True), (1, 200, 2, 1, True), (1, 320, 2, 2, False),
                                               (1, 1024, 8, 2, True)])
def test_flash_bwd(B, S, Hq, Hkv, causal):
    torch.manual_seed(S + Hq + 1)
    D = 128
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
    out, lse = ops.flash_fwd(qkv, B, S, Hq, Hkv, D, causal)
    do = torch.randn_like(out)
    dqkv = ops.flash_bwd(qkv, out, lse, do, B, S, Hq, Hkv, D, causal)
    leaf = qkv.float().requires_grad_(True)
    ro, _ = _ref(leaf, B, S, Hq, Hkv, D, causal)
    (ref,) = torch.autograd.grad(ro, leaf, do.float())
    for name, lo, hi in (("dq", 0, Hq * D), ("dk", Hq * D, (Hq + Hkv) * D), ("dv", (Hq + Hkv) * D, (Hq + 2 * Hkv) * D)):
        g, r = dqkv[:, lo:hi].float(), ref[:, lo:hi]
        rel = (g - r).norm() / (r.norm() + 1e-9)
        assert rel.item() < 3e-2, (name, rel.item())


def test_attention_packed_autograd_any_backend():
    torch.manual_seed(3)
    B, S, Hq, Hkv, D = 1, 256, 4, 2, 128
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16).requires_grad_(True)
    o = ops.attention_packed(qkv, B, S, Hq, Hkv, D, True)
    g = torch.randn_like(o)
    o.backward(g)
    leaf = qkv.detach().float().requires_grad_(True)
    ro, _ = _ref(leaf, B, S, Hq, Hkv, D, True)
    (ref,) = torch.autograd.grad(ro, leaf, g.float())
    assert (o.float() - ro).abs().max().item() < 2e-2
    assert ((qkv.grad.float() - ref).norm() / ref.norm()).item() < 3e-2


@pytest.mark.parametrize("D,causal,Hq,Hkv,S", [(64, False, 4, 4, 197), (64, True, 4, 2, 256), (96, False, 2, 2, 130), (32, False, 2, 1, 64)])
def test_small_head_dims_run_on_the_padded_tcgen05_route(D, causal, Hq, Hkv, S):
    """Head dimensions below 128 are zero-padded into the D = 128 kernels: values and gradients against the f32 materialised form."""
    import ferrotorch_b200.nn as nn
    torch.manual_seed(0)
    B = 2
    q = torch.randn(B, Hq, S, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, Hkv, S, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, Hkv, S, D, device="cuda", dtype=torch.bfloat16)
    assert nn.attention_backend(q, k) == "tcgen05"
    qa, ka, va = (t.clone().requires_grad_() for t in (q, k, v))
    qb, kb, vb = (t.float().clone().requires_grad_() for t in (q, k, v))
    o = nn.flash_attention(qa, ka, va, causal)
    rep = Hq // Hkv
    ref = nn.standard_attention(qb, nn.repeat_kv(kb, rep), nn.repeat_kv(vb, rep), causal)
    assert o.shape == ref.shape
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()  # noqa: E731
    assert rel(o, ref) < 2e-2
    w = torch.randn_like(ref)
    (o.float() * w).sum().backward()
    (ref * w).sum().backward()
    for a, b in ((qa, qb), (ka, kb), (va, vb)):
        assert rel(a.grad, b.grad) < 3e-2
