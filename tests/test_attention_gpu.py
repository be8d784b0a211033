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
