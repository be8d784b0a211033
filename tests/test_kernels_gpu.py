"""Bandwidth-bound kernels (norms, RoPE, SwiGLU, embedding, cross-entropy, optimizers) against f32 PyTorch references."""
import math

import pytest
import torch

from ferrotorch_b200 import ops

pytestmark = pytest.mark.gpu


def _close(got, ref, rtol=2e-2, atol=2e-2):
    assert torch.allclose(got.float(), ref.float(), rtol=rtol, atol=atol), (got.float() - ref.float()).abs().max().item()


@pytest.mark.parametrize("rows,d", [(5, 256), (300, 4096), (17, 8192), (3, 12288), (1, 4096), (4096, 4096), (5003, 1024), (2401, 8192)])
def test_rmsnorm_fwd_bwd(rows, d):
    torch.manual_seed(rows + d)
    x = torch.randn(rows, d, device="cuda").to(torch.bfloat16).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    y = ops.rms_norm(x, w, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    yr.backward(g.float())
    _close(y, yr)
    _close(x.grad, xr.grad, 3e-2, 3e-2)
    assert ((w.grad.float() - wr.grad).norm() / wr.grad.norm()).item() < 2e-2


@pytest.mark.parametrize("rows", [64, 67, 4801])
def test_rmsnorm_residual_fused(rows):
    torch.manual_seed(0)
    x = torch.randn(rows, 1024, device="cuda").to(torch.bfloat16)
    r = torch.randn(rows, 1024, device="cuda").to(torch.bfloat16)
    w = torch.ones(1024, device="cuda", dtype=torch.bfloat16)
    y, rstd, xs = ops.rmsnorm_fwd(x, w, 1e-5, residual=r)
    s = (x.float() + r.float()).to(torch.bfloat16)
    assert torch.equal(xs, s)
    sf = s.float()
    _close(y, sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + 1e-5))


@pytest.mark.parametrize("rows,d", [(9, 512), (130, 1024)])
def test_layernorm_fwd_bwd(rows, d):
    torch.manual_seed(1)
    x = torch.randn(rows, d, device="cuda").to(torch.bfloat16).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    b = (0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    y = ops.layer_norm(x, w, b, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.layer_norm(xr, (d,), wr, br, 1e-5)
    yr.backward(g.float())
    _close(y, yr)
    _close(x.grad, xr.grad, 3e-2, 3e-2)
    assert ((w.grad.float() - wr.grad).norm() / wr.grad.norm()).item() < 2e-2
    assert ((b.grad.float() - br.grad).norm() / br.grad.norm()).item() < 2e-2


def test_rope_forward_inverse():
    torch.manual_seed(2)
    B, S, H, D = 2, 48, 6, 128
    cos, sin = ops.rope_tables(64, D, 5e5, "cuda")
    x = torch.randn(B, S, H, D, device="cuda").to(torch.bfloat16)
    y = ops.apply_rope(x, cos, sin)
    xf = x.float()
    c, s = cos[:S].view(1, S, 1, D // 2), sin[:S].view(1, S, 1, D // 2)
    a, b = xf[..., : D // 2], xf[..., D // 2:]
    ref = torch.cat([a * c - b * s, b * c + a * s], -1)
    _close(y, ref)
    z = y.reshape(B * S, H * D).clone()
    ops.rope_inplace(z, cos, sin, S, 0, H, D, inverse=True)
    _close(z.reshape(B, S, H, D), x, 3e-2, 3e-2)


def test_swiglu_fwd_bwd():
    torch.manual_seed(3)
    gu = torch.randn(37, 2 * 264, device="cuda").to(torch.bfloat16).requires_grad_(True)
    y = ops.swiglu(gu)
    g = torch.randn_like(y)
    y.backward(g)
    r = gu.detach().float().requires_grad_(True)
    yr = torch.nn.functional.silu(r[:, :264]) * r[:, 264:]
    yr.backward(g.float())
    _close(y, yr)
    _close(gu.grad, r.grad, 3e-2, 3e-2)


def test_embedding_fwd_bwd():
    torch.manual_seed(4)
    V, d = 1000, 256
    table = torch.randn(V, d, device="cuda").to(torch.bfloat16).requires_grad_(True)
    ids = torch.randint(0, V, (4, 33), device="cuda")
    y = ops.embedding(ids, table)
    assert torch.equal(y, table.detach()[ids])
    g = torch.randn_like(y)
    y.backward(g)
    ref = torch.zeros(V, d, device="cuda")
    ref.index_add_(0, ids.reshape(-1), g.reshape(-1, d).float())
    _close(table.grad, ref, 5e-2, 5e-2)


@pytest.mark.parametrize("V", [1000, 128256, 32003])
def test_cross_entropy(V):
    torch.manual_seed(5)
    rows = 19
    logits = (torch.randn(rows, V, device="cuda") * 3).to(torch.bfloat16)
    if V % 8:
        pad = torch.zeros(rows, (V + 7) // 8 * 8, device="cuda", dtype=torch.bfloat16)
        pad[:, :V] = logits
        logits = pad[:, :V]
    t = torch.randint(0, V, (rows,), device="cuda")
    t[3] = -100
    l = logits.detach().clone().requires_grad_(True) if V % 8 == 0 else None
    loss, dl, cnt = ops.cross_entropy_fwd_bwd(logits, t, ignore_index=-100, grad_scale=1.0 / 18, inplace_grad=False)
    lr = logits.float().detach().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lr, t, ignore_index=-100)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * max(1.0, abs(ref.item()))
    assert cnt.item() == 18
    assert (dl.float() - lr.grad).abs().max().item() < 2e-3
    if l is not None:
        lo = ops.cross_entropy(l, t)
        lo.backward()
        assert (l.grad.float() - lr.grad).abs().max().item() < 2e-3


def test_cross_entropy_label_smoothing_f32():
    torch.manual_seed(6)
    logits = torch.randn(11, 516, device="cuda")
    t = torch.randint(0, 516, (11,), device="cuda")
    loss, dl, _ = ops.cross_entropy_fwd_bwd(logits, t, label_smoothing=0.1, inplace_grad=False)
    lr = logits.clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lr, t, label_smoothing=0.1)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-4
    assert (dl - lr.grad).abs().max().item() < 1e-5


@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
def test_adamw_flat_matches_torch(gdtype):
    torch.manual_seed(7)
    n = 10007
    p0 = torch.randn(n, device="cuda")
    master, m, v = p0.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ref = torch.nn.Parameter(p0.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        g = torch.randn(n, device="cuda").to(gdtype)
        ops.adamw_flat_(master, pb, m, v, g, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
        ref.grad = g.float()
        opt.step()
    assert (master - ref.detach()).abs().max().item() < 1e-5
    assert torch.equal(pb, master.to(torch.bfloat16))


def test_sgd_flat_matches_torch():
    torch.manual_seed(8)
    n = 4099
    p0 = torch.randn(n, device="cuda")
    master, buf = p0.clone(), torch.zeros(n, device="cuda")
    ref = torch.nn.Parameter(p0.clone())
    opt = torch.optim.SGD([ref], lr=0.1, momentum=0.9, weight_decay=1e-4, nesterov=True)
    for step in range(3):
        g = torch.randn(n, device="cuda")
        ops.sgd_flat_(master, None, buf, g, lr=0.1, momentum=0.9, weight_decay=1e-4, nesterov=True, first_step=(step == 0))
        ref.grad = g.clone()
        opt.step()
    assert (master - ref.detach()).abs().max().item() < 1e-5


def test_grad_norm_and_scale():
    torch.manual_seed(9)
    a = torch.randn(100003, device="cuda")
    b = torch.randn(5001, device="cuda").to(torch.bfloat16)
    nrm, coef = ops.grad_norm_([a, b], max_norm=1.0)
    ref = math.sqrt(a.pow(2).sum().item() + b.float().pow(2).sum().item())
    assert abs(nrm.item() - ref) / ref < 1e-4
    assert abs(coef.item() - 1.0 / (ref + 1e-6)) < 1e-6
    a2 = a.clone()
    ops.scale_(a2, 1.0, coef)
    assert torch.allclose(a2, a * coef, rtol=1e-6, atol=1e-7)


def test_elementwise_optimizer_kernel_matches_the_tensor_operation_forms():
    """ft_foreach_opt (one launch per parameter) against the same recurrences evaluated as tensor operations on the CPU."""
    from ferrotorch_b200 import optim as O
    from tests.test_optim_elementwise_cpu import CASES, _run
    for ours, _, kw in CASES:
        dev, _ = _run(ours, kw, steps=12, device="cuda")
        cpu, _ = _run(ours, kw, steps=12, device="cpu")
        assert (dev - cpu).abs().max().item() < 2e-5, (ours.__name__, kw, (dev - cpu).abs().max().item())
