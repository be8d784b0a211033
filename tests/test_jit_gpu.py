"""Generated sm_100a fused kernels against eager execution."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _f(x, y, b):
    h = F.gelu(x * y + b) * torch.sigmoid(x) - 0.5
    return torch.where(h > 0, h, h * 0.1).sum(-1), torch.tanh(h)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_fused_kernel_vectorised_and_strided(dtype, tol):
    from ferrotorch_b200 import _lib, jit
    g = torch.Generator(device="cuda").manual_seed(0)
    x, y = (torch.randn(512, 1027, device="cuda", generator=g).to(dtype) for _ in range(2))
    b = torch.randn(1027, device="cuda", generator=g).to(dtype)
    cf = jit.compile(_f, backend="cuda")
    l0 = _lib.launch_calls
    out = cf(x, y, b)                                # b is broadcast -> strided kernel
    ref = _f(x, y, b)                                # eager in the same dtype: the generated code rounds through the storage type after every op, as eager does
    assert cf.stats.fused_kernels == 1 and _lib.launch_calls > l0
    rel = lambda a, r: ((a.float() - r.float()).abs() / (1 + r.float().abs())).max()   # noqa: E731
    assert rel(out[1], ref[1]) < tol
    assert rel(out[0], ref[0]) < tol * 4
    f2 = lambda p, q: torch.tanh(p) * q + F.silu(p)  # noqa: E731  all operands dense -> 16-byte vector kernel, ragged tail (512*1027 % 8 != 0 for bf16)
    c2 = jit.compile(f2, backend="cuda")
    assert rel(c2(x, y), f2(x, y)) < tol
    xs = x[:, ::2]                                   # strided view
    assert rel(c2(xs, y[:, ::2]), f2(xs, y[:, ::2])) < tol
    assert _lib.read_status() == 0


def test_compiled_mlp_block_matches_eager():
    from ferrotorch_b200 import jit
    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.GELU(), torch.nn.Linear(512, 256)).cuda()
    x = torch.randn(64, 256, device="cuda")
    f = lambda t: F.silu(m(t)) * torch.sigmoid(t) + t     # noqa: E731
    cf = jit.compile(f, backend="cuda")
    assert (cf(x) - f(x)).abs().max() < 1e-4 and cf.stats.fused_kernels >= 1


def test_fused_row_reduction_kernel():
    from ferrotorch_b200 import jit

    def f(x, b):
        e = torch.exp(x * 0.1) * b
        return e.sum(-1, keepdim=True), torch.tanh(e)
    x, b = torch.randn(300, 1027, device="cuda"), torch.randn(1027, device="cuda")
    cf = jit.compile(f, backend="cuda")
    out, ref = cf(x, b), f(x, b)
    assert cf.stats.fused_kernels == 1
    assert (out[0] - ref[0]).abs().max() < 1e-2 and (out[1] - ref[1]).abs().max() < 1e-5
    sm = lambda t: torch.exp(t - t.amax(-1, keepdim=True))                 # noqa: E731
    assert (jit.compile(sm, backend="cuda")(x) - sm(x)).abs().max() < 1e-5
