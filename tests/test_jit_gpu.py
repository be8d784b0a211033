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
    ref = _f(x.float(), y.float(), b.float())
    assert cf.stats.fused_kernels == 1 and _lib.launch_calls > l0
    assert (out[1].float() - ref[1]).abs().max() < tol
    assert (out[0].float() - ref[0]).abs().max() < tol * 1027 ** 0.5 * 4
    f2 = lambda p, q: torch.tanh(p) * q + F.silu(p)  # noqa: E731  all operands dense -> 16-byte vector kernel, ragged tail (512*1027 % 8 != 0 for bf16)
    c2 = jit.compile(f2, backend="cuda")
    assert (c2(x, y).float() - f2(x.float(), y.float())).abs().max() < tol
    xs = x[:, ::2]                                   # strided view
    assert (c2(xs, y[:, ::2]).float() - f2(xs.float(), y[:, ::2].float())).abs().max() < tol
    assert _lib.read_status() == 0


def test_compiled_mlp_block_matches_eager():
    from ferrotorch_b200 import jit
    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.GELU(), torch.nn.Linear(512, 256)).cuda()
    x = torch.randn(64, 256, device="cuda")
    f = lambda t: F.silu(m(t)) * torch.sigmoid(t) + t     # noqa: E731
    cf = jit.compile(f, backend="cuda")
    assert (cf(x) - f(x)).abs().max() < 1e-4 and cf.stats.fused_kernels >= 1
