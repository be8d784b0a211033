"""End-to-end training on the device: parameters and gradients live on cuda:0, the loss falls, and the framework's kernels are the ones launched."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_mlp_bf16_trains_on_device_with_native_kernels():
    from ferrotorch_b200 import _lib, nn, optim
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    X = torch.randn(512, 64, device=dev)
    y = (X[:, :4].sum(1) > 0).long()
    model = nn.Sequential(nn.Linear(64, 256), nn.GELU(), nn.Linear(256, 8)).to(dev).to(torch.bfloat16)
    opt = optim.AdamW(model.parameters(), lr=3e-3)
    l0 = _lib.launch_calls
    first = last = None
    for _ in range(60):
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(model(X.bfloat16()).float(), y)
        loss.backward()
        opt.step()
        first = float(loss.detach()) if first is None else first
        last = float(loss.detach())
    assert last < 0.6 * first
    assert _lib.launch_calls - l0 >= 60 * 4                     # two GEMMs forward, dgrad / wgrad backward, fused optimizer
    for p in model.parameters():
        assert p.device == dev and p.grad is not None and p.grad.device == dev
    assert _lib.read_status() == 0


def test_resnet18_step_channels_last_autocast():
    from ferrotorch_b200 import _lib, nn, optim
    from ferrotorch_b200.vision import resnet18
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    m = resnet18(num_classes=10).to(dev).to(memory_format=torch.channels_last)
    opt = optim.Sgd(m.parameters(), lr=0.05, momentum=0.9)
    x = torch.randn(16, 3, 64, 64, device=dev).contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 10, (16,), device=dev)
    losses = []
    l0 = _lib.launch_calls
    for _ in range(12):
        opt.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(m(x).float(), y)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < 0.7 * losses[0], losses
    assert _lib.launch_calls - l0 > 12 * 20                     # batch-norm, 3x3 convolution and pooling kernels of every block
    assert all(p.grad is not None and p.grad.is_cuda for p in m.parameters())
    assert _lib.read_status() == 0

