"""The long-tail layers of ``ferrotorch_b200.nn`` against ``torch.nn`` given the same parameters: forward values and input gradients."""
import math

import pytest
import torch

import ferrotorch_b200.nn as nn
import ferrotorch_b200.nn.functional as FF
from ferrotorch_b200.errors import InvalidArgument, ShapeMismatch

tnn = torch.nn
TF = torch.nn.functional


def _close(a, b, tol=1e-5):
    assert a.shape == b.shape, (a.shape, b.shape)
    assert torch.allclose(a, b, atol=tol, rtol=tol), (a - b).abs().max().item()


def _fwd_bwd(ours, theirs, *inputs, tol=1e-5):
    """Runs both modules on clones of the inputs and compares outputs and the gradient of ``sum(out * w)`` w.r.t. every float input."""
    ia = [i.clone().requires_grad_(i.is_floating_point()) for i in inputs]
    ib = [i.clone().requires_grad_(i.is_floating_point()) for i in inputs]
    ya, yb = ours(*ia), theirs(*ib)
    ya0, yb0 = (ya[0], yb[0]) if isinstance(ya, tuple) else (ya, yb)
    _close(ya0, yb0, tol)
    w = torch.randn_like(yb0)
    (ya0 * w).sum().backward()
    (yb0 * w).sum().backward()
    for a, b in zip(ia, ib):
        if a.requires_grad and b.grad is not None:
            ok = torch.isfinite(b.grad)          # torch's own gradient w.r.t. a target can be NaN (y log y at y = 0)
            _close(torch.where(ok, a.grad, torch.zeros_like(a.grad)), torch.where(ok, b.grad, torch.zeros_like(b.grad)), tol * 10)
    return ya, yb


def test_no_layer_is_a_torch_subclass_alias():
    """Every exported layer class is defined in this package (only the torch Module base is shared)."""
    for name in dir(nn):
        obj = getattr(nn, name)
        if isinstance(obj, type) and issubclass(obj, torch.nn.Module):
            assert obj.__module__.startswith("ferrotorch_b200."), (name, obj.__module__)
            foreign = [b for b in obj.__mro__ if b.__module__.startswith("torch.nn.modules.") and b.__name__ not in
                       ("Module", "Sequential", "ModuleList", "ModuleDict", "ParameterList", "ParameterDict", "Container")]
            assert not foreign, (name, foreign)


ACTS = [("ReLU", {}), ("ReLU6", {}), ("SELU", {}), ("SiLU", {}), ("Mish", {}), ("Sigmoid", {}), ("Tanh", {}), ("LogSigmoid", {}), ("Tanhshrink", {}),
        ("Softsign", {}), ("LeakyReLU", {"negative_slope": 0.2}), ("ELU", {"alpha": 1.3}), ("CELU", {"alpha": 0.7}), ("Hardtanh", {"min_val": -0.5, "max_val": 0.8}),
        ("Softplus", {"beta": 2.0, "threshold": 3.0}), ("Softmax", {"dim": 1}), ("LogSoftmax", {"dim": -1}), ("Softmin", {"dim": 0}), ("GLU", {"dim": 1}),
        ("Threshold", {"threshold": 0.1, "value": -2.0}), ("Softshrink", {"lambd": 0.3}), ("Hardshrink", {"lambd": 0.3}), ("GELU", {})]


@pytest.mark.parametrize("name,kw", ACTS)
def test_activation_matches_torch(name, kw):
    torch.manual_seed(0)
    x = torch.randn(4, 6, 5) * 3
    _fwd_bwd(getattr(nn, name)(**kw), getattr(tnn, name)(**kw), x)


def test_hard_sigmoid_swish_prelu_rrelu_softmax2d():
    torch.manual_seed(1)
    x = torch.randn(3, 4, 5, 5) * 4
    _fwd_bwd(nn.HardSigmoid(), tnn.Hardsigmoid(), x)
    _fwd_bwd(nn.HardSwish(), tnn.Hardswish(), x)
    _fwd_bwd(nn.Softmax2d(), tnn.Softmax2d(), x)
    for n in (1, 4):
        a, b = nn.PReLU(n, 0.1), tnn.PReLU(n, 0.1)
        _fwd_bwd(a, b, x)
    r = nn.RReLU(0.1, 0.3).eval()
    _close(r(x), tnn.RReLU(0.1, 0.3).eval()(x))
    y = nn.RReLU(0.1, 0.3).train()(x)
    ratio = (y / x)[x < 0]
    assert ratio.min() >= 0.1 - 1e-6 and ratio.max() <= 0.3 + 1e-6 and torch.equal(y[x >= 0], x[x >= 0])
    with pytest.raises(InvalidArgument):
        nn.Hardtanh(1.0, -1.0)


def test_relu_inplace_writes_through_without_autograd():
    x = torch.tensor([-1.0, 2.0])
    y = nn.ReLU(inplace=True)(x)
    assert y.data_ptr() == x.data_ptr() and x.tolist() == [0.0, 2.0]


LOSSES = [("MSELoss", {}, 2), ("L1Loss", {}, 2), ("SmoothL1Loss", {"beta": 0.5}, 2), ("HuberLoss", {"delta": 0.7}, 2)]


@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
@pytest.mark.parametrize("name,kw,_n", LOSSES)
def test_regression_losses(name, kw, _n, reduction):
    torch.manual_seed(2)
    x, y = torch.randn(5, 7), torch.randn(5, 7)
    _fwd_bwd(getattr(nn, name)(reduction=reduction, **kw), getattr(tnn, name)(reduction=reduction, **kw), x, y)


def test_classification_and_ranking_losses():
    torch.manual_seed(3)
    x, t = torch.randn(6, 5), torch.randint(0, 5, (6,))
    w = torch.rand(5) + 0.5
    p = torch.sigmoid(torch.randn(6, 5))
    y01 = torch.randint(0, 2, (6, 5)).float()
    for red in ("mean", "sum", "none"):
        _fwd_bwd(nn.BCELoss(reduction=red), tnn.BCELoss(reduction=red), p, y01)
        _fwd_bwd(nn.BCELoss(weight=w, reduction=red), tnn.BCELoss(weight=w, reduction=red), p, y01)
        _fwd_bwd(nn.BCEWithLogitsLoss(reduction=red), tnn.BCEWithLogitsLoss(reduction=red), x * 5, y01)
        _fwd_bwd(nn.BCEWithLogitsLoss(weight=w, pos_weight=w * 2, reduction=red), tnn.BCEWithLogitsLoss(weight=w, pos_weight=w * 2, reduction=red), x, y01)
        lp = torch.log_softmax(x, 1)
        _fwd_bwd(nn.NLLLoss(reduction=red), tnn.NLLLoss(reduction=red), lp, t)
        tt = t.clone()
        tt[1] = -100
        _fwd_bwd(nn.NLLLoss(weight=w, reduction=red), tnn.NLLLoss(weight=w, reduction=red), lp, tt)
        _fwd_bwd(nn.MultiMarginLoss(reduction=red), tnn.MultiMarginLoss(reduction=red), x, t)
        _fwd_bwd(nn.MultiMarginLoss(p=2, margin=0.5, weight=w, reduction=red), tnn.MultiMarginLoss(p=2, margin=0.5, weight=w, reduction=red), x, t)
        _fwd_bwd(nn.MultiLabelSoftMarginLoss(reduction=red), tnn.MultiLabelSoftMarginLoss(reduction=red), x, y01)
        _fwd_bwd(nn.MultiLabelSoftMarginLoss(weight=w, reduction=red), tnn.MultiLabelSoftMarginLoss(weight=w, reduction=red), x, y01)
        ypm = torch.randint(0, 2, (6,)).float() * 2 - 1
        a, b = torch.randn(6), torch.randn(6)
        _fwd_bwd(nn.MarginRankingLoss(0.3, reduction=red), tnn.MarginRankingLoss(0.3, reduction=red), a, b, ypm)
        _fwd_bwd(nn.HingeEmbeddingLoss(0.8, reduction=red), tnn.HingeEmbeddingLoss(0.8, reduction=red), a, ypm)
        u, v = torch.randn(6, 8), torch.randn(6, 8)
        _fwd_bwd(nn.CosineEmbeddingLoss(0.2, reduction=red), tnn.CosineEmbeddingLoss(0.2, reduction=red), u, v, ypm)
        n_ = torch.randn(6, 8)
        for swap in (False, True):
            _fwd_bwd(nn.TripletMarginLoss(0.9, swap=swap, reduction=red), tnn.TripletMarginLoss(0.9, swap=swap, reduction=red), u, v, n_)
    # 4-D NLL
    lp4, t4 = torch.log_softmax(torch.randn(2, 5, 3, 3), 1), torch.randint(0, 5, (2, 3, 3))
    _fwd_bwd(nn.NLLLoss(), tnn.NLLLoss(), lp4, t4)
    with pytest.raises(InvalidArgument):
        nn.NLLLoss()(torch.log_softmax(x, 1), torch.full((6,), 9))


def test_distribution_losses():
    torch.manual_seed(4)
    lq = torch.log_softmax(torch.randn(4, 6), 1)
    pt = torch.softmax(torch.randn(4, 6), 1)
    for red in ("mean", "sum", "none", "batchmean"):
        _fwd_bwd(nn.KLDivLoss(reduction=red), tnn.KLDivLoss(reduction=red), lq, pt)
        _fwd_bwd(nn.KLDivLoss(reduction=red, log_target=True), tnn.KLDivLoss(reduction=red, log_target=True), lq, pt.log())
    x, y = torch.randn(4, 6), torch.poisson(torch.rand(4, 6) * 4)
    for log_input in (True, False):
        for full in (True, False):
            xi = x if log_input else x.abs() + 0.1
            _fwd_bwd(nn.PoissonNLLLoss(log_input, full), tnn.PoissonNLLLoss(log_input, full), xi, y)
    var = torch.rand(4, 6) + 0.1
    for full in (True, False):
        _fwd_bwd(nn.GaussianNLLLoss(full=full), tnn.GaussianNLLLoss(full=full), x, torch.randn(4, 6), var)
    _fwd_bwd(nn.GaussianNLLLoss(), tnn.GaussianNLLLoss(), x, torch.randn(4, 6), torch.rand(4) + 0.1)
    a, b = torch.randn(5, 7), torch.randn(5, 7)
    _fwd_bwd(nn.CosineSimilarity(1), tnn.CosineSimilarity(1), a, b)
    for p in (1.0, 2.0, 3.0):
        _fwd_bwd(nn.PairwiseDistance(p), tnn.PairwiseDistance(p), a, b)


@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_ctc_loss_matches_torch(reduction):
    torch.manual_seed(5)
    T, N, C, S = 12, 3, 6, 5
    logits = torch.randn(T, N, C)
    lp = torch.log_softmax(logits, 2)
    targets = torch.randint(1, C, (N, S))
    targets[0, 1] = targets[0, 0]                 # a repeated label needs a blank between its two copies
    il, tl = torch.tensor([12, 10, 7]), torch.tensor([5, 3, 0])
    # gradients are compared at the logits: the library's backward is written for log-softmax inputs
    a = logits.clone().requires_grad_()
    b = logits.clone().requires_grad_()
    la = nn.CTCLoss(reduction=reduction)(torch.log_softmax(a, 2), targets, il, tl)
    lb = tnn.CTCLoss(reduction=reduction)(torch.log_softmax(b, 2), targets, il, tl)
    _close(la, lb, 1e-4)
    la.sum().backward()
    lb.sum().backward()
    _close(a.grad, b.grad, 1e-4)
    # concatenated targets, and an impossible alignment (input shorter than the labels)
    flat = torch.cat([targets[i, : tl[i]] for i in range(N)])
    _close(nn.CTCLoss(reduction=reduction)(lp, flat, il, tl), lb.detach(), 1e-4)
    bad = nn.CTCLoss(reduction="none", zero_infinity=True)(lp, targets, torch.tensor([12, 2, 7]), tl)
    assert bad[1] == 0 and torch.isinf(nn.CTCLoss(reduction="none")(lp, targets, torch.tensor([12, 2, 7]), tl)[1])


def _copy_params(ours, theirs):
    sd = theirs.state_dict()
    missing = ours.load_state_dict(sd, strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys


CONVS = [
    ("Conv1d", (4, 6, 3), dict(stride=2, padding=1), (2, 4, 11)),
    ("Conv1d", (4, 6, 3), dict(padding="same", dilation=2), (2, 4, 11)),
    ("Conv1d", (4, 6, 4), dict(padding="same"), (2, 4, 11)),
    ("Conv2d", (4, 8, 3), dict(stride=(2, 1), padding=(1, 2), dilation=(1, 2)), (2, 4, 9, 10)),
    ("Conv2d", (4, 8, 3), dict(groups=2, bias=False), (2, 4, 9, 10)),
    ("Conv2d", (4, 8, 3), dict(padding=1, padding_mode="reflect"), (2, 4, 9, 10)),
    ("Conv2d", (4, 8, 3), dict(padding=2, padding_mode="circular"), (2, 4, 9, 10)),
    ("Conv2d", (4, 8, 3), dict(padding=1, padding_mode="replicate"), (4, 9, 10)),
    ("Conv2d", (4, 8, (2, 3)), dict(padding="valid"), (2, 4, 9, 10)),
    ("Conv3d", (2, 4, 3), dict(stride=2, padding=1), (2, 2, 7, 8, 9)),
    ("ConvTranspose1d", (4, 6, 3), dict(stride=2, padding=1, output_padding=1), (2, 4, 7)),
    ("ConvTranspose2d", (4, 6, 3), dict(stride=2, padding=1, output_padding=1, groups=2, dilation=1), (2, 4, 5, 6)),
    ("ConvTranspose2d", (4, 6, 4), dict(stride=2, padding=1), (2, 4, 5, 6)),
    ("ConvTranspose3d", (2, 4, 3), dict(stride=2), (1, 2, 3, 4, 5)),
]


@pytest.mark.parametrize("name,args,kw,shape", CONVS)
def test_conv_layers_match_torch(name, args, kw, shape):
    torch.manual_seed(6)
    ours, theirs = getattr(nn, name)(*args, **kw), getattr(tnn, name)(*args, **kw)
    assert {k: v.shape for k, v in ours.state_dict().items()} == {k: v.shape for k, v in theirs.state_dict().items()}
    _copy_params(ours, theirs)
    _fwd_bwd(ours, theirs, torch.randn(*shape), tol=1e-4)


def test_conv_init_errors_lazy_and_output_size():
    c = nn.Conv2d(16, 32, 3)
    bound = math.sqrt(2.0) * math.sqrt(3.0 / (16 * 9))
    assert c.weight.abs().max() <= bound and c.weight.abs().max() > 0.8 * bound and float(c.bias.abs().sum()) == 0.0
    with pytest.raises(InvalidArgument):
        nn.Conv2d(3, 8, 3, groups=2)
    with pytest.raises(InvalidArgument):
        nn.Conv2d(4, 8, 3, stride=2, padding="same")
    with pytest.raises(ShapeMismatch):
        c(torch.randn(1, 3, 8, 8))
    lz = nn.LazyConv2d(8, 3, padding=1)
    assert not lz.is_initialized()
    assert lz(torch.randn(2, 5, 6, 6)).shape == (2, 8, 6, 6) and lz.inner.in_channels == 5
    lt = nn.LazyConvTranspose1d(4, 3, stride=2)
    assert lt(torch.randn(2, 6, 5)).shape == (2, 4, 11)
    ct, tt = nn.ConvTranspose2d(3, 4, 3, stride=2, padding=1), tnn.ConvTranspose2d(3, 4, 3, stride=2, padding=1)
    _copy_params(ct, tt)
    x = torch.randn(1, 3, 5, 5)
    _close(ct(x, output_size=(10, 10)), tt(x, output_size=(10, 10)), 1e-5)
    assert ct.output_size((5, 5)) == (9, 9)
    with pytest.raises(InvalidArgument):
        ct(x, output_size=(12, 12))


NORMS = [("BatchNorm1d", (6,), {}, (8, 6)), ("BatchNorm1d", (6,), {"momentum": None}, (8, 6, 5)), ("BatchNorm2d", (6,), {"affine": False}, (4, 6, 5, 5)),
         ("BatchNorm2d", (6,), {"track_running_stats": False}, (4, 6, 5, 5)), ("BatchNorm3d", (4,), {"eps": 1e-3, "momentum": 0.3}, (2, 4, 3, 4, 5)),
         ("GroupNorm", (3, 6), {}, (4, 6, 5, 5)), ("GroupNorm", (2, 6), {"affine": False}, (4, 6, 7)),
         ("InstanceNorm1d", (6,), {}, (4, 6, 9)), ("InstanceNorm2d", (6,), {"affine": True, "track_running_stats": True}, (4, 6, 5, 5)),
         ("InstanceNorm3d", (3,), {"affine": True}, (2, 3, 4, 4, 4)), ("LocalResponseNorm", (3,), {}, (2, 7, 5, 5)),
         ("LocalResponseNorm", (4,), {"alpha": 1e-2, "beta": 0.5, "k": 2.0}, (2, 7, 9))]


@pytest.mark.parametrize("name,args,kw,shape", NORMS)
def test_norm_layers_match_torch_over_train_and_eval(name, args, kw, shape):
    torch.manual_seed(7)
    ours, theirs = getattr(nn, name)(*args, **kw), getattr(tnn, name)(*args, **kw)
    with torch.no_grad():
        for p in theirs.parameters():
            p.uniform_(0.5, 1.5)
    _copy_params(ours, theirs)
    for step in range(3):
        _fwd_bwd(ours, theirs, torch.randn(*shape) * 2 + 1, tol=2e-5)
    for (ka, va), (kb, vb) in zip(sorted(ours.state_dict().items()), sorted(theirs.state_dict().items())):
        assert ka == kb
        _close(va.float(), vb.float(), 1e-5)
    ours.eval(), theirs.eval()
    _fwd_bwd(ours, theirs, torch.randn(*shape), tol=2e-5)


def test_lazy_batch_norm_and_shape_errors():
    lz = nn.LazyBatchNorm2d()
    y = lz(torch.randn(4, 5, 3, 3))
    assert lz.inner.num_features == 5 and y.shape == (4, 5, 3, 3)
    with pytest.raises(ShapeMismatch):
        nn.BatchNorm2d(4)(torch.randn(2, 4, 3))
    with pytest.raises(InvalidArgument):
        nn.GroupNorm(4, 6)


POOLS = [
    ("MaxPool1d", (3,), dict(stride=2, padding=1), (2, 3, 11)),
    ("MaxPool2d", (3,), dict(stride=2, padding=1), (2, 3, 11, 12)),
    ("MaxPool2d", ((2, 3),), dict(stride=(2, 1), dilation=(1, 2), ceil_mode=True), (2, 3, 11, 12)),
    ("MaxPool2d", (2,), dict(ceil_mode=True), (3, 7, 7)),
    ("MaxPool3d", (2,), dict(stride=2, padding=1), (1, 2, 5, 6, 7)),
    ("AvgPool1d", (3,), dict(stride=2, padding=1, count_include_pad=False), (2, 3, 11)),
    ("AvgPool2d", (3,), dict(stride=2, padding=1), (2, 3, 11, 12)),
    ("AvgPool2d", (3,), dict(stride=2, padding=1, ceil_mode=True, count_include_pad=False), (2, 3, 10, 12)),
    ("AvgPool2d", (3,), dict(stride=2, padding=1, ceil_mode=True), (2, 3, 10, 12)),
    ("AvgPool2d", (2,), dict(divisor_override=3), (2, 3, 8, 8)),
    ("AvgPool3d", (2,), dict(stride=1, padding=1), (1, 2, 4, 5, 6)),
    ("AdaptiveAvgPool1d", (4,), {}, (2, 3, 11)),
    ("AdaptiveAvgPool2d", ((3, 5),), {}, (2, 3, 11, 12)),
    ("AdaptiveAvgPool2d", (1,), {}, (2, 3, 7, 7)),
    ("AdaptiveAvgPool2d", ((None, 4),), {}, (2, 3, 6, 8)),
    ("AdaptiveAvgPool3d", (2,), {}, (1, 2, 5, 6, 7)),
    ("AdaptiveMaxPool1d", (4,), {}, (2, 3, 11)),
    ("AdaptiveMaxPool2d", ((3, 5),), {}, (2, 3, 11, 12)),
    ("AdaptiveMaxPool3d", (2,), {}, (1, 2, 5, 6, 7)),
    ("LPPool1d", (2, 3), dict(stride=2), (2, 3, 11)),
    ("LPPool2d", (3, 2), dict(stride=1, ceil_mode=True), (2, 3, 7, 8)),
    ("PixelShuffle", (2,), {}, (2, 8, 3, 4)),
    ("PixelUnshuffle", (2,), {}, (2, 3, 6, 8)),
    ("Unfold", ((2, 3),), dict(dilation=(1, 2), padding=1, stride=(2, 1)), (2, 3, 7, 9)),
]


@pytest.mark.parametrize("name,args,kw,shape", POOLS)
def test_pooling_matches_torch(name, args, kw, shape):
    torch.manual_seed(8)
    x = torch.randn(*shape)
    if name.startswith("LPPool"):
        x = x.abs() + 0.1
    _fwd_bwd(getattr(nn, name)(*args, **kw), getattr(tnn, name)(*args, **kw), x)


def test_pool_indices_unpool_fold_fractional():
    torch.manual_seed(9)
    x = torch.randn(2, 3, 8, 9)
    for kw in (dict(kernel_size=2), dict(kernel_size=3, stride=2, padding=1), dict(kernel_size=2, stride=2, ceil_mode=True)):
        va, ia = nn.MaxPool2d(return_indices=True, **kw)(x)
        vb, ib = tnn.MaxPool2d(return_indices=True, **kw)(x)
        _close(va, vb)
        assert torch.equal(ia, ib)
    va, ia = nn.MaxPool1d(3, 2, return_indices=True)(x[:, :, 0])
    vb, ib = tnn.MaxPool1d(3, 2, return_indices=True)(x[:, :, 0])
    assert torch.equal(ia, ib)
    va, ia = nn.AdaptiveMaxPool2d((3, 4), return_indices=True)(x)
    vb, ib = tnn.AdaptiveMaxPool2d((3, 4), return_indices=True)(x)
    _close(va, vb)
    assert torch.equal(ia, ib)
    v, i = tnn.MaxPool2d(2, return_indices=True)(x)
    _close(nn.MaxUnpool2d(2)(v, i, output_size=(8, 9)), tnn.MaxUnpool2d(2)(v, i, output_size=(8, 9)))
    v8, i8 = tnn.MaxPool2d(2, return_indices=True)(x[..., :8])
    _close(nn.MaxUnpool2d(2)(v8, i8), tnn.MaxUnpool2d(2)(v8, i8))
    with pytest.raises(InvalidArgument):
        nn.MaxUnpool2d(2)(v, i)                   # indices of an 8x9 plane do not fit the default 8x8 output
    cols = torch.randn(2, 3 * 2 * 3, 4 * 7)
    kw = dict(output_size=(7, 9), kernel_size=(2, 3), dilation=(1, 2), padding=1, stride=(2, 1))
    _fwd_bwd(nn.Fold(**kw), tnn.Fold(**kw), cols)
    samples = torch.rand(2, 3, 2)
    for kw in (dict(output_size=(4, 5)), dict(output_ratio=(0.5, 0.6))):
        a = nn.FractionalMaxPool2d(2, return_indices=True, _random_samples=samples, **kw)(x)
        b = tnn.FractionalMaxPool2d(2, return_indices=True, _random_samples=samples, **kw)(x)
        _close(a[0], b[0])
        assert torch.equal(a[1], b[1])
    with pytest.raises(ShapeMismatch):
        nn.MaxPool2d(5)(torch.randn(1, 1, 3, 3))


PADS = [("ConstantPad1d", ((2, 1), 1.5), (2, 3, 5)), ("ConstantPad2d", ((1, 2, 0, 3), -1.0), (2, 3, 4, 5)), ("ConstantPad3d", (1, 0.5), (1, 2, 3, 4, 5)),
        ("ZeroPad1d", ((1, 2),), (2, 3, 5)), ("ZeroPad2d", ((1, -1, 2, 0),), (2, 3, 4, 5)), ("ZeroPad3d", (1,), (1, 2, 3, 4, 5)),
        ("ReflectionPad1d", ((2, 3),), (2, 3, 5)), ("ReflectionPad2d", ((1, 2, 3, 0),), (2, 3, 4, 5)), ("ReflectionPad3d", (1,), (1, 2, 3, 4, 5)),
        ("ReplicationPad1d", ((2, 3),), (2, 3, 5)), ("ReplicationPad2d", ((1, 2, 3, 0),), (3, 4, 5)), ("ReplicationPad3d", ((1, 0, 2, 1, 0, 2),), (1, 2, 3, 4, 5)),
        ("CircularPad1d", ((2, 3),), (2, 3, 5)), ("CircularPad2d", ((1, 2, 3, 0),), (2, 3, 4, 5)), ("CircularPad3d", (1,), (1, 2, 3, 4, 5))]


@pytest.mark.parametrize("name,args,shape", PADS)
def test_padding_matches_torch(name, args, shape):
    torch.manual_seed(10)
    _fwd_bwd(getattr(nn, name)(*args), getattr(tnn, name)(*args), torch.randn(*shape))


def test_padding_limits():
    with pytest.raises(InvalidArgument):
        nn.ReflectionPad1d(5)(torch.randn(1, 2, 5))
    with pytest.raises(InvalidArgument):
        nn.CircularPad1d(6)(torch.randn(1, 2, 5))
    with pytest.raises(ShapeMismatch):
        nn.ZeroPad2d(1)(torch.randn(5))
    _close(FF.pad(torch.arange(6.0).view(2, 3), (1, 1, 0, 1), "constant", 9.0), TF.pad(torch.arange(6.0).view(2, 3), (1, 1, 0, 1), "constant", 9.0))


@pytest.mark.parametrize("name,gates", [("RNN", 1), ("LSTM", 4), ("GRU", 3)])
@pytest.mark.parametrize("bidirectional,layers,batch_first,bias", [(False, 1, False, True), (True, 2, True, True), (False, 2, False, False)])
def test_recurrent_layers_match_torch(name, gates, bidirectional, layers, batch_first, bias):
    torch.manual_seed(11)
    kw = dict(num_layers=layers, bidirectional=bidirectional, batch_first=batch_first, bias=bias)
    ours, theirs = getattr(nn, name)(5, 7, **kw), getattr(tnn, name)(5, 7, **kw)
    assert [k for k, _ in ours.named_parameters()] == [k for k, _ in theirs.named_parameters()]
    _copy_params(ours, theirs)
    x = torch.randn(3, 6, 5) if batch_first else torch.randn(6, 3, 5)
    D = 2 if bidirectional else 1
    h0 = torch.randn(layers * D, 3, 7)
    hx = (h0, torch.randn(layers * D, 3, 7)) if name == "LSTM" else h0
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    (ya, sa), (yb, sb) = ours(xa, hx), theirs(xb, hx)
    _close(ya, yb, 1e-5)
    for a, b in zip(sa if name == "LSTM" else (sa,), sb if name == "LSTM" else (sb,)):
        _close(a, b, 1e-5)
    w = torch.randn_like(yb)
    (ya * w).sum().backward()
    (yb * w).sum().backward()
    _close(xa.grad, xb.grad, 1e-4)
    for (n, pa), (_, pb) in zip(ours.named_parameters(), theirs.named_parameters()):
        _close(pa.grad, pb.grad, 1e-4)
    # default zero state and un-batched input
    _close(ours(x)[0], theirs(x)[0], 1e-5)
    xu = torch.randn(6, 5)
    _close(ours(xu)[0], theirs(xu)[0], 1e-5)


def test_recurrent_cells_relu_rnn_and_packed_sequences():
    torch.manual_seed(12)
    for name in ("RNNCell", "LSTMCell", "GRUCell"):
        ours, theirs = getattr(nn, name)(4, 6), getattr(tnn, name)(4, 6)
        _copy_params(ours, theirs)
        x = torch.randn(3, 4)
        a, b = ours(x), theirs(x)
        for u, v in zip(a if isinstance(a, tuple) else (a,), b if isinstance(b, tuple) else (b,)):
            _close(u, v, 1e-5)
        _close((ours(x[0])[0] if name == "LSTMCell" else ours(x[0])), (theirs(x[0])[0] if name == "LSTMCell" else theirs(x[0])), 1e-5)
    ours, theirs = nn.RNN(4, 6, nonlinearity="relu"), tnn.RNN(4, 6, nonlinearity="relu")
    _copy_params(ours, theirs)
    _close(ours(torch.ones(5, 2, 4))[0], theirs(torch.ones(5, 2, 4))[0], 1e-5)
    # variable-length batch through packing, both directions
    ours, theirs = nn.LSTM(4, 6, bidirectional=True), tnn.LSTM(4, 6, bidirectional=True)
    _copy_params(ours, theirs)
    x, lengths = torch.randn(7, 3, 4), torch.tensor([4, 7, 2])
    pa = nn.utils.pack_padded_sequence(x, lengths, enforce_sorted=False)
    pb = tnn.utils.rnn.pack_padded_sequence(x, lengths, enforce_sorted=False)
    _close(pa.data, pb.data)
    assert torch.equal(pa.batch_sizes, pb.batch_sizes) and torch.equal(pa.sorted_indices, pb.sorted_indices)
    (oa, (ha, ca)), (ob, (hb, cb)) = ours(pa), theirs(pb)
    ua, la = nn.utils.pad_packed_sequence(oa)
    ub, lb = tnn.utils.rnn.pad_packed_sequence(ob)
    _close(ua, ub, 1e-5)
    assert torch.equal(la, lb)
    _close(ha, hb, 1e-5)
    _close(ca, cb, 1e-5)
    # a torch PackedSequence is accepted and answered in kind
    oc, _ = ours(pb)
    assert isinstance(oc, tnn.utils.rnn.PackedSequence)
    seqs = [torch.randn(n, 2) for n in (5, 3, 1)]
    _close(nn.utils.pad_sequence(seqs, batch_first=True), tnn.utils.rnn.pad_sequence(seqs, batch_first=True))
    _close(nn.utils.pack_sequence(seqs).data, tnn.utils.rnn.pack_sequence(seqs).data)
    with pytest.raises(InvalidArgument):
        nn.utils.pack_padded_sequence(x, torch.tensor([4, 7, 2]))


def _load_attn(ours, theirs):
    E = ours.embed_dim
    with torch.no_grad():
        wq, wk, wv = theirs.in_proj_weight.split(E)
        bq, bk, bv = theirs.in_proj_bias.split(E)
        for lin, w, b in ((ours.q_proj, wq, bq), (ours.k_proj, wk, bk), (ours.v_proj, wv, bv), (ours.out_proj, theirs.out_proj.weight, theirs.out_proj.bias)):
            lin.weight.copy_(w)
            lin.bias.copy_(b)


def _load_block(ours, theirs):
    _load_attn(ours.self_attn, theirs.self_attn)
    if hasattr(theirs, "multihead_attn"):
        _load_attn(ours.multihead_attn, theirs.multihead_attn)
    with torch.no_grad():
        for n in ("linear1", "linear2", "norm1", "norm2", "norm3"):
            if hasattr(theirs, n):
                getattr(ours, n).weight.copy_(getattr(theirs, n).weight)
                getattr(ours, n).bias.copy_(getattr(theirs, n).bias)


@pytest.mark.parametrize("norm_first,batch_first,act", [(False, True, "relu"), (True, False, "gelu")])
def test_transformer_stacks_match_torch(norm_first, batch_first, act):
    torch.manual_seed(13)
    kw = dict(d_model=16, nhead=4, num_encoder_layers=2, num_decoder_layers=2, dim_feedforward=32, dropout=0.0, activation=act,
              batch_first=batch_first, norm_first=norm_first)
    ours, theirs = nn.Transformer(**kw), tnn.Transformer(**kw)
    for a, b in zip(ours.encoder.layers, theirs.encoder.layers):
        _load_block(a, b)
    for a, b in zip(ours.decoder.layers, theirs.decoder.layers):
        _load_block(a, b)
    with torch.no_grad():
        for a, b in ((ours.encoder.norm, theirs.encoder.norm), (ours.decoder.norm, theirs.decoder.norm)):
            a.weight.copy_(b.weight)
            a.bias.copy_(b.bias)
    ours.eval(), theirs.eval()
    B, S, T = 2, 5, 4
    src, tgt = torch.randn(B, S, 16), torch.randn(B, T, 16)
    if not batch_first:
        src, tgt = src.transpose(0, 1).contiguous(), tgt.transpose(0, 1).contiguous()
    tgt_mask = nn.Transformer.generate_square_subsequent_mask(T)
    assert torch.equal(tgt_mask, tnn.Transformer.generate_square_subsequent_mask(T))
    pad = torch.zeros(B, S, dtype=torch.bool)
    pad[1, -2:] = True
    with torch.no_grad():
        ya = ours(src, tgt, tgt_mask=tgt_mask, src_key_padding_mask=pad, memory_key_padding_mask=pad)
        yb = theirs(src, tgt, tgt_mask=tgt_mask, src_key_padding_mask=pad, memory_key_padding_mask=pad)
    _close(ya, yb, 2e-5)
    # boolean mask and is_causal give the same answer as the float mask
    with torch.no_grad():
        yc = ours(src, tgt, tgt_mask=torch.ones(T, T, dtype=torch.bool).triu(1), src_key_padding_mask=pad, memory_key_padding_mask=pad)
        yd = ours(src, tgt, tgt_is_causal=True, src_key_padding_mask=pad, memory_key_padding_mask=pad)
    _close(yc, ya, 1e-6)
    _close(yd, ya, 1e-5)
    # encoder alone, gradient flows to every parameter
    out = ours.encoder(src, src_key_padding_mask=pad)
    out.sum().backward()
    assert all(p.grad is not None for p in ours.encoder.parameters())


def test_dropout_family_and_misc_layers():
    torch.manual_seed(14)
    x = torch.ones(64, 32, 8)
    d = nn.Dropout(0.25)
    y = d(x)
    kept = (y != 0).float().mean().item()
    assert abs(kept - 0.75) < 0.02 and torch.allclose(y[y != 0], torch.tensor(1 / 0.75))
    assert torch.equal(d.eval()(x), x)
    y1 = nn.Dropout1d(0.5)(x)
    per_channel = (y1 != 0).float().mean(-1)
    assert set(per_channel.unique().tolist()) <= {0.0, 1.0}
    y2 = nn.Dropout2d(0.5)(torch.ones(8, 16, 4, 4))
    assert set((y2 != 0).float().mean((-1, -2)).unique().tolist()) <= {0.0, 1.0}
    assert nn.Dropout3d(0.0)(torch.ones(1, 2, 2, 2, 2)).sum() == 16
    z = torch.selu(torch.randn(200000))
    za = nn.AlphaDropout(0.2)(z)
    assert abs(za.mean() - z.mean()) < 0.02 and abs(za.std() - z.std()) < 0.03
    with pytest.raises(InvalidArgument):
        nn.Dropout(1.5)
    t = torch.randn(2, 6, 4, 4)
    _close(nn.ChannelShuffle(3)(t), tnn.ChannelShuffle(3)(t))
    _close(nn.Flatten()(t), tnn.Flatten()(t))
    _close(nn.Unflatten(1, (2, 3))(t), tnn.Unflatten(1, (2, 3))(t))
    assert nn.Identity(1, a=2)(t) is t
    _close(nn.Upsample(scale_factor=2, mode="bilinear", align_corners=False)(t), tnn.Upsample(scale_factor=2, mode="bilinear", align_corners=False)(t))
    se = nn.SqueezeExcitation(6, 2)
    assert se(t).shape == t.shape


@pytest.mark.parametrize("mode", ["sum", "mean", "max"])
def test_embedding_bag_matches_torch(mode):
    torch.manual_seed(15)
    w = torch.randn(10, 4)
    ours, theirs = nn.EmbeddingBag(10, 4, mode=mode, _weight=w.clone()), tnn.EmbeddingBag(10, 4, mode=mode, _weight=w.clone())
    ids2 = torch.randint(0, 10, (3, 5))
    _close(ours(ids2), theirs(ids2))
    ids1, off = torch.randint(0, 10, (11,)), torch.tensor([0, 3, 3, 8])
    _close(ours(ids1, off), theirs(ids1, off))
    ya, yb = ours(ids1, off), theirs(ids1, off)
    ya.sum().backward(), yb.sum().backward()
    _close(ours.weight.grad, theirs.weight.grad)
    if mode == "sum":
        psw = torch.rand(11)
        _close(ours(ids1, off, psw), theirs(ids1, off, psw))
    pa, pb = nn.EmbeddingBag(10, 4, mode=mode, padding_idx=2, _weight=w.clone()), tnn.EmbeddingBag(10, 4, mode=mode, padding_idx=2, _weight=w.clone())
    ids2[0, :2] = 2
    _close(pa(ids2), pb(ids2))


def test_functional_forms_are_this_packages():
    x = torch.randn(3, 5)
    for name in ("relu", "softmax", "mse_loss", "max_pool2d", "batch_norm", "pad", "dropout", "one_hot", "normalize", "embedding"):
        assert getattr(FF, name).__module__.startswith("ferrotorch_b200."), name
    _close(FF.normalize(x, 3.0, 1), TF.normalize(x, 3.0, 1))
    _close(FF.one_hot(torch.tensor([0, 2]), 3), TF.one_hot(torch.tensor([0, 2]), 3))
    w = torch.randn(6, 4, requires_grad=True)
    ids = torch.tensor([[1, 2], [2, 5]])
    FF.embedding(ids, w, padding_idx=2).sum().backward()
    assert float(w.grad[2].abs().sum()) == 0 and float(w.grad[1].sum()) == 4.0
    _close(FF.layer_norm(x, (5,)), TF.layer_norm(x, (5,)))


@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_cross_entropy_loss_takes_class_weights(reduction):
    import ferrotorch_b200.nn as ftnn
    g = torch.Generator().manual_seed(4)
    logits = torch.randn(9, 5, generator=g)
    target = torch.randint(0, 5, (9,), generator=g)
    w = torch.rand(5, generator=g) + 0.5
    a, b = logits.clone().requires_grad_(True), logits.clone().requires_grad_(True)
    got = ftnn.CrossEntropyLoss(reduction=reduction, label_smoothing=0.1, weight=w)(a, target)
    want = torch.nn.CrossEntropyLoss(weight=w, reduction=reduction, label_smoothing=0.1)(b, target)
    torch.testing.assert_close(got, want)
    got.sum().backward(); want.sum().backward()
    torch.testing.assert_close(a.grad, b.grad)


def test_torch_transformer_checkpoints_with_packed_projections_load_and_match():
    torch.manual_seed(0)
    x, y = torch.randn(2, 5, 8), torch.randn(2, 3, 8)
    ref = torch.nn.Transformer(8, 2, 2, 2, 16, dropout=0.0, batch_first=True).eval()
    mine = nn.Transformer(8, 2, 2, 2, 16, dropout=0.0, batch_first=True).eval()
    assert any(k.endswith("in_proj_weight") for k in ref.state_dict())
    result = mine.load_state_dict(ref.state_dict())
    assert not result.missing_keys and not result.unexpected_keys
    torch.testing.assert_close(mine(x, y), ref(x, y), rtol=1e-4, atol=1e-5)
    bad = {k: (v[:-1] if k.endswith("in_proj_weight") else v) for k, v in ref.state_dict().items()}
    with pytest.raises(ShapeMismatch):
        mine.load_state_dict(bad)
