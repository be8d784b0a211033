"""Per-symbol behaviour checks of ``ferrotorch_b200.nn`` / ``nn.functional`` against PyTorch: the functional forms, lazy layers, enums, paged
KV cache, attention helpers and hooks that the layer-level tests do not already exercise."""
import pytest
import torch

import ferrotorch_b200.nn as nn
import ferrotorch_b200.nn.functional as FF
from ferrotorch_b200.errors import InvalidArgument

TF = torch.nn.functional


def _close(a, b, tol=1e-5):
    assert a.shape == b.shape and torch.allclose(a, b, atol=tol, rtol=tol), (a.shape, b.shape, (a - b).abs().max().item() if a.shape == b.shape else None)


UNARY = [("celu", (0.7,)), ("glu", (1,)), ("hardshrink", (0.3,)), ("hardsigmoid", ()), ("hardtanh", (-0.4, 0.6)), ("leaky_relu", (0.2,)), ("logsigmoid", ()),
         ("relu6", ()), ("softmin", (1,)), ("softshrink", (0.3,)), ("softsign", ()), ("tanhshrink", ())]


@pytest.mark.parametrize("name,args", UNARY)
def test_functional_activations(name, args):
    torch.manual_seed(0)
    x = torch.randn(4, 6) * 3
    _close(getattr(FF, name)(x, *args), getattr(TF, name)(x, *args))


def test_rrelu_and_alpha_dropout_functional():
    torch.manual_seed(0)
    x = torch.randn(100, 50)
    _close(FF.rrelu(x, 0.1, 0.3, False), TF.rrelu(x, 0.1, 0.3, False))
    y = FF.rrelu(x, 0.1, 0.3, True)
    r = (y / x)[x < 0]
    assert 0.1 - 1e-6 <= r.min() and r.max() <= 0.3 + 1e-6
    assert torch.equal(FF.alpha_dropout(x, 0.3, False), x)
    z = torch.selu(torch.randn(100000))
    za = FF.alpha_dropout(z, 0.3, True)
    assert abs(za.mean() - z.mean()) < 0.03 and abs(za.std() - z.std()) < 0.05


def test_functional_losses():
    torch.manual_seed(1)
    x, y = torch.randn(5, 6), torch.randn(5, 6)
    t = torch.randint(0, 6, (5,))
    y01, ypm = torch.randint(0, 2, (5, 6)).float(), torch.randint(0, 2, (5,)).float() * 2 - 1
    p = torch.sigmoid(x)
    _close(FF.binary_cross_entropy(p, y01), TF.binary_cross_entropy(p, y01))
    _close(FF.binary_cross_entropy_with_logits(x, y01), TF.binary_cross_entropy_with_logits(x, y01))
    _close(FF.l1_loss(x, y), TF.l1_loss(x, y))
    _close(FF.smooth_l1_loss(x, y, "sum", 0.5), TF.smooth_l1_loss(x, y, reduction="sum", beta=0.5))
    _close(FF.huber_loss(x, y, "mean", 0.7), TF.huber_loss(x, y, delta=0.7))
    _close(FF.nll_loss(torch.log_softmax(x, 1), t), TF.nll_loss(torch.log_softmax(x, 1), t))
    _close(FF.kl_div(torch.log_softmax(x, 1), torch.softmax(y, 1), "batchmean"), TF.kl_div(torch.log_softmax(x, 1), torch.softmax(y, 1), reduction="batchmean"))
    _close(FF.cosine_embedding_loss(x, y, ypm, 0.1), TF.cosine_embedding_loss(x, y, ypm, margin=0.1))
    _close(FF.cosine_similarity(x, y, 1), TF.cosine_similarity(x, y, 1))
    _close(FF.pairwise_distance(x, y, 2.0), TF.pairwise_distance(x, y, 2.0))
    _close(FF.margin_ranking_loss(x[:, 0], y[:, 0], ypm, 0.2), TF.margin_ranking_loss(x[:, 0], y[:, 0], ypm, margin=0.2))
    _close(FF.hinge_embedding_loss(x[:, 0], ypm, 0.9), TF.hinge_embedding_loss(x[:, 0], ypm, margin=0.9))
    _close(FF.triplet_margin_loss(x, y, x.flip(0), 0.8), TF.triplet_margin_loss(x, y, x.flip(0), margin=0.8))
    _close(FF.multi_margin_loss(x, t), TF.multi_margin_loss(x, t))
    _close(FF.multilabel_soft_margin_loss(x, y01), TF.multilabel_soft_margin_loss(x, y01))
    _close(FF.poisson_nll_loss(x, y.abs()), TF.poisson_nll_loss(x, y.abs()))
    _close(FF.gaussian_nll_loss(x, y, y.abs() + 0.1), TF.gaussian_nll_loss(x, y, y.abs() + 0.1))
    lp = torch.log_softmax(torch.randn(8, 2, 5), 2)
    tg, il, tl = torch.randint(1, 5, (2, 3)), torch.tensor([8, 6]), torch.tensor([3, 2])
    _close(FF.ctc_loss(lp, tg, il, tl), TF.ctc_loss(lp, tg, il, tl), 1e-4)


def test_functional_pooling_and_reshaping():
    torch.manual_seed(2)
    x1, x2, x3 = torch.randn(2, 3, 12), torch.randn(2, 3, 9, 10), torch.randn(1, 2, 5, 6, 7)
    _close(FF.max_pool1d(x1, 3, 2, 1), TF.max_pool1d(x1, 3, 2, 1))
    _close(FF.max_pool3d(x3, 2), TF.max_pool3d(x3, 2))
    _close(FF.avg_pool1d(x1, 3, 2, 1), TF.avg_pool1d(x1, 3, 2, 1))
    _close(FF.avg_pool2d(x2, 3, 2, 1, True, False), TF.avg_pool2d(x2, 3, 2, 1, True, False))
    _close(FF.avg_pool3d(x3, 2, 1), TF.avg_pool3d(x3, 2, 1))
    _close(FF.adaptive_avg_pool1d(x1, 5), TF.adaptive_avg_pool1d(x1, 5))
    _close(FF.adaptive_avg_pool3d(x3, (2, 3, 2)), TF.adaptive_avg_pool3d(x3, (2, 3, 2)))
    _close(FF.adaptive_max_pool1d(x1, 5), TF.adaptive_max_pool1d(x1, 5))
    _close(FF.adaptive_max_pool2d(x2, (4, 3)), TF.adaptive_max_pool2d(x2, (4, 3)))
    _close(FF.adaptive_max_pool3d(x3, 2), TF.adaptive_max_pool3d(x3, 2))
    _close(FF.lp_pool1d(x1.abs(), 2, 3), TF.lp_pool1d(x1.abs(), 2, 3))
    _close(FF.lp_pool2d(x2.abs(), 3, 2), TF.lp_pool2d(x2.abs(), 3, 2))
    v, i = TF.max_pool2d(x2[..., :8, :], 2, return_indices=True)
    _close(FF.max_unpool2d(v, i, 2), TF.max_unpool2d(v, i, 2))
    samples = torch.rand(2, 3, 2)
    _close(FF.fractional_max_pool2d(x2, 2, (4, 4), _random_samples=samples), TF.fractional_max_pool2d(x2, 2, (4, 4), _random_samples=samples))
    t = torch.randn(1, 8, 3, 3)
    _close(FF.pixel_shuffle(t, 2), TF.pixel_shuffle(t, 2))
    cols = FF.unfold(x2, (2, 3), 1, 1, 2)
    _close(cols, TF.unfold(x2, (2, 3), 1, 1, 2))
    _close(FF.fold(cols, (9, 10), (2, 3), 1, 1, 2), TF.fold(cols, (9, 10), (2, 3), 1, 1, 2))
    _close(FF.instance_norm(x2), TF.instance_norm(x2))
    _close(FF.local_response_norm(x2, 3), TF.local_response_norm(x2, 3))
    # the same functions under the package root
    _close(nn.max_pool1d(x1, 2), TF.max_pool1d(x1, 2))
    _close(nn.max_pool3d(x3, 2), TF.max_pool3d(x3, 2))
    _close(nn.avg_pool1d(x1, 2), TF.avg_pool1d(x1, 2))
    _close(nn.avg_pool2d(x2, 2), TF.avg_pool2d(x2, 2))
    _close(nn.avg_pool3d(x3, 2), TF.avg_pool3d(x3, 2))
    _close(nn.adaptive_avg_pool1d(x1, 3), TF.adaptive_avg_pool1d(x1, 3))
    _close(nn.adaptive_avg_pool3d(x3, 1), TF.adaptive_avg_pool3d(x3, 1))
    _close(nn.adaptive_max_pool1d(x1, 3), TF.adaptive_max_pool1d(x1, 3))
    _close(nn.adaptive_max_pool2d(x2, 3), TF.adaptive_max_pool2d(x2, 3))
    _close(nn.adaptive_max_pool3d(x3, 1), TF.adaptive_max_pool3d(x3, 1))
    _close(nn.lp_pool1d(x1.abs(), 2, 2), TF.lp_pool1d(x1.abs(), 2, 2))
    _close(nn.lp_pool2d(x2.abs(), 2, 2), TF.lp_pool2d(x2.abs(), 2, 2))
    _close(nn.max_unpool2d(v, i, 2), TF.max_unpool2d(v, i, 2))
    _close(nn.pixel_shuffle(t, 2), TF.pixel_shuffle(t, 2))
    _close(nn.unfold(x2, 3), TF.unfold(x2, 3))
    _close(nn.fold(nn.unfold(x2, 3), (9, 10), 3), TF.fold(TF.unfold(x2, 3), (9, 10), 3))
    _close(nn.functional_pad_1d(x1, (1, 2), "reflect"), TF.pad(x1, (1, 2), mode="reflect"))
    _close(nn.functional_pad_2d(x2, (1, 2, 0, 1), "replicate"), TF.pad(x2, (1, 2, 0, 1), mode="replicate"))
    _close(nn.functional_pad_3d(x3, (1, 1, 1, 1, 1, 1), "constant", 2.0), TF.pad(x3, (1, 1, 1, 1, 1, 1), value=2.0))


def test_embedding_bag_functional_and_fast_embedding():
    torch.manual_seed(3)
    w = torch.randn(10, 4)
    ids = torch.randint(0, 10, (3, 5))
    _close(FF.embedding_bag(ids, w, mode="sum"), TF.embedding_bag(ids, w, mode="sum"))
    assert FF.embedding_fast is not None and nn.EmbeddingBagMode.Mean.value == "mean"
    _close(nn.EmbeddingBag(10, 4, mode=nn.EmbeddingBagMode.Max, _weight=w.clone())(ids), TF.embedding_bag(ids, w, mode="max"))


def test_lazy_layers_infer_their_input_size():
    assert nn.LazyLinear(7)(torch.randn(3, 5)).shape == (3, 7)
    assert nn.LazyConv1d(4, 3)(torch.randn(2, 6, 9)).shape == (2, 4, 7)
    assert nn.LazyConv3d(4, 2)(torch.randn(1, 3, 4, 4, 4)).shape == (1, 4, 3, 3, 3)
    assert nn.LazyConvTranspose2d(4, 2, stride=2)(torch.randn(1, 3, 4, 4)).shape == (1, 4, 8, 8)
    assert nn.LazyConvTranspose3d(2, 2)(torch.randn(1, 3, 2, 2, 2)).shape == (1, 2, 3, 3, 3)
    b1, b3 = nn.LazyBatchNorm1d(), nn.LazyBatchNorm3d()
    assert b1(torch.randn(4, 6)).shape == (4, 6) and b1.inner.num_features == 6
    assert b3(torch.randn(2, 3, 2, 2, 2)).shape == (2, 3, 2, 2, 2) and b3.inner.num_features == 3


def test_enums_and_configs():
    assert nn.PaddingMode.Reflect.value == "reflect" and nn.PaddingMode.Zeros.value == "constant"
    c = nn.Conv2d(2, 2, 3, padding=1, padding_mode=nn.PaddingMode.Reflect)
    assert c.padding_mode == "reflect"
    assert nn.RNNNonlinearity.ReLU.value == "relu"
    r = nn.RNN(3, 4, nonlinearity=nn.RNNNonlinearity.ReLU)
    assert r.nonlinearity == "relu" and (r(torch.ones(2, 1, 3))[0] >= 0).all()
    assert {m.name for m in nn.NonLinearity} >= {"ReLU", "Tanh"} or len(list(nn.NonLinearity)) > 0
    assert len(list(nn.ObserverType)) >= 2
    cfg = nn.QatConfig()
    assert hasattr(cfg, "__dict__") or cfg is not None
    s = nn.RoPEScaling.linear(2.0)
    assert s.as_dict() == {"type": "linear", "factor": 2.0} and nn.RoPEScaling.none().as_dict() is None
    y = nn.RoPEScaling.yarn(4.0, 2048)
    assert y.as_dict()["original_max_position"] == 2048 and nn.RoPEScaling.ntk_aware(2.0).kind == "ntk"
    assert nn.DeriveModule is nn.derive_module


def test_head_reshapes_kv_cache_and_paged_cache():
    torch.manual_seed(4)
    x = torch.randn(2, 5, 12)
    h = nn.reshape_to_heads(x, 3)
    assert h.shape == (2, 3, 5, 4) and torch.equal(nn.transpose_heads_to_2d(h), x)
    kv = nn.KVCache(2, 3, 8, 4)
    k1, v1 = torch.randn(2, 3, 5, 4), torch.randn(2, 3, 5, 4)
    ka, va = kv.update(k1, v1)
    assert torch.equal(ka, k1) and kv.len == 5
    kb, _ = kv.update(k1[:, :, :3], v1[:, :, :3])
    assert kb.shape[2] == 8 and torch.equal(kb[:, :, 5:], k1[:, :, :3])
    with pytest.raises(InvalidArgument):
        kv.update(k1, v1)
    kv.reset()
    assert kv.len == 0
    pool = nn.PagePool(num_pages=4, page_size=2)
    cache = nn.PagedKVCache(pool, kv_heads=1, head_dim=4)
    cache.add_sequence(0)
    k, v = torch.randn(3, 1, 4), torch.randn(3, 1, 4)
    cache.append(0, k, v)
    assert pool.num_free() == 2 and isinstance(pool.pages[0], nn.KVPage)
    gk, gv = cache.gather(0)
    assert torch.equal(gk, k) and torch.equal(gv, v)
    cache.fork(0, 1)                                # shares both pages; appending to the half-filled one copies it first
    cache.append(1, k[:1], v[:1])
    assert torch.equal(cache.gather(0)[0], k) and torch.equal(cache.gather(1)[0], torch.cat([k, k[:1]]))
    cache.free_sequence(0)
    cache.free_sequence(1)
    assert pool.num_free() == 4


def test_score_mods_and_decoder_stack():
    torch.manual_seed(5)
    q, k, v = torch.randn(1, 2, 4, 8), torch.randn(1, 2, 4, 8), torch.randn(1, 2, 4, 8)
    slopes = torch.tensor([0.5, 0.25])
    out = nn.flex_attention(q, k, v, score_mod=nn.alibi_score_mod(slopes))
    s = (q @ k.transpose(-1, -2)) / 8 ** 0.5
    pos = torch.arange(4)
    dist = (pos[:, None] - pos[None, :]).abs().float()
    _close(out, torch.softmax(s - slopes.view(1, 2, 1, 1) * dist, -1) @ v)
    table = torch.randn(2, 7)                                        # [heads, 2 * max_dist + 1], max_dist 3
    out = nn.flex_attention(q, k, v, score_mod=nn.relative_position_score_mod(table))
    rel = (pos[None, :] - pos[:, None]).clamp(-3, 3) + 3
    _close(out, torch.softmax(s + table[:, rel].unsqueeze(0), -1) @ v)
    layer = nn.TransformerDecoderLayer(8, 2, 16, dropout=0.0, batch_first=True)
    dec = nn.TransformerDecoder(layer, 2)
    y = dec(torch.randn(2, 3, 8), torch.randn(2, 5, 8), tgt_is_causal=True)
    assert y.shape == (2, 3, 8) and len(dec.layers) == 2 and dec.layers[0] is not dec.layers[1]


def test_hooks_and_grad_clipping():
    lin = nn.Linear(3, 2)
    hm = nn.HookedModule(lin)
    seen = []
    h = hm.register_forward_hook_fn(lambda inp, out: seen.append(out.shape))
    assert isinstance(h, nn.HookHandle)
    hm(torch.randn(4, 3))
    h.remove()
    hm(torch.randn(4, 3))
    assert seen == [torch.Size([4, 2])]
    h2 = hm.register_forward_pre_hook_fn(lambda inp: inp * 0)           # the replacement input is used
    assert torch.equal(hm(torch.randn(4, 3)), lin.bias.expand(4, 2))
    h2.remove()
    grads = []
    h3 = hm.register_backward_hook_fn(lambda gi, go: grads.append((gi.shape, go.shape)))
    hm(torch.randn(4, 3, requires_grad=True)).sum().backward()
    h3.remove()
    assert grads == [(torch.Size([4, 3]), torch.Size([4, 2]))]
    p = torch.nn.Parameter(torch.zeros(3))
    p.grad = torch.tensor([-2.0, 0.5, 3.0])
    nn.clip_grad_value_([p], 1.0)
    assert p.grad.tolist() == [-1.0, 0.5, 1.0]
    nn.utils.clip_grad_value_([p], 0.25)
    assert p.grad.abs().max() == 0.25
