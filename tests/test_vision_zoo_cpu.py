"""Vision model zoo against torchvision: identical parameter names and (with the same weights) identical outputs."""
import warnings

import pytest
import torch

torchvision = pytest.importorskip("torchvision")
warnings.filterwarnings("ignore")


def _same(ours, tv, x, atol=1e-5):
    ours.eval()
    tv.eval()
    r = ours.load_state_dict(tv.state_dict(), strict=False)
    assert not r.missing_keys and all("num_batches_tracked" in k for k in r.unexpected_keys), (r.missing_keys[:3], r.unexpected_keys[:3])
    with torch.no_grad():
        a, b = ours(x), tv(x)
    if isinstance(b, dict):
        for k in b:
            assert (a[k] - b[k]).abs().max() < atol, k
    else:
        assert (a - b).abs().max() < atol


def test_classification_backbones_match_torchvision():
    from ferrotorch_b200 import vision as V
    x = torch.randn(1, 3, 96, 96)
    tvm = torchvision.models
    _same(V.mobilenet_v3_small(), tvm.mobilenet_v3_small(), x)
    _same(V.mobilenet_v3_large(), tvm.mobilenet_v3_large(), x)
    _same(V.swin_tiny(), tvm.swin_t(), torch.randn(1, 3, 64, 64))
    _same(V.inception_v3(), tvm.inception_v3(init_weights=False), torch.randn(1, 3, 128, 128))
    assert {"swin_tiny", "fasterrcnn_resnet50_fpn", "deeplabv3_resnet50", "resnet50"} <= set(V.list_models())


def test_segmentation_models_match_torchvision():
    from ferrotorch_b200 import vision as V
    x = torch.randn(1, 3, 64, 64)
    tvs = torchvision.models.segmentation
    _same(V.fcn_resnet50(), tvs.fcn_resnet50(weights=None, weights_backbone=None, aux_loss=True), x)
    _same(V.deeplabv3_resnet50(), tvs.deeplabv3_resnet50(weights=None, weights_backbone=None, aux_loss=True), x)
    _same(V.lraspp_mobilenet_v3_large(), tvs.lraspp_mobilenet_v3_large(weights=None, weights_backbone=None), x)


def test_detection_building_blocks_and_models_match_torchvision():
    from ferrotorch_b200 import vision as V
    from torchvision.models.detection import _utils as tvu
    from torchvision.models.detection import anchor_utils as tva
    torch.manual_seed(0)
    boxes = torch.rand(50, 4) * 50
    boxes[:, 2:] += boxes[:, :2] + 1
    deltas = torch.randn(50, 8) * 0.3
    coder = tvu.BoxCoder((10.0, 10.0, 5.0, 5.0))
    assert torch.allclose(V.decode_boxes(deltas, boxes, (10.0, 10.0, 5.0, 5.0)), coder.decode_single(deltas, boxes).view(50, 2, 4), atol=1e-4)
    gt = boxes + torch.rand(50, 4)
    assert torch.allclose(V.encode_boxes(gt, boxes, (10.0, 10.0, 5.0, 5.0)), coder.encode_single(gt, boxes), atol=1e-5)
    feats = [torch.zeros(1, 8, 16, 20), torch.zeros(1, 8, 8, 10)]
    ag_t = tva.AnchorGenerator(((32,), (64,)), ((0.5, 1.0, 2.0),) * 2)
    from torchvision.models.detection.image_list import ImageList
    ref = ag_t(ImageList(torch.zeros(1, 3, 128, 160), [(128, 160)]), feats)[0]
    assert torch.equal(V.AnchorGenerator(((32,), (64,)), ((0.5, 1.0, 2.0),) * 2)((128, 160), feats), ref)
    tvd = torchvision.models.detection
    imgs = [torch.rand(3, 100, 130), torch.rand(3, 90, 120)]
    kw = dict(weights=None, weights_backbone=None, min_size=128, max_size=160)
    for ours, tv in ((V.fasterrcnn_resnet50_fpn(min_size=128, max_size=160, box_score_thresh=0.0), tvd.fasterrcnn_resnet50_fpn(box_score_thresh=0.0, **kw)),
                     (V.retinanet_resnet50_fpn(min_size=128, max_size=160, score_thresh=0.0), tvd.retinanet_resnet50_fpn(score_thresh=0.0, **kw)),
                     (V.fcos_resnet50_fpn(min_size=128, max_size=160, score_thresh=0.0), tvd.fcos_resnet50_fpn(score_thresh=0.0, **kw))):
        ours.eval()
        tv.eval()
        r = ours.load_state_dict(tv.state_dict(), strict=False)
        assert not r.missing_keys and all("num_batches_tracked" in k for k in r.unexpected_keys)
        with torch.no_grad():
            a, b = ours(imgs), tv(imgs)
        for x, y in zip(a, b):
            assert len(x["boxes"]) == len(y["boxes"]) and (x["scores"] - y["scores"]).abs().max() < 1e-4
            assert (x["boxes"] - y["boxes"]).abs().max() < 1e-2 and torch.equal(x["labels"], y["labels"])
    for ours, tv in ((V.maskrcnn_resnet50_fpn(), tvd.maskrcnn_resnet50_fpn(weights=None, weights_backbone=None)),
                     (V.keypointrcnn_resnet50_fpn(), tvd.keypointrcnn_resnet50_fpn(weights=None, weights_backbone=None)),
                     (V.ssd300_vgg16(), tvd.ssd300_vgg16(weights=None, weights_backbone=None))):
        extra = set(tv.state_dict()) - set(ours.state_dict())
        assert not (set(ours.state_dict()) - set(tv.state_dict())) and all("num_batches_tracked" in k for k in extra)
    masks = V.postprocess_masks(torch.randn(2, 3, 28, 28), torch.tensor([1, 2]), torch.tensor([[10.0, 12.0, 40.0, 50.0], [0.0, 0.0, 20.0, 20.0]]), (64, 64))
    assert masks.shape == (2, 1, 64, 64) and masks.dtype == torch.bool and not masks[0, 0, :5].any()
