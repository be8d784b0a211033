"""Per-symbol behaviour checks of ``ferrotorch_b200.vision`` against torchvision: the remaining classification backbones, box algebra, focal
losses, RoI pooling, detection post-processing, augmentation transforms, raw-image I/O, folder datasets and the model registry."""
import warnings

import pytest
import torch

torchvision = pytest.importorskip("torchvision")
warnings.filterwarnings("ignore")

from ferrotorch_b200 import vision as V  # noqa: E402
from ferrotorch_b200.errors import FerrotorchError  # noqa: E402

tvo = torchvision.ops


def _same(ours, tv, x, atol=2e-5):
    ours.eval(), tv.eval()
    r = ours.load_state_dict(tv.state_dict(), strict=False)
    assert not r.missing_keys and all("num_batches_tracked" in k for k in r.unexpected_keys), (r.missing_keys[:3], r.unexpected_keys[:3])
    with torch.no_grad():
        a, b = ours(x), tv(x)
    assert a.shape == b.shape and (a - b).abs().max() < atol, (a - b).abs().max().item()


@pytest.mark.parametrize("name,tv_name,size", [("resnet34", "resnet34", 64), ("vgg11", "vgg11", 64), ("vgg16", "vgg16", 64), ("mobilenet_v2", "mobilenet_v2", 64),
                                               ("densenet121", "densenet121", 64), ("convnext_tiny", "convnext_tiny", 64),
                                               ("efficientnet_b0", "efficientnet_b0", 64), ("vit_b_16", "vit_b_16", 224)])
def test_classification_backbones_match_torchvision(name, tv_name, size):
    torch.manual_seed(0)
    ours, tv = getattr(V, name)(num_classes=10), getattr(torchvision.models, tv_name)(num_classes=10)
    _same(ours, tv, torch.randn(1, 3, size, size), atol=1e-4)
    cls = {"resnet34": V.ResNet, "vgg11": V.VGG, "vgg16": V.VGG, "mobilenet_v2": V.MobileNetV2, "densenet121": V.DenseNet, "convnext_tiny": V.ConvNeXt,
           "efficientnet_b0": V.EfficientNet, "vit_b_16": V.VisionTransformer}[name]
    assert isinstance(ours, cls)


def test_dilated_resnet_and_block_types():
    m = V.resnet50_dilated(num_classes=5)
    tv = torchvision.models.resnet50(num_classes=5, replace_stride_with_dilation=[False, True, True])
    _same(m, tv, torch.randn(1, 3, 64, 64), atol=1e-4)
    assert isinstance(m.layer1[0], V.Bottleneck) and isinstance(m.layer1[0].conv1, V.Conv1x1)
    small, large = V.mobilenet_v3_small(), V.mobilenet_v3_large()
    assert isinstance(small, V.MobileNetV3) and isinstance(large, V.MobileNetV3) and V.MobileNetV3Small is not None and V.MobileNetV3Large is not None
    for n, cls in (("inception_v3", V.InceptionV3), ("swin_tiny", V.SwinTransformer), ("fcn_resnet50", V.Fcn), ("deeplabv3_resnet50", V.DeepLabV3),
                   ("lraspp_mobilenet_v3_large", V.Lraspp)):
        assert isinstance(getattr(V, n)(), cls)
    d = V.deeplabv3_resnet50()
    assert isinstance(d.classifier, V.DeepLabV3Head) and isinstance(d.classifier[0], V.Aspp)
    y = V.Yolo(num_classes=3, width=8)(torch.randn(1, 3, 64, 64))
    assert (y[0] if isinstance(y, (list, tuple)) else y).shape[0] == 1


def test_detection_model_types():
    kw = dict(min_size=64, max_size=96)
    assert isinstance(V.fasterrcnn_resnet50_fpn(**kw), V.FasterRcnn) and isinstance(V.retinanet_resnet50_fpn(**kw), V.RetinaNet)
    assert isinstance(V.fcos_resnet50_fpn(**kw), V.Fcos) and isinstance(V.ssd300_vgg16(), V.Ssd300)
    mk, kp = V.maskrcnn_resnet50_fpn(), V.keypointrcnn_resnet50_fpn()
    assert isinstance(mk, V.MaskRcnn) and isinstance(kp, V.KeypointRcnn) and any(isinstance(m, V.MaskHead) for m in mk.modules())
    fpn = V.FeaturePyramidNetwork([8, 16], 4)
    tv = tvo.FeaturePyramidNetwork([8, 16], 4)
    fpn.load_state_dict(tv.state_dict())
    from collections import OrderedDict
    feats = OrderedDict([("0", torch.randn(1, 8, 16, 16)), ("1", torch.randn(1, 16, 8, 8))])
    a, b = fpn(feats), tv(feats)
    assert all(torch.allclose(a[k], b[k], atol=1e-5) for k in b)
    assert V.SsdDetections is not None


def test_box_algebra_matches_torchvision():
    torch.manual_seed(1)
    a = torch.rand(20, 4) * 50
    a[:, 2:] += a[:, :2] + 0.5
    b = torch.rand(15, 4) * 50
    b[:, 2:] += b[:, :2] + 0.5
    assert torch.allclose(V.box_area(a), tvo.box_area(a))
    assert torch.allclose(V.box_iou(a, b), tvo.box_iou(a, b), atol=1e-6)
    assert torch.allclose(V.generalized_box_iou(a, b), tvo.generalized_box_iou(a, b), atol=1e-6)
    assert torch.allclose(V.distance_box_iou(a, b), tvo.distance_box_iou(a, b), atol=1e-5)
    assert torch.allclose(V.complete_box_iou(a, b), tvo.complete_box_iou(a, b), atol=1e-5)
    for i, o in (("xyxy", "cxcywh"), ("xyxy", "xywh"), ("cxcywh", "xyxy"), ("xywh", "cxcywh")):
        assert torch.allclose(V.box_convert(a, i, o), tvo.box_convert(a, i, o), atol=1e-5)
    assert torch.equal(V.clip_boxes_to_image(a - 10, (30, 40)), tvo.clip_boxes_to_image(a - 10, (30, 40)))
    assert torch.equal(V.remove_small_boxes(a, 20.0), tvo.remove_small_boxes(a, 20.0))
    feat = torch.randn(2, 4, 16, 16)
    rois = torch.tensor([[0, 1.0, 2.0, 9.0, 12.0], [1, 0.0, 0.0, 15.0, 15.0], [0, 4.0, 4.0, 6.0, 5.0]])
    assert torch.allclose(V.roi_pool(feat, rois, (3, 3), 1.0), tvo.roi_pool(feat, rois, (3, 3), 1.0), atol=1e-6)
    assert torch.allclose(V.roi_pool(feat, rois, 2, 0.5), tvo.roi_pool(feat, rois, 2, 0.5), atol=1e-6)


def test_focal_losses_and_postprocessing():
    torch.manual_seed(2)
    x, t = torch.randn(6, 5), torch.randint(0, 2, (6, 5)).float()
    for red in ("none", "mean", "sum"):
        assert torch.allclose(V.sigmoid_focal_loss(x, t, 0.25, 2.0, red), tvo.sigmoid_focal_loss(x, t, 0.25, 2.0, red), atol=1e-6)
    y = torch.randint(0, 5, (6,))
    logp = torch.log_softmax(x, 1).gather(1, y[:, None]).squeeze(1)
    ref = (-(1 - logp.exp()) ** 2 * logp).mean()
    assert torch.allclose(V.focal_loss(x, y, 2.0), ref, atol=1e-6)
    assert torch.allclose(V.focal_loss(x, y, 0.0), torch.nn.functional.cross_entropy(x, y), atol=1e-6)
    props = [torch.tensor([[10.0, 10.0, 30.0, 30.0], [20.0, 20.0, 40.0, 40.0]])]
    logits = torch.tensor([[0.0, 5.0, 0.0], [0.0, 0.0, 5.0]])
    out = V.postprocess_detections(logits, torch.zeros(2, 12), props, [(50, 50)], score_thresh=0.5)
    (boxes, scores, labels, rows), = out                                # per image: boxes, scores, labels, proposal row of each detection
    assert sorted(labels.tolist()) == [1, 2] and torch.allclose(boxes.sort(0).values, props[0], atol=1e-4) and (scores > 0.9).all()
    assert sorted(rows.tolist()) == [0, 1]


def test_augmentation_transforms_keep_shape_and_range():
    torch.manual_seed(3)
    img = torch.rand(3, 32, 40)
    assert torch.equal(V.RandomVerticalFlip(1.0)(img), img.flip(-2)) and torch.equal(V.RandomVerticalFlip(0.0)(img), img)
    assert V.RandomResizedCrop(16)(img).shape == (3, 16, 16)
    assert torch.allclose(V.RandomRotation(0.0)(img), img, atol=1e-5) and V.RandomRotation(30.0)(img).shape == img.shape
    blurred = V.RandomGaussianBlur(5, (1.0, 1.0), p=1.0)(img)
    assert blurred.shape == img.shape and blurred.var() < img.var()
    assert torch.equal(V.RandomApply([lambda t: t * 0], p=0.0)(img), img) and V.RandomApply([lambda t: t * 0], p=1.0)(img).abs().sum() == 0
    e = V.ElasticTransform(5.0, 3.0)(img)
    assert e.shape == img.shape and 0.0 <= e.min() and e.max() <= 1.0 + 1e-5
    t = V.TrivialAugmentWide()(img)
    assert t.shape == img.shape and torch.isfinite(t).all()


def test_raw_images_folders_and_registry(tmp_path):
    raw = V.RawImage(bytes(range(24)), width=4, height=2, channels=3)
    t = V.raw_image_to_tensor(raw)
    assert t.shape == (3, 2, 4)
    back = V.tensor_to_raw_image(t)
    assert (back.width, back.height, back.channels) == (4, 2, 3) and back.data == raw.data
    p = tmp_path / "img.ppm"
    V.write_raw_image(p, raw)
    again = V.read_image_raw(p)
    assert again.data == raw.data and again.width == 4
    for cls_name, k in (("cat", 2), ("dog", 1)):
        (tmp_path / "ds" / cls_name).mkdir(parents=True)
        for i in range(k):
            V.write_raw_image(tmp_path / "ds" / cls_name / f"{i}.ppm", raw)
    ds = V.ImageFolder(tmp_path / "ds")
    assert isinstance(ds, V.DatasetFolder) and len(ds) == 3 and ds.classes == ["cat", "dog"] and ds[2][1] == 1 and ds[0][0].shape == (3, 2, 4)
    c = V.Cifar100(torch.zeros(5, 3, 32, 32, dtype=torch.uint8), torch.arange(5))
    assert len(c) == 5 and c[3][1] == 3
    V.register_model("unit_test_tiny_vgg", lambda num_classes=3: V.VGG(11, num_classes))
    assert "unit_test_tiny_vgg" in V.list_models() and isinstance(V.get_model("unit_test_tiny_vgg", num_classes=3), V.VGG)
    reg = V.ModelRegistry()
    reg.register("m", lambda: 7)
    assert reg.names() == ["m"] and reg.get("m") == 7
    with pytest.raises(FerrotorchError):
        V.get_model("no_such_model")
