"""Semantic segmentation heads on the classification backbones, torchvision parameter names: FCN, DeepLabV3 (ASPP), LR-ASPP.

Reference parity: ferrotorch-vision/src/models/{fcn.rs:177,338, deeplabv3.rs:363,487, aspp.rs:361, lraspp.rs:315,498}.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, Optional

import torch
import torch.nn.functional as F

from .. import nn
from . import models as M
from . import models2 as M2


class _ResNetBody(nn.Module):
    """ResNet trunk returning the ``layer3`` ("aux") and ``layer4`` ("out") feature maps; parameter names as in the full model."""

    def __init__(self, net: M.ResNet):
        super().__init__()
        for n in ("conv1", "bn1", "relu", "maxpool", "layer1", "layer2", "layer3", "layer4"):
            setattr(self, n, getattr(net, n))

    def forward(self, x) -> Dict[str, torch.Tensor]:
        x = M.max_pool(M.bn_act(self.bn1, self.conv1(x)), 3, 2, 1)
        x = self.layer2(self.layer1(x))
        aux = self.layer3(x)
        return {"aux": aux, "out": self.layer4(aux)}


class FCNHead(nn.Sequential):
    def __init__(self, cin, channels):
        inter = cin // 4
        super().__init__(nn.Conv2d(cin, inter, 3, padding=1, bias=False), nn.BatchNorm2d(inter), nn.ReLU(), nn.Dropout(0.1), nn.Conv2d(inter, channels, 1))


class _ASPPConv(nn.Sequential):
    def __init__(self, cin, cout, dilation):
        super().__init__(nn.Conv2d(cin, cout, 3, padding=dilation, dilation=dilation, bias=False), nn.BatchNorm2d(cout), nn.ReLU())


class _ASPPPooling(nn.Sequential):
    def __init__(self, cin, cout):
        super().__init__(nn.AdaptiveAvgPool2d(1), nn.Conv2d(cin, cout, 1, bias=False), nn.BatchNorm2d(cout), nn.ReLU())

    def forward(self, x):
        size = x.shape[-2:]
        return F.interpolate(super().forward(x), size=size, mode="bilinear", align_corners=False)


class Aspp(nn.Module):
    """Atrous spatial pyramid pooling: 1x1 branch, three dilated 3x3 branches, image pooling branch, projection."""

    def __init__(self, cin, rates=(12, 24, 36), cout=256):
        super().__init__()
        mods = [nn.Sequential(nn.Conv2d(cin, cout, 1, bias=False), nn.BatchNorm2d(cout), nn.ReLU())]
        mods += [_ASPPConv(cin, cout, r) for r in rates]
        mods.append(_ASPPPooling(cin, cout))
        self.convs = nn.ModuleList(mods)
        self.project = nn.Sequential(nn.Conv2d(len(mods) * cout, cout, 1, bias=False), nn.BatchNorm2d(cout), nn.ReLU(), nn.Dropout(0.5))

    def forward(self, x):
        return self.project(torch.cat([c(x) for c in self.convs], 1))


class DeepLabHead(nn.Sequential):
    def __init__(self, cin, num_classes):
        super().__init__(Aspp(cin), nn.Conv2d(256, 256, 3, padding=1, bias=False), nn.BatchNorm2d(256), nn.ReLU(), nn.Conv2d(256, num_classes, 1))


class _SegModel(nn.Module):
    def __init__(self, backbone, classifier, aux_classifier=None):
        super().__init__()
        self.backbone, self.classifier, self.aux_classifier = backbone, classifier, aux_classifier

    def forward(self, x) -> "OrderedDict[str, torch.Tensor]":
        size = x.shape[-2:]
        f = self.backbone(x)
        out = OrderedDict(out=F.interpolate(self.classifier(f["out"]), size=size, mode="bilinear", align_corners=False))
        if self.aux_classifier is not None:
            out["aux"] = F.interpolate(self.aux_classifier(f["aux"]), size=size, mode="bilinear", align_corners=False)
        return out


class Fcn(_SegModel):
    pass


class DeepLabV3(_SegModel):
    pass


FcnHead, DeepLabV3Head = FCNHead, DeepLabHead                 # ferrotorch-vision/src/models/segmentation/{fcn.rs, deeplabv3.rs}


class ResNet50Dilated(_ResNetBody):
    """ResNet-50 trunk with layers 3 and 4 dilated instead of strided (output stride 8); ``forward`` returns ``{"aux": layer3, "out": layer4}``
    (ferrotorch-vision/src/models/segmentation/backbone.rs)."""

    def __init__(self):
        super().__init__(M.ResNet(M.Bottleneck, [3, 4, 6, 3], replace_stride_with_dilation=(False, True, True)))


def _dilated_resnet50():
    return _ResNetBody(M.ResNet(M.Bottleneck, [3, 4, 6, 3], replace_stride_with_dilation=(False, True, True)))


def fcn_resnet50(num_classes: int = 21, aux_loss: bool = True) -> Fcn:
    return Fcn(_dilated_resnet50(), FCNHead(2048, num_classes), FCNHead(1024, num_classes) if aux_loss else None)


def deeplabv3_resnet50(num_classes: int = 21, aux_loss: bool = True) -> DeepLabV3:
    return DeepLabV3(_dilated_resnet50(), DeepLabHead(2048, num_classes), FCNHead(1024, num_classes) if aux_loss else None)


class _MNV3Body(nn.Module):
    """MobileNetV3 features returning the stride-8 ("low") and the final ("high") maps; modules are numbered as in ``features``."""

    def __init__(self, features: torch.nn.Sequential, low_idx: int):
        super().__init__()
        for i, m in enumerate(features):
            self.add_module(str(i), m)
        self.low_idx, self.n = low_idx, len(features)

    def forward(self, x):
        out = {}
        for i in range(self.n):
            x = getattr(self, str(i))(x)
            if i == self.low_idx:
                out["low"] = x
        out["high"] = x
        return out


class LrasppHead(nn.Module):
    def __init__(self, low, high, num_classes, inter):
        super().__init__()
        self.cbr = nn.Sequential(nn.Conv2d(high, inter, 1, bias=False), nn.BatchNorm2d(inter), nn.ReLU())
        self.scale = nn.Sequential(nn.AdaptiveAvgPool2d(1), nn.Conv2d(high, inter, 1, bias=False), nn.Sigmoid())
        self.low_classifier, self.high_classifier = nn.Conv2d(low, num_classes, 1), nn.Conv2d(inter, num_classes, 1)

    def forward(self, f):
        x = self.cbr(f["high"]) * self.scale(f["high"])
        x = F.interpolate(x, size=f["low"].shape[-2:], mode="bilinear", align_corners=False)
        return self.low_classifier(f["low"]) + self.high_classifier(x)


class Lraspp(nn.Module):
    def __init__(self, backbone, low, high, num_classes, inter=128):
        super().__init__()
        self.backbone, self.classifier = backbone, LrasppHead(low, high, num_classes, inter)

    def forward(self, x):
        return OrderedDict(out=F.interpolate(self.classifier(self.backbone(x)), size=x.shape[-2:], mode="bilinear", align_corners=False))


def lraspp_mobilenet_v3_large(num_classes: int = 21) -> Lraspp:
    net = M2.mobilenet_v3_large(dilated=True)
    return Lraspp(_MNV3Body(net.features, 4), 40, 960, num_classes)
