"""Classification backbones: ResNet-18/34/50 (+dilated), VGG-11/16, ViT-B/16, MobileNetV2, DenseNet-121, ConvNeXt-Tiny,
EfficientNet-B0, U-Net and a compact YOLO-style detector head, plus the model registry and a feature extractor.

Architectures (layer structure, parameter names and counts) follow torchvision's definitions so pretrained state dicts load
unchanged. 1x1 convolutions on bf16 channels-last CUDA tensors run on the tcgen05 GEMM (a 1x1 convolution over NHWC data is
exactly ``[N*H*W, Cin] x [Cout, Cin]^T``); other kernel sizes use the framework's Conv2d.

Reference parity: ferrotorch-vision/src/models/{resnet.rs:100-1066, vgg.rs, vit.rs, mobilenet.rs, densenet.rs, convnext.rs,
efficientnet.rs, unet.rs, yolo.rs, registry.rs:75-442, feature_extractor.rs:136}.
"""
from __future__ import annotations

import math
from collections import OrderedDict
from functools import partial
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from .. import nn, ops
from ..errors import InvalidArgument
from ..nn.compute_copy import compute_copy


def _autocast_bf16() -> bool:
    return torch.is_autocast_enabled() and torch.get_autocast_dtype("cuda") == torch.bfloat16


class Conv1x1(nn.Conv2d):
    """1x1 convolution; bf16 channels-last CUDA inputs are evaluated as one GEMM over the pixel rows (stride handled by subsampling)."""

    def __init__(self, cin: int, cout: int, stride: int = 1, bias: bool = False):
        super().__init__(cin, cout, 1, stride, 0, bias=bias)

    def forward(self, x):
        w = self.weight
        wc = compute_copy(w) if (x.is_cuda and w.dtype == torch.float32 and _autocast_bf16()) else None
        if wc is not None and wc.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and self.out_channels % 8 == 0:
            # bf16 copy kept current by the optimizer: no cast launch here, f32 weight gradient straight from the GEMM
            x = x.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
            if self.stride[0] > 1:
                x = x[:, :, :: self.stride[0], :: self.stride[1]].contiguous(memory_format=torch.channels_last)
            N, C, H, W = x.shape
            rows = x.permute(0, 2, 3, 1).reshape(N * H * W, C)
            y = ops.linear_master(rows, w, wc, None if self.bias is None else self.bias.to(torch.bfloat16))
            return y.view(N, H, W, self.out_channels).permute(0, 3, 1, 2)
        if x.is_cuda and torch.is_autocast_enabled() and torch.get_autocast_dtype("cuda") == torch.bfloat16:
            x, w = x.to(torch.bfloat16), w.to(torch.bfloat16)        # autocast policy: convolutions run in the reduced dtype
        if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and self.out_channels % 8 == 0 \
                and x.is_contiguous(memory_format=torch.channels_last):
            if self.stride[0] > 1:
                x = x[:, :, :: self.stride[0], :: self.stride[1]].contiguous(memory_format=torch.channels_last)
            N, C, H, W = x.shape
            rows = x.permute(0, 2, 3, 1).reshape(N * H * W, C)
            y = ops.linear(rows, w.view(self.out_channels, C), None if self.bias is None else self.bias.to(torch.bfloat16))
            return y.view(N, H, W, self.out_channels).permute(0, 3, 1, 2)
        return super().forward(x)


def bn_act(bn: "nn.BatchNorm2d", x: torch.Tensor, residual: Optional[torch.Tensor] = None, relu: bool = True) -> torch.Tensor:
    """BatchNorm (+ residual add) (+ ReLU). Channels-last CUDA f32/bf16 activations take the fused two-stage-statistics kernels; everything else
    (CPU, NCHW, SyncBatchNorm subclasses with their own forward) the module's own path."""
    sync = hasattr(bn, "_reducer")                  # SyncBatchNorm2d: same kernels, the two small sums reduced over the group
    fused = ((sync or type(bn).forward in (nn.BatchNorm2d.forward, torch.nn.BatchNorm2d.forward)) and x.is_cuda and x.dim() == 4
             and x.dtype in (torch.float32, torch.bfloat16) and x.shape[1] % 8 == 0 and x.is_contiguous(memory_format=torch.channels_last)
             and bn.affine and bn.track_running_stats and bn.momentum is not None
             and (residual is None or (residual.dtype == x.dtype and residual.is_contiguous(memory_format=torch.channels_last))))
    if not fused:
        out = bn(x)
        if residual is not None:
            out = out + residual
        return torch.relu(out) if relu else out
    group = None
    if sync and bn.training:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(bn.pg) > 1:
            group = bn._reducer(x.device)
    if bn.training and bn.num_batches_tracked is not None:
        bn.num_batches_tracked.add_(1)
    return ops.nn_ops.batch_norm_nhwc(x, bn.weight, bn.bias, bn.running_mean, bn.running_var, residual=residual, relu=relu, training=bn.training,
                                      momentum=bn.momentum, eps=bn.eps, group=group)


def max_pool(x: torch.Tensor, k: int, s: int, p: int) -> torch.Tensor:
    if x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and x.shape[1] % 8 == 0 and x.is_contiguous(memory_format=torch.channels_last):
        return ops.nn_ops.max_pool2d_nhwc(x, k, s, p)
    return F.max_pool2d(x, k, s, p)


class Conv3x3(nn.Conv2d):
    """3x3 convolution; stride-1 bf16 channels-last CUDA inputs (autocast included) run on the implicit-GEMM tcgen05 kernel."""

    def __init__(self, cin, cout, stride=1, groups=1, dilation=1):
        super().__init__(cin, cout, 3, stride, dilation, dilation, groups, bias=False)

    def forward(self, x):
        if x.is_cuda and torch.is_autocast_enabled() and torch.get_autocast_dtype("cuda") == torch.bfloat16 and x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)
        if ops.conv.conv3x3_rows_eligible(x, self.weight, self.stride, self.padding, self.dilation, self.groups):
            return ops.conv.conv3x3_autograd_rows(x, self.weight, self.stride[0])          # opt-in: every pass on the GEMM's row-shift tables
        if ops.conv.conv3x3_eligible(x, self.weight, self.stride, self.padding, self.dilation, self.groups):
            wc = compute_copy(self.weight) if self.weight.dtype == torch.float32 else None
            if wc is not None and wc.dtype == torch.bfloat16:
                return ops.conv.conv3x3_master(x, self.weight, wc)
            return ops.conv3x3(x, self.weight)
        return super().forward(x)


def conv3x3(cin, cout, stride=1, groups=1, dilation=1):
    return Conv3x3(cin, cout, stride, groups, dilation)


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, inplanes, planes, stride=1, downsample=None, dilation=1):
        super().__init__()
        self.conv1, self.bn1 = conv3x3(inplanes, planes, stride), nn.BatchNorm2d(planes)
        self.relu = nn.ReLU(inplace=True)
        self.conv2, self.bn2 = conv3x3(planes, planes), nn.BatchNorm2d(planes)
        self.downsample = downsample

    def forward(self, x):
        idt = x if self.downsample is None else bn_act(self.downsample[1], self.downsample[0](x), relu=False)
        out = bn_act(self.bn1, self.conv1(x))
        return bn_act(self.bn2, self.conv2(out), residual=idt)


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, inplanes, planes, stride=1, downsample=None, dilation=1):
        super().__init__()
        self.conv1, self.bn1 = Conv1x1(inplanes, planes), nn.BatchNorm2d(planes)
        self.conv2, self.bn2 = conv3x3(planes, planes, stride, dilation=dilation), nn.BatchNorm2d(planes)
        self.conv3, self.bn3 = Conv1x1(planes, planes * 4), nn.BatchNorm2d(planes * 4)
        self.relu = nn.ReLU(inplace=True)
        self.downsample = downsample

    def forward(self, x):
        idt = x if self.downsample is None else bn_act(self.downsample[1], self.downsample[0](x), relu=False)
        out = bn_act(self.bn1, self.conv1(x))
        out = bn_act(self.bn2, self.conv2(out))
        return bn_act(self.bn3, self.conv3(out), residual=idt)


class ResNet(nn.Module):
    def __init__(self, block, layers: Sequence[int], num_classes: int = 1000, replace_stride_with_dilation=(False, False, False), zero_init_residual: bool = False):
        super().__init__()
        self.inplanes, self.dilation = 64, 1
        self.conv1 = nn.Conv2d(3, 64, 7, 2, 3, bias=False)
        self.bn1, self.relu = nn.BatchNorm2d(64), nn.ReLU(inplace=True)
        self.maxpool = nn.MaxPool2d(3, 2, 1)
        self.layer1 = self._make(block, 64, layers[0])
        self.layer2 = self._make(block, 128, layers[1], 2, replace_stride_with_dilation[0])
        self.layer3 = self._make(block, 256, layers[2], 2, replace_stride_with_dilation[1])
        self.layer4 = self._make(block, 512, layers[3], 2, replace_stride_with_dilation[2])
        self.avgpool = nn.AdaptiveAvgPool2d(1)
        self.fc = nn.Linear(512 * block.expansion, num_classes)
        for m in self.modules():
            if isinstance(m, (nn.Conv2d, torch.nn.Conv2d)):
                torch.nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
            elif isinstance(m, (nn.BatchNorm2d, torch.nn.BatchNorm2d)):
                torch.nn.init.ones_(m.weight)
                torch.nn.init.zeros_(m.bias)
        if zero_init_residual:
            for m in self.modules():
                if isinstance(m, Bottleneck):
                    torch.nn.init.zeros_(m.bn3.weight)
                elif isinstance(m, BasicBlock):
                    torch.nn.init.zeros_(m.bn2.weight)

    def _make(self, block, planes, blocks, stride=1, dilate=False):
        prev_dil = self.dilation
        if dilate:
            self.dilation *= stride
            stride = 1
        down = None
        if stride != 1 or self.inplanes != planes * block.expansion:
            down = nn.Sequential(Conv1x1(self.inplanes, planes * block.expansion, stride), nn.BatchNorm2d(planes * block.expansion))
        layers = [block(self.inplanes, planes, stride, down, prev_dil)]
        self.inplanes = planes * block.expansion
        layers += [block(self.inplanes, planes, dilation=self.dilation) for _ in range(1, blocks)]
        return nn.Sequential(*layers)

    def features(self, x):
        x = max_pool(bn_act(self.bn1, self.conv1(x)), 3, 2, 1)
        return self.layer4(self.layer3(self.layer2(self.layer1(x))))

    def forward(self, x):
        x = self.avgpool(self.features(x)).flatten(1)
        return self.fc(x)


def resnet18(num_classes=1000):
    return ResNet(BasicBlock, [2, 2, 2, 2], num_classes)


def resnet34(num_classes=1000):
    return ResNet(BasicBlock, [3, 4, 6, 3], num_classes)


def resnet50(num_classes=1000, zero_init_residual=False):
    return ResNet(Bottleneck, [3, 4, 6, 3], num_classes, zero_init_residual=zero_init_residual)


def resnet50_dilated(num_classes=1000):
    return ResNet(Bottleneck, [3, 4, 6, 3], num_classes, (False, True, True))


# -- VGG -------------------------------------------------------------------------------------------------------------------------
_VGG = {11: [64, "M", 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
        16: [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"]}


class VGG(nn.Module):
    def __init__(self, depth: int = 16, num_classes: int = 1000, batch_norm: bool = False, dropout: float = 0.5):
        super().__init__()
        layers, c = [], 3
        for v in _VGG[depth]:
            if v == "M":
                layers.append(nn.MaxPool2d(2, 2))
            else:
                layers += [nn.Conv2d(c, v, 3, padding=1)] + ([nn.BatchNorm2d(v)] if batch_norm else []) + [nn.ReLU(inplace=True)]
                c = v
        self.features = nn.Sequential(*layers)
        self.avgpool = nn.AdaptiveAvgPool2d(7)
        self.classifier = nn.Sequential(nn.Linear(512 * 49, 4096), nn.ReLU(True), nn.Dropout(dropout), nn.Linear(4096, 4096), nn.ReLU(True),
                                        nn.Dropout(dropout), nn.Linear(4096, num_classes))

    def forward(self, x):
        return self.classifier(self.avgpool(self.features(x)).flatten(1))


def vgg11(num_classes=1000):
    return VGG(11, num_classes)


def vgg16(num_classes=1000):
    return VGG(16, num_classes)


# -- ViT -------------------------------------------------------------------------------------------------------------------------
class _PackedSelfAttention(nn.Module):
    """Self-attention with the packed ``in_proj_weight [3E, E]`` / ``in_proj_bias`` / ``out_proj`` parameter layout of published ViT
    checkpoints. One GEMM produces q, k, v; the attention itself is :func:`nn.flash_attention` (the tcgen05 kernels for bf16 CUDA inputs)."""

    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.dim, self.heads = dim, heads
        self.in_proj_weight = nn.Parameter(torch.empty(3 * dim, dim))
        self.in_proj_bias = nn.Parameter(torch.zeros(3 * dim))
        self.out_proj = nn.Linear(dim, dim)
        torch.nn.init.xavier_uniform_(self.in_proj_weight)

    def forward(self, x):
        B, S, E = x.shape
        qkv = ops.linear(x, self.in_proj_weight, self.in_proj_bias).view(B, S, 3, self.heads, E // self.heads)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        o = nn.flash_attention(q, k, v)
        return self.out_proj(o.transpose(1, 2).reshape(B, S, E))


class _EncoderBlock(nn.Module):
    def __init__(self, dim, heads, mlp_dim, dropout=0.0):
        super().__init__()
        self.ln_1 = nn.LayerNorm(dim, eps=1e-6)
        self.self_attention = _PackedSelfAttention(dim, heads)
        self.dropout = nn.Dropout(dropout)
        self.ln_2 = nn.LayerNorm(dim, eps=1e-6)
        self.mlp = nn.Sequential(nn.Linear(dim, mlp_dim), nn.GELU(), nn.Dropout(dropout), nn.Linear(mlp_dim, dim), nn.Dropout(dropout))

    def forward(self, x):
        x = x + self.dropout(self.self_attention(self.ln_1(x)))
        return x + self.mlp(self.ln_2(x))


class _ViTEncoder(nn.Module):
    def __init__(self, seq_len, num_layers, num_heads, hidden_dim, mlp_dim, dropout=0.0):
        super().__init__()
        self.pos_embedding = nn.Parameter(torch.empty(1, seq_len, hidden_dim).normal_(std=0.02))
        self.dropout = nn.Dropout(dropout)
        self.layers = nn.Sequential(OrderedDict((f"encoder_layer_{i}", _EncoderBlock(hidden_dim, num_heads, mlp_dim, dropout)) for i in range(num_layers)))
        self.ln = nn.LayerNorm(hidden_dim, eps=1e-6)

    def forward(self, x):
        return self.ln(self.layers(self.dropout(x + self.pos_embedding)))


class VisionTransformer(nn.Module):
    """ViT with the module tree of the published checkpoints: ``conv_proj``, ``class_token``, ``encoder.{pos_embedding, layers.encoder_layer_N, ln}``,
    ``heads.head``."""

    def __init__(self, image_size=224, patch_size=16, num_layers=12, num_heads=12, hidden_dim=768, mlp_dim=3072, num_classes=1000):
        super().__init__()
        self.patch_size, self.hidden_dim = patch_size, hidden_dim
        self.conv_proj = nn.Conv2d(3, hidden_dim, patch_size, patch_size)
        n = (image_size // patch_size) ** 2 + 1
        self.class_token = nn.Parameter(torch.zeros(1, 1, hidden_dim))
        self.encoder = _ViTEncoder(n, num_layers, num_heads, hidden_dim, mlp_dim)
        self.heads = nn.Sequential(OrderedDict([("head", nn.Linear(hidden_dim, num_classes))]))

    def forward(self, x):
        x = self.conv_proj(x).flatten(2).transpose(1, 2)
        x = torch.cat([self.class_token.expand(x.shape[0], -1, -1).to(x.dtype), x], 1)
        return self.heads(self.encoder(x)[:, 0])


def vit_b_16(num_classes=1000, image_size=224):
    return VisionTransformer(image_size, 16, 12, 12, 768, 3072, num_classes)


# -- MobileNetV2 ----------------------------------------------------------------------------------------------------------------------
def _cbr(cin, cout, k=3, s=1, g=1, act=nn.ReLU6):
    return nn.Sequential(nn.Conv2d(cin, cout, k, s, (k - 1) // 2, groups=g, bias=False), nn.BatchNorm2d(cout), act(inplace=True))


class InvertedResidual(nn.Module):
    def __init__(self, cin, cout, stride, expand):
        super().__init__()
        hid = int(round(cin * expand))
        self.use_res = stride == 1 and cin == cout
        layers = ([_cbr(cin, hid, 1)] if expand != 1 else []) + [_cbr(hid, hid, 3, stride, hid), nn.Conv2d(hid, cout, 1, bias=False), nn.BatchNorm2d(cout)]
        self.conv = nn.Sequential(*layers)

    def forward(self, x):
        return x + self.conv(x) if self.use_res else self.conv(x)


class MobileNetV2(nn.Module):
    def __init__(self, num_classes=1000, width=1.0):
        super().__init__()
        cfg = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]
        c = int(32 * width)
        feats = [_cbr(3, c, 3, 2)]
        for t, ch, n, s in cfg:
            oc = int(ch * width)
            for i in range(n):
                feats.append(InvertedResidual(c, oc, s if i == 0 else 1, t))
                c = oc
        self.last = int(1280 * max(1.0, width))
        feats.append(_cbr(c, self.last, 1))
        self.features = nn.Sequential(*feats)
        self.classifier = nn.Sequential(nn.Dropout(0.2), nn.Linear(self.last, num_classes))

    def forward(self, x):
        return self.classifier(F.adaptive_avg_pool2d(self.features(x), 1).flatten(1))


def mobilenet_v2(num_classes=1000):
    return MobileNetV2(num_classes)


# -- DenseNet ---------------------------------------------------------------------------------------------------------------------------
class _DenseLayer(nn.Module):
    def __init__(self, cin, growth, bn_size):
        super().__init__()
        self.norm1, self.relu1, self.conv1 = nn.BatchNorm2d(cin), nn.ReLU(inplace=True), nn.Conv2d(cin, bn_size * growth, 1, bias=False)
        self.norm2, self.relu2, self.conv2 = nn.BatchNorm2d(bn_size * growth), nn.ReLU(inplace=True), nn.Conv2d(bn_size * growth, growth, 3, padding=1, bias=False)

    def forward(self, xs):
        x = torch.cat(xs, 1) if isinstance(xs, list) else xs
        return self.conv2(self.relu2(self.norm2(self.conv1(self.relu1(self.norm1(x))))))


class _DenseBlock(torch.nn.ModuleDict):
    def __init__(self, n, cin, bn_size, growth):
        super().__init__()
        for i in range(n):
            self[f"denselayer{i + 1}"] = _DenseLayer(cin + i * growth, growth, bn_size)

    def forward(self, x):
        feats = [x]
        for l in self.values():
            feats.append(l(feats))
        return torch.cat(feats, 1)


class DenseNet(nn.Module):
    def __init__(self, growth=32, blocks=(6, 12, 24, 16), init=64, bn_size=4, num_classes=1000):
        super().__init__()
        f = OrderedDict([("conv0", nn.Conv2d(3, init, 7, 2, 3, bias=False)), ("norm0", nn.BatchNorm2d(init)), ("relu0", nn.ReLU(inplace=True)),
                         ("pool0", nn.MaxPool2d(3, 2, 1))])
        c = init
        for i, n in enumerate(blocks):
            f[f"denseblock{i + 1}"] = _DenseBlock(n, c, bn_size, growth)
            c += n * growth
            if i != len(blocks) - 1:
                f[f"transition{i + 1}"] = nn.Sequential(OrderedDict([("norm", nn.BatchNorm2d(c)), ("relu", nn.ReLU(inplace=True)),
                                                                      ("conv", nn.Conv2d(c, c // 2, 1, bias=False)), ("pool", nn.AvgPool2d(2, 2))]))
                c //= 2
        f["norm5"] = nn.BatchNorm2d(c)
        self.features = nn.Sequential(f)
        self.classifier = nn.Linear(c, num_classes)

    def forward(self, x):
        return self.classifier(F.adaptive_avg_pool2d(F.relu(self.features(x)), 1).flatten(1))


def densenet121(num_classes=1000):
    return DenseNet(num_classes=num_classes)


# -- ConvNeXt ---------------------------------------------------------------------------------------------------------------------------
class _LayerNorm2d(nn.LayerNorm):
    def forward(self, x):
        return F.layer_norm(x.permute(0, 2, 3, 1), self.normalized_shape, self.weight, self.bias, self.eps).permute(0, 3, 1, 2)


class _CNBlock(nn.Module):
    def __init__(self, dim, layer_scale=1e-6):
        super().__init__()
        self.block = nn.Sequential(nn.Conv2d(dim, dim, 7, padding=3, groups=dim), _Permute(0, 2, 3, 1), nn.LayerNorm(dim, eps=1e-6), nn.Linear(dim, 4 * dim),
                                   nn.GELU(), nn.Linear(4 * dim, dim), _Permute(0, 3, 1, 2))
        self.layer_scale = nn.Parameter(torch.ones(dim, 1, 1) * layer_scale)

    def forward(self, x):
        return x + self.layer_scale * self.block(x)


class _Permute(nn.Module):
    def __init__(self, *dims):
        super().__init__()
        self.dims = dims

    def forward(self, x):
        return x.permute(*self.dims)


class ConvNeXt(nn.Module):
    def __init__(self, depths=(3, 3, 9, 3), dims=(96, 192, 384, 768), num_classes=1000):
        super().__init__()
        layers = [nn.Sequential(nn.Conv2d(3, dims[0], 4, 4), _LayerNorm2d(dims[0], eps=1e-6))]
        for i, (d, c) in enumerate(zip(depths, dims)):
            layers.append(nn.Sequential(*[_CNBlock(c) for _ in range(d)]))
            if i < 3:
                layers.append(nn.Sequential(_LayerNorm2d(c, eps=1e-6), nn.Conv2d(c, dims[i + 1], 2, 2)))
        self.features = nn.Sequential(*layers)
        self.avgpool = nn.AdaptiveAvgPool2d(1)
        self.classifier = nn.Sequential(_LayerNorm2d(dims[-1], eps=1e-6), nn.Flatten(1), nn.Linear(dims[-1], num_classes))

    def forward(self, x):
        return self.classifier(self.avgpool(self.features(x)))


def convnext_tiny(num_classes=1000):
    return ConvNeXt(num_classes=num_classes)


# -- EfficientNet-B0 ----------------------------------------------------------------------------------------------------------------------
class _MBConv(nn.Module):
    def __init__(self, cin, cout, k, s, expand, se_ratio=0.25):
        super().__init__()
        hid = cin * expand
        self.use_res = s == 1 and cin == cout
        layers = []
        if expand != 1:
            layers.append(_cbr(cin, hid, 1, act=nn.SiLU))
        layers.append(_cbr(hid, hid, k, s, hid, act=nn.SiLU))
        layers.append(nn.SqueezeExcitation(hid, max(1, int(cin * se_ratio)), activation=F.silu))
        layers.append(nn.Sequential(nn.Conv2d(hid, cout, 1, bias=False), nn.BatchNorm2d(cout)))      # projection: no activation
        self.block = nn.Sequential(*layers)

    def forward(self, x):
        return x + self.block(x) if self.use_res else self.block(x)


class EfficientNet(nn.Module):
    def __init__(self, num_classes=1000, dropout=0.2):
        super().__init__()
        cfg = [(1, 3, 1, 32, 16, 1), (6, 3, 2, 16, 24, 2), (6, 5, 2, 24, 40, 2), (6, 3, 2, 40, 80, 3), (6, 5, 1, 80, 112, 3), (6, 5, 2, 112, 192, 4),
               (6, 3, 1, 192, 320, 1)]
        feats = [_cbr(3, 32, 3, 2, act=nn.SiLU)]
        for e, k, s, ci, co, n in cfg:
            feats.append(nn.Sequential(*[_MBConv(ci if i == 0 else co, co, k, s if i == 0 else 1, e) for i in range(n)]))
        feats.append(_cbr(320, 1280, 1, act=nn.SiLU))
        self.features = nn.Sequential(*feats)
        self.classifier = nn.Sequential(nn.Dropout(dropout), nn.Linear(1280, num_classes))

    def forward(self, x):
        return self.classifier(F.adaptive_avg_pool2d(self.features(x), 1).flatten(1))


def efficientnet_b0(num_classes=1000):
    return EfficientNet(num_classes)


# -- U-Net / YOLO head -----------------------------------------------------------------------------------------------------------------------
class _DoubleConv(nn.Sequential):
    def __init__(self, cin, cout):
        super().__init__(nn.Conv2d(cin, cout, 3, padding=1, bias=False), nn.BatchNorm2d(cout), nn.ReLU(inplace=True),
                         nn.Conv2d(cout, cout, 3, padding=1, bias=False), nn.BatchNorm2d(cout), nn.ReLU(inplace=True))


class UNet(nn.Module):
    def __init__(self, in_channels=3, num_classes=2, base=64, depth=4):
        super().__init__()
        chs = [base * 2 ** i for i in range(depth + 1)]
        self.downs = nn.ModuleList([_DoubleConv(in_channels if i == 0 else chs[i - 1], chs[i]) for i in range(depth + 1)])
        self.ups = nn.ModuleList([nn.ConvTranspose2d(chs[i + 1], chs[i], 2, 2) for i in reversed(range(depth))])
        self.dec = nn.ModuleList([_DoubleConv(chs[i] * 2, chs[i]) for i in reversed(range(depth))])
        self.head = nn.Conv2d(base, num_classes, 1)

    def forward(self, x):
        skips = []
        for i, d in enumerate(self.downs):
            x = d(x if i == 0 else F.max_pool2d(x, 2))
            skips.append(x)
        for up, dec, sk in zip(self.ups, self.dec, reversed(skips[:-1])):
            x = up(x)
            if x.shape[-2:] != sk.shape[-2:]:
                x = F.interpolate(x, sk.shape[-2:])
            x = dec(torch.cat([sk, x], 1))
        return self.head(x)


class Yolo(nn.Module):
    """Single-scale YOLO-style detector: conv backbone -> grid of (x, y, w, h, objectness, classes) per anchor."""

    def __init__(self, num_classes=20, anchors=((10, 13), (16, 30), (33, 23)), width=32):
        super().__init__()
        self.num_classes, self.anchors = num_classes, torch.tensor(anchors, dtype=torch.float32)
        c = width
        self.backbone = nn.Sequential(_cbr(3, c, 3, 2, act=nn.SiLU), _cbr(c, 2 * c, 3, 2, act=nn.SiLU), _cbr(2 * c, 4 * c, 3, 2, act=nn.SiLU),
                                      _cbr(4 * c, 8 * c, 3, 2, act=nn.SiLU), _cbr(8 * c, 8 * c, 3, 1, act=nn.SiLU))
        self.head = nn.Conv2d(8 * c, len(anchors) * (5 + num_classes), 1)

    def forward(self, x):
        p = self.head(self.backbone(x))
        B, _, H, W = p.shape
        return p.view(B, len(self.anchors), 5 + self.num_classes, H, W).permute(0, 1, 3, 4, 2)

    @torch.no_grad()
    def decode(self, pred, stride=16, conf=0.25):
        B, A, H, W, _ = pred.shape
        gy, gx = torch.meshgrid(torch.arange(H, device=pred.device), torch.arange(W, device=pred.device), indexing="ij")
        xy = (pred[..., :2].sigmoid() + torch.stack([gx, gy], -1)) * stride
        wh = pred[..., 2:4].exp() * self.anchors.to(pred.device).view(1, A, 1, 1, 2)
        obj, cls = pred[..., 4].sigmoid(), pred[..., 5:].sigmoid()
        score, label = (obj.unsqueeze(-1) * cls).max(-1)
        boxes = torch.cat([xy - wh / 2, xy + wh / 2], -1)
        keep = score > conf
        return [(boxes[b][keep[b]], score[b][keep[b]], label[b][keep[b]]) for b in range(B)]


# -- registry ---------------------------------------------------------------------------------------------------------------------------
class ModelRegistry:
    def __init__(self):
        self._m: Dict[str, Callable] = {}

    def register(self, name: str, ctor: Callable) -> None:
        self._m[name] = ctor

    def get(self, name: str, **kw):
        if name not in self._m:
            raise InvalidArgument(f"unknown model {name!r}; known: {sorted(self._m)}")
        return self._m[name](**kw)

    def names(self) -> List[str]:
        return sorted(self._m)


_REG = ModelRegistry()
for _n, _c in [("resnet18", resnet18), ("resnet34", resnet34), ("resnet50", resnet50), ("resnet50_dilated", resnet50_dilated), ("vgg11", vgg11),
               ("vgg16", vgg16), ("vit_b_16", vit_b_16), ("mobilenet_v2", mobilenet_v2), ("densenet121", densenet121), ("convnext_tiny", convnext_tiny),
               ("efficientnet_b0", efficientnet_b0), ("unet", UNet), ("yolo", Yolo)]:
    _REG.register(_n, _c)


def list_models() -> List[str]:
    return _REG.names()


def get_model(name: str, **kw):
    return _REG.get(name, **kw)


def register_model(name: str, ctor: Callable) -> None:
    _REG.register(name, ctor)


class FeatureExtractor(nn.Module):
    """``forward`` returns ``{node: output}`` for the named submodules, captured by forward hooks during one pass of ``model``
    (ferrotorch-vision/src/models/feature_extractor.rs:63)."""

    def __init__(self, model: torch.nn.Module, return_nodes: Sequence[str]):
        super().__init__()
        self.model, self.nodes = model, list(return_nodes)
        mods = dict(model.named_modules())
        missing = [n for n in self.nodes if n not in mods]
        if missing:
            raise InvalidArgument(f"no submodule named {missing}")
        self._out: Dict[str, torch.Tensor] = {}
        for n in self.nodes:
            mods[n].register_forward_hook(lambda m, i, o, n=n: self._out.__setitem__(n, o))

    def return_nodes(self) -> List[str]:
        return list(self.nodes)

    def forward(self, x):
        self._out.clear()
        self.model(x)
        return dict(self._out)


def create_feature_extractor(model: torch.nn.Module, return_nodes: Sequence[str]) -> FeatureExtractor:
    return FeatureExtractor(model, return_nodes)


ModelConstructor = Callable[..., torch.nn.Module]            # what the registry stores (ferrotorch-vision/src/models/registry.rs:71)
