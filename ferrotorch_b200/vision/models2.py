"""Further classification backbones with torchvision parameter names: MobileNetV3 (small / large), InceptionV3, Swin Transformer.

Reference parity: ferrotorch-vision/src/models/{mobilenet.rs:1218,1392,1471,1732, inception.rs:990,1284, swin.rs:1213,1461}.
"""
from __future__ import annotations

from functools import partial
from typing import Callable, List, Optional, Sequence

import torch
import torch.nn.functional as F

from .. import nn


def _make_divisible(v: float, divisor: int = 8) -> int:
    new = max(divisor, int(v + divisor / 2) // divisor * divisor)
    return new + divisor if new < 0.9 * v else new


class _ConvBNAct(nn.Sequential):
    def __init__(self, cin, cout, k=3, s=1, g=1, d=1, act: Optional[Callable] = nn.ReLU, eps=1e-3, momentum=0.01):
        layers = [nn.Conv2d(cin, cout, k, s, (k - 1) // 2 * d, d, g, bias=False), nn.BatchNorm2d(cout, eps=eps, momentum=momentum)]
        if act is not None:
            layers.append(act())
        super().__init__(*layers)


class _SE(nn.Module):
    def __init__(self, ch, squeeze, act=nn.ReLU, gate=nn.HardSigmoid):
        super().__init__()
        self.fc1, self.fc2 = nn.Conv2d(ch, squeeze, 1), nn.Conv2d(squeeze, ch, 1)
        self.activation, self.scale_activation = act(), gate()

    def forward(self, x):
        s = F.adaptive_avg_pool2d(x, 1)
        return x * self.scale_activation(self.fc2(self.activation(self.fc1(s))))


class _MNV3Block(nn.Module):
    def __init__(self, cin, k, exp, cout, se, hs, stride, dilation=1):
        super().__init__()
        self.use_res = stride == 1 and cin == cout
        act = nn.HardSwish if hs else nn.ReLU
        layers = []
        if exp != cin:
            layers.append(_ConvBNAct(cin, exp, 1, act=act))
        layers.append(_ConvBNAct(exp, exp, k, 1 if dilation > 1 else stride, exp, dilation, act=act))
        if se:
            layers.append(_SE(exp, _make_divisible(exp // 4)))
        layers.append(_ConvBNAct(exp, cout, 1, act=None))
        self.block = nn.Sequential(*layers)
        self.out_channels = cout

    def forward(self, x):
        y = self.block(x)
        return x + y if self.use_res else y


_MNV3_LARGE = [(16, 3, 16, 16, False, False, 1), (16, 3, 64, 24, False, False, 2), (24, 3, 72, 24, False, False, 1), (24, 5, 72, 40, True, False, 2),
               (40, 5, 120, 40, True, False, 1), (40, 5, 120, 40, True, False, 1), (40, 3, 240, 80, False, True, 2), (80, 3, 200, 80, False, True, 1),
               (80, 3, 184, 80, False, True, 1), (80, 3, 184, 80, False, True, 1), (80, 3, 480, 112, True, True, 1), (112, 3, 672, 112, True, True, 1),
               (112, 5, 672, 160, True, True, 2), (160, 5, 960, 160, True, True, 1), (160, 5, 960, 160, True, True, 1)]
_MNV3_SMALL = [(16, 3, 16, 16, True, False, 2), (16, 3, 72, 24, False, False, 2), (24, 3, 88, 24, False, False, 1), (24, 5, 96, 40, True, True, 2),
               (40, 5, 240, 40, True, True, 1), (40, 5, 240, 40, True, True, 1), (40, 5, 120, 48, True, True, 1), (48, 5, 144, 48, True, True, 1),
               (48, 5, 288, 96, True, True, 2), (96, 5, 576, 96, True, True, 1), (96, 5, 576, 96, True, True, 1)]


class MobileNetV3(nn.Module):
    def __init__(self, cfg, last_channel: int, num_classes: int = 1000, dilated: bool = False):
        super().__init__()
        layers: List[torch.nn.Module] = [_ConvBNAct(3, cfg[0][0], 3, 2, act=nn.HardSwish)]
        dilation = 1
        for i, (cin, k, exp, cout, se, hs, s) in enumerate(cfg):
            if dilated and s == 2 and i >= len(cfg) - 3:          # the last stride-2 stage runs dilated (segmentation backbones)
                dilation, s_eff = 2, 1
                layers.append(_MNV3Block(cin, k, exp, cout, se, hs, 2, dilation))
                continue
            layers.append(_MNV3Block(cin, k, exp, cout, se, hs, s, dilation))
        last_in = cfg[-1][3]
        layers.append(_ConvBNAct(last_in, 6 * last_in, 1, act=nn.HardSwish))
        self.features = nn.Sequential(*layers)
        self.avgpool = nn.AdaptiveAvgPool2d(1)
        self.classifier = nn.Sequential(nn.Linear(6 * last_in, last_channel), nn.HardSwish(), nn.Dropout(0.2), nn.Linear(last_channel, num_classes))

    def forward(self, x):
        return self.classifier(self.avgpool(self.features(x)).flatten(1))


MobileNetV3Small = MobileNetV3Large = MobileNetV3


def mobilenet_v3_large(num_classes=1000, dilated=False):
    return MobileNetV3(_MNV3_LARGE, 1280, num_classes, dilated)


def mobilenet_v3_small(num_classes=1000, dilated=False):
    return MobileNetV3(_MNV3_SMALL, 1024, num_classes, dilated)


# ----------------------------------------------------------------------------------------------------------------------
class _BasicConv2d(nn.Module):
    def __init__(self, cin, cout, **kw):
        super().__init__()
        self.conv = nn.Conv2d(cin, cout, bias=False, **kw)
        self.bn = nn.BatchNorm2d(cout, eps=0.001)

    def forward(self, x):
        return F.relu(self.bn(self.conv(x)))


class _InceptionA(nn.Module):
    def __init__(self, cin, pool):
        super().__init__()
        C = _BasicConv2d
        self.branch1x1 = C(cin, 64, kernel_size=1)
        self.branch5x5_1, self.branch5x5_2 = C(cin, 48, kernel_size=1), C(48, 64, kernel_size=5, padding=2)
        self.branch3x3dbl_1, self.branch3x3dbl_2, self.branch3x3dbl_3 = C(cin, 64, kernel_size=1), C(64, 96, kernel_size=3, padding=1), C(96, 96, kernel_size=3, padding=1)
        self.branch_pool = C(cin, pool, kernel_size=1)

    def forward(self, x):
        return torch.cat([self.branch1x1(x), self.branch5x5_2(self.branch5x5_1(x)), self.branch3x3dbl_3(self.branch3x3dbl_2(self.branch3x3dbl_1(x))),
                          self.branch_pool(F.avg_pool2d(x, 3, 1, 1))], 1)


class _InceptionB(nn.Module):
    def __init__(self, cin):
        super().__init__()
        C = _BasicConv2d
        self.branch3x3 = C(cin, 384, kernel_size=3, stride=2)
        self.branch3x3dbl_1, self.branch3x3dbl_2, self.branch3x3dbl_3 = C(cin, 64, kernel_size=1), C(64, 96, kernel_size=3, padding=1), C(96, 96, kernel_size=3, stride=2)

    def forward(self, x):
        return torch.cat([self.branch3x3(x), self.branch3x3dbl_3(self.branch3x3dbl_2(self.branch3x3dbl_1(x))), F.max_pool2d(x, 3, 2)], 1)


class _InceptionC(nn.Module):
    def __init__(self, cin, c7):
        super().__init__()
        C = _BasicConv2d
        self.branch1x1 = C(cin, 192, kernel_size=1)
        self.branch7x7_1, self.branch7x7_2, self.branch7x7_3 = C(cin, c7, kernel_size=1), C(c7, c7, kernel_size=(1, 7), padding=(0, 3)), C(c7, 192, kernel_size=(7, 1), padding=(3, 0))
        self.branch7x7dbl_1, self.branch7x7dbl_2 = C(cin, c7, kernel_size=1), C(c7, c7, kernel_size=(7, 1), padding=(3, 0))
        self.branch7x7dbl_3, self.branch7x7dbl_4 = C(c7, c7, kernel_size=(1, 7), padding=(0, 3)), C(c7, c7, kernel_size=(7, 1), padding=(3, 0))
        self.branch7x7dbl_5 = C(c7, 192, kernel_size=(1, 7), padding=(0, 3))
        self.branch_pool = C(cin, 192, kernel_size=1)

    def forward(self, x):
        b7 = self.branch7x7_3(self.branch7x7_2(self.branch7x7_1(x)))
        d = self.branch7x7dbl_5(self.branch7x7dbl_4(self.branch7x7dbl_3(self.branch7x7dbl_2(self.branch7x7dbl_1(x)))))
        return torch.cat([self.branch1x1(x), b7, d, self.branch_pool(F.avg_pool2d(x, 3, 1, 1))], 1)


class _InceptionD(nn.Module):
    def __init__(self, cin):
        super().__init__()
        C = _BasicConv2d
        self.branch3x3_1, self.branch3x3_2 = C(cin, 192, kernel_size=1), C(192, 320, kernel_size=3, stride=2)
        self.branch7x7x3_1, self.branch7x7x3_2 = C(cin, 192, kernel_size=1), C(192, 192, kernel_size=(1, 7), padding=(0, 3))
        self.branch7x7x3_3, self.branch7x7x3_4 = C(192, 192, kernel_size=(7, 1), padding=(3, 0)), C(192, 192, kernel_size=3, stride=2)

    def forward(self, x):
        return torch.cat([self.branch3x3_2(self.branch3x3_1(x)), self.branch7x7x3_4(self.branch7x7x3_3(self.branch7x7x3_2(self.branch7x7x3_1(x)))), F.max_pool2d(x, 3, 2)], 1)


class _InceptionE(nn.Module):
    def __init__(self, cin):
        super().__init__()
        C = _BasicConv2d
        self.branch1x1 = C(cin, 320, kernel_size=1)
        self.branch3x3_1, self.branch3x3_2a, self.branch3x3_2b = C(cin, 384, kernel_size=1), C(384, 384, kernel_size=(1, 3), padding=(0, 1)), C(384, 384, kernel_size=(3, 1), padding=(1, 0))
        self.branch3x3dbl_1, self.branch3x3dbl_2 = C(cin, 448, kernel_size=1), C(448, 384, kernel_size=3, padding=1)
        self.branch3x3dbl_3a, self.branch3x3dbl_3b = C(384, 384, kernel_size=(1, 3), padding=(0, 1)), C(384, 384, kernel_size=(3, 1), padding=(1, 0))
        self.branch_pool = C(cin, 192, kernel_size=1)

    def forward(self, x):
        b3 = self.branch3x3_1(x)
        b3 = torch.cat([self.branch3x3_2a(b3), self.branch3x3_2b(b3)], 1)
        d = self.branch3x3dbl_2(self.branch3x3dbl_1(x))
        d = torch.cat([self.branch3x3dbl_3a(d), self.branch3x3dbl_3b(d)], 1)
        return torch.cat([self.branch1x1(x), b3, d, self.branch_pool(F.avg_pool2d(x, 3, 1, 1))], 1)


class _InceptionAux(nn.Module):
    def __init__(self, cin, num_classes):
        super().__init__()
        self.conv0, self.conv1 = _BasicConv2d(cin, 128, kernel_size=1), _BasicConv2d(128, 768, kernel_size=5)
        self.fc = nn.Linear(768, num_classes)

    def forward(self, x):
        x = self.conv1(self.conv0(F.avg_pool2d(x, 5, 3)))
        return self.fc(F.adaptive_avg_pool2d(x, 1).flatten(1))


class InceptionV3(nn.Module):
    def __init__(self, num_classes: int = 1000, aux_logits: bool = True, transform_input: bool = False):
        super().__init__()
        C = _BasicConv2d
        self.aux_logits, self.transform_input = aux_logits, transform_input
        self.Conv2d_1a_3x3, self.Conv2d_2a_3x3, self.Conv2d_2b_3x3 = C(3, 32, kernel_size=3, stride=2), C(32, 32, kernel_size=3), C(32, 64, kernel_size=3, padding=1)
        self.Conv2d_3b_1x1, self.Conv2d_4a_3x3 = C(64, 80, kernel_size=1), C(80, 192, kernel_size=3)
        self.Mixed_5b, self.Mixed_5c, self.Mixed_5d = _InceptionA(192, 32), _InceptionA(256, 64), _InceptionA(288, 64)
        self.Mixed_6a = _InceptionB(288)
        self.Mixed_6b, self.Mixed_6c, self.Mixed_6d, self.Mixed_6e = _InceptionC(768, 128), _InceptionC(768, 160), _InceptionC(768, 160), _InceptionC(768, 192)
        self.AuxLogits = _InceptionAux(768, num_classes) if aux_logits else None
        self.Mixed_7a, self.Mixed_7b, self.Mixed_7c = _InceptionD(768), _InceptionE(1280), _InceptionE(2048)
        self.dropout = nn.Dropout(0.5)
        self.fc = nn.Linear(2048, num_classes)

    def forward(self, x):
        if self.transform_input:
            x = torch.cat([x[:, 0:1] * (0.229 / 0.5) + (0.485 - 0.5) / 0.5, x[:, 1:2] * (0.224 / 0.5) + (0.456 - 0.5) / 0.5, x[:, 2:3] * (0.225 / 0.5) + (0.406 - 0.5) / 0.5], 1)
        x = self.Conv2d_2b_3x3(self.Conv2d_2a_3x3(self.Conv2d_1a_3x3(x)))
        x = F.max_pool2d(x, 3, 2)
        x = F.max_pool2d(self.Conv2d_4a_3x3(self.Conv2d_3b_1x1(x)), 3, 2)
        x = self.Mixed_5d(self.Mixed_5c(self.Mixed_5b(x)))
        x = self.Mixed_6e(self.Mixed_6d(self.Mixed_6c(self.Mixed_6b(self.Mixed_6a(x)))))
        aux = self.AuxLogits(x) if self.AuxLogits is not None and self.training else None
        x = self.Mixed_7c(self.Mixed_7b(self.Mixed_7a(x)))
        out = self.fc(self.dropout(F.adaptive_avg_pool2d(x, 1).flatten(1)))
        return (out, aux) if aux is not None else out


def inception_v3(num_classes=1000, aux_logits=True):
    return InceptionV3(num_classes, aux_logits)


# ----------------------------------------------------------------------------------------------------------------------
class _PatchMerging(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.reduction, self.norm = nn.Linear(4 * dim, 2 * dim, bias=False), nn.LayerNorm(4 * dim)

    def forward(self, x):                                     # [B, H, W, C]
        H, W = x.shape[1:3]
        x = F.pad(x, (0, 0, 0, W % 2, 0, H % 2))
        x = torch.cat([x[:, 0::2, 0::2], x[:, 1::2, 0::2], x[:, 0::2, 1::2], x[:, 1::2, 1::2]], -1)
        return self.reduction(self.norm(x))


class _ShiftedWindowAttention(nn.Module):
    def __init__(self, dim, window, shift, heads):
        super().__init__()
        self.window, self.shift, self.heads = window, shift, heads
        self.qkv, self.proj = nn.Linear(dim, dim * 3), nn.Linear(dim, dim)
        self.relative_position_bias_table = nn.Parameter(torch.zeros((2 * window - 1) ** 2, heads))
        torch.nn.init.trunc_normal_(self.relative_position_bias_table, std=0.02)
        c = torch.stack(torch.meshgrid(torch.arange(window), torch.arange(window), indexing="ij")).flatten(1)
        rel = (c[:, :, None] - c[:, None, :]).permute(1, 2, 0) + (window - 1)
        self.register_buffer("relative_position_index", (rel[..., 0] * (2 * window - 1) + rel[..., 1]).flatten())

    def forward(self, x):                                     # [B, H, W, C]
        B, H, W, C = x.shape
        ws = self.window
        ph, pw = (ws - H % ws) % ws, (ws - W % ws) % ws
        x = F.pad(x, (0, 0, 0, pw, 0, ph))
        Hp, Wp = x.shape[1:3]
        sh = [0 if ws >= Hp else self.shift, 0 if ws >= Wp else self.shift]
        if sum(sh):
            x = torch.roll(x, (-sh[0], -sh[1]), (1, 2))
        nw = (Hp // ws) * (Wp // ws)
        xw = x.view(B, Hp // ws, ws, Wp // ws, ws, C).permute(0, 1, 3, 2, 4, 5).reshape(B * nw, ws * ws, C)
        qkv = self.qkv(xw).reshape(B * nw, ws * ws, 3, self.heads, C // self.heads).permute(2, 0, 3, 1, 4)
        q, k, v = qkv[0] * (C // self.heads) ** -0.5, qkv[1], qkv[2]
        attn = q @ k.transpose(-2, -1)
        bias = self.relative_position_bias_table[self.relative_position_index].view(ws * ws, ws * ws, -1).permute(2, 0, 1)
        attn = attn + bias[None]
        if sum(sh):
            m = x.new_zeros(Hp, Wp)
            cnt = 0
            for hs in ((0, -ws), (-ws, -sh[0]), (-sh[0], None)):
                for wsl in ((0, -ws), (-ws, -sh[1]), (-sh[1], None)):
                    m[hs[0]:hs[1], wsl[0]:wsl[1]] = cnt
                    cnt += 1
            m = m.view(Hp // ws, ws, Wp // ws, ws).permute(0, 2, 1, 3).reshape(nw, ws * ws)
            am = m[:, None, :] - m[:, :, None]
            am = am.masked_fill(am != 0, -100.0).masked_fill(am == 0, 0.0)
            attn = (attn.view(B, nw, self.heads, ws * ws, ws * ws) + am[None, :, None]).view(-1, self.heads, ws * ws, ws * ws)
        out = (attn.softmax(-1) @ v).transpose(1, 2).reshape(B * nw, ws * ws, C)
        out = self.proj(out).view(B, Hp // ws, Wp // ws, ws, ws, C).permute(0, 1, 3, 2, 4, 5).reshape(B, Hp, Wp, C)
        if sum(sh):
            out = torch.roll(out, (sh[0], sh[1]), (1, 2))
        return out[:, :H, :W].contiguous()


class _SwinMLP(nn.Sequential):
    def __init__(self, dim, hidden):
        super().__init__(nn.Linear(dim, hidden), nn.GELU(), nn.Dropout(0.0), nn.Linear(hidden, dim), nn.Dropout(0.0))


class _SwinBlock(nn.Module):
    def __init__(self, dim, heads, window, shift):
        super().__init__()
        self.norm1, self.norm2 = nn.LayerNorm(dim, eps=1e-5), nn.LayerNorm(dim, eps=1e-5)
        self.attn = _ShiftedWindowAttention(dim, window, shift, heads)
        self.mlp = _SwinMLP(dim, 4 * dim)

    def forward(self, x):
        x = x + self.attn(self.norm1(x))
        return x + self.mlp(self.norm2(x))


class SwinTransformer(nn.Module):
    def __init__(self, embed_dim=96, depths=(2, 2, 6, 2), heads=(3, 6, 12, 24), window=7, num_classes=1000, patch=4):
        super().__init__()
        layers: List[torch.nn.Module] = [nn.Sequential(nn.Conv2d(3, embed_dim, patch, patch), _ToNHWC(), nn.LayerNorm(embed_dim, eps=1e-5))]
        dim = embed_dim
        for i, (d, h) in enumerate(zip(depths, heads)):
            layers.append(nn.Sequential(*[_SwinBlock(dim, h, window, 0 if j % 2 == 0 else window // 2) for j in range(d)]))
            if i < len(depths) - 1:
                layers.append(_PatchMerging(dim))
                dim *= 2
        self.features = nn.Sequential(*layers)
        self.norm = nn.LayerNorm(dim, eps=1e-5)
        self.head = nn.Linear(dim, num_classes)

    def forward(self, x):
        x = self.norm(self.features(x))
        return self.head(x.permute(0, 3, 1, 2).mean((2, 3)))


class _ToNHWC(nn.Module):
    def forward(self, x):
        return x.permute(0, 2, 3, 1)


def swin_tiny(num_classes=1000):
    return SwinTransformer(96, (2, 2, 6, 2), (3, 6, 12, 24), 7, num_classes)
