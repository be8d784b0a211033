"""Object detection: FPN, anchors, box coding, RPN, RoI heads (Faster / Mask / Keypoint R-CNN), RetinaNet, FCOS and SSD300, with torchvision
parameter names so published checkpoints load by name. Inference paths are complete (transform, proposals, heads, post-processing);
training losses are left to the caller (``vision.ops`` has the focal / IoU losses).

Reference parity: ferrotorch-vision/src/models/{fpn.rs:52, anchor_utils.rs:32,236, rpn.rs:153, roi_heads_postprocess.rs:184,371,
faster_rcnn.rs:206,556, mask_rcnn.rs:218,553, keypoint_rcnn.rs:275,622, retinanet.rs:626,996, fcos.rs:482,850, ssd.rs:644,1344}.
"""
from __future__ import annotations

import math
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import nn
from . import models as M
from . import ops as V


# ----------------------------------------------------------------------------------------------------------------------
# backbone + FPN
# ----------------------------------------------------------------------------------------------------------------------
class _ConvNorm(nn.Sequential):
    """torchvision's Conv2dNormActivation naming: ``0`` = conv, ``1`` = norm."""

    def __init__(self, cin, cout, k, padding=None, norm=None, act=None, bias=True, stride=1):
        layers: List[torch.nn.Module] = [nn.Conv2d(cin, cout, k, stride, (k - 1) // 2 if padding is None else padding, bias=bias)]
        if norm is not None:
            layers.append(norm(cout))
        if act is not None:
            layers.append(act())
        super().__init__(*layers)


class LastLevelMaxPool(nn.Module):
    def forward(self, results, x, names):
        return results + [F.max_pool2d(results[-1], 1, 2, 0)], names + ["pool"]


class LastLevelP6P7(nn.Module):
    def __init__(self, cin, cout):
        super().__init__()
        self.p6, self.p7 = nn.Conv2d(cin, cout, 3, 2, 1), nn.Conv2d(cout, cout, 3, 2, 1)
        self.use_P5 = cin == cout

    def forward(self, results, x, names):
        p6 = self.p6(results[-1] if self.use_P5 else x[-1])
        return results + [p6, self.p7(F.relu(p6))], names + ["p6", "p7"]


class FeaturePyramidNetwork(nn.Module):
    def __init__(self, in_channels: Sequence[int], out_channels: int, extra_blocks: Optional[torch.nn.Module] = None):
        super().__init__()
        self.inner_blocks = nn.ModuleList([_ConvNorm(c, out_channels, 1, padding=0) for c in in_channels])
        self.layer_blocks = nn.ModuleList([_ConvNorm(out_channels, out_channels, 3) for _ in in_channels])
        self.extra_blocks = extra_blocks

    def forward(self, feats: "OrderedDict[str, torch.Tensor]") -> "OrderedDict[str, torch.Tensor]":
        names, xs = list(feats.keys()), list(feats.values())
        last = self.inner_blocks[-1](xs[-1])
        results = [self.layer_blocks[-1](last)]
        for i in range(len(xs) - 2, -1, -1):
            lat = self.inner_blocks[i](xs[i])
            last = lat + F.interpolate(last, size=lat.shape[-2:], mode="nearest")
            results.insert(0, self.layer_blocks[i](last))
        if self.extra_blocks is not None:
            results, names = self.extra_blocks(results, xs, names)
        return OrderedDict(zip(names, results))


class _FrozenBatchNorm2d(nn.Module):
    def __init__(self, n, eps=1e-5):
        super().__init__()
        self.eps = eps
        for name, v in (("weight", torch.ones(n)), ("bias", torch.zeros(n)), ("running_mean", torch.zeros(n)), ("running_var", torch.ones(n))):
            self.register_buffer(name, v)

    def forward(self, x):
        scale = self.weight * (self.running_var + self.eps).rsqrt()
        return x * scale[None, :, None, None] + (self.bias - self.running_mean * scale)[None, :, None, None]


class _ResNetLayers(nn.Module):
    def __init__(self, net: M.ResNet, returned: Sequence[int]):
        super().__init__()
        for n in ("conv1", "bn1", "relu", "maxpool", "layer1", "layer2", "layer3", "layer4"):
            setattr(self, n, getattr(net, n))
        self.returned = list(returned)

    def forward(self, x):
        x = M.max_pool(M.bn_act(self.bn1, self.conv1(x)), 3, 2, 1)
        out = OrderedDict()
        for i in range(1, 5):
            x = getattr(self, f"layer{i}")(x)
            if i in self.returned:
                out[str(self.returned.index(i))] = x
        return out


def _freeze_bn(m: torch.nn.Module) -> None:
    for name, child in m.named_children():
        if isinstance(child, (nn.BatchNorm2d, torch.nn.BatchNorm2d)):
            setattr(m, name, _FrozenBatchNorm2d(child.num_features, child.eps))
        else:
            _freeze_bn(child)


class BackboneWithFPN(nn.Module):
    def __init__(self, returned_layers=(1, 2, 3, 4), out_channels=256, extra_blocks=None, frozen_bn=True):
        super().__init__()
        net = M.resnet50()
        if frozen_bn:
            _freeze_bn(net)
        self.body = _ResNetLayers(net, returned_layers)
        self.fpn = FeaturePyramidNetwork([256 * 2 ** (i - 1) for i in returned_layers], out_channels, extra_blocks or LastLevelMaxPool())
        self.out_channels = out_channels

    def forward(self, x):
        return self.fpn(self.body(x))


# ----------------------------------------------------------------------------------------------------------------------
# anchors + box coding
# ----------------------------------------------------------------------------------------------------------------------
class AnchorGenerator(nn.Module):
    def __init__(self, sizes=((32,), (64,), (128,), (256,), (512,)), aspect_ratios=((0.5, 1.0, 2.0),) * 5):
        super().__init__()
        self.sizes, self.aspect_ratios = sizes, aspect_ratios

    def base_anchors(self, scales, ratios, device) -> torch.Tensor:
        s, r = torch.as_tensor(scales, dtype=torch.float32, device=device), torch.as_tensor(ratios, dtype=torch.float32, device=device)
        h, w = torch.sqrt(r), 1 / torch.sqrt(r)
        ws, hs = (w[:, None] * s[None]).view(-1), (h[:, None] * s[None]).view(-1)
        return (torch.stack([-ws, -hs, ws, hs], 1) / 2).round()

    def num_anchors_per_location(self) -> List[int]:
        return [len(s) * len(a) for s, a in zip(self.sizes, self.aspect_ratios)]

    def forward(self, image_size: Tuple[int, int], feature_maps: Sequence[torch.Tensor]) -> torch.Tensor:
        out = []
        for fm, sz, ar in zip(feature_maps, self.sizes, self.aspect_ratios):
            gh, gw = fm.shape[-2:]
            sh, sw = image_size[0] // gh, image_size[1] // gw
            ys, xs = torch.meshgrid(torch.arange(gh, device=fm.device) * sh, torch.arange(gw, device=fm.device) * sw, indexing="ij")
            shifts = torch.stack([xs, ys, xs, ys], -1).view(-1, 1, 4).float()
            out.append((shifts + self.base_anchors(sz, ar, fm.device)[None]).view(-1, 4))
        return torch.cat(out)


def encode_boxes(ref: torch.Tensor, proposals: torch.Tensor, weights=(1.0, 1.0, 1.0, 1.0)) -> torch.Tensor:
    wx, wy, ww, wh = weights
    pw, ph = proposals[:, 2] - proposals[:, 0], proposals[:, 3] - proposals[:, 1]
    px, py = proposals[:, 0] + 0.5 * pw, proposals[:, 1] + 0.5 * ph
    gw, gh = ref[:, 2] - ref[:, 0], ref[:, 3] - ref[:, 1]
    gx, gy = ref[:, 0] + 0.5 * gw, ref[:, 1] + 0.5 * gh
    return torch.stack([wx * (gx - px) / pw, wy * (gy - py) / ph, ww * torch.log(gw / pw), wh * torch.log(gh / ph)], 1)


def decode_boxes(deltas: torch.Tensor, boxes: torch.Tensor, weights=(1.0, 1.0, 1.0, 1.0), clip: float = math.log(1000.0 / 16)) -> torch.Tensor:
    """``deltas [N, 4*k]`` relative to ``boxes [N, 4]`` -> ``[N, k, 4]`` corner boxes."""
    wx, wy, ww, wh = weights
    w, h = boxes[:, 2] - boxes[:, 0], boxes[:, 3] - boxes[:, 1]
    cx, cy = boxes[:, 0] + 0.5 * w, boxes[:, 1] + 0.5 * h
    dx, dy = deltas[:, 0::4] / wx, deltas[:, 1::4] / wy
    dw, dh = (deltas[:, 2::4] / ww).clamp(max=clip), (deltas[:, 3::4] / wh).clamp(max=clip)
    pcx, pcy = dx * w[:, None] + cx[:, None], dy * h[:, None] + cy[:, None]
    pw, ph = torch.exp(dw) * w[:, None], torch.exp(dh) * h[:, None]
    return torch.stack([pcx - 0.5 * pw, pcy - 0.5 * ph, pcx + 0.5 * pw, pcy + 0.5 * ph], 2)


# ----------------------------------------------------------------------------------------------------------------------
# transform
# ----------------------------------------------------------------------------------------------------------------------
class DetectionTransform(nn.Module):
    def __init__(self, min_size=800, max_size=1333, mean=(0.485, 0.456, 0.406), std=(0.229, 0.224, 0.225), divisor=32, fixed_size=None):
        super().__init__()
        self.min_size, self.max_size, self.mean, self.std, self.divisor, self.fixed_size = min_size, max_size, mean, std, divisor, fixed_size

    def forward(self, images: Sequence[torch.Tensor]):
        out, sizes = [], []
        for im in images:
            m, s = im.new_tensor(self.mean)[:, None, None], im.new_tensor(self.std)[:, None, None]
            im = (im - m) / s
            h, w = im.shape[-2:]
            if self.fixed_size is not None:
                im = F.interpolate(im[None], size=self.fixed_size, mode="bilinear", align_corners=False)[0]
            else:
                scale = min(self.min_size / min(h, w), self.max_size / max(h, w))
                im = F.interpolate(im[None], scale_factor=scale, mode="bilinear", recompute_scale_factor=True, align_corners=False)[0]
            out.append(im)
            sizes.append(tuple(im.shape[-2:]))
        H = max(s[0] for s in sizes)
        Wd = max(s[1] for s in sizes)
        H, Wd = int(math.ceil(H / self.divisor) * self.divisor), int(math.ceil(Wd / self.divisor) * self.divisor)
        batch = out[0].new_zeros(len(out), 3, H, Wd)
        for i, im in enumerate(out):
            batch[i, :, : im.shape[1], : im.shape[2]] = im
        return batch, sizes

    @staticmethod
    def rescale(boxes: torch.Tensor, from_size, to_size) -> torch.Tensor:
        rh, rw = to_size[0] / from_size[0], to_size[1] / from_size[1]
        return boxes * boxes.new_tensor([rw, rh, rw, rh])


# ----------------------------------------------------------------------------------------------------------------------
# RPN
# ----------------------------------------------------------------------------------------------------------------------
class Detections(dict):
    """Detections of one image: a dict with ``boxes [N, 4]`` (xyxy, image pixels), ``scores [N]``, ``labels [N]`` that also reads as attributes
    (ferrotorch-vision/src/models/detection/faster_rcnn.rs:92, retinanet.rs:612, fcos.rs:467)."""

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError:
            raise AttributeError(k) from None


class MaskDetections(Detections):
    """:class:`Detections` plus ``masks [N, 1, H, W]`` pasted into the image (mask_rcnn.rs:192)."""


class SsdDetections(Detections):
    """ssd.rs:1325."""


FPN_OUT_CHANNELS = 256                                       # fpn.rs:39
SSD_ANCHORS_PER_SCALE = (4, 6, 6, 6, 4, 4)                   # ssd.rs:436-465
SSD_FM_SIZES = (38, 19, 10, 5, 3, 1)
SSD_TOTAL_ANCHORS = 8732
SSD_SCORE_THRESH, SSD_NMS_THRESH, SSD_TOPK_CANDIDATES, SSD_DETECTIONS_PER_IMG = 0.01, 0.45, 400, 200


@dataclass
class RpnConfig:
    """Proposal filtering knobs (rpn.rs:115); ``default_eval`` carries torchvision's inference values."""
    pre_nms_top_n: int = 1000
    post_nms_top_n: int = 1000
    nms_thresh: float = 0.7
    min_size: float = 1e-3
    score_thresh: float = 0.0
    image_size: Tuple[int, int] = (800, 800)

    @classmethod
    def default_eval(cls, image_size) -> "RpnConfig":
        return cls(image_size=tuple(image_size))


class RPNHead(nn.Module):
    def __init__(self, ch, num_anchors):
        super().__init__()
        self.conv = nn.Sequential(_ConvNorm(ch, ch, 3, act=nn.ReLU))
        self.cls_logits, self.bbox_pred = nn.Conv2d(ch, num_anchors, 1), nn.Conv2d(ch, num_anchors * 4, 1)

    def forward(self, feats):
        ts = [self.conv(f) for f in feats]
        return [self.cls_logits(t) for t in ts], [self.bbox_pred(t) for t in ts]


def _flatten_levels(xs: Sequence[torch.Tensor], c: int) -> torch.Tensor:
    """per-level ``[B, A*c, H, W]`` -> ``[B, sum(H*W*A), c]`` in (H, W, A) order, the order of the generated anchors."""
    return torch.cat([x.view(x.shape[0], -1, c, x.shape[-2], x.shape[-1]).permute(0, 3, 4, 1, 2).reshape(x.shape[0], -1, c) for x in xs], 1)


class Rpn(nn.Module):
    def __init__(self, anchor_generator: AnchorGenerator, head: RPNHead, pre_nms_top_n=1000, post_nms_top_n=1000, nms_thresh=0.7, score_thresh=0.0, min_size=1e-3):
        super().__init__()
        if isinstance(pre_nms_top_n, RpnConfig):
            c = pre_nms_top_n
            pre_nms_top_n, post_nms_top_n, nms_thresh, score_thresh, min_size = c.pre_nms_top_n, c.post_nms_top_n, c.nms_thresh, c.score_thresh, c.min_size
        self.anchor_generator, self.head = anchor_generator, head
        self.pre, self.post, self.nms_thresh, self.score_thresh, self.min_size = pre_nms_top_n, post_nms_top_n, nms_thresh, score_thresh, min_size

    @torch.no_grad()
    def forward(self, batch: torch.Tensor, image_sizes, feats: "OrderedDict[str, torch.Tensor]") -> List[torch.Tensor]:
        fl = list(feats.values())
        logits, deltas = self.head(fl)
        anchors = self.anchor_generator(tuple(batch.shape[-2:]), fl)
        per_level = [l.shape[1] * l.shape[2] * l.shape[3] for l in logits]
        obj, reg = _flatten_levels(logits, 1).squeeze(-1), _flatten_levels(deltas, 4)
        levels = torch.cat([torch.full((n,), i, device=batch.device) for i, n in enumerate(per_level)])
        out = []
        for b in range(batch.shape[0]):
            boxes = decode_boxes(reg[b], anchors)[:, 0]
            keep_idx = []
            off = 0
            for n in per_level:
                k = min(self.pre, n)
                keep_idx.append(obj[b, off: off + n].topk(k).indices + off)
                off += n
            idx = torch.cat(keep_idx)
            bx, sc, lv = V.clip_boxes_to_image(boxes[idx], image_sizes[b]), torch.sigmoid(obj[b, idx]), levels[idx]
            k = V.remove_small_boxes(bx, self.min_size)
            bx, sc, lv = bx[k], sc[k], lv[k]
            k = sc >= self.score_thresh
            bx, sc, lv = bx[k], sc[k], lv[k]
            k = V.batched_nms(bx, sc, lv, self.nms_thresh)[: self.post]
            out.append(bx[k])
        return out


# ----------------------------------------------------------------------------------------------------------------------
# RoI heads
# ----------------------------------------------------------------------------------------------------------------------
class MultiScaleRoIAlign(nn.Module):
    def __init__(self, featmap_names=("0", "1", "2", "3"), output_size=7, sampling_ratio=2, canonical_scale=224, canonical_level=4):
        super().__init__()
        self.names, self.out, self.sr, self.s0, self.k0 = list(featmap_names), output_size, sampling_ratio, canonical_scale, canonical_level

    def forward(self, feats: Dict[str, torch.Tensor], boxes: List[torch.Tensor], image_sizes) -> torch.Tensor:
        fl = [feats[n] for n in self.names]
        H = max(s[0] for s in image_sizes)
        scales = [2 ** round(math.log2(f.shape[-2] / H)) for f in fl]
        kmin, kmax = -math.log2(scales[0]), -math.log2(scales[-1])
        rois = torch.cat([torch.cat([torch.full((len(b), 1), i, dtype=b.dtype, device=b.device), b], 1) for i, b in enumerate(boxes)])
        if len(fl) == 1:
            return V.roi_align(fl[0], rois, self.out, scales[0], self.sr)
        area = ((rois[:, 3] - rois[:, 1]) * (rois[:, 4] - rois[:, 2])).sqrt()
        lvl = torch.floor(self.k0 + torch.log2(area / self.s0) + 1e-6).clamp(kmin, kmax).long() - int(kmin)
        osz = (self.out, self.out) if isinstance(self.out, int) else tuple(self.out)
        out = rois.new_zeros(len(rois), fl[0].shape[1], *osz)
        for i, (f, s) in enumerate(zip(fl, scales)):
            idx = torch.where(lvl == i)[0]
            if len(idx):
                out[idx] = V.roi_align(f, rois[idx], self.out, s, self.sr).to(out.dtype)
        return out


class TwoMLPHead(nn.Module):
    def __init__(self, cin, rep):
        super().__init__()
        self.fc6, self.fc7 = nn.Linear(cin, rep), nn.Linear(rep, rep)

    def forward(self, x):
        return F.relu(self.fc7(F.relu(self.fc6(x.flatten(1)))))


class FastRCNNPredictor(nn.Module):
    def __init__(self, cin, num_classes):
        super().__init__()
        self.cls_score, self.bbox_pred = nn.Linear(cin, num_classes), nn.Linear(cin, num_classes * 4)

    def forward(self, x):
        return self.cls_score(x), self.bbox_pred(x)


def postprocess_detections(class_logits, box_regression, proposals: List[torch.Tensor], image_sizes, score_thresh=0.05, nms_thresh=0.5, detections_per_img=100,
                           weights=(10.0, 10.0, 5.0, 5.0)):
    """Softmax scores, per-class box decoding, clipping, score threshold, small-box removal, class-wise NMS, top-k. Returns per image
    ``(boxes, scores, labels, keep_rows)`` where ``keep_rows`` indexes the image's proposals (for the mask / keypoint heads)."""
    n = [len(p) for p in proposals]
    boxes = decode_boxes(box_regression, torch.cat(proposals), weights)
    scores = F.softmax(class_logits, -1)
    out = []
    for bx, sc, size in zip(boxes.split(n), scores.split(n), image_sizes):
        C = sc.shape[1]
        bx = V.clip_boxes_to_image(bx.reshape(-1, 4), size).view(-1, C, 4)
        labels = torch.arange(C, device=sc.device).expand_as(sc)
        rows = torch.arange(len(sc), device=sc.device)[:, None].expand_as(sc)
        bx, sc, labels, rows = bx[:, 1:].reshape(-1, 4), sc[:, 1:].reshape(-1), labels[:, 1:].reshape(-1), rows[:, 1:].reshape(-1)
        k = sc > score_thresh
        bx, sc, labels, rows = bx[k], sc[k], labels[k], rows[k]
        k = V.remove_small_boxes(bx, 1e-2)
        bx, sc, labels, rows = bx[k], sc[k], labels[k], rows[k]
        k = V.batched_nms(bx, sc, labels, nms_thresh)[:detections_per_img]
        out.append((bx[k], sc[k], labels[k], rows[k]))
    return out


def postprocess_masks(mask_logits: torch.Tensor, labels: torch.Tensor, boxes: torch.Tensor, image_size, threshold: Optional[float] = 0.5) -> torch.Tensor:
    """``mask_logits [N, C, m, m]`` -> per-detection masks pasted into the image ``[N, 1, H, W]`` (boolean when ``threshold`` is given)."""
    N = len(labels)
    H, Wd = image_size
    probs = mask_logits.sigmoid()[torch.arange(N, device=labels.device), labels][:, None]
    out = probs.new_zeros(N, 1, H, Wd)
    m = probs.shape[-1]
    pad = 1                                                          # one-pixel border avoids edge artefacts when resizing
    scale = (m + 2 * pad) / m
    probs = F.pad(probs, (pad,) * 4)
    for i in range(N):
        x0, y0, x1, y1 = boxes[i].tolist()
        cx, cy, w, h = (x0 + x1) / 2, (y0 + y1) / 2, (x1 - x0) * scale, (y1 - y0) * scale
        bx0, by0, bx1, by1 = int(cx - w / 2), int(cy - h / 2), int(cx + w / 2), int(cy + h / 2)
        bw, bh = max(bx1 - bx0 + 1, 1), max(by1 - by0 + 1, 1)
        mk = F.interpolate(probs[i][None], size=(bh, bw), mode="bilinear", align_corners=False)[0, 0]
        xs0, ys0, xs1, ys1 = max(bx0, 0), max(by0, 0), min(bx1 + 1, Wd), min(by1 + 1, H)
        if xs1 > xs0 and ys1 > ys0:
            out[i, 0, ys0:ys1, xs0:xs1] = mk[ys0 - by0: ys1 - by0, xs0 - bx0: xs1 - bx0]
    return out > threshold if threshold is not None else out


def heatmaps_to_keypoints(maps: torch.Tensor, rois: torch.Tensor):
    """``maps [N, K, s, s]`` keypoint logits over each RoI -> ``(xy_visible [N, K, 3], scores [N, K])`` in image coordinates."""
    N, K, s, _ = maps.shape
    w, h = (rois[:, 2] - rois[:, 0]).clamp(min=1), (rois[:, 3] - rois[:, 1]).clamp(min=1)
    flat = maps.view(N, K, -1)
    pos = flat.argmax(-1)
    xi, yi = (pos % s).float(), (pos // s).float()
    x = (xi + 0.5) * (w / s)[:, None] + rois[:, 0:1]
    y = (yi + 0.5) * (h / s)[:, None] + rois[:, 1:2]
    return torch.stack([x, y, torch.ones_like(x)], 2), flat.max(-1).values


class MaskRCNNHeads(nn.Sequential):
    def __init__(self, cin, layers=(256, 256, 256, 256)):
        mods, c = [], cin
        for l in layers:
            mods.append(_ConvNorm(c, l, 3, act=nn.ReLU))
            c = l
        super().__init__(*mods)


class MaskRCNNPredictor(nn.Sequential):
    def __init__(self, cin, dim, num_classes):
        super().__init__(OrderedDict([("conv5_mask", nn.ConvTranspose2d(cin, dim, 2, 2, 0)), ("relu", nn.ReLU()), ("mask_fcn_logits", nn.Conv2d(dim, num_classes, 1))]))


class KeypointRCNNHeads(nn.Sequential):
    def __init__(self, cin, layers=(512,) * 8):
        mods, c = [], cin
        for l in layers:
            mods += [nn.Conv2d(c, l, 3, padding=1), nn.ReLU()]
            c = l
        super().__init__(*mods)


class KeypointRCNNPredictor(nn.Module):
    def __init__(self, cin, num_keypoints):
        super().__init__()
        self.kps_score_lowres = nn.ConvTranspose2d(cin, num_keypoints, 4, 2, 1)

    def forward(self, x):
        return F.interpolate(self.kps_score_lowres(x), scale_factor=2.0, mode="bilinear", align_corners=False, recompute_scale_factor=False)


class RoIHeads(nn.Module):
    def __init__(self, box_roi_pool, box_head, box_predictor, score_thresh=0.05, nms_thresh=0.5, detections_per_img=100):
        super().__init__()
        self.box_roi_pool, self.box_head, self.box_predictor = box_roi_pool, box_head, box_predictor
        self.score_thresh, self.nms_thresh, self.detections_per_img = score_thresh, nms_thresh, detections_per_img
        self.mask_roi_pool = self.mask_head = self.mask_predictor = None
        self.keypoint_roi_pool = self.keypoint_head = self.keypoint_predictor = None

    @torch.no_grad()
    def forward(self, feats, proposals, image_sizes) -> List[Dict[str, torch.Tensor]]:
        x = self.box_head(self.box_roi_pool(feats, proposals, image_sizes))
        logits, reg = self.box_predictor(x)
        dets = postprocess_detections(logits, reg, proposals, image_sizes, self.score_thresh, self.nms_thresh, self.detections_per_img)
        out = [Detections(boxes=b, scores=s, labels=l) for b, s, l, _ in dets]
        if self.mask_head is not None:
            bl = [d["boxes"] for d in out]
            ml = self.mask_predictor(self.mask_head(self.mask_roi_pool(feats, bl, image_sizes)))
            for d, m, size in zip(out, ml.split([len(b) for b in bl]), image_sizes):
                d["masks"] = postprocess_masks(m, d["labels"], d["boxes"], size, None)
                d.__class__ = MaskDetections
        if self.keypoint_head is not None:
            bl = [d["boxes"] for d in out]
            kl = self.keypoint_predictor(self.keypoint_head(self.keypoint_roi_pool(feats, bl, image_sizes)))
            for d, k in zip(out, kl.split([len(b) for b in bl])):
                d["keypoints"], d["keypoints_scores"] = heatmaps_to_keypoints(k, d["boxes"])
        return out


class FasterRcnn(nn.Module):
    def __init__(self, num_classes=91, min_size=800, max_size=1333, box_detections_per_img=100, box_score_thresh=0.05):
        super().__init__()
        self.transform = DetectionTransform(min_size, max_size)
        self.backbone = BackboneWithFPN()
        ag = AnchorGenerator()
        self.rpn = Rpn(ag, RPNHead(256, ag.num_anchors_per_location()[0]))
        self.roi_heads = RoIHeads(MultiScaleRoIAlign(output_size=7), TwoMLPHead(256 * 7 * 7, 1024), FastRCNNPredictor(1024, num_classes), box_score_thresh, 0.5,
                                  box_detections_per_img)

    @torch.no_grad()
    def forward(self, images: Sequence[torch.Tensor]) -> List[Dict[str, torch.Tensor]]:
        orig = [tuple(im.shape[-2:]) for im in images]
        batch, sizes = self.transform(images)
        feats = self.backbone(batch)
        props = self.rpn(batch, sizes, feats)
        dets = self.roi_heads(feats, props, sizes)
        for d, s, o in zip(dets, sizes, orig):
            d["boxes"] = DetectionTransform.rescale(d["boxes"], s, o)
            if "keypoints" in d:
                d["keypoints"][..., 0] *= o[1] / s[1]
                d["keypoints"][..., 1] *= o[0] / s[0]
            if "masks" in d:
                d["masks"] = F.interpolate(d["masks"], size=o, mode="bilinear", align_corners=False) if len(d["masks"]) else d["masks"].new_zeros(0, 1, *o)
        return dets


class MaskRcnn(FasterRcnn):
    def __init__(self, num_classes=91, **kw):
        super().__init__(num_classes, **kw)
        self.roi_heads.mask_roi_pool = MultiScaleRoIAlign(output_size=14)
        self.roi_heads.mask_head = MaskRCNNHeads(256)
        self.roi_heads.mask_predictor = MaskRCNNPredictor(256, 256, num_classes)


class KeypointRcnn(FasterRcnn):
    def __init__(self, num_classes=2, num_keypoints=17, **kw):
        super().__init__(num_classes, **kw)
        self.roi_heads.keypoint_roi_pool = MultiScaleRoIAlign(output_size=14)
        self.roi_heads.keypoint_head = KeypointRCNNHeads(256)
        self.roi_heads.keypoint_predictor = KeypointRCNNPredictor(512, num_keypoints)


def fasterrcnn_resnet50_fpn(num_classes=91, **kw): return FasterRcnn(num_classes, **kw)     # noqa: E704
def maskrcnn_resnet50_fpn(num_classes=91, **kw): return MaskRcnn(num_classes, **kw)         # noqa: E704
def keypointrcnn_resnet50_fpn(num_classes=2, num_keypoints=17, **kw): return KeypointRcnn(num_classes, num_keypoints, **kw)  # noqa: E704


# ----------------------------------------------------------------------------------------------------------------------
# one-stage detectors
# ----------------------------------------------------------------------------------------------------------------------
class _TowerHead(nn.Module):
    def __init__(self, ch, out, norm_groups: Optional[int] = None, n_conv=4):
        super().__init__()
        if norm_groups:                      # FCOS: a flat conv / GroupNorm / ReLU sequence
            mods: List[torch.nn.Module] = []
            for _ in range(n_conv):
                mods += [nn.Conv2d(ch, ch, 3, padding=1), nn.GroupNorm(norm_groups, ch), nn.ReLU()]
            self.conv = nn.Sequential(*mods)
        else:                                # RetinaNet: conv + ReLU blocks
            self.conv = nn.Sequential(*[_ConvNorm(ch, ch, 3, act=nn.ReLU) for _ in range(n_conv)])
        self.out = out


class RetinaNetClassificationHead(_TowerHead):
    def __init__(self, ch, num_anchors, num_classes):
        super().__init__(ch, num_classes)
        self.cls_logits = nn.Conv2d(ch, num_anchors * num_classes, 3, padding=1)

    def forward(self, feats):
        return _flatten_levels([self.cls_logits(self.conv(f)) for f in feats], self.out)


class RetinaNetRegressionHead(_TowerHead):
    def __init__(self, ch, num_anchors):
        super().__init__(ch, 4)
        self.bbox_reg = nn.Conv2d(ch, num_anchors * 4, 3, padding=1)

    def forward(self, feats):
        return _flatten_levels([self.bbox_reg(self.conv(f)) for f in feats], 4)


class RetinaNetHead(nn.Module):
    def __init__(self, ch, num_anchors, num_classes):
        super().__init__()
        self.classification_head, self.regression_head = RetinaNetClassificationHead(ch, num_anchors, num_classes), RetinaNetRegressionHead(ch, num_anchors)


def _one_stage_postprocess(scores_per_level, boxes_fn, image_size, score_thresh, topk, nms_thresh, dets):
    bl, sl, ll = [], [], []
    for lvl, sc in enumerate(scores_per_level):
        C = sc.shape[-1]
        flat = sc.flatten()
        keep = torch.where(flat > score_thresh)[0]
        k = min(topk, len(keep))
        top = flat[keep].topk(k)
        idx = keep[top.indices]
        a_idx, labels = idx // C, idx % C
        bl.append(V.clip_boxes_to_image(boxes_fn(lvl, a_idx), image_size))
        sl.append(top.values)
        ll.append(labels)
    b, s, l = torch.cat(bl), torch.cat(sl), torch.cat(ll)
    k = V.batched_nms(b, s, l, nms_thresh)[:dets]
    return Detections(boxes=b[k], scores=s[k], labels=l[k])


class RetinaNet(nn.Module):
    def __init__(self, num_classes=91, min_size=800, max_size=1333, score_thresh=0.05, nms_thresh=0.5, detections_per_img=300, topk_candidates=1000):
        super().__init__()
        self.transform = DetectionTransform(min_size, max_size)
        self.backbone = BackboneWithFPN((2, 3, 4), 256, LastLevelP6P7(256, 256))
        sizes = tuple((x, int(x * 2 ** (1 / 3)), int(x * 2 ** (2 / 3))) for x in (32, 64, 128, 256, 512))
        self.anchor_generator = AnchorGenerator(sizes, ((0.5, 1.0, 2.0),) * 5)
        self.head = RetinaNetHead(256, 9, num_classes)
        self.cfg = (score_thresh, topk_candidates, nms_thresh, detections_per_img)

    @torch.no_grad()
    def forward(self, images):
        orig = [tuple(im.shape[-2:]) for im in images]
        batch, sizes = self.transform(images)
        fl = list(self.backbone(batch).values())
        cls, reg = self.head.classification_head(fl), self.head.regression_head(fl)
        anchors = self.anchor_generator(tuple(batch.shape[-2:]), fl)
        n = [f.shape[-2] * f.shape[-1] * 9 for f in fl]
        out = []
        for b in range(batch.shape[0]):
            sc, rg, an = cls[b].sigmoid().split(n), reg[b].split(n), anchors.split(n)
            d = _one_stage_postprocess(sc, lambda lvl, idx: decode_boxes(rg[lvl][idx], an[lvl][idx])[:, 0], sizes[b], *self.cfg)
            d["boxes"] = DetectionTransform.rescale(d["boxes"], sizes[b], orig[b])
            out.append(d)
        return out


def retinanet_resnet50_fpn(num_classes=91, **kw): return RetinaNet(num_classes, **kw)      # noqa: E704


class FcosClassificationHead(_TowerHead):
    def __init__(self, ch, num_classes):
        super().__init__(ch, num_classes, 32)
        self.cls_logits = nn.Conv2d(ch, num_classes, 3, padding=1)

    def forward(self, feats):
        return _flatten_levels([self.cls_logits(self.conv(f)) for f in feats], self.out)


class FcosRegressionHead(_TowerHead):
    def __init__(self, ch):
        super().__init__(ch, 4, 32)
        self.bbox_reg, self.bbox_ctrness = nn.Conv2d(ch, 4, 3, padding=1), nn.Conv2d(ch, 1, 3, padding=1)

    def forward(self, feats):
        ts = [self.conv(f) for f in feats]
        return _flatten_levels([F.relu(self.bbox_reg(t)) for t in ts], 4), _flatten_levels([self.bbox_ctrness(t) for t in ts], 1)


class FcosHead(nn.Module):
    def __init__(self, ch, num_classes):
        super().__init__()
        self.classification_head, self.regression_head = FcosClassificationHead(ch, num_classes), FcosRegressionHead(ch)


class Fcos(nn.Module):
    def __init__(self, num_classes=91, min_size=800, max_size=1333, score_thresh=0.2, nms_thresh=0.6, detections_per_img=100, topk_candidates=1000):
        super().__init__()
        self.transform = DetectionTransform(min_size, max_size)
        self.backbone = BackboneWithFPN((2, 3, 4), 256, LastLevelP6P7(256, 256))
        self.anchor_generator = AnchorGenerator(((8,), (16,), (32,), (64,), (128,)), ((1.0,),) * 5)
        self.head = FcosHead(256, num_classes)
        self.cfg = (score_thresh, topk_candidates, nms_thresh, detections_per_img)

    @torch.no_grad()
    def forward(self, images):
        orig = [tuple(im.shape[-2:]) for im in images]
        batch, sizes = self.transform(images)
        fl = list(self.backbone(batch).values())
        cls = self.head.classification_head(fl)
        reg, ctr = self.head.regression_head(fl)
        anchors = self.anchor_generator(tuple(batch.shape[-2:]), fl)
        n = [f.shape[-2] * f.shape[-1] for f in fl]
        out = []
        for b in range(batch.shape[0]):
            sc = torch.sqrt(cls[b].sigmoid() * ctr[b].sigmoid()).split(n)
            rg, an = reg[b].split(n), anchors.split(n)

            def boxes(lvl, idx):
                a = an[lvl][idx]
                cx, cy, sz = (a[:, 0] + a[:, 2]) / 2, (a[:, 1] + a[:, 3]) / 2, (a[:, 2] - a[:, 0])[:, None]
                d = rg[lvl][idx] * sz                                # (l, t, r, b) distances in units of the level's stride box
                return torch.stack([cx - d[:, 0], cy - d[:, 1], cx + d[:, 2], cy + d[:, 3]], 1)
            d = _one_stage_postprocess(sc, boxes, sizes[b], *self.cfg)
            d["boxes"] = DetectionTransform.rescale(d["boxes"], sizes[b], orig[b])
            out.append(d)
        return out


def fcos_resnet50_fpn(num_classes=91, **kw): return Fcos(num_classes, **kw)                # noqa: E704


# ----------------------------------------------------------------------------------------------------------------------
# SSD300
# ----------------------------------------------------------------------------------------------------------------------
class DefaultBoxGenerator(nn.Module):
    def __init__(self, aspect_ratios=((2,), (2, 3), (2, 3), (2, 3), (2,), (2,)), scales=(0.07, 0.15, 0.33, 0.51, 0.69, 0.87, 1.05), steps=(8, 16, 32, 64, 100, 300)):
        super().__init__()
        self.aspect_ratios, self.scales, self.steps = aspect_ratios, scales, steps

    def num_anchors_per_location(self):
        return [2 + 2 * len(r) for r in self.aspect_ratios]

    def forward(self, image_size: Tuple[int, int], grid_sizes: Sequence[Tuple[int, int]]) -> torch.Tensor:
        out = []
        for k, (gh, gw) in enumerate(grid_sizes):
            sk, sk1 = self.scales[k], self.scales[k + 1]
            wh = [(sk, sk), (math.sqrt(sk * sk1),) * 2]
            for r in self.aspect_ratios[k]:
                sq = math.sqrt(r)
                wh += [(sk * sq, sk / sq), (sk / sq, sk * sq)]
            wh_t = torch.tensor(wh).clamp(0, 1)
            fy, fx = (image_size[0] / self.steps[k], image_size[1] / self.steps[k]) if self.steps else (gh, gw)
            ys, xs = torch.meshgrid((torch.arange(gh) + 0.5) / fy, (torch.arange(gw) + 0.5) / fx, indexing="ij")
            ctr = torch.stack([xs, ys], -1).view(-1, 1, 2).expand(-1, len(wh), 2)
            out.append(torch.cat([ctr, wh_t[None].expand(gh * gw, -1, 2)], -1).reshape(-1, 4))
        cxcywh = torch.cat(out)
        boxes = torch.cat([cxcywh[:, :2] - cxcywh[:, 2:] / 2, cxcywh[:, :2] + cxcywh[:, 2:] / 2], 1)
        return boxes * torch.tensor([image_size[1], image_size[0], image_size[1], image_size[0]])


class _SsdVggBackbone(nn.Module):
    def __init__(self):
        super().__init__()
        cfg = [64, 64, "M", 128, 128, "M", 256, 256, 256, "C", 512, 512, 512, "M", 512, 512, 512]
        layers, c = [], 3
        for v in cfg:
            if v == "M":
                layers.append(nn.MaxPool2d(2, 2))
            elif v == "C":
                layers.append(nn.MaxPool2d(2, 2, ceil_mode=True))
            else:
                layers += [nn.Conv2d(c, v, 3, padding=1), nn.ReLU()]
                c = v
        self.scale_weight = nn.Parameter(torch.ones(512) * 20)
        self.features = nn.Sequential(*layers[:23])          # up to conv4_3 + ReLU
        fc = nn.Sequential(nn.MaxPool2d(3, 1, 1), nn.Conv2d(512, 1024, 3, padding=6, dilation=6), nn.ReLU(), nn.Conv2d(1024, 1024, 1), nn.ReLU())
        def extra(cin, mid, cout, k2, s2, p2):
            return nn.Sequential(nn.Conv2d(cin, mid, 1), nn.ReLU(), nn.Conv2d(mid, cout, k2, s2, p2), nn.ReLU())
        self.extra = nn.ModuleList([nn.Sequential(*layers[23:], fc), extra(1024, 256, 512, 3, 2, 1), extra(512, 128, 256, 3, 2, 1), extra(256, 128, 256, 3, 1, 0),
                                    extra(256, 128, 256, 3, 1, 0)])

    def forward(self, x):
        x = self.features(x)
        out = [self.scale_weight.view(1, -1, 1, 1) * F.normalize(x, dim=1)]
        for blk in self.extra:
            x = blk(x)
            out.append(x)
        return out


class _SsdScoringHead(nn.Module):
    def __init__(self, chans, anchors, cols):
        super().__init__()
        self.module_list = nn.ModuleList([nn.Conv2d(c, a * cols, 3, padding=1) for c, a in zip(chans, anchors)])
        self.cols = cols

    def forward(self, feats):
        return _flatten_levels([m(f) for m, f in zip(self.module_list, feats)], self.cols)


class _SsdHead(nn.Module):
    def __init__(self, chans, anchors, num_classes):
        super().__init__()
        self.classification_head, self.regression_head = _SsdScoringHead(chans, anchors, num_classes), _SsdScoringHead(chans, anchors, 4)


class Ssd300(nn.Module):
    def __init__(self, num_classes=91, score_thresh=0.01, nms_thresh=0.45, detections_per_img=200, topk_candidates=400):
        super().__init__()
        self.transform = DetectionTransform(mean=(0.48235, 0.45882, 0.40784), std=(1 / 255,) * 3, divisor=1, fixed_size=(300, 300))
        self.backbone = _SsdVggBackbone()
        self.anchor_generator = DefaultBoxGenerator()
        self.head = _SsdHead([512, 1024, 512, 256, 256, 256], self.anchor_generator.num_anchors_per_location(), num_classes)
        self.cfg = (score_thresh, nms_thresh, detections_per_img, topk_candidates)

    @torch.no_grad()
    def forward(self, images):
        orig = [tuple(im.shape[-2:]) for im in images]
        batch, sizes = self.transform(images)
        fl = self.backbone(batch)
        cls, reg = self.head.classification_head(fl), self.head.regression_head(fl)
        anchors = self.anchor_generator((300, 300), [tuple(f.shape[-2:]) for f in fl]).to(batch.device)
        st, nt, dets, topk = self.cfg
        out = []
        for b in range(batch.shape[0]):
            boxes = V.clip_boxes_to_image(decode_boxes(reg[b], anchors, (10.0, 10.0, 5.0, 5.0))[:, 0], (300, 300))
            scores = F.softmax(cls[b], -1)
            bl, sl, ll = [], [], []
            for c in range(1, scores.shape[1]):
                k = scores[:, c] > st
                s = scores[k, c]
                t = s.topk(min(topk, len(s)))
                bl.append(boxes[k][t.indices])
                sl.append(t.values)
                ll.append(torch.full_like(t.values, c, dtype=torch.int64))
            bx, sc, lb = torch.cat(bl), torch.cat(sl), torch.cat(ll)
            k = V.batched_nms(bx, sc, lb, nt)[:dets]
            out.append(SsdDetections(boxes=DetectionTransform.rescale(bx[k], (300, 300), orig[b]), scores=sc[k], labels=lb[k]))
        return out


def ssd300_vgg16(num_classes=91, **kw): return Ssd300(num_classes, **kw)                    # noqa: E704


# the reference's names for the heads (rpn.rs, faster_rcnn.rs:105, mask_rcnn.rs)
RpnHead, TwoMlpHead, MaskHead, MaskPredictor = RPNHead, TwoMLPHead, MaskRCNNHeads, MaskRCNNPredictor
