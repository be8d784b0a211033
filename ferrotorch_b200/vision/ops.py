"""Detection / box operators: conversions, IoU family, NMS, RoI align / pool, focal losses (plain compute, any device).

Reference parity: ferrotorch-vision/src/ops.rs:48-908.
"""
from __future__ import annotations

import math
from typing import List, Tuple

import torch
import torch.nn.functional as F

from ..errors import InvalidArgument


def box_convert(boxes: torch.Tensor, in_fmt: str, out_fmt: str) -> torch.Tensor:
    if in_fmt == out_fmt:
        return boxes.clone()
    if in_fmt == "xywh":
        x, y, w, h = boxes.unbind(-1)
        xyxy = torch.stack([x, y, x + w, y + h], -1)
    elif in_fmt == "cxcywh":
        cx, cy, w, h = boxes.unbind(-1)
        xyxy = torch.stack([cx - w / 2, cy - h / 2, cx + w / 2, cy + h / 2], -1)
    elif in_fmt == "xyxy":
        xyxy = boxes
    else:
        raise InvalidArgument(f"unknown box format {in_fmt}")
    x1, y1, x2, y2 = xyxy.unbind(-1)
    if out_fmt == "xyxy":
        return xyxy
    if out_fmt == "xywh":
        return torch.stack([x1, y1, x2 - x1, y2 - y1], -1)
    if out_fmt == "cxcywh":
        return torch.stack([(x1 + x2) / 2, (y1 + y2) / 2, x2 - x1, y2 - y1], -1)
    raise InvalidArgument(f"unknown box format {out_fmt}")


def box_area(b: torch.Tensor) -> torch.Tensor:
    return (b[..., 2] - b[..., 0]) * (b[..., 3] - b[..., 1])


def _inter_union(a, b):
    lt = torch.max(a[:, None, :2], b[None, :, :2])
    rb = torch.min(a[:, None, 2:], b[None, :, 2:])
    inter = (rb - lt).clamp(min=0).prod(-1)
    return inter, box_area(a)[:, None] + box_area(b)[None] - inter


def box_iou(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    i, u = _inter_union(a, b)
    return i / u


def generalized_box_iou(a, b):
    i, u = _inter_union(a, b)
    lt = torch.min(a[:, None, :2], b[None, :, :2])
    rb = torch.max(a[:, None, 2:], b[None, :, 2:])
    c = (rb - lt).clamp(min=0).prod(-1)
    return i / u - (c - u) / c


def distance_box_iou(a, b, eps: float = 1e-7):
    i, u = _inter_union(a, b)
    lt = torch.min(a[:, None, :2], b[None, :, :2])
    rb = torch.max(a[:, None, 2:], b[None, :, 2:])
    diag = ((rb - lt) ** 2).sum(-1) + eps
    ca, cb = (a[:, :2] + a[:, 2:]) / 2, (b[:, :2] + b[:, 2:]) / 2
    return i / u - ((ca[:, None] - cb[None]) ** 2).sum(-1) / diag


def complete_box_iou(a, b, eps: float = 1e-7):
    iou = box_iou(a, b)
    diou = distance_box_iou(a, b, eps)
    wa, ha = a[:, 2] - a[:, 0], a[:, 3] - a[:, 1]
    wb, hb = b[:, 2] - b[:, 0], b[:, 3] - b[:, 1]
    v = (4 / math.pi ** 2) * (torch.atan(wa / ha)[:, None] - torch.atan(wb / hb)[None]) ** 2
    with torch.no_grad():
        alpha = v / (1 - iou + v + eps)
    return diou - alpha * v


def clip_boxes_to_image(boxes: torch.Tensor, size: Tuple[int, int]) -> torch.Tensor:
    h, w = size
    x = boxes[..., 0::2].clamp(0, w)
    y = boxes[..., 1::2].clamp(0, h)
    return torch.stack([x[..., 0], y[..., 0], x[..., 1], y[..., 1]], -1)


def remove_small_boxes(boxes: torch.Tensor, min_size: float) -> torch.Tensor:
    w, h = boxes[:, 2] - boxes[:, 0], boxes[:, 3] - boxes[:, 1]
    return torch.where((w >= min_size) & (h >= min_size))[0]


def nms(boxes: torch.Tensor, scores: torch.Tensor, iou_threshold: float) -> torch.Tensor:
    """Greedy non-maximum suppression; returns kept indices in decreasing score order. CPU boxes run the native sorted sweep (O(N) memory);
    CUDA boxes the mask + on-device sweep kernels."""
    if boxes.numel() == 0:
        return torch.empty(0, dtype=torch.long, device=boxes.device)
    # a stable sort: tied scores keep their input order, so the host and the device sweep visit the boxes in the same order
    order = scores.argsort(descending=True, stable=True)
    b = boxes[order].float().contiguous()
    n = len(b)
    if boxes.is_cuda:
        from .. import _lib
        words = (n + 63) // 64
        mask = torch.empty(n * words, dtype=torch.int64, device=boxes.device)
        keep = torch.empty(n, dtype=torch.uint8, device=boxes.device)
        _lib.call("ft_nms_sorted", b, n, float(iou_threshold), mask, keep, None, _lib.S())
        return order[keep.bool()]
    import ctypes
    from .. import _lib
    fn = _lib.runtime().ft_nms_sorted_f32
    fn.restype = ctypes.c_int64
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p]
    keep = torch.empty(n, dtype=torch.uint8)
    fn(b.data_ptr(), n, float(iou_threshold), keep.data_ptr())
    return order[keep.bool()]


def batched_nms(boxes, scores, idxs, iou_threshold: float):
    """Class-wise NMS: a coordinate offset per class for small inputs, a per-class loop above 4000 boxes (bounded suppression work)."""
    if boxes.numel() == 0:
        return torch.empty(0, dtype=torch.long, device=boxes.device)
    if len(boxes) <= 4000:
        off = idxs.to(boxes) * (boxes.max() + 1)
        return nms(boxes + off[:, None], scores, iou_threshold)
    keep = torch.zeros(len(boxes), dtype=torch.bool, device=boxes.device)
    for c in torch.unique(idxs):
        sel = torch.where(idxs == c)[0]
        keep[sel[nms(boxes[sel], scores[sel], iou_threshold)]] = True
    k = torch.where(keep)[0]
    return k[scores[k].argsort(descending=True, stable=True)]


def sigmoid_focal_loss(inputs, targets, alpha: float = 0.25, gamma: float = 2.0, reduction: str = "none"):
    p = torch.sigmoid(inputs)
    ce = F.binary_cross_entropy_with_logits(inputs, targets, reduction="none")
    pt = p * targets + (1 - p) * (1 - targets)
    loss = ce * (1 - pt) ** gamma
    if alpha >= 0:
        loss = (alpha * targets + (1 - alpha) * (1 - targets)) * loss
    return loss.mean() if reduction == "mean" else loss.sum() if reduction == "sum" else loss


def focal_loss(logits, target, gamma: float = 2.0, alpha=None, reduction: str = "mean"):
    """Multi-class focal loss on ``[N, C]`` logits with integer targets."""
    logp = F.log_softmax(logits, -1)
    lp = logp.gather(1, target.view(-1, 1)).squeeze(1)
    loss = -((1 - lp.exp()) ** gamma) * lp
    if alpha is not None:
        loss = loss * torch.as_tensor(alpha, device=logits.device, dtype=logits.dtype)[target]
    return loss.mean() if reduction == "mean" else loss.sum() if reduction == "sum" else loss


def roi_align(feat: torch.Tensor, rois: torch.Tensor, output_size, spatial_scale: float = 1.0, sampling_ratio: int = 2, aligned: bool = False):
    """``feat`` ``[N,C,H,W]``, ``rois`` ``[K,5]`` (batch index, x1, y1, x2, y2) -> ``[K,C,ph,pw]`` by bilinear sampling."""
    ph, pw = (output_size, output_size) if isinstance(output_size, int) else output_size
    N, C, H, W = feat.shape
    K = rois.shape[0]
    off = 0.5 if aligned else 0.0
    x1, y1, x2, y2 = (rois[:, i] * spatial_scale - off for i in range(1, 5))
    rw, rh = x2 - x1, y2 - y1
    if not aligned:
        rw, rh = rw.clamp(min=1.0), rh.clamp(min=1.0)
    sr = sampling_ratio if sampling_ratio > 0 else 2
    iy = (torch.arange(ph * sr, device=feat.device, dtype=feat.dtype) + 0.5) / sr
    ix = (torch.arange(pw * sr, device=feat.device, dtype=feat.dtype) + 0.5) / sr
    ys = y1[:, None] + iy[None] * (rh / ph)[:, None]
    xs = x1[:, None] + ix[None] * (rw / pw)[:, None]

    def bilinear(img, y, x):      # img [C,H,W]; y [P], x [Q]
        valid_y, valid_x = (y >= -1) & (y <= H), (x >= -1) & (x <= W)
        y, x = y.clamp(0, H - 1), x.clamp(0, W - 1)
        y0, x0 = y.floor().long(), x.floor().long()
        y1_, x1_ = (y0 + 1).clamp(max=H - 1), (x0 + 1).clamp(max=W - 1)
        ly, lx = (y - y0).view(1, -1, 1), (x - x0).view(1, 1, -1)
        v = (img[:, y0][:, :, x0] * (1 - ly) * (1 - lx) + img[:, y0][:, :, x1_] * (1 - ly) * lx + img[:, y1_][:, :, x0] * ly * (1 - lx)
             + img[:, y1_][:, :, x1_] * ly * lx)
        return v * (valid_y.view(1, -1, 1) & valid_x.view(1, 1, -1))
    out = feat.new_zeros(K, C, ph, pw)
    for k in range(K):
        v = bilinear(feat[int(rois[k, 0])], ys[k], xs[k])
        out[k] = v.view(C, ph, sr, pw, sr).mean((2, 4))
    return out


def roi_pool(feat: torch.Tensor, rois: torch.Tensor, output_size, spatial_scale: float = 1.0):
    ph, pw = (output_size, output_size) if isinstance(output_size, int) else output_size
    N, C, H, W = feat.shape
    out = feat.new_zeros(rois.shape[0], C, ph, pw)
    for k in range(rois.shape[0]):
        b = int(rois[k, 0])
        # half-way cases round away from zero (the C rule), not to even
        x1, y1, x2, y2 = [int(math.copysign(math.floor(abs(float(v) * spatial_scale) + 0.5), float(v))) for v in rois[k, 1:]]
        rw, rh = max(x2 - x1 + 1, 1), max(y2 - y1 + 1, 1)
        for i in range(ph):
            hs, he = min(max(y1 + int(math.floor(i * rh / ph)), 0), H), min(max(y1 + int(math.ceil((i + 1) * rh / ph)), 0), H)
            for j in range(pw):
                ws, we = min(max(x1 + int(math.floor(j * rw / pw)), 0), W), min(max(x1 + int(math.ceil((j + 1) * rw / pw)), 0), W)
                if he > hs and we > ws:
                    out[k, :, i, j] = feat[b, :, hs:he, ws:we].amax((1, 2))
    return out


def roi_align_with_aligned(feat, rois, output_size, spatial_scale: float = 1.0, sampling_ratio: int = 2, aligned: bool = True):
    """:func:`roi_align` with the half-pixel switch spelled out: ``aligned=True`` shifts box coordinates by half a pixel (newer detectors),
    ``False`` is the legacy rule of the published COCO R-CNN weights (ferrotorch-vision/src/ops.rs:773)."""
    return roi_align(feat, rois, output_size, spatial_scale, sampling_ratio, aligned)
