"""Loss layers (ferrotorch-nn/src/loss.rs:48-2290). Each loss is written out from its definition on tensor primitives and
differentiated by autograd; the cross-entropy hot path lives with the fused kernel in ``layers.CrossEntropyLoss``."""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..errors import InvalidArgument, ShapeMismatch
from .module import Module


def _reduce(v: torch.Tensor, reduction: str) -> torch.Tensor:
    if reduction == "mean":
        return v.mean()
    if reduction == "sum":
        return v.sum()
    if reduction == "none":
        return v
    raise InvalidArgument(f"unknown reduction {reduction!r} (mean | sum | none)")


def _same(a: torch.Tensor, b: torch.Tensor, what: str) -> None:
    if a.shape != b.shape:
        try:
            torch.broadcast_shapes(a.shape, b.shape)
        except RuntimeError:
            raise ShapeMismatch(f"{what}: input {list(a.shape)} and target {list(b.shape)} do not broadcast") from None


class _Loss(Module):
    def __init__(self, reduction: str = "mean"):
        super().__init__()
        if hasattr(reduction, "value"):
            reduction = reduction.value
        if reduction not in ("mean", "sum", "none"):
            raise InvalidArgument(f"unknown reduction {reduction!r} (mean | sum | none)")
        self.reduction = reduction


# -- functional forms ---------------------------------------------------------------------------------------------------------------------
def mse_loss(x, y, reduction="mean"):
    _same(x, y, "mse_loss")
    d = x - y
    return _reduce(d * d, reduction)


def l1_loss(x, y, reduction="mean"):
    _same(x, y, "l1_loss")
    return _reduce(torch.abs(x - y), reduction)


def smooth_l1_loss(x, y, reduction="mean", beta: float = 1.0):
    _same(x, y, "smooth_l1_loss")
    if beta < 0:
        raise InvalidArgument("smooth_l1_loss: beta must be >= 0")
    d = torch.abs(x - y)
    if beta == 0:
        return _reduce(d, reduction)
    return _reduce(torch.where(d < beta, 0.5 * d * d / beta, d - 0.5 * beta), reduction)


def huber_loss(x, y, reduction="mean", delta: float = 1.0):
    _same(x, y, "huber_loss")
    if delta <= 0:
        raise InvalidArgument("huber_loss: delta must be > 0")
    d = torch.abs(x - y)
    return _reduce(torch.where(d <= delta, 0.5 * d * d, delta * (d - 0.5 * delta)), reduction)


def binary_cross_entropy(p, y, weight=None, reduction="mean"):
    _same(p, y, "binary_cross_entropy")
    # log terms are clamped at -100 so that p = 0 or 1 gives a finite loss and gradient
    v = -(y * torch.clamp_min(torch.log(p), -100.0) + (1 - y) * torch.clamp_min(torch.log1p(-p), -100.0))
    if weight is not None:
        v = v * weight
    return _reduce(v, reduction)


def binary_cross_entropy_with_logits(x, y, weight=None, pos_weight=None, reduction="mean"):
    _same(x, y, "binary_cross_entropy_with_logits")
    # softplus(-x) = log(1 + exp(-x)), stable for both signs
    sp = torch.clamp_min(-x, 0) + torch.log1p(torch.exp(-torch.abs(x)))
    if pos_weight is None:
        v = (1 - y) * x + sp
    else:
        v = (1 - y) * x + (1 + (pos_weight - 1) * y) * sp
    if weight is not None:
        v = v * weight
    return _reduce(v, reduction)


def kl_div(log_q, p, reduction="mean", log_target: bool = False):
    """Pointwise ``p * (log p - log_q)``; ``batchmean`` divides the sum by the batch size."""
    _same(log_q, p, "kl_div")
    if log_target:
        v = torch.exp(p) * (p - log_q)
    else:
        v = torch.where(p > 0, p * (torch.log(torch.where(p > 0, p, torch.ones_like(p))) - log_q), torch.zeros_like(log_q))
    if reduction == "batchmean":
        return v.sum() / max(1, log_q.shape[0] if log_q.dim() else 1)
    return _reduce(v, reduction)


def nll_loss(logp, target, weight=None, ignore_index: int = -100, reduction="mean"):
    """``logp``: ``[N, C]`` or ``[N, C, d1, ...]`` log-probabilities, ``target``: ``[N]`` or ``[N, d1, ...]`` class indices."""
    if logp.dim() == 1:
        logp, target = logp.unsqueeze(0), target.reshape(1)
    if logp.dim() < 2 or target.shape != logp.shape[:1] + logp.shape[2:]:
        raise ShapeMismatch(f"nll_loss: input {list(logp.shape)} vs target {list(target.shape)}")
    C = logp.shape[1]
    valid = target != ignore_index
    t = torch.where(valid, target, torch.zeros_like(target))
    if bool(((t < 0) | (t >= C)).any()):
        raise InvalidArgument(f"nll_loss: target out of range [0, {C})")
    picked = -logp.gather(1, t.unsqueeze(1)).squeeze(1)
    w = torch.ones_like(picked) if weight is None else weight.to(picked.dtype)[t]
    w = w * valid.to(picked.dtype)
    v = picked * w
    if reduction == "mean":
        return v.sum() / w.sum()
    return _reduce(v, reduction)


def cosine_similarity(a, b, dim: int = 1, eps: float = 1e-8):
    na = torch.clamp_min(torch.sqrt((a * a).sum(dim)), eps)
    nb = torch.clamp_min(torch.sqrt((b * b).sum(dim)), eps)
    return (a * b).sum(dim) / (na * nb)


def pairwise_distance(a, b, p: float = 2.0, eps: float = 1e-6, keepdim: bool = False):
    d = torch.abs(a - b + eps)
    if p == float("inf"):
        return d.amax(-1, keepdim=keepdim)
    if p == 1:
        return d.sum(-1, keepdim=keepdim)
    if p == 2:
        return torch.sqrt((d * d).sum(-1, keepdim=keepdim))
    return d.pow(p).sum(-1, keepdim=keepdim).pow(1.0 / p)


def cosine_embedding_loss(a, b, y, margin: float = 0.0, reduction="mean"):
    eps = 1e-12                                   # added to the squared norms, under the root
    cos = (a * b).sum(-1) / torch.sqrt(((a * a).sum(-1) + eps) * ((b * b).sum(-1) + eps))
    v = torch.where(y > 0, 1 - cos, torch.clamp_min(cos - margin, 0))
    return _reduce(v, reduction)


def margin_ranking_loss(a, b, y, margin: float = 0.0, reduction="mean"):
    return _reduce(torch.clamp_min(-y * (a - b) + margin, 0), reduction)


def triplet_margin_loss(anchor, positive, negative, margin: float = 1.0, p: float = 2.0, eps: float = 1e-6, swap: bool = False, reduction="mean"):
    dp = pairwise_distance(anchor, positive, p, eps)
    dn = pairwise_distance(anchor, negative, p, eps)
    if swap:
        dn = torch.minimum(dn, pairwise_distance(positive, negative, p, eps))
    return _reduce(torch.clamp_min(margin + dp - dn, 0), reduction)


def hinge_embedding_loss(x, y, margin: float = 1.0, reduction="mean"):
    v = torch.where(y == 1, x, torch.zeros_like(x)) + torch.where(y == -1, torch.clamp_min(margin - x, 0), torch.zeros_like(x))
    return _reduce(v, reduction)


def poisson_nll_loss(x, y, log_input: bool = True, full: bool = False, eps: float = 1e-8, reduction="mean"):
    v = (torch.exp(x) - y * x) if log_input else (x - y * torch.log(x + eps))
    if full:
        # Stirling term y log y - y + log(2 pi y)/2 for y > 1
        ys = torch.where(y > 1, y, torch.ones_like(y))
        v = v + torch.where(y > 1, ys * torch.log(ys) - ys + 0.5 * torch.log(2 * math.pi * ys), torch.zeros_like(y))
    return _reduce(v, reduction)


def gaussian_nll_loss(x, y, var, full: bool = False, eps: float = 1e-6, reduction="mean"):
    if bool((var < 0).any()):
        raise InvalidArgument("gaussian_nll_loss: var has negative entries")
    if var.shape != x.shape and var.shape == x.shape[:-1]:
        var = var.unsqueeze(-1)                               # one variance per row
    v_ = var + (torch.clamp_min(var, eps) - var).detach()     # clamped value, gradient of the unclamped variance
    out = 0.5 * (torch.log(v_) + (x - y) ** 2 / v_)
    if full:
        out = out + 0.5 * math.log(2 * math.pi)
    return _reduce(out, reduction)


def multi_margin_loss(x, target, p: int = 1, margin: float = 1.0, weight=None, reduction="mean"):
    if p not in (1, 2):
        raise InvalidArgument("multi_margin_loss: p must be 1 or 2")
    if x.dim() == 1:
        x, target = x.unsqueeze(0), target.reshape(1)
    N, C = x.shape
    xt = x.gather(1, target.unsqueeze(1))
    v = torch.clamp_min(margin - xt + x, 0)
    if p == 2:
        v = v * v
    if weight is not None:
        v = v * weight[target].unsqueeze(1)
    mask = torch.ones_like(v).scatter_(1, target.unsqueeze(1), 0.0)
    return _reduce((v * mask).sum(1) / C, reduction)


def multilabel_soft_margin_loss(x, y, weight=None, reduction="mean"):
    from .activation import logsigmoid
    v = -(y * logsigmoid(x) + (1 - y) * logsigmoid(-x))
    if weight is not None:
        v = v * weight
    return _reduce(v.mean(-1), reduction)


def ctc_loss(log_probs, targets, input_lengths, target_lengths, blank: int = 0, reduction="mean", zero_infinity: bool = False):
    """Connectionist temporal classification. ``log_probs``: ``[T, N, C]`` (or ``[T, C]``) log-softmax outputs; ``targets``: padded ``[N, S]`` or the
    concatenation of all label sequences. The forward variable runs over the blank-extended label sequence in log space; autograd
    differentiates the recursion."""
    if log_probs.dim() == 2:
        log_probs = log_probs.unsqueeze(1)
        targets = targets.reshape(1, -1) if targets.dim() == 1 else targets
    T, N, C = log_probs.shape
    il = torch.as_tensor(input_lengths, dtype=torch.long).reshape(-1).tolist()
    tl = torch.as_tensor(target_lengths, dtype=torch.long).reshape(-1).tolist()
    if len(il) != N or len(tl) != N:
        raise ShapeMismatch("ctc_loss: one input length and one target length per batch element")
    if targets.dim() == 1:
        offs = [0]
        for n in tl:
            offs.append(offs[-1] + n)
        seqs = [targets[offs[i]: offs[i + 1]] for i in range(N)]
    else:
        seqs = [targets[i, : tl[i]] for i in range(N)]
    S = max(tl) if tl else 0
    L = 2 * S + 1
    dev, dt = log_probs.device, log_probs.dtype
    neg = float("-inf")
    ext = torch.full((N, L), blank, dtype=torch.long, device=dev)
    for i, s in enumerate(seqs):
        if len(s):
            ext[i, 1: 2 * len(s): 2] = s.to(dev)
    # a skip from s-2 is allowed onto a label that differs from the label two places back
    skip = torch.zeros(N, L, dtype=torch.bool, device=dev)
    if L > 2:
        skip[:, 2:] = (ext[:, 2:] != blank) & (ext[:, 2:] != ext[:, :-2])
    lp = log_probs.gather(2, ext.unsqueeze(0).expand(T, N, L))             # [T, N, L]
    alpha = torch.full((N, L), neg, device=dev, dtype=dt)
    init = torch.zeros(N, L, dtype=torch.bool, device=dev)
    init[:, 0] = True
    if L > 1:
        init[:, 1] = torch.tensor([n > 0 for n in tl], device=dev)
    alpha = torch.where(init, lp[0], alpha)
    ilt = torch.tensor(il, device=dev)
    negs = torch.full((N, 1), neg, device=dev, dtype=dt)
    for t in range(1, T):
        a1 = torch.cat([negs, alpha[:, :-1]], 1)
        a2 = torch.cat([negs, negs, alpha[:, :-2]], 1) if L > 2 else torch.full_like(alpha, neg)
        a2 = torch.where(skip, a2, torch.full_like(a2, neg))
        stack = torch.stack([alpha, a1, a2], 0)
        m = stack.amax(0)
        msafe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        new = msafe + torch.log(torch.exp(stack - msafe).sum(0)) + lp[t]
        new = torch.where(torch.isinf(m), torch.full_like(new, neg), new)
        alpha = torch.where((t < ilt).unsqueeze(1), new, alpha)             # sequences shorter than T stop advancing
    tlt = torch.tensor(tl, device=dev)
    last = alpha.gather(1, (2 * tlt).unsqueeze(1)).squeeze(1)
    prev = alpha.gather(1, torch.clamp_min(2 * tlt - 1, 0).unsqueeze(1)).squeeze(1)
    prev = torch.where(tlt > 0, prev, torch.full_like(prev, neg))
    m = torch.maximum(last, prev)
    msafe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    ll = msafe + torch.log(torch.exp(last - msafe) + torch.exp(prev - msafe))
    ll = torch.where(torch.isinf(m), torch.full_like(ll, neg), ll)
    loss = -ll
    if zero_infinity:
        loss = torch.where(torch.isinf(loss), torch.zeros_like(loss), loss)
    if reduction == "mean":
        return (loss / torch.clamp_min(tlt, 1).to(dt)).mean()
    return _reduce(loss, reduction)


# -- modules -----------------------------------------------------------------------------------------------------------------------------
class MSELoss(_Loss):
    def forward(self, x, y):
        return mse_loss(x, y, self.reduction)


class L1Loss(_Loss):
    def forward(self, x, y):
        return l1_loss(x, y, self.reduction)


class SmoothL1Loss(_Loss):
    def __init__(self, reduction: str = "mean", beta: float = 1.0):
        super().__init__(reduction)
        self.beta = beta

    def forward(self, x, y):
        return smooth_l1_loss(x, y, self.reduction, self.beta)


class HuberLoss(_Loss):
    def __init__(self, reduction: str = "mean", delta: float = 1.0):
        super().__init__(reduction)
        self.delta = delta

    def forward(self, x, y):
        return huber_loss(x, y, self.reduction, self.delta)


class BCELoss(_Loss):
    def __init__(self, weight: Optional[torch.Tensor] = None, reduction: str = "mean"):
        super().__init__(reduction)
        self.register_buffer("weight", weight)

    def forward(self, p, y):
        return binary_cross_entropy(p, y, self.weight, self.reduction)


class BCEWithLogitsLoss(_Loss):
    def __init__(self, weight: Optional[torch.Tensor] = None, reduction: str = "mean", pos_weight: Optional[torch.Tensor] = None):
        super().__init__(reduction)
        self.register_buffer("weight", weight)
        self.register_buffer("pos_weight", pos_weight)

    def forward(self, x, y):
        return binary_cross_entropy_with_logits(x, y, self.weight, self.pos_weight, self.reduction)


class KLDivLoss(Module):
    def __init__(self, reduction: str = "mean", log_target: bool = False):
        super().__init__()
        if reduction not in ("mean", "sum", "none", "batchmean"):
            raise InvalidArgument(f"unknown reduction {reduction!r}")
        self.reduction, self.log_target = reduction, log_target

    def forward(self, log_q, p):
        return kl_div(log_q, p, self.reduction, self.log_target)


class NLLLoss(_Loss):
    def __init__(self, weight: Optional[torch.Tensor] = None, ignore_index: int = -100, reduction: str = "mean"):
        super().__init__(reduction)
        self.register_buffer("weight", weight)
        self.ignore_index = ignore_index

    def forward(self, logp, target):
        return nll_loss(logp, target, self.weight, self.ignore_index, self.reduction)


class CosineEmbeddingLoss(_Loss):
    def __init__(self, margin: float = 0.0, reduction: str = "mean"):
        super().__init__(reduction)
        self.margin = margin

    def forward(self, a, b, y):
        return cosine_embedding_loss(a, b, y, self.margin, self.reduction)


class MarginRankingLoss(_Loss):
    def __init__(self, margin: float = 0.0, reduction: str = "mean"):
        super().__init__(reduction)
        self.margin = margin

    def forward(self, a, b, y):
        return margin_ranking_loss(a, b, y, self.margin, self.reduction)


class TripletMarginLoss(_Loss):
    def __init__(self, margin: float = 1.0, p: float = 2.0, eps: float = 1e-6, swap: bool = False, reduction: str = "mean"):
        super().__init__(reduction)
        self.margin, self.p, self.eps, self.swap = margin, p, eps, swap

    def forward(self, anchor, positive, negative):
        return triplet_margin_loss(anchor, positive, negative, self.margin, self.p, self.eps, self.swap, self.reduction)


class HingeEmbeddingLoss(_Loss):
    def __init__(self, margin: float = 1.0, reduction: str = "mean"):
        super().__init__(reduction)
        self.margin = margin

    def forward(self, x, y):
        return hinge_embedding_loss(x, y, self.margin, self.reduction)


class PoissonNLLLoss(_Loss):
    def __init__(self, log_input: bool = True, full: bool = False, eps: float = 1e-8, reduction: str = "mean"):
        super().__init__(reduction)
        self.log_input, self.full, self.eps = log_input, full, eps

    def forward(self, x, y):
        return poisson_nll_loss(x, y, self.log_input, self.full, self.eps, self.reduction)


class GaussianNLLLoss(_Loss):
    def __init__(self, full: bool = False, eps: float = 1e-6, reduction: str = "mean"):
        super().__init__(reduction)
        self.full, self.eps = full, eps

    def forward(self, x, y, var):
        return gaussian_nll_loss(x, y, var, self.full, self.eps, self.reduction)


class MultiMarginLoss(_Loss):
    def __init__(self, p: int = 1, margin: float = 1.0, weight: Optional[torch.Tensor] = None, reduction: str = "mean"):
        super().__init__(reduction)
        if p not in (1, 2):
            raise InvalidArgument("MultiMarginLoss: p must be 1 or 2")
        self.p, self.margin = p, margin
        self.register_buffer("weight", weight)

    def forward(self, x, target):
        return multi_margin_loss(x, target, self.p, self.margin, self.weight, self.reduction)


class MultiLabelSoftMarginLoss(_Loss):
    def __init__(self, weight: Optional[torch.Tensor] = None, reduction: str = "mean"):
        super().__init__(reduction)
        self.register_buffer("weight", weight)

    def forward(self, x, y):
        return multilabel_soft_margin_loss(x, y, self.weight, self.reduction)


class CTCLoss(_Loss):
    def __init__(self, blank: int = 0, reduction: str = "mean", zero_infinity: bool = False):
        super().__init__(reduction)
        self.blank, self.zero_infinity = blank, zero_infinity

    def forward(self, log_probs, targets, input_lengths, target_lengths):
        return ctc_loss(log_probs, targets, input_lengths, target_lengths, self.blank, self.reduction, self.zero_infinity)


class CosineSimilarity(Module):
    def __init__(self, dim: int = 1, eps: float = 1e-8):
        super().__init__()
        self.dim, self.eps = dim, eps

    def forward(self, a, b):
        return cosine_similarity(a, b, self.dim, self.eps)


class PairwiseDistance(Module):
    def __init__(self, p: float = 2.0, eps: float = 1e-6, keepdim: bool = False):
        super().__init__()
        self.p, self.eps, self.keepdim = p, eps, keepdim

    def forward(self, a, b):
        return pairwise_distance(a, b, self.p, self.eps, self.keepdim)


__all__ = ["MSELoss", "L1Loss", "SmoothL1Loss", "HuberLoss", "BCELoss", "BCEWithLogitsLoss", "KLDivLoss", "NLLLoss", "CosineEmbeddingLoss",
           "MarginRankingLoss", "TripletMarginLoss", "HingeEmbeddingLoss", "PoissonNLLLoss", "GaussianNLLLoss", "MultiMarginLoss",
           "MultiLabelSoftMarginLoss", "CTCLoss", "CosineSimilarity", "PairwiseDistance"]
