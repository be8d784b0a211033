"""Regression, classification, ranking and clustering metrics on tensors (or arrays), computed in f64 on the host.

Definitions follow scikit-learn, which the reference's metric backend mirrors; the CPU test tier checks every function against scikit-learn.
Reference parity: ferrotorch-ml/src/metrics.rs:63-1180, adapter.rs:52-240.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

from ..errors import InvalidArgument, ShapeMismatch


def _a(x) -> np.ndarray:
    return x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else np.asarray(x)


def _pair(y_true, y_pred, dtype=np.float64) -> Tuple[np.ndarray, np.ndarray]:
    a, b = _a(y_true).astype(dtype).reshape(-1), _a(y_pred).astype(dtype).reshape(-1)
    if a.shape != b.shape:
        raise ShapeMismatch(f"metric inputs differ in length: {a.shape[0]} vs {b.shape[0]}")
    if a.size == 0:
        raise InvalidArgument("metric inputs are empty")
    return a, b


def _labels(y_true, y_pred) -> Tuple[np.ndarray, np.ndarray]:
    a, b = _pair(y_true, y_pred)
    if (a != np.round(a)).any() or (b != np.round(b)).any():
        raise InvalidArgument("class labels must be integers")
    return a.astype(np.int64), b.astype(np.int64)


# -- adapters (adapter.rs) ------------------------------------------------------------------------------------------------------------
def tensor_to_array1(t: torch.Tensor) -> np.ndarray:
    if t.dim() != 1:
        raise ShapeMismatch(f"tensor_to_array1: expected a 1-D tensor, got shape {list(t.shape)}")
    return _a(t).copy()


def tensor_to_array2(t: torch.Tensor) -> np.ndarray:
    if t.dim() != 2:
        raise ShapeMismatch(f"tensor_to_array2: expected a 2-D tensor, got shape {list(t.shape)}")
    return _a(t).copy()


def array1_to_tensor(a, dtype=torch.float32) -> torch.Tensor:
    a = np.asarray(a)
    if a.ndim != 1:
        raise ShapeMismatch(f"array1_to_tensor: expected a 1-D array, got shape {list(a.shape)}")
    return torch.as_tensor(np.ascontiguousarray(a)).to(dtype)


def array2_to_tensor(a, dtype=torch.float32) -> torch.Tensor:
    a = np.asarray(a)
    if a.ndim != 2:
        raise ShapeMismatch(f"array2_to_tensor: expected a 2-D array, got shape {list(a.shape)}")
    return torch.as_tensor(np.ascontiguousarray(a)).to(dtype)


def array1_usize_to_tensor(a, dtype=torch.float32) -> torch.Tensor:
    a = np.asarray(a)
    if a.ndim != 1 or (a < 0).any():
        raise InvalidArgument("array1_usize_to_tensor: a 1-D array of non-negative integers is expected")
    return torch.as_tensor(a.astype(np.int64)).to(dtype)


def tensor_to_array1_usize(t: torch.Tensor) -> np.ndarray:
    a = tensor_to_array1(t).astype(np.float64)
    if (a < 0).any() or (a != np.round(a)).any() or not np.isfinite(a).all():
        raise InvalidArgument("tensor_to_array1_usize: values must be finite non-negative integers")
    return a.astype(np.int64)


# -- regression ----------------------------------------------------------------------------------------------------------------------
def root_mean_squared_error(y_true, y_pred) -> float:
    y, p = _pair(y_true, y_pred)
    return float(np.sqrt(((y - p) ** 2).mean()))


def mean_absolute_percentage_error(y_true, y_pred) -> float:
    y, p = _pair(y_true, y_pred)
    return float((np.abs(y - p) / np.maximum(np.abs(y), np.finfo(np.float64).eps)).mean())


def median_absolute_error(y_true, y_pred) -> float:
    y, p = _pair(y_true, y_pred)
    return float(np.median(np.abs(y - p)))


def max_error(y_true, y_pred) -> float:
    y, p = _pair(y_true, y_pred)
    return float(np.abs(y - p).max())


def explained_variance_score(y_true, y_pred) -> float:
    y, p = _pair(y_true, y_pred)
    num, den = np.var(y - p), np.var(y)
    if den == 0:
        return 1.0 if num == 0 else 0.0
    return float(1.0 - num / den)


# -- classification --------------------------------------------------------------------------------------------------------------------
def _cm(y, p) -> Tuple[np.ndarray, np.ndarray]:
    classes = np.unique(np.concatenate([y, p]))
    idx = {c: i for i, c in enumerate(classes.tolist())}
    cm = np.zeros((len(classes), len(classes)), dtype=np.float64)
    np.add.at(cm, ([idx[v] for v in y.tolist()], [idx[v] for v in p.tolist()]), 1)
    return cm, classes


def hamming_loss(y_true, y_pred) -> float:
    y, p = _labels(y_true, y_pred)
    return float((y != p).mean())


def zero_one_loss(y_true, y_pred, normalize: bool = True) -> float:
    y, p = _labels(y_true, y_pred)
    wrong = float((y != p).sum())
    return wrong / len(y) if normalize else wrong


def balanced_accuracy_score(y_true, y_pred, adjusted: bool = False) -> float:
    y, p = _labels(y_true, y_pred)
    cm, classes = _cm(y, p)
    support = cm.sum(1)
    rec = np.diag(cm)[support > 0] / support[support > 0]
    score = float(rec.mean())
    if adjusted:
        chance = 1.0 / len(rec)
        score = (score - chance) / (1.0 - chance)
    return score


def matthews_corrcoef(y_true, y_pred) -> float:
    y, p = _labels(y_true, y_pred)
    cm, _ = _cm(y, p)
    t, pp, c, s = cm.sum(1), cm.sum(0), np.trace(cm), cm.sum()
    cov_ytyp, cov_ypyp, cov_ytyt = c * s - t @ pp, s * s - pp @ pp, s * s - t @ t
    den = cov_ypyp * cov_ytyt
    return float(cov_ytyp / math.sqrt(den)) if den > 0 else 0.0


def cohen_kappa_score(y_true, y_pred) -> float:
    y, p = _labels(y_true, y_pred)
    cm, _ = _cm(y, p)
    n = cm.sum()
    po, pe = np.trace(cm) / n, float(cm.sum(0) @ cm.sum(1)) / (n * n)
    return float((po - pe) / (1.0 - pe)) if pe != 1.0 else 0.0 if po != 1.0 else float("nan")


def _binary(y_true, y_prob) -> Tuple[np.ndarray, np.ndarray]:
    y, s = _pair(y_true, y_prob)
    if not np.isin(y, (0.0, 1.0)).all():
        raise InvalidArgument("binary metric: y_true must hold 0 / 1 labels")
    return y, s


def brier_score_loss(y_true, y_prob) -> float:
    y, s = _binary(y_true, y_prob)
    if (s < 0).any() or (s > 1).any():
        raise InvalidArgument("brier_score_loss: probabilities must lie in [0, 1]")
    return float(((s - y) ** 2).mean())


def d2_brier_score(y_true, y_prob) -> float:
    """Fraction of the Brier score explained relative to always predicting the positive rate."""
    y, s = _binary(y_true, y_prob)
    ref = float(((y.mean() - y) ** 2).mean())
    return float(1.0 - brier_score_loss(y, s) / ref) if ref > 0 else float("nan")


def top_k_accuracy_score(y_true, y_score, k: int = 2) -> float:
    y = tensor_to_array1_usize(torch.as_tensor(_a(y_true)))
    s = _a(y_score).astype(np.float64)
    if s.ndim != 2 or s.shape[0] != len(y):
        raise ShapeMismatch(f"top_k_accuracy_score: y_score must be [n_samples, n_classes], got shape {list(s.shape)} for {len(y)} labels")
    if not 1 <= k <= s.shape[1] or (y >= s.shape[1]).any():
        raise InvalidArgument(f"top_k_accuracy_score: k = {k} / labels outside the {s.shape[1]} classes")
    true_scores = s[np.arange(len(y)), y]
    better = (s > true_scores[:, None]).sum(1)                # ties resolve in favour of the true class only when fewer than k are strictly better
    return float((better < k).mean())


def average_precision_score(y_true, y_score) -> float:
    """Area under the precision-recall step function: sum over thresholds of ``(R_n - R_{n-1}) * P_n``."""
    y, s = _binary(y_true, y_score)
    if y.sum() == 0:
        raise InvalidArgument("average_precision_score: no positive samples")
    order = np.argsort(-s, kind="mergesort")
    y, s = y[order], s[order]
    last = np.r_[s[1:] != s[:-1], True]                       # one point per distinct threshold
    tp = np.cumsum(y)[last]
    fp = np.cumsum(1 - y)[last]
    prec, rec = tp / (tp + fp), tp / y.sum()
    return float(np.sum(np.diff(np.r_[0.0, rec]) * prec))


def _dcg(rel_sorted: np.ndarray, k: Optional[int]) -> float:
    r = rel_sorted[: k] if k is not None else rel_sorted
    return float((r / np.log2(np.arange(2, len(r) + 2))).sum())


def _tie_averaged_dcg(y: np.ndarray, s: np.ndarray, k: Optional[int]) -> float:
    """DCG with the gains of tied scores averaged over the positions the tie occupies."""
    disc = 1.0 / np.log2(np.arange(2, len(y) + 2))
    if k is not None:
        disc[k:] = 0.0
    order = np.argsort(-s, kind="mergesort")
    ys, ss = y[order], s[order]
    starts = np.flatnonzero(np.r_[True, ss[1:] != ss[:-1]])
    ends = np.r_[starts[1:], len(ss)]
    return float(sum(ys[a:b].mean() * disc[a:b].sum() for a, b in zip(starts, ends)))


def dcg_score(y_true, y_score, k: Optional[int] = None) -> float:
    y, s = _pair(y_true, y_score)
    if k is not None and k < 1:
        raise InvalidArgument("dcg_score: k must be >= 1")
    return _tie_averaged_dcg(y, s, k)


def ndcg_score(y_true, y_score, k: Optional[int] = None) -> float:
    y, s = _pair(y_true, y_score)
    if (y < 0).any():
        raise InvalidArgument("ndcg_score: relevance values must be non-negative")
    ideal = _dcg(np.sort(y)[::-1], k)
    return float(dcg_score(y, s, k) / ideal) if ideal > 0 else 0.0


def _multilabel(y_true, y_score) -> Tuple[np.ndarray, np.ndarray]:
    y, s = _a(y_true).astype(np.float64), _a(y_score).astype(np.float64)
    if y.ndim != 2 or y.shape != s.shape:
        raise ShapeMismatch(f"multilabel metric: [n_samples, n_labels] indicator and scores expected, got {list(y.shape)} and {list(s.shape)}")
    return y, s


def coverage_error(y_true, y_score) -> float:
    y, s = _multilabel(y_true, y_score)
    out = []
    for yi, si in zip(y, s):
        out.append(float((si >= si[yi > 0].min()).sum()) if (yi > 0).any() else 0.0)
    return float(np.mean(out))


def label_ranking_average_precision_score(y_true, y_score) -> float:
    y, s = _multilabel(y_true, y_score)
    total = 0.0
    for yi, si in zip(y, s):
        rel = np.flatnonzero(yi > 0)
        if len(rel) == 0 or len(rel) == len(yi):
            total += 1.0
            continue
        rank = np.array([(si >= si[j]).sum() for j in rel], dtype=np.float64)
        hits = np.array([(si[rel] >= si[j]).sum() for j in rel], dtype=np.float64)
        total += float((hits / rank).mean())
    return total / len(y)


def label_ranking_loss(y_true, y_score) -> float:
    y, s = _multilabel(y_true, y_score)
    total = 0.0
    for yi, si in zip(y, s):
        pos, neg = si[yi > 0], si[yi <= 0]
        if len(pos) == 0 or len(neg) == 0:
            continue
        total += float((neg[None, :] >= pos[:, None]).sum()) / (len(pos) * len(neg))
    return total / len(y)


# -- clustering --------------------------------------------------------------------------------------------------------------------------
def _contingency(a, b) -> np.ndarray:
    ya, yb = _pair(a, b)
    _, ia = np.unique(ya, return_inverse=True)
    _, ib = np.unique(yb, return_inverse=True)
    c = np.zeros((ia.max() + 1, ib.max() + 1), dtype=np.float64)
    np.add.at(c, (ia, ib), 1)
    return c


def _comb2(x):
    return x * (x - 1) / 2.0


def adjusted_rand_score(labels_true, labels_pred) -> float:
    c = _contingency(labels_true, labels_pred)
    n = c.sum()
    sum_ij, sum_a, sum_b = _comb2(c).sum(), _comb2(c.sum(1)).sum(), _comb2(c.sum(0)).sum()
    expected, mx = sum_a * sum_b / _comb2(n) if n > 1 else 0.0, (sum_a + sum_b) / 2.0
    return float((sum_ij - expected) / (mx - expected)) if mx != expected else 1.0


def _entropy(counts: np.ndarray) -> float:
    p = counts[counts > 0] / counts.sum()
    return float(-(p * np.log(p)).sum())


def _mutual_info(c: np.ndarray) -> float:
    n = c.sum()
    nz = c > 0
    outer = np.outer(c.sum(1), c.sum(0))
    return float((c[nz] / n * (np.log(c[nz] * n) - np.log(outer[nz]))).sum())


def _expected_mi(c: np.ndarray) -> float:
    a, b, n = c.sum(1), c.sum(0), c.sum()
    lg = math.lgamma
    emi = 0.0
    for ai in a:
        for bj in b:
            lo, hi = int(max(1, ai + bj - n)), int(min(ai, bj))
            for nij in range(lo, hi + 1):
                logp = (lg(ai + 1) + lg(bj + 1) + lg(n - ai + 1) + lg(n - bj + 1) - lg(n + 1) - lg(nij + 1) - lg(ai - nij + 1) - lg(bj - nij + 1)
                        - lg(n - ai - bj + nij + 1))
                emi += nij / n * math.log(n * nij / (ai * bj)) * math.exp(logp)
    return emi


def normalized_mutual_info_score(labels_true, labels_pred) -> float:
    c = _contingency(labels_true, labels_pred)
    hu, hv = _entropy(c.sum(1)), _entropy(c.sum(0))
    if hu == 0.0 and hv == 0.0:
        return 1.0
    den = (hu + hv) / 2.0
    return float(_mutual_info(c) / den) if den > 0 else 0.0


def adjusted_mutual_info_score(labels_true, labels_pred) -> float:
    c = _contingency(labels_true, labels_pred)
    if c.shape == (1, 1) or (c.shape[0] == c.shape[1] == int(c.sum())):
        return 1.0
    mi, emi, hu, hv = _mutual_info(c), _expected_mi(c), _entropy(c.sum(1)), _entropy(c.sum(0))
    den = (hu + hv) / 2.0 - emi
    den = min(den, -np.finfo(np.float64).eps) if den < 0 else max(den, np.finfo(np.float64).eps)
    return float((mi - emi) / den)


def homogeneity_score(labels_true, labels_pred) -> float:
    c = _contingency(labels_true, labels_pred)
    h = _entropy(c.sum(1))
    return float(_mutual_info(c) / h) if h > 0 else 1.0


def completeness_score(labels_true, labels_pred) -> float:
    c = _contingency(labels_true, labels_pred)
    h = _entropy(c.sum(0))
    return float(_mutual_info(c) / h) if h > 0 else 1.0


def v_measure_score(labels_true, labels_pred, beta: float = 1.0) -> float:
    h, c = homogeneity_score(labels_true, labels_pred), completeness_score(labels_true, labels_pred)
    return float((1 + beta) * h * c / (beta * h + c)) if h + c > 0 else 0.0


def fowlkes_mallows_score(labels_true, labels_pred) -> float:
    c = _contingency(labels_true, labels_pred)
    n = c.sum()
    tk, pk, qk = (c ** 2).sum() - n, (c.sum(0) ** 2).sum() - n, (c.sum(1) ** 2).sum() - n
    return float(math.sqrt(tk / pk) * math.sqrt(tk / qk)) if tk > 0 else 0.0


def _xy(x, labels) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    X = _a(x).astype(np.float64)
    y = _a(labels).reshape(-1)
    if X.ndim != 2 or X.shape[0] != y.shape[0]:
        raise ShapeMismatch(f"cluster metric: X [n, d] and n labels expected, got {list(X.shape)} and {y.shape[0]}")
    cl, inv = np.unique(y, return_inverse=True)
    if not 2 <= len(cl) <= len(y) - 1:
        raise InvalidArgument(f"cluster metric: {len(cl)} clusters for {len(y)} samples (need 2 .. n - 1)")
    return X, inv, cl


def silhouette_score(x, labels) -> float:
    X, inv, cl = _xy(x, labels)
    D = np.sqrt(np.maximum(((X[:, None, :] - X[None, :, :]) ** 2).sum(-1), 0.0))
    k = len(cl)
    sums = np.stack([D[:, inv == c].sum(1) for c in range(k)], 1)          # distance mass of every sample to every cluster
    sizes = np.bincount(inv, minlength=k).astype(np.float64)
    own = sizes[inv]
    a = np.where(own > 1, sums[np.arange(len(X)), inv] / np.maximum(own - 1, 1), 0.0)
    other = sums / sizes[None, :]
    other[np.arange(len(X)), inv] = np.inf
    b = other.min(1)
    s = np.where(own > 1, (b - a) / np.maximum(np.maximum(a, b), 1e-300), 0.0)
    return float(s.mean())


def davies_bouldin_score(x, labels) -> float:
    X, inv, cl = _xy(x, labels)
    k = len(cl)
    cent = np.stack([X[inv == c].mean(0) for c in range(k)])
    spread = np.array([np.sqrt(((X[inv == c] - cent[c]) ** 2).sum(1)).mean() for c in range(k)])
    M = np.sqrt(((cent[:, None] - cent[None]) ** 2).sum(-1))
    if np.allclose(spread, 0) or np.allclose(M, 0):
        return 0.0
    with np.errstate(divide="ignore", invalid="ignore"):
        R = (spread[:, None] + spread[None, :]) / M
    R[~np.isfinite(R)] = 0.0
    np.fill_diagonal(R, 0.0)
    return float(R.max(1).mean())


def calinski_harabasz_score(x, labels) -> float:
    X, inv, cl = _xy(x, labels)
    n, k, mean = len(X), len(cl), X.mean(0)
    extra = intra = 0.0
    for c in range(k):
        pts = X[inv == c]
        extra += len(pts) * ((pts.mean(0) - mean) ** 2).sum()
        intra += ((pts - pts.mean(0)) ** 2).sum()
    return float(extra * (n - k) / (intra * (k - 1))) if intra > 0 else 1.0
