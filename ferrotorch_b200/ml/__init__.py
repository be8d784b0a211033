"""scikit-learn style adapter: tensor <-> ndarray conversion, toy dataset generators, classification/regression metrics.

Reference parity: ferrotorch-ml/src/adapter.rs:52-218, datasets (make_classification:85 ... load_breast_cancer:320), metrics.rs
(r2_score:63 ... confusion_matrix).
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from ..errors import InvalidArgument


def tensor_to_ndarray(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().float().numpy() if t.dtype == torch.bfloat16 else t.detach().cpu().numpy()


def ndarray_to_tensor(a: np.ndarray, dtype: Optional[torch.dtype] = None, device="cpu") -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a))
    return t.to(device=device, dtype=dtype) if (dtype or str(device) != "cpu") else t


class SklearnAdapter:
    """Wraps a module + optimizer factory behind ``fit(X, y)`` / ``predict(X)`` / ``score(X, y)``."""

    def __init__(self, model: torch.nn.Module, lr: float = 1e-2, epochs: int = 50, batch_size: int = 64, task: str = "classification", seed: int = 0):
        self.model, self.lr, self.epochs, self.batch_size, self.task, self.seed = model, lr, epochs, batch_size, task, seed

    def fit(self, X: np.ndarray, y: np.ndarray) -> "SklearnAdapter":
        from ..optim import AdamW
        torch.manual_seed(self.seed)
        Xt = ndarray_to_tensor(X, torch.float32)
        yt = ndarray_to_tensor(y, torch.long if self.task == "classification" else torch.float32)
        opt = AdamW(self.model.parameters(), lr=self.lr, weight_decay=0.0)
        lossf = torch.nn.functional.cross_entropy if self.task == "classification" else torch.nn.functional.mse_loss
        n = Xt.shape[0]
        for _ in range(self.epochs):
            perm = torch.randperm(n)
            for i in range(0, n, self.batch_size):
                idx = perm[i: i + self.batch_size]
                opt.zero_grad()
                out = self.model(Xt[idx])
                loss = lossf(out if self.task == "classification" else out.squeeze(-1), yt[idx])
                loss.backward()
                opt.step()
        return self

    @torch.no_grad()
    def predict(self, X: np.ndarray) -> np.ndarray:
        out = self.model(ndarray_to_tensor(X, torch.float32))
        return tensor_to_ndarray(out.argmax(-1) if self.task == "classification" else out.squeeze(-1))

    @torch.no_grad()
    def predict_proba(self, X: np.ndarray) -> np.ndarray:
        return tensor_to_ndarray(torch.softmax(self.model(ndarray_to_tensor(X, torch.float32)), -1))

    def score(self, X, y) -> float:
        p = self.predict(X)
        return accuracy_score(y, p) if self.task == "classification" else r2_score(y, p)


# -- datasets ----------------------------------------------------------------------------------------------------------------------
def make_classification(n_samples=100, n_features=20, n_informative=2, n_classes=2, class_sep=1.0, seed=0) -> Tuple[np.ndarray, np.ndarray]:
    rng = np.random.default_rng(seed)
    centers = rng.normal(0, class_sep * 2, (n_classes, n_informative))
    y = rng.integers(0, n_classes, n_samples)
    X = rng.normal(0, 1, (n_samples, n_features))
    X[:, :n_informative] += centers[y]
    return X.astype(np.float32), y.astype(np.int64)


def make_regression(n_samples=100, n_features=10, noise=0.1, seed=0):
    rng = np.random.default_rng(seed)
    X = rng.normal(0, 1, (n_samples, n_features))
    w = rng.normal(0, 1, n_features)
    return X.astype(np.float32), (X @ w + rng.normal(0, noise, n_samples)).astype(np.float32)


def make_blobs(n_samples=100, centers=3, n_features=2, cluster_std=1.0, seed=0):
    rng = np.random.default_rng(seed)
    c = rng.uniform(-10, 10, (centers, n_features))
    y = rng.integers(0, centers, n_samples)
    return (c[y] + rng.normal(0, cluster_std, (n_samples, n_features))).astype(np.float32), y.astype(np.int64)


def make_moons(n_samples=100, noise=0.1, seed=0):
    rng = np.random.default_rng(seed)
    n = n_samples // 2
    t = np.linspace(0, np.pi, n)
    X = np.concatenate([np.stack([np.cos(t), np.sin(t)], 1), np.stack([1 - np.cos(t), 0.5 - np.sin(t)], 1)])
    return (X + rng.normal(0, noise, X.shape)).astype(np.float32), np.concatenate([np.zeros(n), np.ones(n)]).astype(np.int64)


def make_circles(n_samples=100, noise=0.05, factor=0.5, seed=0):
    rng = np.random.default_rng(seed)
    n = n_samples // 2
    t = np.linspace(0, 2 * np.pi, n, endpoint=False)
    X = np.concatenate([np.stack([np.cos(t), np.sin(t)], 1), factor * np.stack([np.cos(t), np.sin(t)], 1)])
    return (X + rng.normal(0, noise, X.shape)).astype(np.float32), np.concatenate([np.zeros(n), np.ones(n)]).astype(np.int64)


def _sk(name):
    from sklearn import datasets
    d = getattr(datasets, name)()
    return d.data.astype(np.float32), d.target


def load_iris():
    return _sk("load_iris")


def load_wine():
    return _sk("load_wine")


def load_breast_cancer():
    return _sk("load_breast_cancer")


def load_digits():
    return _sk("load_digits")


def train_test_split(X, y, test_size=0.25, seed=0):
    rng = np.random.default_rng(seed)
    idx = rng.permutation(len(X))
    k = int(len(X) * (1 - test_size))
    return X[idx[:k]], X[idx[k:]], y[idx[:k]], y[idx[k:]]


# -- metrics -----------------------------------------------------------------------------------------------------------------------
def _np(a):
    return tensor_to_ndarray(a) if isinstance(a, torch.Tensor) else np.asarray(a)


def r2_score(y_true, y_pred) -> float:
    y, p = _np(y_true).astype(np.float64), _np(y_pred).astype(np.float64)
    ss_tot = ((y - y.mean()) ** 2).sum()
    return float(1.0 - ((y - p) ** 2).sum() / ss_tot) if ss_tot > 0 else 0.0


def mean_squared_error(y_true, y_pred) -> float:
    return float(((_np(y_true).astype(np.float64) - _np(y_pred)) ** 2).mean())


def mean_absolute_error(y_true, y_pred) -> float:
    return float(np.abs(_np(y_true).astype(np.float64) - _np(y_pred)).mean())


def accuracy_score(y_true, y_pred) -> float:
    return float((_np(y_true) == _np(y_pred)).mean())


def confusion_matrix(y_true, y_pred, n_classes: Optional[int] = None) -> np.ndarray:
    y, p = _np(y_true).astype(np.int64), _np(y_pred).astype(np.int64)
    k = n_classes or int(max(y.max(), p.max())) + 1
    cm = np.zeros((k, k), dtype=np.int64)
    np.add.at(cm, (y, p), 1)
    return cm


def precision_recall_f1(y_true, y_pred, average: str = "macro"):
    cm = confusion_matrix(y_true, y_pred).astype(np.float64)
    tp = np.diag(cm)
    prec = tp / np.maximum(cm.sum(0), 1)
    rec = tp / np.maximum(cm.sum(1), 1)
    f1 = 2 * prec * rec / np.maximum(prec + rec, 1e-12)
    if average == "macro":
        return float(prec.mean()), float(rec.mean()), float(f1.mean())
    if average == "micro":
        a = tp.sum() / max(cm.sum(), 1)
        return float(a), float(a), float(a)
    if average == "weighted":                       # class means weighted by the number of true samples of each class
        w = cm.sum(1) / max(cm.sum(), 1)
        return float((prec * w).sum()), float((rec * w).sum()), float((f1 * w).sum())
    if average is None or average == "none":
        return prec, rec, f1
    raise InvalidArgument(f"unknown average {average!r} (macro, micro, weighted or None)")


def precision_score(y_true, y_pred, average="macro"):
    return precision_recall_f1(y_true, y_pred, average)[0]


def recall_score(y_true, y_pred, average="macro"):
    return precision_recall_f1(y_true, y_pred, average)[1]


def f1_score(y_true, y_pred, average="macro"):
    return precision_recall_f1(y_true, y_pred, average)[2]


def roc_auc_score(y_true, scores) -> float:
    y, s = _np(y_true).astype(np.int64), _np(scores).astype(np.float64)
    # mid-ranks: tied scores share the mean of the ranks they span (the Mann-Whitney statistic with ties counted as one half)
    order = np.argsort(s, kind="mergesort")
    ss = s[order]
    first = np.r_[True, ss[1:] != ss[:-1]]
    group = np.cumsum(first) - 1
    starts = np.flatnonzero(first)
    ends = np.r_[starts[1:], len(ss)]
    mid = (starts + 1 + ends) / 2.0
    ranks = np.empty(len(s))
    ranks[order] = mid[group]
    npos, nneg = y.sum(), (1 - y).sum()
    if npos == 0 or nneg == 0:
        raise InvalidArgument("ROC AUC needs both classes")
    return float((ranks[y == 1].sum() - npos * (npos + 1) / 2) / (npos * nneg))


def log_loss(y_true, proba, eps: float = 1e-12) -> float:
    y, p = _np(y_true).astype(np.int64), np.clip(_np(proba).astype(np.float64), eps, 1 - eps)
    return float(-np.log(p[np.arange(len(y)), y]).mean())


from .metrics_ext import (tensor_to_array1, tensor_to_array2, array1_to_tensor, array2_to_tensor, array1_usize_to_tensor, tensor_to_array1_usize,  # noqa: E402,F401
                          root_mean_squared_error, mean_absolute_percentage_error, median_absolute_error, max_error, explained_variance_score, hamming_loss,
                          zero_one_loss, balanced_accuracy_score, matthews_corrcoef, cohen_kappa_score, brier_score_loss, d2_brier_score, top_k_accuracy_score,
                          average_precision_score, dcg_score, ndcg_score, coverage_error, label_ranking_average_precision_score, label_ranking_loss,
                          adjusted_rand_score, adjusted_mutual_info_score, normalized_mutual_info_score, homogeneity_score, completeness_score,
                          v_measure_score, fowlkes_mallows_score, silhouette_score, davies_bouldin_score, calinski_harabasz_score)
from .sk_bridge import preprocess, decomposition, model_selection, TensorEstimator  # noqa: E402,F401
