"""Every metric of the ml package against scikit-learn on random data with ties, plus the argument checks."""
import numpy as np
import pytest
import torch

from ferrotorch_b200 import ml
from ferrotorch_b200.errors import FerrotorchError

skm = pytest.importorskip("sklearn.metrics")


def _close(a, b, tol=1e-9):
    assert abs(float(a) - float(b)) <= tol * max(1.0, abs(float(b))), (a, b)


def test_regression_metrics_match_sklearn():
    rng = np.random.default_rng(0)
    y, p = rng.normal(size=200), rng.normal(size=200)
    yt, pt = torch.tensor(y), torch.tensor(p)
    _close(ml.root_mean_squared_error(yt, pt), skm.root_mean_squared_error(y, p))
    _close(ml.mean_absolute_percentage_error(yt, pt), skm.mean_absolute_percentage_error(y, p))
    _close(ml.median_absolute_error(yt, pt), skm.median_absolute_error(y, p))
    _close(ml.max_error(yt, pt), skm.max_error(y, p))
    _close(ml.explained_variance_score(yt, pt), skm.explained_variance_score(y, p))
    assert ml.explained_variance_score([1.0, 1.0], [1.0, 1.0]) == 1.0
    with pytest.raises(FerrotorchError):
        ml.max_error(yt, pt[:5])
    with pytest.raises(FerrotorchError):
        ml.max_error([], [])


def test_classification_metrics_match_sklearn():
    rng = np.random.default_rng(1)
    y, p = rng.integers(0, 4, 300), rng.integers(0, 4, 300)
    p[:120] = y[:120]
    _close(ml.hamming_loss(y, p), skm.hamming_loss(y, p))
    _close(ml.zero_one_loss(y, p), skm.zero_one_loss(y, p))
    _close(ml.zero_one_loss(y, p, normalize=False), skm.zero_one_loss(y, p, normalize=False))
    _close(ml.balanced_accuracy_score(y, p), skm.balanced_accuracy_score(y, p))
    _close(ml.balanced_accuracy_score(y, p, adjusted=True), skm.balanced_accuracy_score(y, p, adjusted=True))
    _close(ml.matthews_corrcoef(y, p), skm.matthews_corrcoef(y, p))
    _close(ml.cohen_kappa_score(y, p), skm.cohen_kappa_score(y, p))
    yb = rng.integers(0, 2, 300)
    prob = np.round(np.clip(yb * 0.3 + rng.uniform(size=300) * 0.7, 0, 1), 2)        # rounded: plenty of tied scores
    _close(ml.brier_score_loss(yb, prob), skm.brier_score_loss(yb, prob))
    _close(ml.d2_brier_score(yb, prob), 1 - skm.brier_score_loss(yb, prob) / skm.brier_score_loss(yb, np.full(300, yb.mean())))
    _close(ml.average_precision_score(yb, prob), skm.average_precision_score(yb, prob))
    scores = rng.normal(size=(300, 4))
    for k in (1, 2, 3):
        _close(ml.top_k_accuracy_score(torch.tensor(y), torch.tensor(scores), k), skm.top_k_accuracy_score(y, scores, k=k, labels=[0, 1, 2, 3]))
    for bad in (lambda: ml.hamming_loss([0.5], [1]), lambda: ml.brier_score_loss([0, 2], [0.1, 0.2]), lambda: ml.brier_score_loss([0, 1], [0.1, 1.2]),
                lambda: ml.top_k_accuracy_score(y, scores, 9), lambda: ml.top_k_accuracy_score(y, scores[:, 0], 1), lambda: ml.average_precision_score([0, 0], [0.1, 0.2])):
        with pytest.raises(FerrotorchError):
            bad()


def test_ranking_metrics_match_sklearn():
    rng = np.random.default_rng(2)
    rel, sc = rng.integers(0, 5, 40).astype(float), np.round(rng.normal(size=40), 1)
    for k in (None, 5, 17):
        _close(ml.dcg_score(rel, sc, k), skm.dcg_score(rel[None], sc[None], k=k))
        _close(ml.ndcg_score(rel, sc, k), skm.ndcg_score(rel[None], sc[None], k=k))
    Y = (rng.uniform(size=(30, 6)) < 0.35).astype(int)
    Y[0], Y[1] = 0, 1                                          # rows without / with only relevant labels
    S = np.round(rng.normal(size=(30, 6)), 1)
    _close(ml.coverage_error(Y[2:], S[2:]), skm.coverage_error(Y[2:], S[2:]))
    _close(ml.label_ranking_average_precision_score(Y, S), skm.label_ranking_average_precision_score(Y, S))
    _close(ml.label_ranking_loss(Y, S), skm.label_ranking_loss(Y, S))
    with pytest.raises(FerrotorchError):
        ml.coverage_error(Y, S[:, :3])
    with pytest.raises(FerrotorchError):
        ml.ndcg_score([-1.0, 2.0], [0.1, 0.2])


def test_clustering_metrics_match_sklearn():
    rng = np.random.default_rng(3)
    a, b = rng.integers(0, 4, 120), rng.integers(0, 3, 120)
    b[:60] = a[:60] % 3
    for ours, theirs in ((ml.adjusted_rand_score, skm.adjusted_rand_score), (ml.normalized_mutual_info_score, skm.normalized_mutual_info_score),
                         (ml.adjusted_mutual_info_score, skm.adjusted_mutual_info_score), (ml.homogeneity_score, skm.homogeneity_score),
                         (ml.completeness_score, skm.completeness_score), (ml.v_measure_score, skm.v_measure_score), (ml.fowlkes_mallows_score, skm.fowlkes_mallows_score)):
        _close(ours(a, b), theirs(a, b), 1e-8)
        _close(ours(a, a), 1.0, 1e-8)
    X = rng.normal(size=(120, 5)) + a[:, None] * 2.0
    _close(ml.silhouette_score(torch.tensor(X), torch.tensor(a)), skm.silhouette_score(X, a), 1e-8)
    _close(ml.davies_bouldin_score(X, a), skm.davies_bouldin_score(X, a), 1e-8)
    _close(ml.calinski_harabasz_score(X, a), skm.calinski_harabasz_score(X, a), 1e-8)
    with pytest.raises(FerrotorchError):
        ml.silhouette_score(X, np.zeros(120))
    with pytest.raises(FerrotorchError):
        ml.silhouette_score(X[:10], a)


def test_adapters_round_trip_and_check_rank():
    t = torch.arange(6.0)
    assert ml.tensor_to_array1(t).tolist() == list(range(6)) and ml.tensor_to_array2(t.view(2, 3)).shape == (2, 3)
    assert torch.equal(ml.array1_to_tensor(np.arange(6.0)), t) and ml.array2_to_tensor(np.ones((2, 2))).shape == (2, 2)
    assert ml.array1_usize_to_tensor(np.array([3, 1])).tolist() == [3.0, 1.0] and ml.tensor_to_array1_usize(torch.tensor([2.0, 0.0])).tolist() == [2, 0]
    for bad in (lambda: ml.tensor_to_array1(t.view(2, 3)), lambda: ml.tensor_to_array2(t), lambda: ml.array1_to_tensor(np.ones((2, 2))),
                lambda: ml.tensor_to_array1_usize(torch.tensor([1.5])), lambda: ml.tensor_to_array1_usize(torch.tensor([-1.0])), lambda: ml.array1_usize_to_tensor(np.array([-2]))):
        with pytest.raises(FerrotorchError):
            bad()


def test_classical_estimators_take_and_return_tensors():
    pytest.importorskip("sklearn")
    g = torch.Generator().manual_seed(0)
    X = torch.randn(60, 5, generator=g, dtype=torch.float64) * torch.tensor([1.0, 5.0, 0.2, 3.0, 1.0], dtype=torch.float64) + 2.0
    sc = ml.preprocess.StandardScaler().fit(X)
    assert isinstance(sc, ml.TensorEstimator) and torch.allclose(sc.mean_, X.mean(0)) and torch.allclose(sc.transform(X), (X - X.mean(0)) / X.std(0, unbiased=False))
    Z = sc.fit_transform(X.float())
    assert Z.dtype == torch.float32 and torch.allclose(sc.inverse_transform(Z), X.float(), atol=1e-4)
    mm = ml.preprocess.MinMaxScaler().fit_transform(X)
    assert float(mm.min()) == 0.0 and abs(float(mm.max()) - 1.0) < 1e-12
    filled = ml.preprocess.SimpleImputer(strategy="mean").fit_transform(torch.tensor([[1.0, float("nan")], [3.0, 4.0]]))
    assert filled.tolist() == [[1.0, 4.0], [3.0, 4.0]]
    pca = ml.decomposition.PCA(n_components=2).fit(X)
    U, S, Vh = torch.linalg.svd(X - X.mean(0), full_matrices=False)
    assert pca.components_.shape == (2, 5) and torch.allclose(pca.components_.abs(), Vh[:2].abs(), atol=1e-8)
    assert torch.allclose(pca.explained_variance_, S[:2] ** 2 / 59, atol=1e-8) and pca.transform(X).shape == (60, 2)
    y = (X[:, 1] > 2.0).long()
    folds = list(ml.model_selection.KFold(n_splits=3).split(X))
    assert len(folds) == 3 and all(isinstance(tr, torch.Tensor) and len(tr) + len(te) == 60 for tr, te in folds)
    assert sorted(torch.cat([te for _, te in folds]).tolist()) == list(range(60))
    Xtr, Xte, ytr, yte = ml.model_selection.train_test_split(X, y, test_size=0.25, random_state=0)
    assert Xtr.shape == (45, 5) and yte.shape == (15,) and isinstance(Xtr, torch.Tensor)
    pipe = ml.model_selection.make_pipeline(ml.preprocess.StandardScaler(), ml.model_selection.DummyClassifier(strategy="most_frequent"))
    pred = pipe.fit(X, y).predict(X)
    assert isinstance(pred, torch.Tensor) and pred.unique().numel() == 1
    with pytest.raises(AttributeError):
        ml.preprocess.NoSuchThing
