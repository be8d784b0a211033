"""``ml.preprocess`` / ``ml.decomposition`` / ``ml.model_selection``: the classical estimators, driven with tensors.

The reference re-exports a CPU machine-learning library (preprocessors, dimensionality reduction, cross-validation, pipelines, search) and asks
callers to convert tensors to arrays and back by hand (ferrotorch-ml/src/lib.rs:98-122). Here the same three namespaces resolve their names in
scikit-learn, and every estimator comes wrapped so that tensors go in and tensors come out: arguments that are tensors are converted to host
arrays, array results come back as tensors of the input's dtype on the input's device, and fitted estimators returned by ``fit`` stay wrapped.
Splitters yield index tensors. Without scikit-learn the namespaces raise a clear error on first use.
"""
from __future__ import annotations

import importlib
import types
from typing import Any

import numpy as np
import torch

from ..errors import FerrotorchError


def _to_np(x):
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().numpy()
    if isinstance(x, TensorEstimator):
        return x.inner
    if isinstance(x, (list, tuple)) and any(isinstance(v, (torch.Tensor, TensorEstimator)) or (isinstance(v, (list, tuple)) and v) for v in x):
        return type(x)(_to_np(v) for v in x)
    if isinstance(x, dict):
        return {k: _to_np(v) for k, v in x.items()}
    return x


def _like(args, kwargs):
    for a in list(args) + list(kwargs.values()):
        if isinstance(a, torch.Tensor):
            return a
    return None


def _to_tensor(x, like):
    if isinstance(x, np.ndarray) and x.dtype != object:
        t = torch.from_numpy(np.ascontiguousarray(x))
        if like is not None:
            t = t.to(device=like.device, dtype=like.dtype if t.is_floating_point() and like.is_floating_point() else t.dtype)
        return t
    if isinstance(x, (list, tuple)):
        return type(x)(_to_tensor(v, like) for v in x)
    if hasattr(x, "fit") or hasattr(x, "split") or hasattr(x, "transform"):
        return TensorEstimator(x)
    return x


class TensorEstimator:
    """A scikit-learn object whose methods take and return tensors; attributes (``mean_``, ``components_`` ...) come back as tensors too."""

    def __init__(self, inner):
        object.__setattr__(self, "inner", inner)

    def __getattr__(self, name: str) -> Any:
        v = getattr(self.inner, name)
        if callable(v) and not isinstance(v, type):
            def call(*args, **kwargs):
                like = _like(args, kwargs)
                out = v(*_to_np(args), **_to_np(kwargs))
                if out is self.inner:
                    return self
                if isinstance(out, types.GeneratorType):
                    return (_to_tensor(o, like) for o in out)
                return _to_tensor(out, like)
            call.__name__, call.__doc__ = name, getattr(v, "__doc__", None)
            return call
        return _to_tensor(v, None)

    def __setattr__(self, name, value):
        setattr(self.inner, name, _to_np(value))

    def __repr__(self):
        return f"TensorEstimator({self.inner!r})"


class _Namespace(types.ModuleType):
    def __init__(self, name: str, sk_modules, doc: str):
        super().__init__(name, doc)
        self._sk = sk_modules

    def __getattr__(self, name: str):
        if name.startswith("__"):
            raise AttributeError(name)
        for modname in self._sk:
            try:
                mod = importlib.import_module(modname)
            except ImportError:
                raise FerrotorchError(f"{self.__name__}.{name} needs scikit-learn, which is not installed") from None
            if hasattr(mod, name):
                obj = getattr(mod, name)
                if isinstance(obj, type):
                    def make(*a, _cls=obj, **k):
                        return TensorEstimator(_cls(*_to_np(a), **_to_np(k)))
                    make.__name__, make.__doc__ = name, obj.__doc__
                    return make

                def fn(*a, _f=obj, **k):
                    return _to_tensor(_f(*_to_np(a), **_to_np(k)), _like(a, k))
                fn.__name__, fn.__doc__ = name, getattr(obj, "__doc__", None)
                return fn
        raise AttributeError(f"{self.__name__} has no {name!r}")


preprocess = _Namespace("ferrotorch_b200.ml.preprocess", ("sklearn.preprocessing", "sklearn.impute"),
                        "StandardScaler, MinMaxScaler, OneHotEncoder, PolynomialFeatures, KBinsDiscretizer, SimpleImputer ... on tensors.")
decomposition = _Namespace("ferrotorch_b200.ml.decomposition", ("sklearn.decomposition", "sklearn.manifold"),
                           "PCA, IncrementalPCA, FastICA, NMF, KernelPCA, TruncatedSVD, SparsePCA, FactorAnalysis, TSNE, Isomap, LocallyLinearEmbedding, MDS on tensors.")
model_selection = _Namespace("ferrotorch_b200.ml.model_selection", ("sklearn.model_selection", "sklearn.pipeline", "sklearn.dummy", "sklearn.multiclass", "sklearn.multioutput"),
                             "KFold, StratifiedKFold, GroupKFold, ShuffleSplit, train_test_split, Pipeline, make_pipeline, GridSearchCV, RandomizedSearchCV, dummy and meta estimators.")
