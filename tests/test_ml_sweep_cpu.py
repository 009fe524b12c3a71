"""Every estimator of ghost_flow_b200.ml with a no-argument constructor fits a small problem and predicts or
transforms it: classification, regression, non-negative and unsupervised inputs are tried in that order, time-series
models get a 1-D series."""
import inspect
import warnings

import numpy as np
import pytest

import ghost_flow_b200.ml as ml

_SERIES = {"ARIMA", "SARIMA", "HoltLinear", "HoltWinters", "STLDecomposition", "SimpleExponentialSmoothing",
           "ExponentialSmoothing"}
_TEXT = {"BPETokenizer", "CharTokenizer", "WordTokenizer", "TfidfVectorizer", "CountVectorizer"}
_TWO_ARG = {"IsotonicRegression", "PlattScaling"}
_NEEDS_ESTIMATORS = {"StackingClassifier", "StackingRegressor", "VotingClassifier", "VotingRegressor",
                     "ClassifierChain", "LinearChainCRF"}


def _estimators():
    out = []
    for name in sorted(dir(ml)):
        cls = getattr(ml, name)
        if not inspect.isclass(cls) or name.startswith("_") or not hasattr(cls, "fit"):
            continue
        if name in _NEEDS_ESTIMATORS or inspect.isabstract(cls):
            continue
        try:
            cls()
        except TypeError:
            continue
        out.append(name)
    return out


@pytest.mark.parametrize("name", _estimators())
def test_estimator_fits_and_predicts(name):
    warnings.filterwarnings("ignore")
    cls = getattr(ml, name)
    rng = np.random.default_rng(0)
    X = rng.normal(size=(60, 5)).astype(np.float32)
    yc = (X[:, 0] + X[:, 1] > 0).astype(np.int64)
    yr = (X @ rng.normal(size=5)).astype(np.float32)
    if name in _SERIES:
        t = np.arange(96, dtype=np.float32)
        attempts = [((np.sin(t / 4) + 0.05 * t + 0.1 * rng.normal(size=96)).astype(np.float32) + 3.0,)]
    elif name in _TEXT:
        attempts = [(["the cat sat on the mat", "the dog ate the cat", "a mat is a mat"],)]
    elif name in _TWO_ARG:
        attempts = [(X[:, 0], yc.astype(np.float32))]
    else:
        attempts = [(X, yc), (X, yr), (np.abs(X), yc), (X,)]
    last = None
    for args in attempts:
        try:
            est = cls()
            est.fit(*args)
            if name in _SERIES:
                if hasattr(est, "forecast"):
                    assert len(np.asarray(est.forecast(4)).reshape(-1)) == 4
                return
            for method in ("predict", "transform", "predict_proba"):
                if hasattr(est, method):
                    try:
                        out = getattr(est, method)(args[0])
                    except TypeError:
                        continue  # needs extra arguments (horizon, labels, ...)
                    assert out is not None
            return
        except Exception as e:  # try the next kind of input
            last = e
    raise AssertionError(f"{name} failed on every input kind: {last!r}")
