"""Scalers, encoders, feature engineering and selection (ghostflow-ml/src/preprocessing.rs,
preprocessing_extended.rs, feature_engineering.rs, polynomial.rs, feature_selection.rs)."""
from __future__ import annotations

import enum
import itertools
import zlib

import numpy as np

from ._base import Estimator, TransformerMixin, out, rng_of, to_np


class StandardScaler(Estimator, TransformerMixin):
    _params = ("with_mean", "with_std")

    def __init__(self):
        self._with_mean, self._with_std = True, True

    def fit(self, X, y=None):
        X = to_np(X)
        self.mean_ = X.mean(0)
        s = X.std(0)
        self.scale_ = np.where(s == 0, 1.0, s)
        return self

    def transform(self, X):
        X = to_np(X)
        if self._with_mean:
            X = X - self.mean_
        if self._with_std:
            X = X / self.scale_
        return out(X)

    def inverse_transform(self, X):
        X = to_np(X)
        if self._with_std:
            X = X * self.scale_
        if self._with_mean:
            X = X + self.mean_
        return out(X)


class MinMaxScaler(Estimator, TransformerMixin):
    _params = ("feature_range",)

    def __init__(self):
        self._feature_range = (0.0, 1.0)

    def fit(self, X, y=None):
        X = to_np(X)
        self.min_, self.max_ = X.min(0), X.max(0)
        return self

    def transform(self, X):
        lo, hi = self._feature_range
        span = np.where(self.max_ - self.min_ == 0, 1.0, self.max_ - self.min_)
        return out((to_np(X) - self.min_) / span * (hi - lo) + lo)

    def inverse_transform(self, X):
        lo, hi = self._feature_range
        span = np.where(self.max_ - self.min_ == 0, 1.0, self.max_ - self.min_)
        return out((to_np(X) - lo) / (hi - lo) * span + self.min_)


class RobustScaler(Estimator, TransformerMixin):
    _params = ("quantile_range",)

    def __init__(self):
        self._quantile_range = (25.0, 75.0)

    def fit(self, X, y=None):
        X = to_np(X)
        self.center_ = np.median(X, 0)
        q = np.percentile(X, self._quantile_range, axis=0)
        iqr = q[1] - q[0]
        self.scale_ = np.where(iqr == 0, 1.0, iqr)
        return self

    def transform(self, X):
        return out((to_np(X) - self.center_) / self.scale_)

    def inverse_transform(self, X):
        return out(to_np(X) * self.scale_ + self.center_)


class MaxAbsScaler(Estimator, TransformerMixin):
    def fit(self, X, y=None):
        m = np.abs(to_np(X)).max(0)
        self.scale_ = np.where(m == 0, 1.0, m)
        return self

    def transform(self, X):
        return out(to_np(X) / self.scale_)

    def inverse_transform(self, X):
        return out(to_np(X) * self.scale_)


class Normalizer(Estimator, TransformerMixin):
    def __init__(self, norm="l2"):
        self._norm = getattr(norm, "value", norm)

    def fit(self, X, y=None):
        return self

    def transform(self, X):
        X = to_np(X)
        if self._norm == "l1":
            n = np.abs(X).sum(1, keepdims=True)
        elif self._norm == "max":
            n = np.abs(X).max(1, keepdims=True)
        else:
            n = np.sqrt((X * X).sum(1, keepdims=True))
        return out(X / np.where(n == 0, 1.0, n))


class Binarizer(Estimator, TransformerMixin):
    def __init__(self, threshold=0.0):
        self._threshold = threshold

    def fit(self, X, y=None):
        return self

    def transform(self, X):
        return out((to_np(X) > self._threshold).astype(np.float64))


class LabelEncoder(Estimator):
    def fit(self, y):
        self.classes_ = np.unique(to_np(y, None))
        return self

    def transform(self, y):
        y = to_np(y, None)
        return out(np.searchsorted(self.classes_, y))

    def fit_transform(self, y):
        return self.fit(y).transform(y)

    def inverse_transform(self, codes):
        return self.classes_[to_np(codes).astype(int)]


class OneHotEncoder(Estimator, TransformerMixin):
    _params = ("drop_first", "handle_unknown")

    def __init__(self):
        self._drop_first, self._handle_unknown = False, "ignore"

    def fit(self, X, y=None):
        X = to_np(X)
        X = X[:, None] if X.ndim == 1 else X
        self.categories_ = [np.unique(X[:, j]) for j in range(X.shape[1])]
        return self

    def transform(self, X):
        X = to_np(X)
        X = X[:, None] if X.ndim == 1 else X
        cols = []
        for j, cats in enumerate(self.categories_):
            oh = (X[:, j][:, None] == cats[None, :]).astype(np.float64)
            cols.append(oh[:, 1:] if self._drop_first else oh)
        return out(np.concatenate(cols, 1))

    def inverse_transform(self, X):
        X = to_np(X)
        res, c = [], 0
        for cats in self.categories_:
            k = len(cats) - (1 if self._drop_first else 0)
            blk = X[:, c:c + k]
            if self._drop_first:
                idx = np.where(blk.sum(1) == 0, 0, blk.argmax(1) + 1)
            else:
                idx = blk.argmax(1)
            res.append(cats[idx])
            c += k
        return out(np.stack(res, 1))


class OrdinalEncoder(Estimator, TransformerMixin):
    def fit(self, X, y=None):
        X = to_np(X)
        self.categories_ = [np.unique(X[:, j]) for j in range(X.shape[1])]
        return self

    def transform(self, X):
        X = to_np(X)
        res = np.empty_like(X)
        for j, cats in enumerate(self.categories_):
            idx = np.searchsorted(cats, X[:, j])
            idx = np.clip(idx, 0, len(cats) - 1)
            res[:, j] = np.where(cats[idx] == X[:, j], idx, -1)
        return out(res)

    def inverse_transform(self, X):
        X = to_np(X).astype(int)
        return out(np.stack([cats[np.clip(X[:, j], 0, len(cats) - 1)] for j, cats in enumerate(self.categories_)], 1))


class TargetEncoder(Estimator, TransformerMixin):
    """Mean of the target per category, shrunk towards the global mean: (n * mean_c + s * prior) / (n + s)."""
    _params = ("smoothing",)

    def __init__(self):
        self._smoothing = 1.0

    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        X = X[:, None] if X.ndim == 1 else X
        self.prior_ = y.mean()
        self.maps_ = []
        for j in range(X.shape[1]):
            m = {}
            for c in np.unique(X[:, j]):
                sel = y[X[:, j] == c]
                m[c] = (sel.sum() + self._smoothing * self.prior_) / (len(sel) + self._smoothing)
            self.maps_.append(m)
        return self

    def transform(self, X):
        X = to_np(X)
        X = X[:, None] if X.ndim == 1 else X
        res = np.empty_like(X)
        for j, m in enumerate(self.maps_):
            res[:, j] = [m.get(v, self.prior_) for v in X[:, j]]
        return out(res)


class KBinsDiscretizer(Estimator, TransformerMixin):
    _params = ("strategy", "encode")

    def __init__(self, n_bins=5):
        self._n_bins, self._strategy, self._encode = n_bins, "uniform", "ordinal"

    def fit(self, X, y=None):
        X = to_np(X)
        self.bin_edges_ = []
        for j in range(X.shape[1]):
            c = X[:, j]
            if self._strategy == "quantile":
                e = np.quantile(c, np.linspace(0, 1, self._n_bins + 1))
            elif self._strategy == "kmeans":
                from .cluster import KMeans
                cen = np.sort(to_np(KMeans(self._n_bins).fit(c[:, None]).cluster_centers_).ravel())
                e = np.concatenate(([c.min()], (cen[1:] + cen[:-1]) / 2, [c.max()]))
            else:
                e = np.linspace(c.min(), c.max(), self._n_bins + 1)
            self.bin_edges_.append(e)
        return self

    def transform(self, X):
        X = to_np(X)
        res = np.empty_like(X)
        for j, e in enumerate(self.bin_edges_):
            res[:, j] = np.clip(np.searchsorted(e[1:-1], X[:, j], side="right"), 0, self._n_bins - 1)
        if self._encode == "onehot":
            return out(np.concatenate([(res[:, j][:, None] == np.arange(self._n_bins)).astype(float)
                                       for j in range(res.shape[1])], 1))
        return out(res)

    def inverse_transform(self, X):
        X = to_np(X).astype(int)
        return out(np.stack([(e[:-1] + e[1:])[np.clip(X[:, j], 0, self._n_bins - 1)] / 2
                             for j, e in enumerate(self.bin_edges_)], 1))


class PolynomialFeatures(Estimator, TransformerMixin):
    _params = ("interaction_only", "include_bias")

    def __init__(self, degree=2):
        self._degree, self._interaction_only, self._include_bias = degree, False, True

    def fit(self, X, y=None):
        n = to_np(X).shape[1]
        comb = itertools.combinations if self._interaction_only else itertools.combinations_with_replacement
        self.powers_ = [c for d in range(0 if self._include_bias else 1, self._degree + 1) for c in comb(range(n), d)]
        self.n_output_features_ = len(self.powers_)
        return self

    def transform(self, X):
        X = to_np(X)
        return out(np.stack([np.prod(X[:, list(c)], axis=1) if c else np.ones(len(X)) for c in self.powers_], 1))


class SplineTransformer(Estimator, TransformerMixin):
    """B-spline basis of the given degree on ``n_knots`` uniform (or quantile) knots per feature."""
    _params = ("degree", "knots", "include_bias")

    def __init__(self, n_knots=5):
        self._n_knots, self._degree, self._knots, self._include_bias = n_knots, 3, "uniform", True

    def fit(self, X, y=None):
        X = to_np(X)
        self.knots_ = []
        for j in range(X.shape[1]):
            c = X[:, j]
            base = (np.quantile(c, np.linspace(0, 1, self._n_knots)) if self._knots == "quantile"
                    else np.linspace(c.min(), c.max(), self._n_knots))
            d = self._degree
            step_lo, step_hi = base[1] - base[0], base[-1] - base[-2]
            t = np.concatenate((base[0] - step_lo * np.arange(d, 0, -1), base, base[-1] + step_hi * np.arange(1, d + 1)))
            self.knots_.append(t)
        return self

    @staticmethod
    def _basis(x, t, d):
        n = len(t) - d - 1
        B = np.zeros((len(x), len(t) - 1))
        for i in range(len(t) - 1):
            B[:, i] = (x >= t[i]) & (x < t[i + 1])
        B[x >= t[-d - 1], len(t) - d - 2] = 1.0 * (x[x >= t[-d - 1]] <= t[-d - 1] + 1e-12) + B[x >= t[-d - 1], len(t) - d - 2]
        for k in range(1, d + 1):
            Bn = np.zeros((len(x), len(t) - 1 - k))
            for i in range(len(t) - 1 - k):
                a = (x - t[i]) / (t[i + k] - t[i]) if t[i + k] > t[i] else 0.0
                b = (t[i + k + 1] - x) / (t[i + k + 1] - t[i + 1]) if t[i + k + 1] > t[i + 1] else 0.0
                Bn[:, i] = a * B[:, i] + b * B[:, i + 1]
            B = Bn
        return B[:, :n]

    def transform(self, X):
        X = to_np(X)
        cols = []
        for j, t in enumerate(self.knots_):
            x = np.clip(X[:, j], t[self._degree], t[-self._degree - 1])
            B = self._basis(x, t, self._degree)
            cols.append(B if self._include_bias else B[:, :-1])
        return out(np.concatenate(cols, 1))


class PowerTransformer(Estimator, TransformerMixin):
    """Yeo-Johnson (default) or Box-Cox with the exponent chosen per feature by a grid search on the log-likelihood."""
    _params = ("standardize",)

    def __init__(self, method="yeo-johnson"):
        self._method, self._standardize = getattr(method, "value", method), True

    @staticmethod
    def _yj(x, lam):
        res = np.empty_like(x)
        p, n = x >= 0, x < 0
        res[p] = np.log1p(x[p]) if abs(lam) < 1e-9 else ((x[p] + 1) ** lam - 1) / lam
        res[n] = -np.log1p(-x[n]) if abs(lam - 2) < 1e-9 else -((1 - x[n]) ** (2 - lam) - 1) / (2 - lam)
        return res

    @staticmethod
    def _bc(x, lam):
        return np.log(x) if abs(lam) < 1e-9 else (x ** lam - 1) / lam

    def _f(self, x, lam):
        return self._yj(x, lam) if self._method == "yeo-johnson" else self._bc(x, lam)

    def fit(self, X, y=None):
        X = to_np(X)
        self.lambdas_ = []
        for j in range(X.shape[1]):
            x = X[:, j]
            best, bl = -np.inf, 1.0
            for lam in np.linspace(-2, 2, 41):
                t = self._f(x, lam)
                jac = (np.sign(x) * np.log1p(np.abs(x))).sum() if self._method == "yeo-johnson" else np.log(x).sum()
                ll = -0.5 * len(x) * np.log(t.var() + 1e-300) + (lam - 1) * jac
                if ll > best:
                    best, bl = ll, lam
            self.lambdas_.append(bl)
        T = np.stack([self._f(X[:, j], l) for j, l in enumerate(self.lambdas_)], 1)
        self.mean_, self.std_ = T.mean(0), np.where(T.std(0) == 0, 1.0, T.std(0))
        return self

    def transform(self, X):
        X = to_np(X)
        T = np.stack([self._f(X[:, j], l) for j, l in enumerate(self.lambdas_)], 1)
        return out((T - self.mean_) / self.std_ if self._standardize else T)


class QuantileTransformer(Estimator, TransformerMixin):
    _params = ("n_quantiles", "output_distribution")

    def __init__(self):
        self._n_quantiles, self._output_distribution = 1000, "uniform"

    def fit(self, X, y=None):
        X = to_np(X)
        nq = min(self._n_quantiles, len(X))
        self.references_ = np.linspace(0, 1, nq)
        self.quantiles_ = np.quantile(X, self.references_, axis=0)
        return self

    def transform(self, X):
        X = to_np(X)
        U = np.stack([np.interp(X[:, j], self.quantiles_[:, j], self.references_) for j in range(X.shape[1])], 1)
        if self._output_distribution == "normal":
            from scipy.stats import norm
            U = norm.ppf(np.clip(U, 1e-7, 1 - 1e-7))
        return out(U)

    def inverse_transform(self, X):
        U = to_np(X)
        if self._output_distribution == "normal":
            from scipy.stats import norm
            U = norm.cdf(U)
        return out(np.stack([np.interp(U[:, j], self.references_, self.quantiles_[:, j]) for j in range(U.shape[1])], 1))


class FeatureHasher(Estimator, TransformerMixin):
    """Signed hashing trick on (feature index, value) pairs or on dicts / token lists."""

    def __init__(self, n_features=1024):
        self._n_features = n_features

    def fit(self, X=None, y=None):
        return self

    def _slot(self, key):
        h = zlib.crc32(str(key).encode())
        return h % self._n_features, 1.0 if (h >> 31) & 1 == 0 else -1.0

    def transform(self, X):
        rows = []
        if isinstance(X, (list, tuple)) and X and isinstance(X[0], (dict, list, tuple)) and not np.isscalar(X[0]):
            for r in X:
                v = np.zeros(self._n_features)
                items = r.items() if isinstance(r, dict) else ((t, 1.0) for t in r)
                for k, val in items:
                    i, s = self._slot(k)
                    v[i] += s * float(val)
                rows.append(v)
            return out(np.stack(rows))
        A = to_np(X)
        res = np.zeros((len(A), self._n_features))
        for j in range(A.shape[1]):
            i, s = self._slot(j)
            res[:, i] += s * A[:, j]
        return out(res)


# ----------------------------------------------------------------------------- feature selection
class ScoreFunction(enum.Enum):
    FClassif = "f_classif"
    FRegression = "f_regression"
    Chi2 = "chi2"
    MutualInfo = "mutual_info"


def f_classif(X, y):
    classes = np.unique(y)
    n, k = len(y), len(classes)
    mean = X.mean(0)
    ssb = sum((y == c).sum() * (X[y == c].mean(0) - mean) ** 2 for c in classes)
    ssw = sum(((X[y == c] - X[y == c].mean(0)) ** 2).sum(0) for c in classes)
    return (ssb / max(1, k - 1)) / (ssw / max(1, n - k) + 1e-300)


def f_regression(X, y):
    xc, yc = X - X.mean(0), y - y.mean()
    r = (xc * yc[:, None]).sum(0) / (np.sqrt((xc ** 2).sum(0) * (yc ** 2).sum()) + 1e-300)
    return r ** 2 / (1 - r ** 2 + 1e-300) * (len(y) - 2)


def chi2(X, y):
    classes = np.unique(y)
    Y = (y[:, None] == classes[None, :]).astype(float)
    obs = Y.T @ X
    exp = Y.mean(0)[:, None] * X.sum(0)[None, :]
    return ((obs - exp) ** 2 / (exp + 1e-300)).sum(0)


def mutual_info(X, y, bins=10):
    res = []
    yc = np.unique(y, return_inverse=True)[1]
    for j in range(X.shape[1]):
        xb = np.digitize(X[:, j], np.histogram_bin_edges(X[:, j], bins)[1:-1])
        joint = np.zeros((bins, yc.max() + 1))
        np.add.at(joint, (xb, yc), 1)
        p = joint / joint.sum()
        px, py = p.sum(1, keepdims=True), p.sum(0, keepdims=True)
        nz = p > 0
        res.append((p[nz] * np.log(p[nz] / (px @ py)[nz])).sum())
    return np.array(res)


class VarianceThreshold(Estimator, TransformerMixin):
    def __init__(self, threshold=0.0):
        self._threshold = threshold

    def fit(self, X, y=None):
        self.variances_ = to_np(X).var(0)
        return self

    def get_support(self):
        return self.variances_ > self._threshold

    def transform(self, X):
        return out(to_np(X)[:, self.get_support()])


class SelectKBest(Estimator, TransformerMixin):
    def __init__(self, k=10, score_func=ScoreFunction.FClassif):
        self._k, self._score_func = k, score_func

    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        fn = {"f_classif": f_classif, "f_regression": f_regression, "chi2": chi2, "mutual_info": mutual_info}[
            getattr(self._score_func, "value", self._score_func)]
        self.scores_ = fn(X, y)
        return self

    def get_support(self):
        m = np.zeros(len(self.scores_), bool)
        m[np.argsort(-self.scores_)[:self._k]] = True
        return m

    def transform(self, X):
        return out(to_np(X)[:, self.get_support()])


class RFE(Estimator, TransformerMixin):
    """Recursive feature elimination with a linear model's |coefficients| as importance (ridge regression on the
    standardised features by default; any estimator with ``coef_`` or ``feature_importances_`` can be passed)."""
    _params = ("step", "estimator")

    def __init__(self, n_features_to_select=5):
        self._n_features_to_select, self._step, self._estimator = n_features_to_select, 1, None

    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        active = list(range(X.shape[1]))
        self.ranking_ = np.ones(X.shape[1], int)
        rank = X.shape[1]
        while len(active) > self._n_features_to_select:
            Xa = X[:, active]
            if self._estimator is not None:
                est = self._estimator.clone().fit(out(Xa), out(y))
                imp = np.abs(to_np(getattr(est, "coef_", None) if hasattr(est, "coef_") else est.feature_importances_)).ravel()
            else:
                Xs = (Xa - Xa.mean(0)) / np.where(Xa.std(0) == 0, 1.0, Xa.std(0))
                imp = np.abs(np.linalg.solve(Xs.T @ Xs + 1e-3 * np.eye(len(active)), Xs.T @ (y - y.mean())))
            drop = min(self._step, len(active) - self._n_features_to_select)
            for i in sorted(np.argsort(imp)[:drop], reverse=True):
                self.ranking_[active[i]] = rank
                rank -= 1
                active.pop(i)
        self.support_ = np.zeros(X.shape[1], bool)
        self.support_[active] = True
        self.ranking_[active] = 1
        return self

    def get_support(self):
        return self.support_

    def ranking(self):
        return self.ranking_

    def transform(self, X):
        return out(to_np(X)[:, self.support_])


def train_test_split(X, y, test_size=0.25, shuffle=True, seed=None):
    Xn, yn = to_np(X), to_np(y)
    n = len(Xn)
    idx = rng_of(seed).permutation(n) if shuffle else np.arange(n)
    nt = int(round(n * test_size)) if test_size < 1 else int(test_size)
    te, tr = idx[:nt], idx[nt:]
    return out(Xn[tr]), out(Xn[te]), out(yn[tr]), out(yn[te])
