"""Decision trees, forests, boosting, bagging, stacking, voting, isolation forest (ghostflow-ml/src/tree.rs,
ensemble.rs, ensemble_advanced.rs, stacking.rs, gradient_boosting.rs, lightgbm.rs).

Trees are grown on the host with vectorised split search (sorted prefix sums per feature); the reference trains
forest members in a rayon parallel loop (ensemble.rs:66-107), here members are trained in a thread pool."""
from __future__ import annotations

import enum
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from ._base import ClassifierMixin, Estimator, RegressorMixin, encode_classes, out, rng_of, sigmoid, softmax, to_np


class Criterion(enum.Enum):
    Gini = "gini"
    Entropy = "entropy"
    MSE = "mse"
    MAE = "mae"


class TreeNode:
    __slots__ = ("feature", "threshold", "left", "right", "value", "n", "impurity")

    def __init__(self, value, n, impurity):
        self.feature, self.threshold, self.left, self.right = -1, 0.0, None, None
        self.value, self.n, self.impurity = value, n, impurity

    @property
    def is_leaf(self):
        return self.left is None


def _impurity(counts, crit):
    n = counts.sum(-1, keepdims=True)
    p = counts / np.maximum(n, 1e-300)
    if crit == "entropy":
        return -(p * np.log2(np.where(p > 0, p, 1.0))).sum(-1)
    return 1.0 - (p ** 2).sum(-1)


class _Tree:
    """Greedy CART on arrays. ``Y``: one-hot class matrix (classification) or [n, 1] targets (regression);
    ``w``: sample weights. ``random_splits`` draws one random threshold per feature (extra-trees)."""

    def __init__(self, crit, max_depth, min_split, min_leaf, max_features, rng, random_splits=False, max_leaves=None):
        self.crit, self.max_depth, self.min_split, self.min_leaf = crit, max_depth, min_split, min_leaf
        self.max_features, self.rng, self.random_splits, self.max_leaves = max_features, rng, random_splits, max_leaves

    def _node_stats(self, Y, w):
        tot = (Y * w[:, None]).sum(0)
        if self.crit in ("gini", "entropy"):
            return tot / max(w.sum(), 1e-300), float(_impurity(tot, self.crit))
        mean = tot / max(w.sum(), 1e-300)
        if self.crit == "mae":
            med = np.median(Y[:, 0])
            return np.array([med]), float(np.abs(Y[:, 0] - med).mean())
        return mean, float(((Y - mean) ** 2 * w[:, None]).sum() / max(w.sum(), 1e-300))

    def _best_split(self, X, Y, w):
        n, d = X.shape
        feats = np.arange(d)
        if self.max_features and self.max_features < d:
            feats = self.rng.choice(d, self.max_features, replace=False)
        best = (0.0, -1, 0.0)
        Yw = Y * w[:, None]
        parent = self._node_stats(Y, w)[1] * w.sum()
        for f in feats:
            x = X[:, f]
            if self.random_splits:
                lo, hi = x.min(), x.max()
                if lo == hi:
                    continue
                th = self.rng.uniform(lo, hi)
                m = x <= th
                if m.sum() < self.min_leaf or (~m).sum() < self.min_leaf:
                    continue
                gl = self._node_stats(Y[m], w[m])[1] * w[m].sum()
                gr = self._node_stats(Y[~m], w[~m])[1] * w[~m].sum()
                gain = parent - gl - gr
                if gain > best[0]:
                    best = (gain, f, th)
                continue
            order = np.argsort(x, kind="stable")
            xs = x[order]
            cl = np.cumsum(Yw[order], 0)
            wl = np.cumsum(w[order])
            cr, wr = cl[-1] - cl, wl[-1] - wl
            valid = (xs[1:] != xs[:-1])
            valid &= (np.arange(1, n) >= self.min_leaf) & (np.arange(1, n) <= n - self.min_leaf)
            if not valid.any():
                continue
            cl, cr, wl_, wr_ = cl[:-1], cr[:-1], wl[:-1], wr[:-1]
            if self.crit in ("gini", "entropy"):
                child = _impurity(cl, self.crit) * wl_ + _impurity(cr, self.crit) * wr_
            else:
                # sum of squared deviations = sum y^2 - (sum y)^2 / n, per side
                sq = np.cumsum((Y[order] ** 2) * w[order][:, None], 0)
                sl, sr = sq[:-1], sq[-1] - sq[:-1]
                child = (sl - cl ** 2 / np.maximum(wl_, 1e-300)[:, None]).sum(1) + \
                        (sr - cr ** 2 / np.maximum(wr_, 1e-300)[:, None]).sum(1)
            gain = np.where(valid, parent - child, -np.inf)
            i = int(gain.argmax())
            if gain[i] > best[0] + 1e-12:
                best = (float(gain[i]), f, float((xs[i] + xs[i + 1]) / 2))
        return best

    def fit(self, X, Y, w):
        self.importances = np.zeros(X.shape[1])
        self.n_leaves = 1

        def grow(idx, depth):
            val, imp = self._node_stats(Y[idx], w[idx])
            node = TreeNode(val, len(idx), imp)
            if ((self.max_depth is not None and depth >= self.max_depth) or len(idx) < self.min_split or imp <= 1e-12
                    or (self.max_leaves and self.n_leaves >= self.max_leaves)):
                return node
            gain, f, th = self._best_split(X[idx], Y[idx], w[idx])
            if f < 0:
                return node
            m = X[idx, f] <= th
            if m.all() or not m.any():
                return node
            node.feature, node.threshold = f, th
            self.importances[f] += gain
            self.n_leaves += 1
            node.left, node.right = grow(idx[m], depth + 1), grow(idx[~m], depth + 1)
            return node

        self.root = grow(np.arange(len(X)), 0)
        return self

    def predict_value(self, X):
        res = np.empty((len(X), len(self.root.value)))

        def walk(node, idx):
            if node.is_leaf or len(idx) == 0:
                res[idx] = node.value
                return
            m = X[idx, node.feature] <= node.threshold
            walk(node.left, idx[m])
            walk(node.right, idx[~m])

        walk(self.root, np.arange(len(X)))
        return res

    def apply_depth(self, X):
        """Depth of the leaf reached by every row (isolation forest)."""
        res = np.zeros(len(X))

        def walk(node, idx, d):
            if node.is_leaf or len(idx) == 0:
                res[idx] = d + _c(node.n)
                return
            m = X[idx, node.feature] <= node.threshold
            walk(node.left, idx[m], d + 1)
            walk(node.right, idx[~m], d + 1)

        walk(self.root, np.arange(len(X)), 0)
        return res


def _c(n):
    return 0.0 if n <= 1 else 2.0 * (np.log(n - 1.0) + 0.5772156649) - 2.0 * (n - 1.0) / n if n > 2 else 1.0


def _resolve_max_features(mf, d, default):
    mf = default if mf is None else mf
    if mf == "sqrt":
        return max(1, int(np.sqrt(d)))
    if mf == "log2":
        return max(1, int(np.log2(d)))
    if isinstance(mf, float):
        return max(1, int(mf * d))
    return mf


class _TreeBase(Estimator):
    _params = ("criterion", "max_depth", "min_samples_split", "min_samples_leaf", "max_features", "seed")

    def _mk(self, d, rng=None, random_splits=False, default_mf=None):
        return _Tree(getattr(self._criterion, "value", self._criterion), self._max_depth, self._min_samples_split,
                     self._min_samples_leaf, _resolve_max_features(self._max_features, d, default_mf),
                     rng or rng_of(self._seed), random_splits)

    def feature_importances(self):
        imp = self.feature_importances_
        return out(imp)


class DecisionTreeClassifier(_TreeBase, ClassifierMixin):
    def __init__(self):
        self._criterion, self._max_depth, self._min_samples_split, self._min_samples_leaf = Criterion.Gini, None, 2, 1
        self._max_features, self._seed = None, 0

    def fit(self, X, y, sample_weight=None, _rng=None, _random_splits=False, _classes=None):
        X = to_np(X)
        if _classes is None:
            self.classes_, yc = encode_classes(y)
        else:
            self.classes_, yc = _classes, np.searchsorted(_classes, to_np(y))
        Y = (yc[:, None] == np.arange(len(self.classes_))[None]).astype(float)
        w = np.ones(len(X)) if sample_weight is None else to_np(sample_weight)
        self.tree_ = self._mk(X.shape[1], _rng, _random_splits).fit(X, Y, w)
        s = self.tree_.importances.sum()
        self.feature_importances_ = self.tree_.importances / s if s > 0 else self.tree_.importances
        return self

    def predict_proba(self, X):
        return out(self.tree_.predict_value(to_np(X)))

    def predict(self, X):
        return out(self.classes_[self.tree_.predict_value(to_np(X)).argmax(1)])


class DecisionTreeRegressor(_TreeBase, RegressorMixin):
    def __init__(self):
        self._criterion, self._max_depth, self._min_samples_split, self._min_samples_leaf = Criterion.MSE, None, 2, 1
        self._max_features, self._seed = None, 0

    def fit(self, X, y, sample_weight=None, _rng=None, _random_splits=False):
        X, y = to_np(X), to_np(y)
        w = np.ones(len(X)) if sample_weight is None else to_np(sample_weight)
        self.tree_ = self._mk(X.shape[1], _rng, _random_splits).fit(X, y[:, None], w)
        s = self.tree_.importances.sum()
        self.feature_importances_ = self.tree_.importances / s if s > 0 else self.tree_.importances
        return self

    def predict(self, X):
        return out(self.tree_.predict_value(to_np(X))[:, 0])


# ----------------------------------------------------------------------------- forests / bagging
class _ForestBase(Estimator):
    _params = ("max_depth", "max_features", "min_samples_split", "min_samples_leaf", "bootstrap", "seed", "n_jobs",
               "max_samples")
    _random_splits = False
    _classifier = True

    def __init__(self, n_estimators=100, max_depth=None, **params):
        """``n_estimators`` as in the reference's constructor; every builder-style setting (``max_depth``,
        ``max_features``, ``min_samples_split``, ...) may also be given as a keyword."""
        self._n_estimators, self._max_depth, self._max_features = n_estimators, max_depth, None
        self._min_samples_split, self._min_samples_leaf, self._bootstrap, self._seed, self._n_jobs = 2, 1, True, 0, 8
        self._max_samples = None
        if params:
            self.set(**params)

    def _fit_members(self, X, y):
        n = len(X)
        seeds = rng_of(self._seed).integers(0, 2 ** 31 - 1, self._n_estimators)
        classes = np.unique(y) if self._classifier else None

        def one(seed):
            r = rng_of(int(seed))
            m = int(self._max_samples * n) if isinstance(self._max_samples, float) else (self._max_samples or n)
            idx = r.integers(0, n, m) if self._bootstrap else np.arange(n)
            base = (DecisionTreeClassifier if self._classifier else DecisionTreeRegressor)()
            base.set(max_depth=self._max_depth, min_samples_split=self._min_samples_split,
                     min_samples_leaf=self._min_samples_leaf,
                     max_features=self._max_features or ("sqrt" if self._classifier else 1.0))
            if self._classifier:
                return base.fit(X[idx], y[idx], _rng=r, _random_splits=self._random_splits, _classes=classes)
            return base.fit(X[idx], y[idx], _rng=r, _random_splits=self._random_splits)

        with ThreadPoolExecutor(self._n_jobs) as ex:
            self.estimators_ = list(ex.map(one, seeds))
        self.feature_importances_ = np.mean([e.feature_importances_ for e in self.estimators_], 0)

    def feature_importances(self):
        return out(self.feature_importances_)


class RandomForestClassifier(_ForestBase, ClassifierMixin):
    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        self.classes_ = np.unique(y)
        self._fit_members(X, y)
        return self

    def predict_proba(self, X):
        return out(np.mean([to_np(e.predict_proba(X)) for e in self.estimators_], 0))

    def predict(self, X):
        return out(self.classes_[to_np(self.predict_proba(X)).argmax(1)])


RandomForest = RandomForestClassifier   # the name used in the reference's README example


class RandomForestRegressor(_ForestBase, RegressorMixin):
    _classifier = False

    def fit(self, X, y):
        self._fit_members(to_np(X), to_np(y))
        return self

    def predict(self, X):
        return out(np.mean([to_np(e.predict(X)) for e in self.estimators_], 0))


class ExtraTreesClassifier(RandomForestClassifier):
    _random_splits = True

    def __init__(self, n_estimators=100):
        super().__init__(n_estimators)
        self._bootstrap = False


class BaggingClassifier(RandomForestClassifier):
    """Bagging of full-feature trees (or of any estimator passed with ``base_estimator``)."""
    _params = ("base_estimator",)

    def __init__(self, n_estimators=10):
        super().__init__(n_estimators)
        self._max_features, self._base_estimator = 1.0, None

    def fit(self, X, y):
        if self._base_estimator is None:
            return super().fit(X, y)
        X, y = to_np(X), to_np(y)
        self.classes_ = np.unique(y)
        r = rng_of(self._seed)
        self.estimators_ = []
        for _ in range(self._n_estimators):
            idx = r.integers(0, len(X), int((self._max_samples or 1.0) * len(X)))
            self.estimators_.append(self._base_estimator.clone().fit(out(X[idx]), out(y[idx])))
        return self

    def predict_proba(self, X):
        if self._base_estimator is None:
            return super().predict_proba(X)
        P = np.zeros((len(to_np(X)), len(self.classes_)))
        for e in self.estimators_:
            p = to_np(e.predict(X))
            P += (p[:, None] == self.classes_[None]).astype(float)
        return out(P / len(self.estimators_))


class IsolationForest(Estimator):
    _params = ("contamination", "max_samples", "seed")

    def __init__(self, n_estimators=100):
        self._n_estimators, self._contamination, self._max_samples, self._seed = n_estimators, 0.1, 256, 0

    def fit(self, X, y=None):
        X = to_np(X)
        r = rng_of(self._seed)
        self._psi = min(self._max_samples, len(X))
        depth = int(np.ceil(np.log2(max(self._psi, 2))))
        self.trees_ = []
        for _ in range(self._n_estimators):
            idx = r.choice(len(X), self._psi, replace=False)
            t = _Tree("mse", depth, 2, 1, 1, r, random_splits=True)
            # isolation trees ignore targets: a random target keeps every node impure, so splitting continues
            self.trees_.append(t.fit(X[idx], r.standard_normal((self._psi, 1)), np.ones(self._psi)))
        s = self.score_samples(X)
        self.threshold_ = np.quantile(s, self._contamination)
        return self

    def score_samples(self, X):
        """Negative anomaly score: lower means more abnormal."""
        X = to_np(X)
        h = np.mean([t.apply_depth(X) for t in self.trees_], 0)
        return -(2.0 ** (-h / max(_c(self._psi), 1e-12)))

    def decision_function(self, X):
        return out(self.score_samples(X) - self.threshold_)

    def predict(self, X):
        return out(np.where(self.score_samples(X) < self.threshold_, -1.0, 1.0))


# ----------------------------------------------------------------------------- boosting
class GBLoss(enum.Enum):
    SquaredError = "squared_error"
    AbsoluteError = "absolute_error"
    Huber = "huber"
    Deviance = "deviance"


class GradientBoostingRegressor(Estimator, RegressorMixin):
    _params = ("learning_rate", "max_depth", "subsample", "loss", "min_samples_split", "seed")

    def __init__(self, n_estimators=100):
        self._n_estimators, self._learning_rate, self._max_depth, self._subsample = n_estimators, 0.1, 3, 1.0
        self._loss, self._min_samples_split, self._seed = GBLoss.SquaredError, 2, 0

    def _neg_grad(self, y, f):
        l = getattr(self._loss, "value", self._loss)
        r = y - f
        if l == "absolute_error":
            return np.sign(r)
        if l == "huber":
            d = np.quantile(np.abs(r), 0.9)
            return np.where(np.abs(r) <= d, r, d * np.sign(r))
        return r

    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        r = rng_of(self._seed)
        self.init_ = np.median(y) if getattr(self._loss, "value", self._loss) == "absolute_error" else y.mean()
        f = np.full(len(y), self.init_)
        self.estimators_, imp = [], np.zeros(X.shape[1])
        for _ in range(self._n_estimators):
            idx = r.choice(len(X), int(self._subsample * len(X)), replace=False) if self._subsample < 1 else np.arange(len(X))
            t = DecisionTreeRegressor().set(max_depth=self._max_depth, min_samples_split=self._min_samples_split)
            t.fit(X[idx], self._neg_grad(y, f)[idx], _rng=r)
            f += self._learning_rate * to_np(t.predict(X))
            self.estimators_.append(t)
            imp += t.feature_importances_
        self.feature_importances_ = imp / max(imp.sum(), 1e-300)
        return self

    def predict(self, X):
        return out(self.init_ + self._learning_rate * sum(to_np(t.predict(X)) for t in self.estimators_))

    def feature_importances(self):
        return out(self.feature_importances_)


class GradientBoostingClassifier(Estimator, ClassifierMixin):
    _params = ("learning_rate", "max_depth", "subsample", "min_samples_split", "seed")

    def __init__(self, n_estimators=100):
        self._n_estimators, self._learning_rate, self._max_depth, self._subsample = n_estimators, 0.1, 3, 1.0
        self._min_samples_split, self._seed = 2, 0

    def fit(self, X, y):
        X = to_np(X)
        self.classes_, yc = encode_classes(y)
        k = len(self.classes_)
        Y = (yc[:, None] == np.arange(k)[None]).astype(float)
        r = rng_of(self._seed)
        self.init_ = np.log(np.maximum(Y.mean(0), 1e-12))
        F = np.tile(self.init_, (len(X), 1))
        self.estimators_, imp = [], np.zeros(X.shape[1])
        for _ in range(self._n_estimators):
            P = softmax(F)
            stage = []
            for c in range(k):
                t = DecisionTreeRegressor().set(max_depth=self._max_depth, min_samples_split=self._min_samples_split)
                t.fit(X, Y[:, c] - P[:, c], _rng=r)
                F[:, c] += self._learning_rate * to_np(t.predict(X))
                stage.append(t)
                imp += t.feature_importances_
            self.estimators_.append(stage)
        self.feature_importances_ = imp / max(imp.sum(), 1e-300)
        return self

    def decision_function(self, X):
        F = np.tile(self.init_, (len(to_np(X)), 1))
        for stage in self.estimators_:
            for c, t in enumerate(stage):
                F[:, c] += self._learning_rate * to_np(t.predict(X))
        return F

    def predict_proba(self, X):
        return out(softmax(self.decision_function(X)))

    def predict(self, X):
        return out(self.classes_[self.decision_function(X).argmax(1)])

    def feature_importances(self):
        return out(self.feature_importances_)


class _NewtonTree:
    """Second-order tree (XGBoost gain with L1/L2 leaf regularisation, histogram bins for LightGBM-style growth)."""

    def __init__(self, max_depth, lam, alpha, gamma, min_child_weight, colsample, rng, max_leaves=None, bins=None):
        self.max_depth, self.lam, self.alpha, self.gamma, self.mcw = max_depth, lam, alpha, gamma, min_child_weight
        self.colsample, self.rng, self.max_leaves, self.bins = colsample, rng, max_leaves, bins

    def _w(self, G, H):
        return -np.sign(G) * np.maximum(np.abs(G) - self.alpha, 0) / (H + self.lam)

    def _score(self, G, H):
        return np.maximum(np.abs(G) - self.alpha, 0) ** 2 / (H + self.lam)

    def _split(self, X, g, h):
        d = X.shape[1]
        feats = self.rng.choice(d, max(1, int(self.colsample * d)), replace=False) if self.colsample < 1 else np.arange(d)
        G, H = g.sum(), h.sum()
        best = (0.0, -1, 0.0)
        for f in feats:
            x = X[:, f]
            if self.bins:
                edges = np.unique(np.quantile(x, np.linspace(0, 1, self.bins + 1)[1:-1]))
                if len(edges) == 0:
                    continue
                b = np.searchsorted(edges, x, side="left")
                gl = np.cumsum(np.bincount(b, g, len(edges) + 1))[:-1]
                hl = np.cumsum(np.bincount(b, h, len(edges) + 1))[:-1]
                ths = edges
            else:
                o = np.argsort(x, kind="stable")
                xs = x[o]
                gl, hl = np.cumsum(g[o])[:-1], np.cumsum(h[o])[:-1]
                ok = xs[1:] != xs[:-1]
                if not ok.any():
                    continue
                gl, hl, ths = gl[ok], hl[ok], ((xs[1:] + xs[:-1]) / 2)[ok]
            gr, hr = G - gl, H - hl
            gain = 0.5 * (self._score(gl, hl) + self._score(gr, hr) - self._score(G, H)) - self.gamma
            gain = np.where((hl >= self.mcw) & (hr >= self.mcw), gain, -np.inf)
            i = int(gain.argmax())
            if gain[i] > best[0]:
                best = (float(gain[i]), f, float(ths[i]))
        return best

    def fit(self, X, g, h):
        self.importances = np.zeros(X.shape[1])
        self.n_leaves = 1

        def grow(idx, depth):
            node = TreeNode(np.array([self._w(g[idx].sum(), h[idx].sum())]), len(idx), 0.0)
            if depth >= self.max_depth or len(idx) < 2 or (self.max_leaves and self.n_leaves >= self.max_leaves):
                return node
            gain, f, th = self._split(X[idx], g[idx], h[idx])
            if f < 0:
                return node
            m = X[idx, f] <= th
            if m.all() or not m.any():
                return node
            node.feature, node.threshold = f, th
            self.importances[f] += gain
            self.n_leaves += 1
            node.left, node.right = grow(idx[m], depth + 1), grow(idx[~m], depth + 1)
            return node

        self.root = grow(np.arange(len(X)), 0)
        return self

    predict_value = _Tree.predict_value


class _XGBBase(Estimator):
    _params = ("learning_rate", "max_depth", "subsample", "colsample_bytree", "reg_alpha", "reg_lambda", "gamma",
               "min_child_weight", "seed")
    _bins = None
    _max_leaves = None

    def __init__(self, n_estimators=100):
        self._n_estimators, self._learning_rate, self._max_depth, self._subsample = n_estimators, 0.3, 6, 1.0
        self._colsample_bytree, self._reg_alpha, self._reg_lambda, self._gamma = 1.0, 0.0, 1.0, 0.0
        self._min_child_weight, self._seed = 1.0, 0

    def _tree(self, r):
        return _NewtonTree(self._max_depth if self._max_depth and self._max_depth > 0 else 64, self._reg_lambda,
                           self._reg_alpha, self._gamma, self._min_child_weight, self._colsample_bytree, r,
                           self._max_leaves, self._bins)

    def _boost(self, X, grad_hess, n_out):
        r = rng_of(self._seed)
        F = np.zeros((len(X), n_out))
        self.trees_, imp = [], np.zeros(X.shape[1])
        for _ in range(self._n_estimators):
            G, H = grad_hess(F)
            idx = r.choice(len(X), int(self._subsample * len(X)), replace=False) if self._subsample < 1 else np.arange(len(X))
            stage = []
            for c in range(n_out):
                t = self._tree(r).fit(X[idx], G[idx, c], H[idx, c])
                F[:, c] += self._learning_rate * t.predict_value(X)[:, 0]
                stage.append(t)
                imp += t.importances
            self.trees_.append(stage)
        self.feature_importances_ = imp / max(imp.sum(), 1e-300)

    def _raw(self, X):
        X = to_np(X)
        F = np.zeros((len(X), len(self.trees_[0])))
        for stage in self.trees_:
            for c, t in enumerate(stage):
                F[:, c] += self._learning_rate * t.predict_value(X)[:, 0]
        return F

    def feature_importances(self):
        return out(self.feature_importances_)


class XGBoostRegressor(_XGBBase, RegressorMixin):
    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        self.base_ = y.mean()
        self._boost(X, lambda F: ((F[:, :1] + self.base_ - y[:, None]), np.ones((len(y), 1))), 1)
        return self

    def predict(self, X):
        return out(self._raw(X)[:, 0] + self.base_)


class XGBoostClassifier(_XGBBase, ClassifierMixin):
    def fit(self, X, y):
        X = to_np(X)
        self.classes_, yc = encode_classes(y)
        k = len(self.classes_)
        if k == 2:
            t = yc.astype(float)[:, None]

            def gh(F):
                p = sigmoid(F)
                return p - t, np.maximum(p * (1 - p), 1e-16)
            self._boost(X, gh, 1)
        else:
            Y = (yc[:, None] == np.arange(k)[None]).astype(float)

            def gh(F):
                P = softmax(F)
                return P - Y, np.maximum(2 * P * (1 - P), 1e-16)
            self._boost(X, gh, k)
        return self

    def predict_proba(self, X):
        F = self._raw(X)
        if F.shape[1] == 1:
            p = sigmoid(F[:, 0])
            return out(np.stack((1 - p, p), 1))
        return out(softmax(F))

    def predict(self, X):
        return out(self.classes_[to_np(self.predict_proba(X)).argmax(1)])


class LightGBMClassifier(XGBoostClassifier):
    """Histogram-binned second-order boosting with a leaf budget (``num_leaves``) and feature sub-sampling."""
    _params = ("num_leaves", "feature_fraction", "max_bin")
    _bins = 63

    def __init__(self, n_estimators=100):
        super().__init__(n_estimators)
        self._learning_rate, self._max_depth, self._num_leaves, self._feature_fraction, self._max_bin = 0.1, -1, 31, 1.0, 63

    def _tree(self, r):
        self._max_leaves, self._bins, self._colsample_bytree = self._num_leaves, self._max_bin, self._feature_fraction
        return super()._tree(r)


class AdaBoostClassifier(Estimator, ClassifierMixin):
    _params = ("learning_rate", "algorithm", "max_depth", "seed")

    def __init__(self, n_estimators=50):
        self._n_estimators, self._learning_rate, self._algorithm, self._max_depth, self._seed = n_estimators, 1.0, "SAMME", 1, 0

    def fit(self, X, y):
        X = to_np(X)
        self.classes_, yc = encode_classes(y)
        k, n = len(self.classes_), len(X)
        w = np.full(n, 1.0 / n)
        self.estimators_, self.alphas_ = [], []
        r = rng_of(self._seed)
        real = str(getattr(self._algorithm, "value", self._algorithm)).upper().endswith("R")
        for _ in range(self._n_estimators):
            t = DecisionTreeClassifier().set(max_depth=self._max_depth).fit(X, yc.astype(float), sample_weight=w, _rng=r,
                                                                            _classes=np.arange(k).astype(float))
            if real:
                P = np.clip(to_np(t.predict_proba(X)), 1e-12, 1)
                L = np.log(P)
                code = np.where(yc[:, None] == np.arange(k)[None], 1.0, -1.0 / (k - 1))
                w *= np.exp(-self._learning_rate * (k - 1) / k * (code * L).sum(1))
                self.alphas_.append(1.0)
            else:
                miss = to_np(t.predict(X)).astype(int) != yc
                err = (w * miss).sum() / w.sum()
                if err >= 1 - 1.0 / k:
                    break
                a = self._learning_rate * (np.log((1 - err) / max(err, 1e-12)) + np.log(k - 1))
                w *= np.exp(a * miss)
                self.alphas_.append(a)
            self.estimators_.append(t)
            w /= w.sum()
            if not real and err < 1e-12:
                break
        self._real = real
        return self

    def decision_function(self, X):
        k = len(self.classes_)
        S = np.zeros((len(to_np(X)), k))
        for t, a in zip(self.estimators_, self.alphas_):
            if self._real:
                L = np.log(np.clip(to_np(t.predict_proba(X)), 1e-12, 1))
                S += (k - 1) * (L - L.mean(1, keepdims=True))
            else:
                S[np.arange(len(S)), to_np(t.predict(X)).astype(int)] += a
        return S

    def predict_proba(self, X):
        return out(softmax(self.decision_function(X) / max(1, len(self.estimators_))))

    def predict(self, X):
        return out(self.classes_[self.decision_function(X).argmax(1)])


# ----------------------------------------------------------------------------- voting / stacking
class VotingType(enum.Enum):
    Hard = "hard"
    Soft = "soft"


class VotingClassifier(Estimator, ClassifierMixin):
    _params = ("weights",)

    def __init__(self, voting=VotingType.Hard):
        self._voting, self._weights, self.estimators = voting, None, []

    def add_estimator(self, est, name=None):
        self.estimators.append((name or f"est{len(self.estimators)}", est))
        return self

    def fit(self, X, y):
        self.classes_ = np.unique(to_np(y))
        for _, e in self.estimators:
            e.fit(X, y)
        return self

    def predict_proba(self, X):
        w = self._weights or [1.0] * len(self.estimators)
        if getattr(self._voting, "value", self._voting) == "soft":
            P = sum(wi * to_np(e.predict_proba(X)) for wi, (_, e) in zip(w, self.estimators))
        else:
            P = sum(wi * (to_np(e.predict(X))[:, None] == self.classes_[None]).astype(float)
                    for wi, (_, e) in zip(w, self.estimators))
        return out(P / sum(w))

    def predict(self, X):
        return out(self.classes_[to_np(self.predict_proba(X)).argmax(1)])


class StackMethod(enum.Enum):
    Predict = "predict"
    PredictProba = "predict_proba"


class LinearMeta(Estimator, RegressorMixin):
    def fit(self, X, y):
        from .linear import Ridge
        self._m = Ridge(1e-6).fit(X, y)
        return self

    def predict(self, X):
        return self._m.predict(X)


class LogisticMeta(Estimator, ClassifierMixin):
    def fit(self, X, y):
        from .linear import LogisticRegression
        self._m = LogisticRegression().fit(X, y)
        self.classes_ = self._m.classes_
        return self

    def predict(self, X):
        return self._m.predict(X)

    def predict_proba(self, X):
        return self._m.predict_proba(X)


class _StackingBase(Estimator):
    _params = ("cv", "passthrough", "stack_method", "final_estimator")

    def add_estimator(self, est, name=None):
        self.estimators.append((name or f"est{len(self.estimators)}", est))
        return self

    def _features(self, est, X):
        if getattr(self._stack_method, "value", self._stack_method) == "predict_proba" and hasattr(est, "predict_proba"):
            return to_np(est.predict_proba(X))
        return to_np(est.predict(X))[:, None]

    def fit(self, X, y):
        from .model_selection import KFold
        Xn, yn = to_np(X), to_np(y)
        blocks = []
        for _, e in self.estimators:
            oof = None
            for tr, te in KFold(self._cv, True, 0).split(Xn):
                m = e.clone().fit(out(Xn[tr]), out(yn[tr]))
                f = self._features(m, out(Xn[te]))
                if oof is None:
                    oof = np.zeros((len(Xn), f.shape[1]))
                oof[te] = f
            blocks.append(oof)
            e.fit(X, y)
        Z = np.hstack(blocks + ([Xn] if self._passthrough else []))
        self.final_ = self._final_estimator.clone().fit(out(Z), out(yn))
        return self

    def _meta_in(self, X):
        Z = [self._features(e, X) for _, e in self.estimators]
        return out(np.hstack(Z + ([to_np(X)] if self._passthrough else [])))

    def predict(self, X):
        return self.final_.predict(self._meta_in(X))


class StackingRegressor(_StackingBase, RegressorMixin):
    def __init__(self):
        self.estimators, self._cv, self._passthrough, self._stack_method = [], 5, False, StackMethod.Predict
        self._final_estimator = LinearMeta()


class StackingClassifier(_StackingBase, ClassifierMixin):
    def __init__(self):
        self.estimators, self._cv, self._passthrough, self._stack_method = [], 5, False, StackMethod.PredictProba
        self._final_estimator = LogisticMeta()

    def predict_proba(self, X):
        return self.final_.predict_proba(self._meta_in(X))
