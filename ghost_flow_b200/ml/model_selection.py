"""Splitters, cross-validation, search and hyper-parameter optimisation (ghostflow-ml/src/model_selection.rs,
model_selection_extended.rs, hyperparameter_optimization.rs)."""
from __future__ import annotations

import enum
import itertools
import math

import numpy as np

from ._base import Estimator, out, rng_of, to_np


class KFold:
    def __init__(self, n_splits=5, shuffle=False, seed=None):
        self.n_splits, self.shuffle, self.seed = n_splits, shuffle, seed

    def split(self, X, y=None, groups=None):
        n = len(to_np(X))
        idx = rng_of(self.seed).permutation(n) if self.shuffle else np.arange(n)
        for f in np.array_split(idx, self.n_splits):
            yield np.setdiff1d(idx, f, assume_unique=True), f


class StratifiedKFold(KFold):
    def split(self, X, y, groups=None):
        y = to_np(y)
        folds = [[] for _ in range(self.n_splits)]
        r = rng_of(self.seed)
        for c in np.unique(y):
            idx = np.where(y == c)[0]
            if self.shuffle:
                idx = r.permutation(idx)
            for i, v in enumerate(idx):
                folds[i % self.n_splits].append(v)
        allidx = np.arange(len(y))
        for f in folds:
            f = np.array(sorted(f))
            yield np.setdiff1d(allidx, f), f


class LeaveOneOut:
    def split(self, X, y=None, groups=None):
        n = len(to_np(X))
        for i in range(n):
            yield np.delete(np.arange(n), i), np.array([i])


class TimeSeriesSplit:
    def __init__(self, n_splits=5):
        self.n_splits = n_splits

    def split(self, X, y=None, groups=None):
        n = len(to_np(X))
        ts = n // (self.n_splits + 1)
        for i in range(1, self.n_splits + 1):
            yield np.arange(0, n - (self.n_splits - i + 1) * ts), np.arange(n - (self.n_splits - i + 1) * ts,
                                                                          n - (self.n_splits - i) * ts)


class GroupKFold:
    def __init__(self, n_splits=5):
        self.n_splits = n_splits

    def split(self, X, y=None, groups=None):
        g = to_np(groups)
        ug, counts = np.unique(g, return_counts=True)
        load = np.zeros(self.n_splits)
        assign = {}
        for grp in ug[np.argsort(-counts)]:
            f = int(load.argmin())
            assign[grp] = f
            load[f] += counts[ug == grp][0]
        fold_of = np.array([assign[v] for v in g])
        for f in range(self.n_splits):
            yield np.where(fold_of != f)[0], np.where(fold_of == f)[0]


class RepeatedKFold:
    def __init__(self, n_splits=5, n_repeats=10, seed=0):
        self.n_splits, self.n_repeats, self.seed = n_splits, n_repeats, seed

    def split(self, X, y=None, groups=None):
        for r in range(self.n_repeats):
            yield from KFold(self.n_splits, True, self.seed + r).split(X)


class StratifiedShuffleSplit:
    def __init__(self, n_splits=10, test_size=0.2, seed=None):
        self.n_splits, self.test_size, self.seed = n_splits, test_size, seed

    def split(self, X, y, groups=None):
        y = to_np(y)
        r = rng_of(self.seed)
        for _ in range(self.n_splits):
            te = []
            for c in np.unique(y):
                idx = r.permutation(np.where(y == c)[0])
                te.extend(idx[:max(1, int(round(len(idx) * self.test_size)))])
            te = np.array(sorted(te))
            yield np.setdiff1d(np.arange(len(y)), te), te


def shuffle_split(n, n_splits=10, test_size=0.2, seed=None):
    r = rng_of(seed)
    for _ in range(n_splits):
        p = r.permutation(n)
        nt = int(round(n * test_size))
        yield p[nt:], p[:nt]


def cross_val_score(estimator, X, y, cv=5, scoring=None):
    Xn, yn = to_np(X), to_np(y)
    cv = KFold(cv) if isinstance(cv, int) else cv
    scores = []
    for tr, te in cv.split(Xn, yn):
        est = estimator.clone().fit(out(Xn[tr]), out(yn[tr]))
        scores.append(scoring(yn[te], to_np(est.predict(out(Xn[te])))) if scoring else est.score(out(Xn[te]), out(yn[te])))
    return np.array(scores)


def parameter_grid(grid: dict):
    keys = list(grid)
    return [dict(zip(keys, v)) for v in itertools.product(*(grid[k] for k in keys))]


def learning_curve(estimator, X, y, train_sizes=(0.1, 0.325, 0.55, 0.775, 1.0), cv=5):
    Xn, yn = to_np(X), to_np(y)
    sizes, tr_s, te_s = [], [], []
    for frac in train_sizes:
        a, b = [], []
        for tr, te in KFold(cv).split(Xn):
            sub = tr[:max(2, int(len(tr) * frac))]
            est = estimator.clone().fit(out(Xn[sub]), out(yn[sub]))
            a.append(est.score(out(Xn[sub]), out(yn[sub])))
            b.append(est.score(out(Xn[te]), out(yn[te])))
        sizes.append(int(len(Xn) * (cv - 1) / cv * frac))
        tr_s.append(a)
        te_s.append(b)
    return np.array(sizes), np.array(tr_s), np.array(te_s)


def validation_curve(estimator, X, y, param_name, param_range, cv=5):
    tr_s, te_s = [], []
    Xn, yn = to_np(X), to_np(y)
    for v in param_range:
        a, b = [], []
        for tr, te in KFold(cv).split(Xn):
            est = estimator.clone().set(**{param_name: v}).fit(out(Xn[tr]), out(yn[tr]))
            a.append(est.score(out(Xn[tr]), out(yn[tr])))
            b.append(est.score(out(Xn[te]), out(yn[te])))
        tr_s.append(a)
        te_s.append(b)
    return np.array(tr_s), np.array(te_s)


class GridSearchCV:
    def __init__(self, estimator, param_grid, cv=3):
        self.estimator, self.param_grid, self.cv = estimator, param_grid, cv

    def _candidates(self):
        return parameter_grid(self.param_grid)

    def fit(self, X, y):
        self.results_ = []
        for params in self._candidates():
            s = cross_val_score(self.estimator.clone().set(**params), X, y, self.cv).mean()
            self.results_.append((params, float(s)))
        self.best_params_, self.best_score_ = max(self.results_, key=lambda t: t[1])
        self.best_estimator_ = self.estimator.clone().set(**self.best_params_).fit(X, y)
        return self

    def predict(self, X):
        return self.best_estimator_.predict(X)


class RandomizedSearchCV(GridSearchCV):
    def __init__(self, estimator, param_distributions, n_iter=10, cv=3, seed=0):
        super().__init__(estimator, param_distributions, cv)
        self.n_iter, self.seed = n_iter, seed

    def _candidates(self):
        r = rng_of(self.seed)
        res = []
        for _ in range(self.n_iter):
            res.append({k: (v[int(r.integers(len(v)))] if isinstance(v, (list, tuple)) else v(r))
                        for k, v in self.param_grid.items()})
        return res


# ----------------------------------------------------------------------------- black-box optimisers
class ParameterSpace:
    """name -> ("float", lo, hi) | ("log", lo, hi) | ("int", lo, hi) | ("choice", [values])."""

    def __init__(self, **dims):
        self.dims = dict(dims)

    def add_float(self, name, lo, hi, log=False):
        self.dims[name] = ("log" if log else "float", lo, hi)
        return self

    def add_int(self, name, lo, hi):
        self.dims[name] = ("int", lo, hi)
        return self

    def add_choice(self, name, values):
        self.dims[name] = ("choice", list(values))
        return self

    def sample(self, r):
        return self.decode(r.random(len(self.dims)))

    def decode(self, u):
        p = {}
        for x, (k, d) in zip(u, self.dims.items()):
            x = float(np.clip(x, 0, 1 - 1e-12))
            if d[0] == "float":
                p[k] = d[1] + x * (d[2] - d[1])
            elif d[0] == "log":
                p[k] = float(np.exp(np.log(d[1]) + x * (np.log(d[2]) - np.log(d[1]))))
            elif d[0] == "int":
                p[k] = int(d[1] + math.floor(x * (d[2] - d[1] + 1)))
            else:
                p[k] = d[1][int(x * len(d[1]))]
        return p


class AcquisitionFunction(enum.Enum):
    ExpectedImprovement = "ei"
    UpperConfidenceBound = "ucb"
    ProbabilityOfImprovement = "pi"


class RandomSearch:
    def __init__(self, space: ParameterSpace, n_iter=20, seed=0):
        self.space, self.n_iter, self.seed = space, n_iter, seed

    def optimize(self, objective):
        """Maximises ``objective(params) -> float``. Returns (best params, best value)."""
        r = rng_of(self.seed)
        self.history = []
        for _ in range(self.n_iter):
            p = self.space.sample(r)
            self.history.append((p, float(objective(p))))
        return max(self.history, key=lambda t: t[1])


class GridSearch:
    def __init__(self, grid: dict):
        self.grid = grid

    def optimize(self, objective):
        self.history = [(p, float(objective(p))) for p in parameter_grid(self.grid)]
        return max(self.history, key=lambda t: t[1])


class BayesianOptimization:
    """Gaussian-process surrogate (RBF kernel on the unit cube) with an acquisition maximised over random
    candidates."""

    def __init__(self, space: ParameterSpace, n_iter=25, n_initial=5, acquisition=AcquisitionFunction.ExpectedImprovement,
                 seed=0):
        self.space, self.n_iter, self.n_initial, self.acquisition, self.seed = space, n_iter, n_initial, acquisition, seed

    def _gp(self, U, y, C, ls=0.3, noise=1e-6):
        def k(a, b):
            return np.exp(-0.5 * ((a[:, None, :] - b[None, :, :]) ** 2).sum(-1) / ls ** 2)
        K = k(U, U) + noise * np.eye(len(U))
        L = np.linalg.cholesky(K)
        mu0, sd0 = y.mean(), y.std() + 1e-12
        alpha = np.linalg.solve(L.T, np.linalg.solve(L, (y - mu0) / sd0))
        Ks = k(C, U)
        mu = Ks @ alpha * sd0 + mu0
        v = np.linalg.solve(L, Ks.T)
        var = np.maximum(1.0 - (v ** 2).sum(0), 1e-12) * sd0 ** 2
        return mu, np.sqrt(var)

    def optimize(self, objective):
        from scipy.stats import norm
        r = rng_of(self.seed)
        d = len(self.space.dims)
        U = r.random((self.n_initial, d))
        y = np.array([float(objective(self.space.decode(u))) for u in U])
        for _ in range(self.n_iter - self.n_initial):
            C = r.random((512, d))
            mu, sd = self._gp(U, y, C)
            best = y.max()
            z = (mu - best) / sd
            a = self.acquisition
            acq = ((mu - best) * norm.cdf(z) + sd * norm.pdf(z) if a is AcquisitionFunction.ExpectedImprovement
                   else mu + 2.0 * sd if a is AcquisitionFunction.UpperConfidenceBound else norm.cdf(z))
            u = C[int(acq.argmax())]
            U = np.vstack((U, u))
            y = np.append(y, float(objective(self.space.decode(u))))
        self.history = [(self.space.decode(u), float(v)) for u, v in zip(U, y)]
        return max(self.history, key=lambda t: t[1])


class Hyperband:
    """Successive halving over brackets. ``objective(params, budget) -> float`` (higher is better)."""

    def __init__(self, space: ParameterSpace, max_budget=27, eta=3, seed=0):
        self.space, self.max_budget, self.eta, self.seed = space, max_budget, eta, seed

    def _propose(self, r, n):
        return [self.space.sample(r) for _ in range(n)]

    def optimize(self, objective):
        r = rng_of(self.seed)
        smax = int(math.log(self.max_budget) / math.log(self.eta) + 1e-9)
        self.history = []
        for s in range(smax, -1, -1):
            n = int(math.ceil((smax + 1) / (s + 1) * self.eta ** s))
            configs = self._propose(r, n)
            for i in range(s + 1):
                budget = self.max_budget * self.eta ** (i - s)
                scores = [float(objective(c, budget)) for c in configs]
                self.history += [(c, v, budget) for c, v in zip(configs, scores)]
                keep = max(1, int(len(configs) / self.eta))
                configs = [configs[j] for j in np.argsort(scores)[::-1][:keep]]
        best = max(self.history, key=lambda t: (t[1]))
        return best[0], best[1]


class BOHB(Hyperband):
    """Hyperband whose proposals come from a density-ratio model (good vs bad observations, Gaussian KDE on the
    unit cube) once enough results exist."""

    def _propose(self, r, n):
        obs = [(u, v) for u, v in getattr(self, "_obs", [])]
        d = len(self.space.dims)
        res = []
        for _ in range(n):
            if len(obs) < 2 * d + 2 or r.random() < 0.2:
                u = r.random(d)
            else:
                vals = np.array([v for _, v in obs])
                U = np.stack([u for u, _ in obs])
                good = U[vals >= np.quantile(vals, 0.75)]
                bad = U[vals < np.quantile(vals, 0.75)]
                cand = np.clip(good[r.integers(len(good), size=32)] + 0.1 * r.standard_normal((32, d)), 0, 1)
                kde = lambda P, C: np.exp(-0.5 * ((C[:, None] - P[None]) ** 2).sum(-1) / 0.04).mean(1) + 1e-12  # noqa: E731
                u = cand[int((kde(good, cand) / kde(bad, cand)).argmax())]
            res.append(u)
        self._last_u = res
        return [self.space.decode(u) for u in res]

    def optimize(self, objective):
        self._obs = []
        outer = self

        def wrapped(params, budget):
            v = objective(params, budget)
            for u in outer._last_u:
                if outer.space.decode(u) == params:
                    outer._obs.append((u, float(v)))
                    break
            return v
        return super().optimize(wrapped)
