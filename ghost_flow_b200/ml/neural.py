"""Small neural models with their own back-propagation, RBF networks, linear-chain CRF, calibration,
semi-supervised and multi-class meta estimators, re-sampling for imbalanced data (ghostflow-ml/src/neural_network.rs,
rbf_network.rs, crf.rs, calibration.rs, semi_supervised.rs, multiclass.rs, imbalanced.rs)."""
from __future__ import annotations

import enum

import numpy as np

from ._base import (ClassifierMixin, Estimator, RegressorMixin, encode_classes, out, pairwise_sq_dists, rng_of, sigmoid,
                    softmax, to_np)


class Activation(enum.Enum):
    ReLU = "relu"
    Tanh = "tanh"
    Sigmoid = "sigmoid"
    Identity = "identity"


class MLPSolver(enum.Enum):
    SGD = "sgd"
    Adam = "adam"


def _act(z, kind):
    if kind == "relu":
        return np.maximum(z, 0), (z > 0).astype(float)
    if kind == "tanh":
        a = np.tanh(z)
        return a, 1 - a * a
    if kind == "sigmoid":
        a = sigmoid(z)
        return a, a * (1 - a)
    return z, np.ones_like(z)


class _MLPBase(Estimator):
    _params = ("activation", "solver", "learning_rate", "max_iter", "batch_size", "alpha", "tol", "seed", "momentum")

    def __init__(self, hidden_layer_sizes=(100,)):
        self._hidden, self._activation, self._solver = list(hidden_layer_sizes), Activation.ReLU, MLPSolver.Adam
        self._learning_rate, self._max_iter, self._batch_size, self._alpha = 1e-3, 200, 32, 1e-4
        self._tol, self._seed, self._momentum = 1e-5, 0, 0.9

    def _init(self, sizes, r):
        self.coefs_ = [r.uniform(-1, 1, (a, b)) * np.sqrt(6.0 / (a + b)) for a, b in zip(sizes[:-1], sizes[1:])]
        self.intercepts_ = [np.zeros(b) for b in sizes[1:]]

    def _forward(self, X):
        kind = getattr(self._activation, "value", self._activation)
        acts, ders = [X], []
        for i, (W, b) in enumerate(zip(self.coefs_, self.intercepts_)):
            z = acts[-1] @ W + b
            if i < len(self.coefs_) - 1:
                a, d = _act(z, kind)
                ders.append(d)
            else:
                a = z
            acts.append(a)
        return acts, ders

    def _train(self, X, Y, out_fn):
        r = rng_of(self._seed)
        self._init([X.shape[1]] + self._hidden + [Y.shape[1]], r)
        params = self.coefs_ + self.intercepts_
        m, v, vel = [np.zeros_like(p) for p in params], [np.zeros_like(p) for p in params], [np.zeros_like(p) for p in params]
        t, prev = 0, np.inf
        adam = getattr(self._solver, "value", self._solver) == "adam"
        self.loss_curve_ = []
        for _ in range(self._max_iter):
            perm = r.permutation(len(X))
            tot = 0.0
            for s in range(0, len(X), self._batch_size):
                idx = perm[s:s + self._batch_size]
                acts, ders = self._forward(X[idx])
                P, loss = out_fn(acts[-1], Y[idx])
                tot += loss * len(idx)
                delta = (P - Y[idx]) / len(idx)
                gW, gb = [], []
                for i in range(len(self.coefs_) - 1, -1, -1):
                    gW.insert(0, acts[i].T @ delta + self._alpha * self.coefs_[i] / len(X))
                    gb.insert(0, delta.sum(0))
                    if i > 0:
                        delta = (delta @ self.coefs_[i].T) * ders[i - 1]
                t += 1
                for j, (p, g) in enumerate(zip(params, gW + gb)):
                    if adam:
                        m[j] = 0.9 * m[j] + 0.1 * g
                        v[j] = 0.999 * v[j] + 0.001 * g * g
                        p -= self._learning_rate * (m[j] / (1 - 0.9 ** t)) / (np.sqrt(v[j] / (1 - 0.999 ** t)) + 1e-8)
                    else:
                        vel[j] = self._momentum * vel[j] - self._learning_rate * g
                        p += vel[j]
            tot /= len(X)
            self.loss_curve_.append(tot)
            if abs(prev - tot) < self._tol:
                break
            prev = tot
        self.n_iter_ = len(self.loss_curve_)


class MLPClassifier(_MLPBase, ClassifierMixin):
    def fit(self, X, y):
        X = to_np(X)
        self.classes_, yc = encode_classes(y)
        Y = (yc[:, None] == np.arange(len(self.classes_))[None]).astype(float)

        def out_fn(Z, T):
            P = softmax(Z)
            return P, float(-(T * np.log(P + 1e-12)).sum(1).mean())
        self._train(X, Y, out_fn)
        return self

    def predict_proba(self, X):
        return out(softmax(self._forward(to_np(X))[0][-1]))

    def predict(self, X):
        return out(self.classes_[self._forward(to_np(X))[0][-1].argmax(1)])


class MLPRegressor(_MLPBase, RegressorMixin):
    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        self._1d = y.ndim == 1
        Y = y[:, None] if self._1d else y
        self._train(X, Y, lambda Z, T: (Z, float(0.5 * ((Z - T) ** 2).sum(1).mean())))
        return self

    def predict(self, X):
        Z = self._forward(to_np(X))[0][-1]
        return out(Z[:, 0] if self._1d else Z)


class RBFNetwork(Estimator, RegressorMixin):
    """Gaussian units centred by k-means, widths from the mean centre spacing, linear read-out by ridge regression."""
    _params = ("gamma", "alpha", "seed")

    def __init__(self, n_centers=10):
        self._n_centers, self._gamma, self._alpha, self._seed = n_centers, None, 1e-6, 0

    def _phi(self, X):
        return np.hstack((np.exp(-self.gamma_ * pairwise_sq_dists(X, self.centers_)), np.ones((len(X), 1))))

    def _fit_units(self, X):
        from .cluster import KMeans
        self.centers_ = to_np(KMeans(min(self._n_centers, len(X))).n_init(3).seed(self._seed).fit(X).cluster_centers_)
        d = np.sqrt(pairwise_sq_dists(self.centers_, self.centers_))
        spacing = d[d > 0].mean() if (d > 0).any() else 1.0
        self.gamma_ = self._gamma or 1.0 / (2 * spacing ** 2)

    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        self._fit_units(X)
        P = self._phi(X)
        self.weights_ = np.linalg.solve(P.T @ P + self._alpha * np.eye(P.shape[1]), P.T @ y)
        return self

    def predict(self, X):
        return out(self._phi(to_np(X)) @ self.weights_)


class RBFClassifier(RBFNetwork, ClassifierMixin):
    def fit(self, X, y):
        X = to_np(X)
        self.classes_, yc = encode_classes(y)
        Y = (yc[:, None] == np.arange(len(self.classes_))[None]).astype(float)
        self._fit_units(X)
        P = self._phi(X)
        self.weights_ = np.linalg.solve(P.T @ P + self._alpha * np.eye(P.shape[1]), P.T @ Y)
        return self

    def predict_proba(self, X):
        S = np.clip(self._phi(to_np(X)) @ self.weights_, 1e-9, None)
        return out(S / S.sum(1, keepdims=True))

    def predict(self, X):
        return out(self.classes_[(self._phi(to_np(X)) @ self.weights_).argmax(1)])

    score = ClassifierMixin.score


# ----------------------------------------------------------------------------- CRF
class LinearChainCRF(Estimator):
    """Sequences of feature vectors -> label sequences. Parameters: emission W [labels, features], transition
    T [labels, labels]; trained by gradient ascent on the exact log-likelihood (forward-backward)."""
    _params = ("l2_penalty", "learning_rate", "max_iter")

    def __init__(self, n_labels=2, n_features=1):
        self._n_labels, self._n_features, self._l2_penalty, self._learning_rate, self._max_iter = n_labels, n_features, 0.1, 0.1, 100
        self.W = np.zeros((n_labels, n_features))
        self.T = np.zeros((n_labels, n_labels))

    def _fb(self, X):
        E = X @ self.W.T
        n, k = E.shape
        a, b = np.zeros((n, k)), np.zeros((n, k))
        a[0] = E[0]
        for t in range(1, n):
            m = a[t - 1][:, None] + self.T
            mx = m.max(0)
            a[t] = E[t] + mx + np.log(np.exp(m - mx).sum(0))
        for t in range(n - 2, -1, -1):
            m = self.T + (E[t + 1] + b[t + 1])[None, :]
            mx = m.max(1)
            b[t] = mx + np.log(np.exp(m - mx[:, None]).sum(1))
        mx = a[-1].max()
        logZ = mx + np.log(np.exp(a[-1] - mx).sum())
        return E, a, b, logZ

    def fit(self, sequences, labels):
        seqs = [to_np(s) for s in sequences]
        labs = [to_np(l).astype(int) for l in labels]
        k = self._n_labels
        n_tok = sum(len(s) for s in seqs)
        for _ in range(self._max_iter):
            gW, gT = -self._l2_penalty * self.W, -self._l2_penalty * self.T
            for X, y in zip(seqs, labs):
                E, a, b, logZ = self._fb(X)
                marg = np.exp(a + b - logZ)
                gW = gW + (np.eye(k)[y] - marg).T @ X / n_tok
                for t in range(len(X) - 1):
                    pair = np.exp(a[t][:, None] + self.T + (E[t + 1] + b[t + 1])[None] - logZ)
                    gT = gT - pair / n_tok
                    gT[y[t], y[t + 1]] += 1.0 / n_tok
            self.W += self._learning_rate * gW * 10
            self.T += self._learning_rate * gT * 10
        return self

    def predict_marginals(self, X):
        E, a, b, logZ = self._fb(to_np(X))
        return out(np.exp(a + b - logZ))

    def predict(self, X):
        X = to_np(X)
        E = X @ self.W.T
        n, k = E.shape
        d, psi = np.zeros((n, k)), np.zeros((n, k), int)
        d[0] = E[0]
        for t in range(1, n):
            m = d[t - 1][:, None] + self.T
            psi[t], d[t] = m.argmax(0), m.max(0) + E[t]
        path = np.zeros(n, int)
        path[-1] = d[-1].argmax()
        for t in range(n - 2, -1, -1):
            path[t] = psi[t + 1][path[t + 1]]
        return out(path)


# ----------------------------------------------------------------------------- calibration
class IsotonicRegression(Estimator, RegressorMixin):
    _params = ("increasing",)

    def __init__(self):
        self._increasing = True

    def fit(self, X, y):
        x, y = to_np(X).ravel(), to_np(y)
        o = np.argsort(x)
        x, y = x[o], (y[o] if self._increasing else -y[o])
        vals, wts, starts = [], [], []
        for i, v in enumerate(y):                       # pool adjacent violators
            vals.append(v)
            wts.append(1.0)
            starts.append(i)
            while len(vals) > 1 and vals[-2] > vals[-1]:
                w = wts[-2] + wts[-1]
                vals[-2] = (vals[-2] * wts[-2] + vals[-1] * wts[-1]) / w
                wts[-2] = w
                vals.pop(), wts.pop(), starts.pop()
        fit = np.empty(len(y))
        for j, s in enumerate(starts):
            e = starts[j + 1] if j + 1 < len(starts) else len(y)
            fit[s:e] = vals[j]
        self.X_thresholds_, self.y_thresholds_ = x, fit if self._increasing else -fit
        return self

    def predict(self, X):
        return out(np.interp(to_np(X).ravel(), self.X_thresholds_, self.y_thresholds_))

    transform = predict


class PlattScaling(Estimator):
    """Sigmoid 1 / (1 + exp(a f + b)) fitted by Newton iterations on the regularised targets of Platt (1999)."""

    def fit(self, scores, y):
        f, y = to_np(scores).ravel(), to_np(y)
        npos, nneg = (y > 0).sum(), (y <= 0).sum()
        t = np.where(y > 0, (npos + 1) / (npos + 2), 1 / (nneg + 2))
        a, b = 0.0, np.log((nneg + 1) / (npos + 1))
        for _ in range(100):
            p = sigmoid(-(a * f + b))
            g = np.array([((p - t) * -f).sum(), -(p - t).sum()])
            w = p * (1 - p)
            H = np.array([[(w * f * f).sum(), (w * f).sum()], [(w * f).sum(), w.sum()]]) + 1e-10 * np.eye(2)
            step = np.linalg.solve(H, g)
            a, b = a - step[0], b - step[1]
            if np.abs(step).max() < 1e-10:
                break
        self.a_, self.b_ = a, b
        return self

    def predict_proba(self, scores):
        return out(sigmoid(-(self.a_ * to_np(scores).ravel() + self.b_)))

    transform = predict_proba


class CalibratedClassifier(Estimator, ClassifierMixin):
    _params = ("cv",)

    def __init__(self, base_estimator=None, method="sigmoid"):
        self._base, self._method, self._cv = base_estimator, getattr(method, "value", method), 3

    def _score(self, est, X):
        if hasattr(est, "decision_function"):
            s = to_np(est.decision_function(X))
            return s if s.ndim == 1 else s[:, -1]
        return to_np(est.predict_proba(X))[:, -1]

    def fit(self, X, y):
        from .linear import LogisticRegression
        from .model_selection import KFold
        Xn, yn = to_np(X), to_np(y)
        self.classes_ = np.unique(yn)
        base = self._base or LogisticRegression()
        s = np.zeros(len(Xn))
        for tr, te in KFold(self._cv, True, 0).split(Xn):
            s[te] = self._score(base.clone().fit(out(Xn[tr]), out(yn[tr])), out(Xn[te]))
        t = (yn == self.classes_[-1]).astype(float)
        self.calibrator_ = (IsotonicRegression().fit(s, t) if self._method == "isotonic" else PlattScaling().fit(s, t))
        self.estimator_ = base.clone().fit(X, y)
        return self

    def predict_proba(self, X):
        s = self._score(self.estimator_, X)
        p = np.clip(to_np(self.calibrator_.transform(s)), 0, 1)
        return out(np.stack((1 - p, p), 1))

    def predict(self, X):
        return out(self.classes_[(to_np(self.predict_proba(X))[:, 1] > 0.5).astype(int)])


# ----------------------------------------------------------------------------- semi-supervised (label -1 = unlabelled)
class LabelPropagation(Estimator, ClassifierMixin):
    _params = ("gamma", "max_iter", "tol", "kernel", "n_neighbors")
    _alpha = None

    def __init__(self):
        self._gamma, self._max_iter, self._tol, self._kernel, self._n_neighbors = 20.0, 1000, 1e-4, "rbf", 7

    def _graph(self, X):
        D = pairwise_sq_dists(X, X)
        if self._kernel == "knn":
            W = np.zeros_like(D)
            idx = np.argsort(D, 1)[:, :self._n_neighbors + 1]
            W[np.arange(len(X))[:, None], idx] = 1
            return np.maximum(W, W.T)
        return np.exp(-self._gamma * D)

    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        self.X_ = X
        lab = y >= 0
        self.classes_ = np.unique(y[lab])
        Y0 = (y[:, None] == self.classes_[None]).astype(float)
        W = self._graph(X)
        if self._alpha is None:
            T = W / W.sum(1, keepdims=True)
        else:
            np.fill_diagonal(W, 0)
            d = np.sqrt(W.sum(1))
            T = W / np.outer(d, d)
        F = Y0.copy()
        for _ in range(self._max_iter):
            Fn = T @ F
            if self._alpha is None:
                Fn[lab] = Y0[lab]
            else:
                Fn = self._alpha * Fn + (1 - self._alpha) * Y0
            if np.abs(Fn - F).max() < self._tol:
                F = Fn
                break
            F = Fn
        self.label_distributions_ = F / np.maximum(F.sum(1, keepdims=True), 1e-300)
        self.transduction_ = self.classes_[F.argmax(1)]
        return self

    def predict_proba(self, X):
        W = np.exp(-self._gamma * pairwise_sq_dists(to_np(X), self.X_))
        P = W @ self.label_distributions_
        return out(P / np.maximum(P.sum(1, keepdims=True), 1e-300))

    def predict(self, X):
        return out(self.classes_[to_np(self.predict_proba(X)).argmax(1)])


class LabelSpreading(LabelPropagation):
    _params = ("alpha",)
    _alpha = 0.2


class SelfTrainingClassifier(Estimator, ClassifierMixin):
    _params = ("max_iter",)

    def __init__(self, base_estimator=None, threshold=0.75):
        self._base, self._threshold, self._max_iter = base_estimator, threshold, 10

    def fit(self, X, y):
        from .linear import LogisticRegression
        Xn, yn = to_np(X), to_np(y).copy()
        base = self._base or LogisticRegression()
        for _ in range(self._max_iter):
            lab = yn >= 0
            self.estimator_ = base.clone().fit(out(Xn[lab]), out(yn[lab]))
            if lab.all():
                break
            P = to_np(self.estimator_.predict_proba(out(Xn[~lab])))
            conf = P.max(1) >= self._threshold
            if not conf.any():
                break
            idx = np.where(~lab)[0][conf]
            yn[idx] = self.estimator_.classes_[P[conf].argmax(1)]
        self.classes_, self.transduction_ = self.estimator_.classes_, yn
        return self

    def predict(self, X):
        return self.estimator_.predict(X)

    def predict_proba(self, X):
        return self.estimator_.predict_proba(X)


# ----------------------------------------------------------------------------- multi-class meta estimators
def _default_binary():
    from .linear import LogisticRegression
    return LogisticRegression()


def _margin(est, X):
    if hasattr(est, "decision_function"):
        s = to_np(est.decision_function(X))
        return s if s.ndim == 1 else s[:, -1]
    return to_np(est.predict_proba(X))[:, -1] - 0.5


class OneVsRestClassifier(Estimator, ClassifierMixin):
    def __init__(self, estimator=None):
        self._estimator = estimator

    def fit(self, X, y):
        yn = to_np(y)
        self.classes_ = np.unique(yn)
        base = self._estimator or _default_binary()
        self.estimators_ = [base.clone().fit(X, out((yn == c).astype(float))) for c in self.classes_]
        return self

    def decision_function(self, X):
        return np.stack([_margin(e, X) for e in self.estimators_], 1)

    def predict(self, X):
        return out(self.classes_[self.decision_function(X).argmax(1)])


class OneVsOneClassifier(Estimator, ClassifierMixin):
    def __init__(self, estimator=None):
        self._estimator = estimator

    def fit(self, X, y):
        Xn, yn = to_np(X), to_np(y)
        self.classes_ = np.unique(yn)
        base = self._estimator or _default_binary()
        self.pairs_ = []
        for i in range(len(self.classes_)):
            for j in range(i + 1, len(self.classes_)):
                m = (yn == self.classes_[i]) | (yn == self.classes_[j])
                self.pairs_.append((i, j, base.clone().fit(out(Xn[m]), out((yn[m] == self.classes_[j]).astype(float)))))
        return self

    def predict(self, X):
        votes = np.zeros((len(to_np(X)), len(self.classes_)))
        for i, j, e in self.pairs_:
            s = _margin(e, X)
            votes[:, j] += s > 0
            votes[:, i] += s <= 0
        return out(self.classes_[votes.argmax(1)])


class OutputCodeClassifier(Estimator, ClassifierMixin):
    _params = ("code_size", "seed")

    def __init__(self, estimator=None):
        self._estimator, self._code_size, self._seed = estimator, 1.5, 0

    def fit(self, X, y):
        yn = to_np(y)
        self.classes_, yc = encode_classes(yn)
        r = rng_of(self._seed)
        nb = max(2, int(len(self.classes_) * self._code_size))
        while True:
            code = (r.random((len(self.classes_), nb)) > 0.5).astype(float)
            if all(0 < code[:, b].sum() < len(self.classes_) for b in range(nb)) and len(np.unique(code, axis=0)) == len(code):
                break
        self.code_book_ = code
        base = self._estimator or _default_binary()
        self.estimators_ = [base.clone().fit(X, out(code[yc, b])) for b in range(nb)]
        return self

    def predict(self, X):
        S = np.stack([(_margin(e, X) > 0).astype(float) for e in self.estimators_], 1)
        return out(self.classes_[pairwise_sq_dists(S, self.code_book_).argmin(1)])


class ClassifierChain(Estimator):
    """Multi-label: label j is predicted from the features plus the predictions of labels before it in the order."""
    _params = ("order",)

    def __init__(self, estimator=None):
        self._estimator, self._order = estimator, None

    def fit(self, X, Y):
        Xn, Yn = to_np(X), to_np(Y)
        self.order_ = list(self._order) if self._order is not None else list(range(Yn.shape[1]))
        base = self._estimator or _default_binary()
        self.estimators_ = []
        aug = Xn
        for j in self.order_:
            self.estimators_.append(base.clone().fit(out(aug), out(Yn[:, j])))
            aug = np.hstack((aug, Yn[:, [j]]))
        return self

    def predict(self, X):
        aug = to_np(X)
        res = np.zeros((len(aug), len(self.order_)))
        for j, e in zip(self.order_, self.estimators_):
            p = to_np(e.predict(out(aug)))
            res[:, j] = p
            aug = np.hstack((aug, p[:, None]))
        return out(res)


# ----------------------------------------------------------------------------- imbalanced data
class _Sampler(Estimator):
    _params = ("seed", "k_neighbors")

    def _targets(self, y):
        cl, cnt = np.unique(y, return_counts=True)
        return cl, cnt, cnt.max()


class RandomOverSampler(_Sampler):
    def __init__(self):
        self._seed = 0

    def fit_resample(self, X, y):
        X, y = to_np(X), to_np(y)
        r = rng_of(self._seed)
        cl, cnt, mx = self._targets(y)
        idx = np.concatenate([np.concatenate((np.where(y == c)[0], r.choice(np.where(y == c)[0], mx - n))) for c, n in zip(cl, cnt)])
        return out(X[idx]), out(y[idx])


class RandomUnderSampler(_Sampler):
    def __init__(self):
        self._seed = 0

    def fit_resample(self, X, y):
        X, y = to_np(X), to_np(y)
        r = rng_of(self._seed)
        cl, cnt, _ = self._targets(y)
        idx = np.concatenate([r.choice(np.where(y == c)[0], cnt.min(), replace=False) for c in cl])
        return out(X[idx]), out(y[idx])


class SMOTE(_Sampler):
    def __init__(self):
        self._seed, self._k_neighbors = 0, 5

    def _seeds(self, X, y, c, Xc):
        return np.arange(len(Xc)), None

    def _synth(self, Xc, seeds, n_new, r, weights=None):
        k = min(self._k_neighbors, len(Xc) - 1)
        if k < 1 or n_new <= 0:
            return np.empty((0, Xc.shape[1]))
        nn = np.argsort(pairwise_sq_dists(Xc, Xc), 1)[:, 1:k + 1]
        base = r.choice(seeds, n_new, p=weights)
        nb = nn[base, r.integers(0, k, n_new)]
        return Xc[base] + r.random((n_new, 1)) * (Xc[nb] - Xc[base])

    def fit_resample(self, X, y):
        X, y = to_np(X), to_np(y)
        r = rng_of(self._seed)
        cl, cnt, mx = self._targets(y)
        Xs, ys = [X], [y]
        for c, n in zip(cl, cnt):
            if n == mx:
                continue
            Xc = X[y == c]
            seeds, w = self._seeds(X, y, c, Xc)
            if len(seeds) == 0:
                seeds, w = np.arange(len(Xc)), None
            S = self._synth(Xc, seeds, mx - n, r, w)
            Xs.append(S)
            ys.append(np.full(len(S), c))
        return out(np.vstack(Xs)), out(np.concatenate(ys))


class BorderlineSMOTE(SMOTE):
    """Only minority points whose neighbourhood is dominated (but not fully) by other classes seed new points."""

    def _seeds(self, X, y, c, Xc):
        k = min(self._k_neighbors, len(X) - 1)
        nn = np.argsort(pairwise_sq_dists(Xc, X), 1)[:, 1:k + 1]
        other = (y[nn] != c).sum(1)
        return np.where((other >= k / 2) & (other < k))[0], None


class ADASYN(SMOTE):
    """Seeds are drawn proportionally to the share of other-class points among their neighbours."""

    def _seeds(self, X, y, c, Xc):
        k = min(self._k_neighbors, len(X) - 1)
        nn = np.argsort(pairwise_sq_dists(Xc, X), 1)[:, 1:k + 1]
        ratio = (y[nn] != c).mean(1)
        if ratio.sum() == 0:
            return np.arange(len(Xc)), None
        return np.arange(len(Xc)), ratio / ratio.sum()
