"""Linear, SGD, robust, Bayesian and kernel models (ghostflow-ml/src/linear.rs, linear_sgd.rs, robust.rs,
bayesian.rs, svm.rs, kernel.rs, discriminant_analysis.rs, naive_bayes.rs, neighbors.rs, gaussian_process.rs)."""
from __future__ import annotations

import enum

import numpy as np

from ._base import (ClassifierMixin, Estimator, RegressorMixin, TransformerMixin, encode_classes, out,
                    pairwise_sq_dists, rng_of, sigmoid, softmax, to_np)


class LinearSolver(enum.Enum):
    Normal = "normal"
    SVD = "svd"
    GradientDescent = "gd"


class Penalty(enum.Enum):
    Null = "none"
    L1 = "l1"
    L2 = "l2"
    ElasticNet = "elasticnet"


class MultiClass(enum.Enum):
    OvR = "ovr"
    Multinomial = "multinomial"


def _center(X, y, fit_intercept):
    if fit_intercept:
        xm, ym = X.mean(0), y.mean(0)
        return X - xm, y - ym, xm, ym
    return X, y, np.zeros(X.shape[1]), 0.0 * y.mean(0)


class _LinearRegBase(Estimator, RegressorMixin):
    _params = ("fit_intercept", "solver", "max_iter", "tol", "learning_rate")

    def predict(self, X):
        return out(to_np(X) @ self.coef_ + self.intercept_)

    def _finish(self, w, xm, ym):
        self.coef_ = w
        self.intercept_ = ym - xm @ w


class LinearRegression(_LinearRegBase):
    def __init__(self):
        self._fit_intercept, self._solver, self._max_iter, self._tol, self._learning_rate = True, LinearSolver.SVD, 1000, 1e-8, 0.01

    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        Xc, yc, xm, ym = _center(X, y, self._fit_intercept)
        s = getattr(self._solver, "value", self._solver)
        if s == "normal":
            w = np.linalg.solve(Xc.T @ Xc + 1e-10 * np.eye(X.shape[1]), Xc.T @ yc)
        elif s == "gd":
            w = np.zeros(X.shape[1:] + y.shape[1:])
            lr = 1.0 / max(np.linalg.norm(Xc, 2) ** 2, 1e-12)
            for _ in range(self._max_iter * 10):
                g = Xc.T @ (Xc @ w - yc)
                w -= lr * g
                if np.abs(g).max() < self._tol:
                    break
        else:
            w = np.linalg.lstsq(Xc, yc, rcond=None)[0]
        self._finish(w, xm, ym)
        return self


class Ridge(_LinearRegBase):
    def __init__(self, alpha=1.0):
        self._alpha, self._fit_intercept = alpha, True

    def alpha(self, a):
        self._alpha = a
        return self

    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        Xc, yc, xm, ym = _center(X, y, self._fit_intercept)
        self._finish(np.linalg.solve(Xc.T @ Xc + self._alpha * np.eye(X.shape[1]), Xc.T @ yc), xm, ym)
        return self


def _coordinate_descent(X, y, alpha, l1_ratio, max_iter, tol):
    n, d = X.shape
    w = np.zeros(d)
    col_sq = (X ** 2).sum(0)
    r = y.copy()
    l1, l2 = alpha * l1_ratio * n, alpha * (1 - l1_ratio) * n
    for _ in range(max_iter):
        mx = 0.0
        for j in range(d):
            if col_sq[j] == 0:
                continue
            rho = X[:, j] @ r + col_sq[j] * w[j]
            nw = np.sign(rho) * max(abs(rho) - l1, 0.0) / (col_sq[j] + l2)
            if nw != w[j]:
                r -= X[:, j] * (nw - w[j])
                mx = max(mx, abs(nw - w[j]))
                w[j] = nw
        if mx < tol:
            break
    return w


class ElasticNet(_LinearRegBase):
    """min 1/(2n) |y - Xw|^2 + alpha * l1_ratio * |w|_1 + alpha * (1 - l1_ratio) / 2 * |w|^2 by coordinate descent."""

    def __init__(self, alpha=1.0, l1_ratio=0.5):
        self._alpha, self._l1_ratio, self._fit_intercept, self._max_iter, self._tol = alpha, l1_ratio, True, 1000, 1e-6

    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        Xc, yc, xm, ym = _center(X, y, self._fit_intercept)
        self._finish(_coordinate_descent(Xc, yc, self._alpha, self._l1_ratio, self._max_iter, self._tol), xm, ym)
        return self


class Lasso(ElasticNet):
    def __init__(self, alpha=1.0):
        super().__init__(alpha, 1.0)


class LogisticRegression(Estimator, ClassifierMixin):
    """L-BFGS-free: full-batch gradient descent with backtracking would be slow, so Newton/IRLS for two classes and
    gradient descent with momentum on the softmax loss for multinomial; L1/L2 penalty with strength 1/C."""
    _params = ("c", "penalty", "multi_class", "max_iter", "learning_rate", "fit_intercept", "tol")

    def __init__(self):
        self._c, self._penalty, self._multi_class = 1.0, Penalty.L2, MultiClass.Multinomial
        self._max_iter, self._learning_rate, self._fit_intercept, self._tol = 300, 0.5, True, 1e-6

    def fit(self, X, y):
        X = to_np(X)
        self.classes_, yc = encode_classes(y)
        n, d = X.shape
        k = len(self.classes_)
        Xb = np.hstack((X, np.ones((n, 1)))) if self._fit_intercept else X
        pen = getattr(self._penalty, "value", self._penalty)
        lam = 0.0 if pen == "none" else 1.0 / (self._c * n)
        W = np.zeros((Xb.shape[1], k if k > 2 else 1))
        Y = (yc[:, None] == np.arange(k)[None, :]).astype(float) if k > 2 else yc[:, None].astype(float)
        vel = np.zeros_like(W)
        L = 0.25 * np.linalg.norm(Xb, 2) ** 2 / n + lam
        lr = 1.0 / L
        for _ in range(self._max_iter * 4):
            Z = Xb @ W
            P = softmax(Z) if k > 2 else sigmoid(Z)
            G = Xb.T @ (P - Y) / n
            reg = W.copy()
            if self._fit_intercept:
                reg[-1] = 0
            if pen in ("l2", "elasticnet"):
                G += lam * reg
            vel = 0.9 * vel - lr * G
            W = W + vel
            if pen in ("l1", "elasticnet"):
                body = W[:-1] if self._fit_intercept else W
                body[...] = np.sign(body) * np.maximum(np.abs(body) - lr * lam, 0)
            if np.abs(G).max() < self._tol:
                break
        self.coef_ = (W[:-1] if self._fit_intercept else W).T
        self.intercept_ = W[-1] if self._fit_intercept else np.zeros(W.shape[1])
        return self

    def decision_function(self, X):
        return to_np(X) @ self.coef_.T + self.intercept_

    def predict_proba(self, X):
        Z = self.decision_function(X)
        if Z.shape[1] == 1:
            p = sigmoid(Z[:, 0])
            return out(np.stack((1 - p, p), 1))
        return out(softmax(Z))

    def predict(self, X):
        return out(self.classes_[to_np(self.predict_proba(X)).argmax(1)])


# ----------------------------------------------------------------------------- SGD family
class SGDLoss(enum.Enum):
    Hinge = "hinge"
    Log = "log"
    SquaredError = "squared_error"
    Huber = "huber"
    ModifiedHuber = "modified_huber"
    Perceptron = "perceptron"
    EpsilonInsensitive = "epsilon_insensitive"


class LearningRate(enum.Enum):
    Constant = "constant"
    Optimal = "optimal"
    InvScaling = "invscaling"
    Adaptive = "adaptive"


def _sgd(X, y, loss, penalty, alpha, l1_ratio, eta0, schedule, epochs, seed, epsilon=0.1, fit_intercept=True):
    r = rng_of(seed)
    n, d = X.shape
    w, b, t = np.zeros(d), 0.0, 1
    for _ in range(epochs):
        for i in r.permutation(n):
            eta = {"constant": eta0, "optimal": 1.0 / (alpha * (t + 1.0 / (alpha * eta0 + 1e-12))),
                   "invscaling": eta0 / t ** 0.25, "adaptive": eta0}[schedule]
            z = X[i] @ w + b
            if loss == "hinge":
                g = -y[i] if y[i] * z < 1 else 0.0
            elif loss == "perceptron":
                g = -y[i] if y[i] * z <= 0 else 0.0
            elif loss == "log":
                g = -y[i] * sigmoid(-y[i] * z)
            elif loss == "modified_huber":
                m = y[i] * z
                g = 0.0 if m >= 1 else (-2 * y[i] * (1 - m) if m >= -1 else -4 * y[i])
            elif loss == "huber":
                e = z - y[i]
                g = e if abs(e) <= epsilon else epsilon * np.sign(e)
            elif loss == "epsilon_insensitive":
                e = z - y[i]
                g = np.sign(e) if abs(e) > epsilon else 0.0
            else:
                g = z - y[i]
            if penalty in ("l2", "elasticnet"):
                w *= 1 - eta * alpha * (1 - l1_ratio if penalty == "elasticnet" else 1.0)
            w -= eta * g * X[i]
            if penalty in ("l1", "elasticnet"):
                th = eta * alpha * (l1_ratio if penalty == "elasticnet" else 1.0)
                w = np.sign(w) * np.maximum(np.abs(w) - th, 0)
            if fit_intercept:
                b -= eta * g
            t += 1
    return w, b


class _SGDBase(Estimator):
    _params = ("alpha", "loss", "penalty", "l1_ratio", "eta0", "learning_rate", "max_iter", "seed", "epsilon")

    def _common(self):
        return dict(loss=getattr(self._loss, "value", self._loss), penalty=getattr(self._penalty, "value", self._penalty),
                    alpha=self._alpha, l1_ratio=self._l1_ratio, eta0=self._eta0,
                    schedule=getattr(self._learning_rate, "value", self._learning_rate), epochs=self._max_iter,
                    seed=self._seed, epsilon=self._epsilon)


class SGDClassifier(_SGDBase, ClassifierMixin):
    def __init__(self):
        self._alpha, self._loss, self._penalty, self._l1_ratio = 1e-4, SGDLoss.Hinge, Penalty.L2, 0.15
        self._eta0, self._learning_rate, self._max_iter, self._seed, self._epsilon = 0.01, LearningRate.InvScaling, 30, 0, 0.1

    def fit(self, X, y):
        X = to_np(X)
        self.classes_, yc = encode_classes(y)
        ks = [1] if len(self.classes_) == 2 else range(len(self.classes_))
        W, B = [], []
        for c in ks:
            w, b = _sgd(X, np.where(yc == c, 1.0, -1.0), **self._common())
            W.append(w)
            B.append(b)
        self.coef_, self.intercept_ = np.stack(W), np.array(B)
        return self

    def decision_function(self, X):
        Z = to_np(X) @ self.coef_.T + self.intercept_
        return Z[:, 0] if Z.shape[1] == 1 else Z

    def predict(self, X):
        Z = self.decision_function(X)
        idx = (Z > 0).astype(int) if Z.ndim == 1 else Z.argmax(1)
        return out(self.classes_[idx])


class SGDRegressor(_SGDBase, RegressorMixin):
    def __init__(self):
        self._alpha, self._loss, self._penalty, self._l1_ratio = 1e-4, SGDLoss.SquaredError, Penalty.L2, 0.15
        self._eta0, self._learning_rate, self._max_iter, self._seed, self._epsilon = 0.01, LearningRate.InvScaling, 50, 0, 0.1

    def fit(self, X, y):
        self.coef_, self.intercept_ = _sgd(to_np(X), to_np(y), **self._common())
        return self

    def predict(self, X):
        return out(to_np(X) @ self.coef_ + self.intercept_)


class RidgeClassifier(Estimator, ClassifierMixin):
    _params = ("alpha",)

    def __init__(self):
        self._alpha = 1.0

    def fit(self, X, y):
        X = to_np(X)
        self.classes_, yc = encode_classes(y)
        Y = np.where(yc[:, None] == np.arange(len(self.classes_))[None, :], 1.0, -1.0)
        self._ridge = Ridge(self._alpha).fit(X, Y)
        return self

    def decision_function(self, X):
        return to_np(self._ridge.predict(X))

    def predict(self, X):
        return out(self.classes_[self.decision_function(X).argmax(1)])


class Perceptron(SGDClassifier):
    def __init__(self):
        super().__init__()
        self._loss, self._penalty, self._learning_rate, self._eta0 = SGDLoss.Perceptron, Penalty.Null, LearningRate.Constant, 1.0


class PassiveAggressiveRegressor(Estimator, RegressorMixin):
    _params = ("c", "epsilon", "max_iter", "seed")

    def __init__(self):
        self._c, self._epsilon, self._max_iter, self._seed = 1.0, 0.1, 50, 0

    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        w, b, r = np.zeros(X.shape[1]), 0.0, rng_of(self._seed)
        for _ in range(self._max_iter):
            for i in r.permutation(len(X)):
                e = y[i] - (X[i] @ w + b)
                l = max(0.0, abs(e) - self._epsilon)
                tau = min(self._c, l / (X[i] @ X[i] + 1.0))
                w += tau * np.sign(e) * X[i]
                b += tau * np.sign(e)
        self.coef_, self.intercept_ = w, b
        return self

    def predict(self, X):
        return out(to_np(X) @ self.coef_ + self.intercept_)


# ----------------------------------------------------------------------------- robust
class HuberRegressor(Estimator, RegressorMixin):
    """Iteratively re-weighted least squares on the Huber loss with a robust (MAD) scale."""
    _params = ("epsilon", "alpha", "max_iter")

    def __init__(self):
        self._epsilon, self._alpha, self._max_iter = 1.35, 1e-4, 100

    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        Xb = np.hstack((X, np.ones((len(X), 1))))
        w = np.linalg.lstsq(Xb, y, rcond=None)[0]
        R = self._alpha * np.eye(Xb.shape[1])
        R[-1, -1] = 0
        for _ in range(self._max_iter):
            r = y - Xb @ w
            s = max(np.median(np.abs(r - np.median(r))) / 0.6745, 1e-12)
            wt = np.where(np.abs(r / s) <= self._epsilon, 1.0, self._epsilon / np.maximum(np.abs(r / s), 1e-300))
            nw = np.linalg.solve(Xb.T @ (Xb * wt[:, None]) + R, Xb.T @ (wt * y))
            if np.abs(nw - w).max() < 1e-10:
                w = nw
                break
            w = nw
        self.coef_, self.intercept_, self.scale_ = w[:-1], w[-1], s
        self.outliers_ = np.abs((y - Xb @ w) / s) > self._epsilon
        return self

    def predict(self, X):
        return out(to_np(X) @ self.coef_ + self.intercept_)


class RANSACRegressor(Estimator, RegressorMixin):
    _params = ("max_trials", "min_samples", "residual_threshold", "seed")

    def __init__(self):
        self._max_trials, self._min_samples, self._residual_threshold, self._seed = 100, None, None, 0

    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        n, d = X.shape
        ms = self._min_samples or d + 1
        th = self._residual_threshold or np.median(np.abs(y - np.median(y)))
        r = rng_of(self._seed)
        best = None
        for _ in range(self._max_trials):
            idx = r.choice(n, ms, replace=False)
            m = LinearRegression().fit(X[idx], y[idx])
            inl = np.abs(y - to_np(m.predict(X))) <= th
            if best is None or inl.sum() > best.sum():
                best = inl
        self.inlier_mask_ = best
        self.estimator_ = LinearRegression().fit(X[best], y[best])
        self.coef_, self.intercept_ = self.estimator_.coef_, self.estimator_.intercept_
        return self

    def inlier_mask(self):
        return self.inlier_mask_

    def predict(self, X):
        return self.estimator_.predict(X)


class TheilSenRegressor(Estimator, RegressorMixin):
    """Spatial median of least-squares fits on random subsets of d + 1 points."""
    _params = ("n_subsamples", "max_subpopulation", "seed")

    def __init__(self):
        self._n_subsamples, self._max_subpopulation, self._seed = None, 500, 0

    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        n, d = X.shape
        ns = self._n_subsamples or d + 1
        r = rng_of(self._seed)
        Xb = np.hstack((X, np.ones((n, 1))))
        W = []
        for _ in range(self._max_subpopulation):
            idx = r.choice(n, ns, replace=False)
            W.append(np.linalg.lstsq(Xb[idx], y[idx], rcond=None)[0])
        W = np.array(W)
        m = np.median(W, 0)
        for _ in range(100):                            # Weiszfeld iterations towards the spatial median
            dist = np.maximum(np.linalg.norm(W - m, axis=1), 1e-12)
            nm = (W / dist[:, None]).sum(0) / (1 / dist).sum()
            if np.linalg.norm(nm - m) < 1e-10:
                break
            m = nm
        self.coef_, self.intercept_ = m[:-1], m[-1]
        return self

    def predict(self, X):
        return out(to_np(X) @ self.coef_ + self.intercept_)


class QuantileRegressor(Estimator, RegressorMixin):
    """Pinball loss minimised as a linear program (scipy ``linprog``, HiGHS)."""
    _params = ("alpha",)

    def __init__(self, quantile=0.5):
        self._quantile, self._alpha = quantile, 0.0

    def fit(self, X, y):
        from scipy.optimize import linprog
        X, y = to_np(X), to_np(y)
        n, d = X.shape
        Xb = np.hstack((X, np.ones((n, 1))))
        q = self._quantile
        # variables: w+ (d+1), w- (d+1), u (n), v (n); Xb (w+ - w-) + u - v = y
        c = np.concatenate((np.full(d, self._alpha), [0], np.full(d, self._alpha), [0], np.full(n, q / n), np.full(n, (1 - q) / n)))
        A = np.hstack((Xb, -Xb, np.eye(n), -np.eye(n)))
        res = linprog(c, A_eq=A, b_eq=y, bounds=(0, None), method="highs")
        w = res.x[:d + 1] - res.x[d + 1:2 * d + 2]
        self.coef_, self.intercept_ = w[:-1], w[-1]
        return self

    def predict(self, X):
        return out(to_np(X) @ self.coef_ + self.intercept_)


# ----------------------------------------------------------------------------- Bayesian linear
class BayesianRidge(Estimator, RegressorMixin):
    _params = ("max_iter", "tol")

    def __init__(self):
        self._max_iter, self._tol = 300, 1e-6

    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        Xc, yc, xm, ym = _center(X, y, True)
        n, d = X.shape
        U, s, Vt = np.linalg.svd(Xc, full_matrices=False)
        eig = s ** 2
        alpha, lam = 1.0 / max(yc.var(), 1e-12), 1.0
        w = np.zeros(d)
        for _ in range(self._max_iter):
            w_new = Vt.T @ ((s / (eig + lam / alpha)) * (U.T @ yc))
            gamma = (alpha * eig / (lam + alpha * eig)).sum()
            lam = (gamma + 2e-6) / (w_new @ w_new + 2e-6)
            alpha = (n - gamma + 2e-6) / (((yc - Xc @ w_new) ** 2).sum() + 2e-6)
            if np.abs(w - w_new).sum() < self._tol:
                w = w_new
                break
            w = w_new
        self.alpha_, self.lambda_ = alpha, lam
        self.sigma_ = np.linalg.inv(alpha * Xc.T @ Xc + lam * np.eye(d))
        self.coef_, self.intercept_, self._xm = w, ym - xm @ w, xm
        return self

    def predict(self, X):
        return out(to_np(X) @ self.coef_ + self.intercept_)

    def predict_with_std(self, X):
        Xc = to_np(X) - self._xm
        var = 1.0 / self.alpha_ + ((Xc @ self.sigma_) * Xc).sum(1)
        return self.predict(X), out(np.sqrt(var))


class ARDRegression(BayesianRidge):
    """One precision per weight; weights whose precision exceeds ``threshold_lambda`` are pruned."""
    _params = ("threshold_lambda",)

    def __init__(self):
        super().__init__()
        self._threshold_lambda = 1e4

    def fit(self, X, y):
        X, y = to_np(X), to_np(y)
        Xc, yc, xm, ym = _center(X, y, True)
        n, d = X.shape
        alpha, lam = 1.0 / max(yc.var(), 1e-12), np.ones(d)
        keep = np.ones(d, bool)
        w = np.zeros(d)
        for _ in range(self._max_iter):
            Xk = Xc[:, keep]
            S = np.linalg.inv(alpha * Xk.T @ Xk + np.diag(lam[keep]))
            wk = alpha * S @ Xk.T @ yc
            gamma = 1 - lam[keep] * np.diag(S)
            lam[keep] = (gamma + 2e-6) / (wk ** 2 + 2e-6)
            alpha = (n - gamma.sum() + 2e-6) / (((yc - Xk @ wk) ** 2).sum() + 2e-6)
            w_new = np.zeros(d)
            w_new[keep] = wk
            keep = lam < self._threshold_lambda
            done = np.abs(w - w_new).sum() < self._tol
            w = w_new * keep
            if done or not keep.any():
                break
        self.alpha_, self.lambda_ = alpha, lam
        S = np.zeros((d, d))
        if keep.any():
            Xk = Xc[:, keep]
            S[np.ix_(keep, keep)] = np.linalg.inv(alpha * Xk.T @ Xk + np.diag(lam[keep]))
        self.sigma_ = S
        self.coef_, self.intercept_, self._xm = w, ym - xm @ w, xm
        return self


# ----------------------------------------------------------------------------- kernels, SVM
class Kernel:
    """``Kernel.rbf(gamma)``, ``Kernel.polynomial(degree, gamma, coef0)``, ``Kernel.linear()``, ``Kernel.sigmoid(...)``."""

    def __init__(self, kind="rbf", gamma=None, degree=3, coef0=1.0):
        self.kind, self.gamma, self.degree, self.coef0 = kind, gamma, degree, coef0

    @classmethod
    def rbf(cls, gamma=None): return cls("rbf", gamma)
    @classmethod
    def linear(cls): return cls("linear")
    @classmethod
    def polynomial(cls, degree=3, gamma=None, coef0=1.0): return cls("poly", gamma, degree, coef0)
    @classmethod
    def sigmoid(cls, gamma=None, coef0=0.0): return cls("sigmoid", gamma, coef0=coef0)

    def compute(self, A, B=None):
        A = to_np(A)
        B = A if B is None else to_np(B)
        g = self.gamma if self.gamma is not None else 1.0 / A.shape[1]
        if self.kind == "linear":
            return A @ B.T
        if self.kind == "poly":
            return (g * A @ B.T + self.coef0) ** self.degree
        if self.kind == "sigmoid":
            return np.tanh(g * A @ B.T + self.coef0)
        return np.exp(-g * pairwise_sq_dists(A, B))


def _smo(K, y, C, tol=1e-3, max_passes=5, seed=0, max_iter=2000):
    n = len(y)
    a, b, r = np.zeros(n), 0.0, rng_of(seed)
    passes = it = 0
    while passes < max_passes and it < max_iter:
        changed = 0
        it += 1
        for i in range(n):
            Ei = (a * y) @ K[:, i] + b - y[i]
            if (y[i] * Ei < -tol and a[i] < C) or (y[i] * Ei > tol and a[i] > 0):
                j = int(r.integers(n - 1))
                j += j >= i
                Ej = (a * y) @ K[:, j] + b - y[j]
                ai, aj = a[i], a[j]
                L, H = (max(0, aj - ai), min(C, C + aj - ai)) if y[i] != y[j] else (max(0, ai + aj - C), min(C, ai + aj))
                eta = 2 * K[i, j] - K[i, i] - K[j, j]
                if L == H or eta >= 0:
                    continue
                a[j] = np.clip(aj - y[j] * (Ei - Ej) / eta, L, H)
                if abs(a[j] - aj) < 1e-7:
                    continue
                a[i] = ai + y[i] * y[j] * (aj - a[j])
                b1 = b - Ei - y[i] * (a[i] - ai) * K[i, i] - y[j] * (a[j] - aj) * K[i, j]
                b2 = b - Ej - y[i] * (a[i] - ai) * K[i, j] - y[j] * (a[j] - aj) * K[j, j]
                b = b1 if 0 < a[i] < C else b2 if 0 < a[j] < C else (b1 + b2) / 2
                changed += 1
        passes = passes + 1 if changed == 0 else 0
    return a, b


class SVC(Estimator, ClassifierMixin):
    """Soft-margin SVM trained with SMO; one-vs-rest for more than two classes."""
    _params = ("c", "gamma", "kernel", "tol", "seed")

    def __init__(self):
        self._c, self._gamma, self._kernel, self._tol, self._seed = 1.0, None, Kernel.rbf(), 1e-3, 0

    def _k(self):
        k = self._kernel if isinstance(self._kernel, Kernel) else Kernel(str(self._kernel))
        if self._gamma is not None:
            k.gamma = self._gamma
        return k

    def fit(self, X, y):
        self.X_ = to_np(X)
        self.classes_, yc = encode_classes(y)
        K = self._k().compute(self.X_)
        ks = [1] if len(self.classes_) == 2 else range(len(self.classes_))
        self.models_ = []
        for c in ks:
            t = np.where(yc == c, 1.0, -1.0)
            a, b = _smo(K, t, self._c, self._tol, seed=self._seed)
            self.models_.append((a * t, b))
        self.support_ = np.where(np.any([np.abs(m[0]) > 1e-8 for m in self.models_], 0))[0]
        return self

    def decision_function(self, X):
        K = self._k().compute(to_np(X), self.X_)
        Z = np.stack([K @ ay + b for ay, b in self.models_], 1)
        return Z[:, 0] if Z.shape[1] == 1 else Z

    def predict(self, X):
        Z = self.decision_function(X)
        return out(self.classes_[(Z > 0).astype(int) if Z.ndim == 1 else Z.argmax(1)])


class SVR(Estimator, RegressorMixin):
    """Epsilon-insensitive kernel regression solved in the dual by projected gradient on beta = alpha - alpha*."""
    _params = ("c", "gamma", "kernel", "epsilon", "max_iter")

    def __init__(self):
        self._c, self._gamma, self._kernel, self._epsilon, self._max_iter = 1.0, None, Kernel.rbf(), 0.1, 2000

    _k = SVC._k

    def fit(self, X, y):
        self.X_, y = to_np(X), to_np(y)
        K = self._k().compute(self.X_) + 1e-8 * np.eye(len(y))
        Kb = K + 1.0                                  # bias absorbed as a constant feature
        beta = np.zeros(len(y))
        lr = 1.0 / np.linalg.norm(Kb, 2)
        for _ in range(self._max_iter):
            g = Kb @ beta - y + self._epsilon * np.sign(beta)
            nb = np.clip(beta - lr * g, -self._c, self._c)
            # soft-threshold around zero for the epsilon term
            z = beta - lr * (Kb @ beta - y)
            nb = np.clip(np.sign(z) * np.maximum(np.abs(z) - lr * self._epsilon, 0), -self._c, self._c)
            if np.abs(nb - beta).max() < 1e-8:
                beta = nb
                break
            beta = nb
        self.dual_coef_, self.intercept_ = beta, beta.sum()
        return self

    def predict(self, X):
        return out(self._k().compute(to_np(X), self.X_) @ self.dual_coef_ + self.intercept_)


class KernelRidge(Estimator, RegressorMixin):
    _params = ("alpha", "kernel")

    def __init__(self):
        self._alpha, self._kernel = 1.0, Kernel.rbf()

    def fit(self, X, y):
        self.X_ = to_np(X)
        K = self._kernel.compute(self.X_)
        self.dual_coef_ = np.linalg.solve(K + self._alpha * np.eye(len(K)), to_np(y))
        return self

    def predict(self, X):
        return out(self._kernel.compute(to_np(X), self.X_) @ self.dual_coef_)


class KernelPCA(Estimator, TransformerMixin):
    _params = ("kernel",)

    def __init__(self, n_components=2):
        self._n_components, self._kernel = n_components, Kernel.rbf()

    def fit(self, X, y=None):
        self.X_ = to_np(X)
        K = self._kernel.compute(self.X_)
        n = len(K)
        self._col_mean, self._all_mean = K.mean(0), K.mean()
        Kc = K - K.mean(0) - K.mean(1)[:, None] + K.mean()
        vals, vecs = np.linalg.eigh(Kc)
        idx = np.argsort(vals)[::-1][:self._n_components]
        self.lambdas_, self.alphas_ = np.maximum(vals[idx], 1e-12), vecs[:, idx]
        return self

    def transform(self, X):
        K = self._kernel.compute(to_np(X), self.X_)
        Kc = K - self._col_mean - K.mean(1)[:, None] + self._all_mean
        return out(Kc @ self.alphas_ / np.sqrt(self.lambdas_))


class Nystrom(Estimator, TransformerMixin):
    _params = ("kernel", "seed")

    def __init__(self, n_components=100):
        self._n_components, self._kernel, self._seed = n_components, Kernel.rbf(), 0

    def fit(self, X, y=None):
        X = to_np(X)
        idx = rng_of(self._seed).permutation(len(X))[:min(self._n_components, len(X))]
        self.components_ = X[idx]
        K = self._kernel.compute(self.components_)
        U, s, _ = np.linalg.svd(K)
        self.normalization_ = U / np.sqrt(np.maximum(s, 1e-12))
        return self

    def transform(self, X):
        return out(self._kernel.compute(to_np(X), self.components_) @ self.normalization_)


# ----------------------------------------------------------------------------- neighbours, naive Bayes, LDA/QDA, GP
class Weights(enum.Enum):
    Uniform = "uniform"
    Distance = "distance"


class Metric(enum.Enum):
    Euclidean = "euclidean"
    Manhattan = "manhattan"
    Chebyshev = "chebyshev"
    Cosine = "cosine"


def _dists(A, B, metric):
    m = getattr(metric, "value", metric)
    if m == "manhattan":
        return np.abs(A[:, None] - B[None]).sum(-1)
    if m == "chebyshev":
        return np.abs(A[:, None] - B[None]).max(-1)
    if m == "cosine":
        An = A / np.maximum(np.linalg.norm(A, axis=1, keepdims=True), 1e-12)
        Bn = B / np.maximum(np.linalg.norm(B, axis=1, keepdims=True), 1e-12)
        return 1 - An @ Bn.T
    return np.sqrt(pairwise_sq_dists(A, B))


class _KNNBase(Estimator):
    _params = ("weights", "metric")

    def __init__(self, n_neighbors=5):
        self._n_neighbors, self._weights, self._metric = n_neighbors, Weights.Uniform, Metric.Euclidean

    def _neigh(self, X):
        D = _dists(to_np(X), self.X_, self._metric)
        k = min(self._n_neighbors, len(self.X_))
        idx = np.argpartition(D, k - 1, axis=1)[:, :k]
        d = np.take_along_axis(D, idx, 1)
        w = np.ones_like(d) if getattr(self._weights, "value", self._weights) == "uniform" else 1.0 / np.maximum(d, 1e-12)
        return idx, w


class KNeighborsClassifier(_KNNBase, ClassifierMixin):
    def fit(self, X, y):
        self.X_ = to_np(X)
        self.classes_, self.y_ = encode_classes(y)
        return self

    def predict_proba(self, X):
        idx, w = self._neigh(X)
        P = np.zeros((len(idx), len(self.classes_)))
        for c in range(len(self.classes_)):
            P[:, c] = (w * (self.y_[idx] == c)).sum(1)
        return out(P / P.sum(1, keepdims=True))

    def predict(self, X):
        return out(self.classes_[to_np(self.predict_proba(X)).argmax(1)])


class KNeighborsRegressor(_KNNBase, RegressorMixin):
    def fit(self, X, y):
        self.X_, self.y_ = to_np(X), to_np(y)
        return self

    def predict(self, X):
        idx, w = self._neigh(X)
        return out((w * self.y_[idx]).sum(1) / w.sum(1))


class GaussianNB(Estimator, ClassifierMixin):
    _params = ("var_smoothing",)

    def __init__(self):
        self._var_smoothing = 1e-9

    def fit(self, X, y):
        X = to_np(X)
        self.classes_, yc = encode_classes(y)
        self.theta_ = np.stack([X[yc == c].mean(0) for c in range(len(self.classes_))])
        self.var_ = np.stack([X[yc == c].var(0) for c in range(len(self.classes_))]) + self._var_smoothing * X.var(0).max()
        self.class_prior_ = np.bincount(yc) / len(yc)
        return self

    def _jll(self, X):
        X = to_np(X)
        return (np.log(self.class_prior_)[None] - 0.5 * (np.log(2 * np.pi * self.var_)[None]
                + (X[:, None] - self.theta_[None]) ** 2 / self.var_[None]).sum(-1))

    def predict_proba(self, X):
        return out(softmax(self._jll(X)))

    def predict(self, X):
        return out(self.classes_[self._jll(X).argmax(1)])


class MultinomialNB(Estimator, ClassifierMixin):
    _params = ("alpha",)

    def __init__(self):
        self._alpha = 1.0

    def _counts(self, X, yc):
        return np.stack([X[yc == c].sum(0) for c in range(len(self.classes_))])

    def fit(self, X, y):
        X = to_np(X)
        self.classes_, yc = encode_classes(y)
        fc = self._counts(X, yc) + self._alpha
        self.feature_log_prob_ = np.log(fc / fc.sum(1, keepdims=True))
        self.class_log_prior_ = np.log(np.bincount(yc) / len(yc))
        return self

    def _jll(self, X):
        return to_np(X) @ self.feature_log_prob_.T + self.class_log_prior_

    predict_proba = GaussianNB.predict_proba
    predict = GaussianNB.predict


class ComplementNB(MultinomialNB):
    def fit(self, X, y):
        X = to_np(X)
        self.classes_, yc = encode_classes(y)
        fc = self._counts(X, yc)
        comp = fc.sum(0, keepdims=True) - fc + self._alpha
        w = -np.log(comp / comp.sum(1, keepdims=True))
        self.feature_log_prob_ = w / np.abs(w).sum(1, keepdims=True)
        self.class_log_prior_ = np.zeros(len(self.classes_))
        return self


class BernoulliNB(MultinomialNB):
    _params = ("binarize",)

    def __init__(self):
        super().__init__()
        self._binarize = 0.0

    def _b(self, X):
        X = to_np(X)
        return (X > self._binarize).astype(float) if self._binarize is not None else X

    def fit(self, X, y):
        X = self._b(X)
        self.classes_, yc = encode_classes(y)
        n_c = np.bincount(yc)[:, None]
        p = (self._counts(X, yc) + self._alpha) / (n_c + 2 * self._alpha)
        self.feature_log_prob_, self._neg = np.log(p), np.log(1 - p)
        self.class_log_prior_ = np.log(n_c[:, 0] / len(yc))
        return self

    def _jll(self, X):
        X = self._b(X)
        return X @ (self.feature_log_prob_ - self._neg).T + self._neg.sum(1) + self.class_log_prior_


class LDASolver(enum.Enum):
    SVD = "svd"
    Eigen = "eigen"
    LSQR = "lsqr"


class LinearDiscriminantAnalysis(Estimator, ClassifierMixin, TransformerMixin):
    _params = ("solver", "shrinkage", "n_components")

    def __init__(self):
        self._solver, self._shrinkage, self._n_components = LDASolver.Eigen, None, None

    def fit(self, X, y):
        X = to_np(X)
        self.classes_, yc = encode_classes(y)
        k, d = len(self.classes_), X.shape[1]
        self.priors_ = np.bincount(yc) / len(yc)
        self.means_ = np.stack([X[yc == c].mean(0) for c in range(k)])
        Sw = sum((X[yc == c] - self.means_[c]).T @ (X[yc == c] - self.means_[c]) for c in range(k)) / len(X)
        if self._shrinkage is not None:
            Sw = (1 - self._shrinkage) * Sw + self._shrinkage * np.trace(Sw) / d * np.eye(d)
        Sw += 1e-9 * np.eye(d)
        self.covariance_ = Sw
        Si = np.linalg.inv(Sw)
        self.coef_ = self.means_ @ Si
        self.intercept_ = -0.5 * (self.coef_ * self.means_).sum(1) + np.log(self.priors_)
        mean = self.priors_ @ self.means_
        Sb = ((self.means_ - mean).T * self.priors_) @ (self.means_ - mean)
        vals, vecs = np.linalg.eig(Si @ Sb)
        order = np.argsort(-vals.real)[:self._n_components or min(k - 1, d)]
        self.scalings_ = vecs[:, order].real
        self.explained_variance_ratio_ = vals.real[order] / max(vals.real.sum(), 1e-300)
        return self

    def decision_function(self, X):
        return to_np(X) @ self.coef_.T + self.intercept_

    def predict_proba(self, X):
        return out(softmax(self.decision_function(X)))

    def predict(self, X):
        return out(self.classes_[self.decision_function(X).argmax(1)])

    def transform(self, X):
        return out(to_np(X) @ self.scalings_)


class QuadraticDiscriminantAnalysis(Estimator, ClassifierMixin):
    _params = ("reg_param",)

    def __init__(self):
        self._reg_param = 0.0

    def fit(self, X, y):
        X = to_np(X)
        self.classes_, yc = encode_classes(y)
        d = X.shape[1]
        self.priors_ = np.bincount(yc) / len(yc)
        self.means_, self._inv, self._logdet = [], [], []
        for c in range(len(self.classes_)):
            Xc = X[yc == c]
            S = np.cov(Xc.T).reshape(d, d) if len(Xc) > 1 else np.eye(d)
            S = (1 - self._reg_param) * S + self._reg_param * np.eye(d) + 1e-9 * np.eye(d)
            self.means_.append(Xc.mean(0))
            self._inv.append(np.linalg.inv(S))
            self._logdet.append(np.linalg.slogdet(S)[1])
        return self

    def decision_function(self, X):
        X = to_np(X)
        return np.stack([-0.5 * (((X - m) @ Si) * (X - m)).sum(1) - 0.5 * ld + np.log(p)
                         for m, Si, ld, p in zip(self.means_, self._inv, self._logdet, self.priors_)], 1)

    predict_proba = LinearDiscriminantAnalysis.predict_proba
    predict = LinearDiscriminantAnalysis.predict


class GPKernel:
    def __init__(self, kind="rbf", length_scale=1.0, nu=1.5, variance=1.0):
        self.kind, self.length_scale, self.nu, self.variance = kind, length_scale, nu, variance

    @classmethod
    def rbf(cls, length_scale=1.0, variance=1.0): return cls("rbf", length_scale, variance=variance)
    @classmethod
    def matern(cls, length_scale=1.0, nu=1.5, variance=1.0): return cls("matern", length_scale, nu, variance)

    def __call__(self, A, B=None):
        A = to_np(A)
        B = A if B is None else to_np(B)
        d = np.sqrt(pairwise_sq_dists(A, B)) / self.length_scale
        if self.kind == "rbf":
            return self.variance * np.exp(-0.5 * d ** 2)
        if self.nu == 0.5:
            return self.variance * np.exp(-d)
        if self.nu == 2.5:
            return self.variance * (1 + np.sqrt(5) * d + 5 / 3 * d ** 2) * np.exp(-np.sqrt(5) * d)
        return self.variance * (1 + np.sqrt(3) * d) * np.exp(-np.sqrt(3) * d)


class GaussianProcessRegressor(Estimator, RegressorMixin):
    _params = ("alpha", "normalize_y")

    def __init__(self, kernel=None):
        self._kernel, self._alpha, self._normalize_y = kernel or GPKernel.rbf(), 1e-10, False

    def fit(self, X, y):
        self.X_, y = to_np(X), to_np(y)
        self._ym, self._ys = (y.mean(), y.std() or 1.0) if self._normalize_y else (0.0, 1.0)
        K = self._kernel(self.X_) + self._alpha * np.eye(len(y))
        self.L_ = np.linalg.cholesky(K + 1e-10 * np.eye(len(y)))
        self.alpha_ = np.linalg.solve(self.L_.T, np.linalg.solve(self.L_, (y - self._ym) / self._ys))
        return self

    def predict(self, X):
        return out(self._kernel(to_np(X), self.X_) @ self.alpha_ * self._ys + self._ym)

    def predict_with_std(self, X):
        Ks = self._kernel(to_np(X), self.X_)
        v = np.linalg.solve(self.L_, Ks.T)
        var = np.maximum(np.diag(self._kernel(to_np(X))) - (v ** 2).sum(0), 0)
        return out(Ks @ self.alpha_ * self._ys + self._ym), out(np.sqrt(var) * self._ys)

    def log_marginal_likelihood(self):
        y = self.L_ @ (self.L_.T @ self.alpha_)
        return float(-0.5 * y @ self.alpha_ - np.log(np.diag(self.L_)).sum() - 0.5 * len(y) * np.log(2 * np.pi))


class GaussianProcessClassifier(Estimator, ClassifierMixin):
    """Binary (one-vs-rest beyond two classes) GP classification with the Laplace approximation."""
    _params = ("max_iter",)

    def __init__(self, kernel=None):
        self._kernel, self._max_iter = kernel or GPKernel.rbf(), 50

    def _laplace(self, K, t):
        f = np.zeros(len(t))
        for _ in range(self._max_iter):
            pi = sigmoid(f)
            W = pi * (1 - pi)
            sW = np.sqrt(W)
            B = np.eye(len(t)) + sW[:, None] * K * sW[None]
            L = np.linalg.cholesky(B)
            b = W * f + (t - pi)
            a = b - sW * np.linalg.solve(L.T, np.linalg.solve(L, sW * (K @ b)))
            nf = K @ a
            if np.abs(nf - f).max() < 1e-8:
                f = nf
                break
            f = nf
        return f, t - sigmoid(f)

    def fit(self, X, y):
        self.X_ = to_np(X)
        self.classes_, yc = encode_classes(y)
        K = self._kernel(self.X_) + 1e-8 * np.eye(len(yc))
        ks = [1] if len(self.classes_) == 2 else range(len(self.classes_))
        self._grad = [self._laplace(K, (yc == c).astype(float))[1] for c in ks]
        return self

    def predict_proba(self, X):
        Ks = self._kernel(to_np(X), self.X_)
        P = np.stack([sigmoid(Ks @ g) for g in self._grad], 1)
        if P.shape[1] == 1:
            return out(np.hstack((1 - P, P)))
        return out(P / P.sum(1, keepdims=True))

    def predict(self, X):
        return out(self.classes_[to_np(self.predict_proba(X)).argmax(1)])
