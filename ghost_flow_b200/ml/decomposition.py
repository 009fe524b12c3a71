"""Matrix decompositions and manifold learning (ghostflow-ml/src/decomposition.rs, decomposition_advanced.rs,
decomposition_incremental.rs, manifold.rs)."""
from __future__ import annotations

import numpy as np

from ._base import Estimator, TransformerMixin, out, pairwise_sq_dists, rng_of, to_np


class PCA(Estimator, TransformerMixin):
    _params = ("whiten",)

    def __init__(self, n_components=2):
        self._n_components, self._whiten = n_components, False

    def fit(self, X, y=None):
        X = to_np(X)
        self.mean_ = X.mean(0)
        U, s, Vt = np.linalg.svd(X - self.mean_, full_matrices=False)
        # deterministic sign: largest-magnitude loading of every component is positive
        sign = np.sign(Vt[np.arange(len(Vt)), np.abs(Vt).argmax(1)])
        Vt = Vt * sign[:, None]
        k = self._n_components
        var = s ** 2 / max(1, len(X) - 1)
        self.components_, self.explained_variance_ = Vt[:k], var[:k]
        self.explained_variance_ratio_ = var[:k] / var.sum()
        self.singular_values_ = s[:k]
        return self

    def transform(self, X):
        Z = (to_np(X) - self.mean_) @ self.components_.T
        return out(Z / np.sqrt(self.explained_variance_ + 1e-300) if self._whiten else Z)

    def inverse_transform(self, Z):
        Z = to_np(Z)
        if self._whiten:
            Z = Z * np.sqrt(self.explained_variance_)
        return out(Z @ self.components_ + self.mean_)


class SVD(Estimator, TransformerMixin):
    """Truncated SVD without centring."""

    def __init__(self, n_components=None):
        self._n_components = n_components

    def fit(self, X, y=None):
        X = to_np(X)
        U, s, Vt = np.linalg.svd(X, full_matrices=False)
        k = self._n_components or len(s)
        self.u_, self.singular_values_, self.components_ = U[:, :k], s[:k], Vt[:k]
        return self

    def transform(self, X):
        return out(to_np(X) @ self.components_.T)

    def inverse_transform(self, Z):
        return out(to_np(Z) @ self.components_)


class NMF(Estimator, TransformerMixin):
    """Multiplicative updates for the Frobenius objective."""
    _params = ("max_iter", "tol", "seed")

    def __init__(self, n_components=2):
        self._n_components, self._max_iter, self._tol, self._seed = n_components, 500, 1e-5, 0

    def _solve_w(self, X, H, W, iters):
        for _ in range(iters):
            W *= (X @ H.T) / np.maximum(W @ (H @ H.T), 1e-12)
        return W

    def fit_transform(self, X, y=None):
        X = to_np(X)
        r = rng_of(self._seed)
        k = self._n_components
        sc = np.sqrt(max(X.mean(), 1e-12) / k)
        W, H = np.abs(r.standard_normal((len(X), k))) * sc, np.abs(r.standard_normal((k, X.shape[1]))) * sc
        prev = np.inf
        for _ in range(self._max_iter):
            H *= (W.T @ X) / np.maximum(W.T @ W @ H, 1e-12)
            W *= (X @ H.T) / np.maximum(W @ (H @ H.T), 1e-12)
            err = np.linalg.norm(X - W @ H)
            if abs(prev - err) < self._tol * max(err, 1e-12):
                break
            prev = err
        self.components_, self.reconstruction_err_ = H, float(err)
        return out(W)

    def fit(self, X, y=None):
        self.fit_transform(X)
        return self

    def transform(self, X):
        X = to_np(X)
        W = np.full((len(X), self._n_components), np.sqrt(max(X.mean(), 1e-12) / self._n_components))
        return out(self._solve_w(X, self.components_, W, 200))

    def inverse_transform(self, W):
        return out(to_np(W) @ self.components_)


class FactorAnalysis(Estimator, TransformerMixin):
    """EM for x = W z + mu + eps, eps ~ N(0, diag(psi))."""
    _params = ("max_iter", "tol")

    def __init__(self, n_components=2):
        self._n_components, self._max_iter, self._tol = n_components, 200, 1e-4

    def fit(self, X, y=None):
        X = to_np(X)
        n, d = X.shape
        self.mean_ = X.mean(0)
        Xc = X - self.mean_
        S = Xc.T @ Xc / n
        k = self._n_components
        W = np.linalg.svd(Xc, full_matrices=False)[2][:k].T * np.sqrt(np.diag(S).mean())
        psi = np.diag(S).copy()
        prev = -np.inf
        for _ in range(self._max_iter):
            G = np.linalg.inv(np.eye(k) + (W.T / psi) @ W)
            B = G @ W.T / psi                                    # E[z|x] = B x
            Ezz = G + B @ S @ B.T
            W = S @ B.T @ np.linalg.inv(Ezz)
            psi = np.maximum(np.diag(S - W @ B @ S), 1e-8)
            C = W @ W.T + np.diag(psi)
            ll = -0.5 * n * (np.linalg.slogdet(C)[1] + np.trace(np.linalg.solve(C, S)) + d * np.log(2 * np.pi))
            if abs(ll - prev) < self._tol * abs(ll):
                break
            prev = ll
        self.components_, self.noise_variance_, self.loglike_ = W.T, psi, float(ll)
        return self

    def transform(self, X):
        W, psi = self.components_.T, self.noise_variance_
        G = np.linalg.inv(np.eye(W.shape[1]) + (W.T / psi) @ W)
        return out((to_np(X) - self.mean_) @ (G @ W.T / psi).T)


class FastICA(Estimator, TransformerMixin):
    """Symmetric fixed-point iteration with the log-cosh contrast on whitened data."""
    _params = ("max_iter", "tol", "seed")

    def __init__(self, n_components=2):
        self._n_components, self._max_iter, self._tol, self._seed = n_components, 200, 1e-5, 0

    @staticmethod
    def _sym(W):
        s, u = np.linalg.eigh(W @ W.T)
        return u @ np.diag(1 / np.sqrt(np.maximum(s, 1e-12))) @ u.T @ W

    def fit(self, X, y=None):
        X = to_np(X)
        self.mean_ = X.mean(0)
        Xc = X - self.mean_
        U, s, Vt = np.linalg.svd(Xc, full_matrices=False)
        k = self._n_components
        self.whitening_ = (Vt[:k] / s[:k, None]) * np.sqrt(len(X))
        Z = Xc @ self.whitening_.T
        W = self._sym(rng_of(self._seed).standard_normal((k, k)))
        for _ in range(self._max_iter):
            Y = Z @ W.T
            g, gp = np.tanh(Y), 1 - np.tanh(Y) ** 2
            Wn = self._sym(g.T @ Z / len(Z) - gp.mean(0)[:, None] * W)
            lim = np.abs(np.abs((Wn * W).sum(1)) - 1).max()
            W = Wn
            if lim < self._tol:
                break
        self.components_ = W @ self.whitening_
        self.mixing_ = np.linalg.pinv(self.components_)
        return self

    def transform(self, X):
        return out((to_np(X) - self.mean_) @ self.components_.T)

    def inverse_transform(self, S):
        return out(to_np(S) @ self.mixing_.T + self.mean_)


def _lasso_codes(X, D, alpha, iters=100):
    """argmin_C 1/2 |X - C D|^2 + alpha |C|_1 by ISTA."""
    L = max(np.linalg.norm(D @ D.T, 2), 1e-12)
    C = np.zeros((len(X), len(D)))
    for _ in range(iters):
        Z = C - (C @ D - X) @ D.T / L
        C = np.sign(Z) * np.maximum(np.abs(Z) - alpha / L, 0)
    return C


class DictionaryLearning(Estimator, TransformerMixin):
    _params = ("alpha", "max_iter", "seed")

    def __init__(self, n_components=2):
        self._n_components, self._alpha, self._max_iter, self._seed = n_components, 1.0, 50, 0

    def fit(self, X, y=None):
        X = to_np(X)
        r = rng_of(self._seed)
        D = X[r.choice(len(X), self._n_components, replace=len(X) < self._n_components)].copy()
        D /= np.maximum(np.linalg.norm(D, axis=1, keepdims=True), 1e-12)
        for _ in range(self._max_iter):
            C = _lasso_codes(X, D, self._alpha, 30)
            A, B = C.T @ C, C.T @ X
            for j in range(len(D)):
                if A[j, j] > 1e-12:
                    D[j] += (B[j] - A[j] @ D) / A[j, j]
                    D[j] /= max(np.linalg.norm(D[j]), 1.0)
        self.components_ = D
        return self

    def transform(self, X):
        return out(_lasso_codes(to_np(X), self.components_, self._alpha))


class SparsePCA(DictionaryLearning):
    """Sparse loadings: dictionary learning on the transposed problem (sparse components, dense codes)."""

    def fit(self, X, y=None):
        X = to_np(X)
        self.mean_ = X.mean(0)
        Xc = X - self.mean_
        U, s, Vt = np.linalg.svd(Xc, full_matrices=False)
        k = self._n_components
        Ucode = U[:, :k] * s[:k]
        V = Vt[:k].copy()
        for _ in range(self._max_iter):
            # components: lasso of X^T on the codes; codes: ridge-regularised least squares, unit norm columns
            Un = Ucode / np.maximum(np.linalg.norm(Ucode, axis=0, keepdims=True), 1e-12)
            V = _lasso_codes(Xc.T, Un.T, self._alpha, 30).T
            G = V @ V.T + 1e-6 * np.eye(k)
            Ucode = Xc @ V.T @ np.linalg.inv(G)
        self.components_ = V / np.maximum(np.linalg.norm(V, axis=1, keepdims=True), 1e-12)
        return self

    def transform(self, X):
        V = self.components_
        return out((to_np(X) - self.mean_) @ V.T @ np.linalg.inv(V @ V.T + 1e-6 * np.eye(len(V))))


class MiniBatchSparsePCA(SparsePCA):
    _params = ("batch_size",)

    def __init__(self, n_components=2):
        super().__init__(n_components)
        self._batch_size, self._max_iter = 50, 20

    def fit(self, X, y=None):
        X = to_np(X)
        r = rng_of(self._seed)
        sub = X[r.choice(len(X), min(len(X), self._batch_size * self._max_iter), replace=False)]
        return super().fit(sub)

    def partial_fit(self, X):
        return self.fit(X)


class IncrementalPCA(PCA):
    """Batch-wise SVD update (stack of previous singular directions, new centred batch and the mean correction)."""
    _params = ("batch_size",)

    def __init__(self, n_components=2):
        super().__init__(n_components)
        self._batch_size, self.n_samples_seen_ = None, 0

    def partial_fit(self, X, y=None):
        X = to_np(X)
        n, k = len(X), self._n_components
        if self.n_samples_seen_ == 0:
            self.mean_ = X.mean(0)
            M = X - self.mean_
        else:
            tot = self.n_samples_seen_ + n
            bm = X.mean(0)
            corr = np.sqrt(self.n_samples_seen_ * n / tot) * (self.mean_ - bm)
            M = np.vstack((self.singular_values_[:, None] * self.components_, X - bm, corr))
            self.mean_ = (self.n_samples_seen_ * self.mean_ + n * bm) / tot
        U, s, Vt = np.linalg.svd(M, full_matrices=False)
        sign = np.sign(Vt[np.arange(len(Vt)), np.abs(Vt).argmax(1)])
        Vt = Vt * sign[:, None]
        self.n_samples_seen_ += n
        self.components_, self.singular_values_ = Vt[:k], s[:k]
        var = s ** 2 / max(1, self.n_samples_seen_ - 1)
        self.explained_variance_ = var[:k]
        self.explained_variance_ratio_ = var[:k] / max(var.sum(), 1e-300)
        return self

    def fit(self, X, y=None):
        X = to_np(X)
        self.n_samples_seen_ = 0
        bs = self._batch_size or max(5 * X.shape[1], self._n_components + 1)
        for i in range(0, len(X), bs):
            if len(X) - i < self._n_components and i > 0:
                break
            self.partial_fit(X[i:i + bs] if len(X) - (i + bs) >= self._n_components else X[i:])
            if len(X) - (i + bs) < self._n_components:
                break
        return self


# ----------------------------------------------------------------------------- manifold
def _classical_mds(D2, k):
    n = len(D2)
    J = np.eye(n) - 1.0 / n
    B = -0.5 * J @ D2 @ J
    vals, vecs = np.linalg.eigh(B)
    idx = np.argsort(vals)[::-1][:k]
    return vecs[:, idx] * np.sqrt(np.maximum(vals[idx], 0))


class MDS(Estimator):
    """Classical scaling followed by SMACOF majorisation of the metric stress."""
    _params = ("max_iter", "eps", "metric")

    def __init__(self, n_components=2):
        self._n_components, self._max_iter, self._eps, self._metric = n_components, 300, 1e-6, True

    def fit_transform(self, X, y=None):
        X = to_np(X)
        D = np.sqrt(pairwise_sq_dists(X, X))
        Z = _classical_mds(D ** 2, self._n_components)
        prev = np.inf
        for _ in range(self._max_iter):
            d = np.sqrt(pairwise_sq_dists(Z, Z))
            stress = ((d - D) ** 2).sum() / 2
            if abs(prev - stress) < self._eps * max(stress, 1e-12):
                break
            prev = stress
            B = -D / np.maximum(d, 1e-12)
            np.fill_diagonal(B, 0)
            np.fill_diagonal(B, -B.sum(1))
            Z = B @ Z / len(Z)
        self.embedding_, self.stress_ = Z, float(stress)
        return out(Z)

    def fit(self, X, y=None):
        self.fit_transform(X)
        return self


class Isomap(Estimator):
    _params = ("n_neighbors",)

    def __init__(self, n_components=2):
        self._n_components, self._n_neighbors = n_components, 5

    def fit_transform(self, X, y=None):
        from scipy.sparse.csgraph import shortest_path
        X = to_np(X)
        D = np.sqrt(pairwise_sq_dists(X, X))
        G = np.full_like(D, np.inf)
        idx = np.argsort(D, 1)[:, 1:self._n_neighbors + 1]
        rows = np.arange(len(X))[:, None]
        G[rows, idx] = D[rows, idx]
        G = np.minimum(G, G.T)
        SP = shortest_path(np.where(np.isfinite(G), G, 0), directed=False)
        SP[~np.isfinite(SP)] = SP[np.isfinite(SP)].max() * 2
        self.dist_matrix_ = SP
        self.embedding_ = _classical_mds(SP ** 2, self._n_components)
        return out(self.embedding_)

    def fit(self, X, y=None):
        self.fit_transform(X)
        return self


class LocallyLinearEmbedding(Estimator):
    _params = ("n_neighbors", "reg")

    def __init__(self, n_components=2):
        self._n_components, self._n_neighbors, self._reg = n_components, 5, 1e-3

    def fit_transform(self, X, y=None):
        X = to_np(X)
        n, k = len(X), self._n_neighbors
        idx = np.argsort(pairwise_sq_dists(X, X), 1)[:, 1:k + 1]
        W = np.zeros((n, n))
        for i in range(n):
            Z = X[idx[i]] - X[i]
            C = Z @ Z.T
            C += np.eye(k) * self._reg * max(np.trace(C), 1e-12)
            w = np.linalg.solve(C, np.ones(k))
            W[i, idx[i]] = w / w.sum()
        M = (np.eye(n) - W).T @ (np.eye(n) - W)
        vals, vecs = np.linalg.eigh(M)
        self.embedding_ = vecs[:, 1:self._n_components + 1] * np.sqrt(n)
        self.reconstruction_error_ = float(vals[1:self._n_components + 1].sum())
        return out(self.embedding_)

    def fit(self, X, y=None):
        self.fit_transform(X)
        return self


class TSNE(Estimator):
    """Exact t-SNE: perplexity-calibrated affinities, early exaggeration, momentum gradient descent."""
    _params = ("perplexity", "n_iter", "learning_rate", "early_exaggeration", "seed")

    def __init__(self, n_components=2):
        self._n_components, self._perplexity, self._n_iter, self._learning_rate = n_components, 30.0, 500, 200.0
        self._early_exaggeration, self._seed = 12.0, 0

    def _affinities(self, D2):
        n = len(D2)
        P = np.zeros((n, n))
        target = np.log(min(self._perplexity, (n - 1) / 3))
        for i in range(n):
            lo, hi, beta = 0.0, np.inf, 1.0
            d = np.delete(D2[i], i)
            for _ in range(50):
                p = np.exp(-(d - d.min()) * beta)
                sp = p.sum()
                H = np.log(sp) + beta * ((d - d.min()) * p).sum() / sp
                if abs(H - target) < 1e-5:
                    break
                if H > target:
                    lo, beta = beta, beta * 2 if hi == np.inf else (beta + hi) / 2
                else:
                    hi, beta = beta, (beta + lo) / 2
            P[i, np.arange(n) != i] = p / sp
        P = (P + P.T) / (2 * n)
        return np.maximum(P, 1e-12)

    def fit_transform(self, X, y=None):
        X = to_np(X)
        n = len(X)
        P = self._affinities(pairwise_sq_dists(X, X))
        r = rng_of(self._seed)
        Y = r.standard_normal((n, self._n_components)) * 1e-4
        vel, gains = np.zeros_like(Y), np.ones_like(Y)
        for it in range(self._n_iter):
            ex = self._early_exaggeration if it < min(250, self._n_iter // 2) else 1.0
            num = 1.0 / (1.0 + pairwise_sq_dists(Y, Y))
            np.fill_diagonal(num, 0)
            Q = np.maximum(num / num.sum(), 1e-12)
            PQ = (ex * P - Q) * num
            grad = 4 * ((np.diag(PQ.sum(1)) - PQ) @ Y)
            gains = np.where(np.sign(grad) != np.sign(vel), gains + 0.2, gains * 0.8).clip(0.01)
            mom = 0.5 if it < 250 else 0.8
            vel = mom * vel - self._learning_rate * gains * grad
            Y = Y + vel
            Y -= Y.mean(0)
        self.embedding_ = Y
        self.kl_divergence_ = float((P * np.log(P / Q)).sum())
        return out(Y)

    def fit(self, X, y=None):
        self.fit_transform(X)
        return self
