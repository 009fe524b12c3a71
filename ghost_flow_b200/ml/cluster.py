"""Clustering, mixtures, hidden Markov model, outlier detection (ghostflow-ml/src/clustering.rs,
clustering_advanced.rs, clustering_more.rs, gmm.rs, mixture.rs, hmm.rs, outlier_detection.rs)."""
from __future__ import annotations

import enum

import numpy as np

from ._base import Estimator, TransformerMixin, out, pairwise_sq_dists, rng_of, to_np


class KMeansInit(enum.Enum):
    Random = "random"
    KMeansPlusPlus = "k-means++"


class DistanceMetric(enum.Enum):
    Euclidean = "euclidean"
    Manhattan = "manhattan"
    Cosine = "cosine"


class Linkage(enum.Enum):
    Ward = "ward"
    Complete = "complete"
    Average = "average"
    Single = "single"


def _kpp(X, k, r):
    c = [X[r.integers(len(X))]]
    for _ in range(1, k):
        d = pairwise_sq_dists(X, np.array(c)).min(1)
        c.append(X[r.choice(len(X), p=d / d.sum())] if d.sum() > 0 else X[r.integers(len(X))])
    return np.array(c)


class KMeans(Estimator, TransformerMixin):
    _params = ("n_init", "max_iter", "tol", "init", "seed")

    def __init__(self, n_clusters=8):
        self._n_clusters, self._n_init, self._max_iter, self._tol = n_clusters, 10, 300, 1e-4
        self._init, self._seed = KMeansInit.KMeansPlusPlus, 0

    def _run(self, X, r):
        k = self._n_clusters
        C = _kpp(X, k, r) if getattr(self._init, "value", self._init) == "k-means++" else X[r.choice(len(X), k, replace=False)]
        for _ in range(self._max_iter):
            lab = pairwise_sq_dists(X, C).argmin(1)
            nC = np.stack([X[lab == j].mean(0) if (lab == j).any() else C[j] for j in range(k)])
            shift = ((nC - C) ** 2).sum()
            C = nC
            if shift < self._tol:
                break
        D = pairwise_sq_dists(X, C)
        lab = D.argmin(1)
        return C, lab, D[np.arange(len(X)), lab].sum()

    def fit(self, X, y=None):
        X = to_np(X)
        r = rng_of(self._seed)
        best = min((self._run(X, r) for _ in range(self._n_init)), key=lambda t: t[2])
        self.cluster_centers_, self.labels_, self.inertia_ = out(best[0]), best[1], float(best[2])
        return self

    def predict(self, X):
        return out(pairwise_sq_dists(to_np(X), to_np(self.cluster_centers_)).argmin(1))

    def fit_predict(self, X, y=None):
        return out(self.fit(X).labels_)

    def transform(self, X):
        return out(np.sqrt(pairwise_sq_dists(to_np(X), to_np(self.cluster_centers_))))


class MiniBatchKMeans(KMeans):
    _params = ("batch_size",)

    def __init__(self, n_clusters=8):
        super().__init__(n_clusters)
        self._batch_size, self._max_iter = 100, 100

    def fit(self, X, y=None):
        X = to_np(X)
        r = rng_of(self._seed)
        C = _kpp(X, self._n_clusters, r)
        counts = np.zeros(self._n_clusters)
        for _ in range(self._max_iter):
            B = X[r.integers(0, len(X), min(self._batch_size, len(X)))]
            lab = pairwise_sq_dists(B, C).argmin(1)
            for x, j in zip(B, lab):
                counts[j] += 1
                C[j] += (x - C[j]) / counts[j]
        D = pairwise_sq_dists(X, C)
        self.cluster_centers_, self.labels_ = out(C), D.argmin(1)
        self.inertia_ = float(D.min(1).sum())
        return self

    def partial_fit(self, X):
        X = to_np(X)
        if not hasattr(self, "_C"):
            self._C, self._counts = _kpp(X, self._n_clusters, rng_of(self._seed)), np.zeros(self._n_clusters)
        for x, j in zip(X, pairwise_sq_dists(X, self._C).argmin(1)):
            self._counts[j] += 1
            self._C[j] += (x - self._C[j]) / self._counts[j]
        self.cluster_centers_ = out(self._C)
        return self


def _region_query(D, i, eps):
    return np.where(D[i] <= eps)[0]


class DBSCAN(Estimator):
    _params = ("metric",)

    def __init__(self, eps=0.5, min_samples=5):
        self._eps, self._min_samples, self._metric = eps, min_samples, DistanceMetric.Euclidean

    def fit(self, X, y=None):
        from .linear import _dists
        X = to_np(X)
        D = _dists(X, X, self._metric)
        n = len(X)
        lab = np.full(n, -2)
        core = (D <= self._eps).sum(1) >= self._min_samples
        c = 0
        for i in range(n):
            if lab[i] != -2:
                continue
            if not core[i]:
                lab[i] = -1
                continue
            lab[i] = c
            stack = list(_region_query(D, i, self._eps))
            while stack:
                j = stack.pop()
                if lab[j] == -1:
                    lab[j] = c
                if lab[j] != -2:
                    continue
                lab[j] = c
                if core[j]:
                    stack.extend(_region_query(D, j, self._eps))
            c += 1
        self.labels_, self.core_sample_indices_ = lab, np.where(core)[0]
        return self

    def fit_predict(self, X, y=None):
        return out(self.fit(X).labels_)


class AgglomerativeClustering(Estimator):
    _params = ("linkage",)

    def __init__(self, n_clusters=2):
        self._n_clusters, self._linkage = n_clusters, Linkage.Ward

    def fit(self, X, y=None):
        from scipy.cluster.hierarchy import fcluster, linkage
        X = to_np(X)
        Z = linkage(X, method=getattr(self._linkage, "value", self._linkage))
        self.children_ = Z[:, :2].astype(int)
        self.labels_ = fcluster(Z, self._n_clusters, "maxclust") - 1
        return self

    def fit_predict(self, X, y=None):
        return out(self.fit(X).labels_)


class SpectralClustering(Estimator):
    _params = ("gamma", "affinity", "n_neighbors", "seed")

    def __init__(self, n_clusters=8):
        self._n_clusters, self._gamma, self._affinity, self._n_neighbors, self._seed = n_clusters, 1.0, "rbf", 10, 0

    def fit(self, X, y=None):
        X = to_np(X)
        D = pairwise_sq_dists(X, X)
        if self._affinity == "nearest_neighbors":
            idx = np.argsort(D, 1)[:, 1:self._n_neighbors + 1]
            A = np.zeros_like(D)
            A[np.arange(len(X))[:, None], idx] = 1
            A = np.maximum(A, A.T)
        else:
            A = np.exp(-self._gamma * D)
            np.fill_diagonal(A, 0)
        d = A.sum(1)
        L = np.eye(len(X)) - A / np.sqrt(np.outer(d, d) + 1e-300)
        _, vecs = np.linalg.eigh(L)
        U = vecs[:, :self._n_clusters]
        U /= np.maximum(np.linalg.norm(U, axis=1, keepdims=True), 1e-12)
        self.labels_ = KMeans(self._n_clusters).seed(self._seed).fit(U).labels_
        return self

    def fit_predict(self, X, y=None):
        return out(self.fit(X).labels_)


class MeanShift(Estimator):
    _params = ("bandwidth", "max_iter")

    def __init__(self):
        self._bandwidth, self._max_iter = None, 100

    def fit(self, X, y=None):
        X = to_np(X)
        bw = self._bandwidth or float(np.sort(np.sqrt(pairwise_sq_dists(X, X)), 1)[:, max(1, int(0.3 * len(X)) - 1)].mean())
        P = X.copy()
        for _ in range(self._max_iter):
            W = np.exp(-0.5 * pairwise_sq_dists(P, X) / bw ** 2)
            nP = W @ X / W.sum(1, keepdims=True)
            if np.abs(nP - P).max() < 1e-5 * bw:
                P = nP
                break
            P = nP
        centers = []
        for p in P:
            if not any(np.linalg.norm(p - c) < bw / 2 for c in centers):
                centers.append(p)
        self.cluster_centers_ = out(np.array(centers))
        self.labels_ = pairwise_sq_dists(X, np.array(centers)).argmin(1)
        return self

    def predict(self, X):
        return out(pairwise_sq_dists(to_np(X), to_np(self.cluster_centers_)).argmin(1))

    def fit_predict(self, X, y=None):
        return out(self.fit(X).labels_)


class AffinityPropagation(Estimator):
    _params = ("damping", "max_iter", "preference")

    def __init__(self):
        self._damping, self._max_iter, self._preference = 0.5, 200, None

    def fit(self, X, y=None):
        X = to_np(X)
        n = len(X)
        S = -pairwise_sq_dists(X, X)
        np.fill_diagonal(S, self._preference if self._preference is not None else np.median(S))
        R, A = np.zeros((n, n)), np.zeros((n, n))
        for _ in range(self._max_iter):
            AS = A + S
            idx = AS.argmax(1)
            first = AS[np.arange(n), idx]
            AS[np.arange(n), idx] = -np.inf
            second = AS.max(1)
            Rn = S - first[:, None]
            Rn[np.arange(n), idx] = S[np.arange(n), idx] - second
            R = self._damping * R + (1 - self._damping) * Rn
            Rp = np.maximum(R, 0)
            np.fill_diagonal(Rp, R.diagonal())
            An = Rp.sum(0)[None, :] - Rp
            dA = An.diagonal().copy()
            An = np.minimum(An, 0)
            np.fill_diagonal(An, dA)
            A = self._damping * A + (1 - self._damping) * An
        ex = np.where((A + R).diagonal() > 0)[0]
        if len(ex) == 0:
            ex = np.array([int((A + R).diagonal().argmax())])
        self.cluster_centers_indices_ = ex
        self.labels_ = S[:, ex].argmax(1)
        self.labels_[ex] = np.arange(len(ex))
        self.cluster_centers_ = out(X[ex])
        return self

    def fit_predict(self, X, y=None):
        return out(self.fit(X).labels_)


class OPTICS(Estimator):
    _params = ("max_eps", "xi", "eps")

    def __init__(self, min_samples=5):
        self._min_samples, self._max_eps, self._xi, self._eps = min_samples, np.inf, 0.05, None

    def fit(self, X, y=None):
        X = to_np(X)
        n = len(X)
        D = np.sqrt(pairwise_sq_dists(X, X))
        core = np.sort(D, 1)[:, min(self._min_samples, n - 1)]
        reach = np.full(n, np.inf)
        done = np.zeros(n, bool)
        order = []
        for s in range(n):
            if done[s]:
                continue
            cur = s
            while cur is not None:
                done[cur] = True
                order.append(cur)
                if core[cur] <= self._max_eps:
                    nd = np.maximum(core[cur], D[cur])
                    m = ~done & (nd < reach) & (D[cur] <= self._max_eps)
                    reach[m] = nd[m]
                cand = np.where(~done & np.isfinite(reach))[0]
                cur = cand[reach[cand].argmin()] if len(cand) else None
        self.ordering_, self.reachability_, self.core_distances_ = np.array(order), reach, core
        eps = self._eps or np.quantile(reach[np.isfinite(reach)], 0.9) if np.isfinite(reach).any() else 1.0
        lab = np.full(n, -1)
        c = -1
        for i in self.ordering_:
            if reach[i] > eps:
                if core[i] <= eps:
                    c += 1
                    lab[i] = c
            else:
                lab[i] = max(c, 0)
        self.labels_ = lab
        return self

    def fit_predict(self, X, y=None):
        return out(self.fit(X).labels_)


class BIRCH(Estimator):
    """Clustering-feature summaries (count, linear sum, squared sum) absorbed within ``threshold``, followed by a
    global clustering of the sub-cluster centroids."""
    _params = ("threshold", "n_clusters", "branching_factor")

    def __init__(self):
        self._threshold, self._n_clusters, self._branching_factor = 0.5, 3, 50

    def fit(self, X, y=None):
        X = to_np(X)
        N, LS, SS = [], [], []
        for x in X:
            if N:
                cen = np.array(LS) / np.array(N)[:, None]
                j = int(((cen - x) ** 2).sum(1).argmin())
                n2, ls2, ss2 = N[j] + 1, LS[j] + x, SS[j] + x @ x
                radius = np.sqrt(max(ss2 / n2 - (ls2 / n2) @ (ls2 / n2), 0))
                if radius <= self._threshold:
                    N[j], LS[j], SS[j] = n2, ls2, ss2
                    continue
            N.append(1)
            LS.append(x.copy())
            SS.append(x @ x)
        self.subcluster_centers_ = np.array(LS) / np.array(N)[:, None]
        k = min(self._n_clusters or len(N), len(N))
        if k < len(N):
            glob = AgglomerativeClustering(k).fit(self.subcluster_centers_).labels_
        else:
            glob = np.arange(len(N))
        self._glob = glob
        self.labels_ = glob[pairwise_sq_dists(X, self.subcluster_centers_).argmin(1)]
        return self

    def predict(self, X):
        return out(self._glob[pairwise_sq_dists(to_np(X), self.subcluster_centers_).argmin(1)])

    def fit_predict(self, X, y=None):
        return out(self.fit(X).labels_)


class HDBSCAN(Estimator):
    """Mutual-reachability minimum spanning tree, single-linkage hierarchy, clusters chosen by stability (excess of
    mass) among those with at least ``min_cluster_size`` points."""
    _params = ("min_samples",)

    def __init__(self, min_cluster_size=5):
        self._min_cluster_size, self._min_samples = min_cluster_size, None

    def fit(self, X, y=None):
        from scipy.cluster.hierarchy import linkage
        from scipy.spatial.distance import squareform
        X = to_np(X)
        n = len(X)
        ms = self._min_samples or self._min_cluster_size
        D = np.sqrt(pairwise_sq_dists(X, X))
        core = np.sort(D, 1)[:, min(ms, n - 1)]
        MR = np.maximum(np.maximum(core[:, None], core[None, :]), D)
        np.fill_diagonal(MR, 0)
        Z = linkage(squareform(MR, checks=False), "single")
        size = {i: 1 for i in range(n)}
        members = {i: [i] for i in range(n)}
        children = {}
        for k, (a, b, d, s) in enumerate(Z):
            nid = n + k
            children[nid] = (int(a), int(b), d)
            size[nid] = int(s)
            members[nid] = members[int(a)] + members[int(b)]
        mcs = self._min_cluster_size
        stability, selected = {}, {}

        def walk(node, birth_lambda):
            """Returns (stability of best selection under node, list of selected clusters)."""
            if node < n:
                return 0.0, []
            a, b, d = children[node]
            lam = 1.0 / max(d, 1e-12)
            big_a, big_b = size[a] >= mcs, size[b] >= mcs
            if big_a and big_b:                       # true split: this cluster dies at lam
                own = size[node] * (lam - birth_lambda)
                sa, ca = walk(a, lam)
                sb, cb = walk(b, lam)
                if own >= sa + sb:
                    return own, [node]
                return sa + sb, ca + cb
            # points fall out; the cluster continues in the big child (if any)
            cont = a if big_a else b if big_b else None
            lost = size[node] - (size[cont] if cont is not None else 0)
            own_part = lost * (lam - birth_lambda)
            if cont is None:
                return size[node] * (lam - birth_lambda), [node]
            s, c = walk(cont, birth_lambda)
            if c == [cont]:
                return s + own_part, [node]
            return s, c

        import sys
        sys.setrecursionlimit(max(10000, 4 * n))
        root = n + len(Z) - 1
        _, chosen = walk(root, 0.0)
        lab = np.full(n, -1)
        if chosen == [root]:
            chosen = [c for c in children[root][:2] if size[c] >= mcs] or [root]
        for ci, node in enumerate(chosen):
            lab[members[node]] = ci
        self.labels_ = lab
        return self

    def fit_predict(self, X, y=None):
        return out(self.fit(X).labels_)


# ----------------------------------------------------------------------------- mixtures
class CovarianceType(enum.Enum):
    Full = "full"
    Diag = "diag"
    Spherical = "spherical"
    Tied = "tied"


def _log_gauss(X, mean, cov):
    d = X.shape[1]
    L = np.linalg.cholesky(cov + 1e-9 * np.eye(d))
    z = np.linalg.solve(L, (X - mean).T)
    return -0.5 * (z ** 2).sum(0) - np.log(np.diag(L)).sum() - 0.5 * d * np.log(2 * np.pi)


class GaussianMixture(Estimator):
    _params = ("covariance_type", "max_iter", "tol", "reg_covar", "seed", "n_init")

    def __init__(self, n_components=1):
        self._n_components, self._covariance_type, self._max_iter, self._tol = n_components, CovarianceType.Full, 100, 1e-4
        self._reg_covar, self._seed, self._n_init = 1e-6, 0, 1

    def _regularise(self, S, d):
        ct = getattr(self._covariance_type, "value", self._covariance_type)
        if ct == "diag":
            S = np.diag(np.diag(S))
        elif ct == "spherical":
            S = np.eye(d) * np.trace(S) / d
        return S + self._reg_covar * np.eye(d)

    def _e(self, X):
        lp = np.stack([np.log(w + 1e-300) + _log_gauss(X, m, S) for w, m, S in
                       zip(self.weights_, self.means_, self.covariances_)], 1)
        mx = lp.max(1, keepdims=True)
        ll = mx[:, 0] + np.log(np.exp(lp - mx).sum(1))
        return np.exp(lp - ll[:, None]), ll

    def _m(self, X, R, prior_w=0.0):
        n, d = X.shape
        nk = R.sum(0) + 1e-10
        self.weights_ = (nk + prior_w) / (n + prior_w * len(nk))
        self.means_ = (R.T @ X) / nk[:, None]
        covs = []
        for k in range(len(nk)):
            Xc = X - self.means_[k]
            covs.append(self._regularise((R[:, k, None] * Xc).T @ Xc / nk[k], d))
        if getattr(self._covariance_type, "value", self._covariance_type) == "tied":
            tied = sum(nk[k] * covs[k] for k in range(len(nk))) / n
            covs = [tied] * len(nk)
        self.covariances_ = np.array(covs)

    def fit(self, X, y=None):
        X = to_np(X)
        best = None
        for init in range(self._n_init):
            km = KMeans(self._n_components).n_init(1).seed(self._seed + init).fit(X)
            R = np.eye(self._n_components)[km.labels_]
            self._m(X, R)
            prev = -np.inf
            for it in range(self._max_iter):
                R, ll = self._e(X)
                self._m(X, R, getattr(self, "_weight_prior", 0.0))
                if abs(ll.mean() - prev) < self._tol:
                    break
                prev = ll.mean()
            if best is None or prev > best[0]:
                best = (prev, self.weights_, self.means_, self.covariances_, it + 1)
        _, self.weights_, self.means_, self.covariances_, self.n_iter_ = best
        self.converged_ = self.n_iter_ < self._max_iter
        return self

    def predict_proba(self, X):
        return out(self._e(to_np(X))[0])

    def predict(self, X):
        return out(self._e(to_np(X))[0].argmax(1))

    def fit_predict(self, X, y=None):
        return self.fit(X).predict(X)

    def score_samples(self, X):
        return out(self._e(to_np(X))[1])

    def score(self, X, y=None):
        return float(self._e(to_np(X))[1].mean())

    def _n_parameters(self, d):
        k = self._n_components
        ct = getattr(self._covariance_type, "value", self._covariance_type)
        cov = {"full": k * d * (d + 1) / 2, "diag": k * d, "spherical": k, "tied": d * (d + 1) / 2}[ct]
        return cov + k * d + k - 1

    def bic(self, X):
        X = to_np(X)
        return float(-2 * self._e(X)[1].sum() + self._n_parameters(X.shape[1]) * np.log(len(X)))

    def aic(self, X):
        X = to_np(X)
        return float(-2 * self._e(X)[1].sum() + 2 * self._n_parameters(X.shape[1]))

    def sample(self, n=1, seed=None):
        r = rng_of(seed)
        comp = r.choice(self._n_components, n, p=self.weights_ / self.weights_.sum())
        return out(np.stack([r.multivariate_normal(self.means_[c], self.covariances_[c]) for c in comp])), out(comp)


class BayesianGaussianMixture(GaussianMixture):
    """Mixture with a sparse Dirichlet prior on the weights (``weight_concentration_prior`` < 1 empties components
    that the data do not support)."""
    _params = ("weight_concentration_prior",)

    def __init__(self, n_components=1):
        super().__init__(n_components)
        self._weight_concentration_prior = None

    def fit(self, X, y=None):
        a = self._weight_concentration_prior if self._weight_concentration_prior is not None else 1.0 / self._n_components
        self._weight_prior = a - 1.0 if a < 1 else 0.0

        def m_step(Xn, R, prior_w=0.0, _orig=GaussianMixture._m):
            _orig(self, Xn, R, 0.0)
            nk = R.sum(0)
            w = np.maximum(nk + a - 1.0, 0.0) if a < 1 else nk + a
            self.weights_ = w / max(w.sum(), 1e-300)
        self._m = m_step
        try:
            return super().fit(X)
        finally:
            del self._m


# ----------------------------------------------------------------------------- HMM
class HMMCovarianceType(enum.Enum):
    Diag = "diag"
    Full = "full"


class GaussianHMM(Estimator):
    _params = ("covariance_type", "max_iter", "tol", "seed")

    def __init__(self, n_components=2, n_features=1):
        self._n_components, self._n_features, self._covariance_type = n_components, n_features, HMMCovarianceType.Diag
        self._max_iter, self._tol, self._seed = 50, 1e-4, 0

    def _logB(self, X):
        return np.stack([_log_gauss(X, m, S) for m, S in zip(self.means_, self.covars_)], 1)

    def _forward_backward(self, X):
        T, k = len(X), self._n_components
        B = self._logB(X)
        sc = B.max(1, keepdims=True)
        Bn = np.exp(B - sc)
        alpha, c = np.zeros((T, k)), np.zeros(T)
        alpha[0] = self.startprob_ * Bn[0]
        c[0] = alpha[0].sum()
        alpha[0] /= c[0]
        for t in range(1, T):
            alpha[t] = (alpha[t - 1] @ self.transmat_) * Bn[t]
            c[t] = alpha[t].sum()
            alpha[t] /= c[t]
        beta = np.ones((T, k))
        for t in range(T - 2, -1, -1):
            beta[t] = (self.transmat_ @ (Bn[t + 1] * beta[t + 1])) / c[t + 1]
        gamma = alpha * beta
        xi = (alpha[:-1, :, None] * self.transmat_[None] * (Bn[1:] * beta[1:])[:, None, :]) / c[1:, None, None]
        return gamma, xi, float(np.log(c).sum() + sc.sum())

    def fit(self, X, lengths=None):
        X = to_np(X)
        X = X[:, None] if X.ndim == 1 else X
        k, d = self._n_components, X.shape[1]
        seqs = np.split(X, np.cumsum(lengths)[:-1]) if lengths is not None else [X]
        km = KMeans(k).seed(self._seed).fit(X)
        self.means_ = to_np(km.cluster_centers_)
        self.covars_ = np.array([np.cov(X[km.labels_ == j].T).reshape(d, d) + 1e-3 * np.eye(d) if (km.labels_ == j).sum() > 1
                                 else np.eye(d) for j in range(k)])
        self.startprob_ = np.full(k, 1.0 / k)
        self.transmat_ = np.full((k, k), 1.0 / k)
        prev = -np.inf
        diag = getattr(self._covariance_type, "value", self._covariance_type) == "diag"
        for _ in range(self._max_iter):
            G, XI, S0, ll = [], np.zeros((k, k)), np.zeros(k), 0.0
            for s in seqs:
                g, xi, l = self._forward_backward(s)
                G.append(g)
                XI += xi.sum(0)
                S0 += g[0]
                ll += l
            g = np.vstack(G)
            self.startprob_ = S0 / S0.sum()
            self.transmat_ = XI / np.maximum(XI.sum(1, keepdims=True), 1e-300)
            nk = g.sum(0) + 1e-10
            self.means_ = g.T @ X / nk[:, None]
            for j in range(k):
                Xc = X - self.means_[j]
                S = (g[:, j, None] * Xc).T @ Xc / nk[j] + 1e-6 * np.eye(d)
                self.covars_[j] = np.diag(np.diag(S)) if diag else S
            if abs(ll - prev) < self._tol:
                break
            prev = ll
        self.log_likelihood_ = ll
        return self

    def score(self, X):
        X = to_np(X)
        return self._forward_backward(X[:, None] if X.ndim == 1 else X)[2]

    def predict_proba(self, X):
        X = to_np(X)
        return out(self._forward_backward(X[:, None] if X.ndim == 1 else X)[0])

    def predict(self, X):
        """Viterbi path."""
        X = to_np(X)
        X = X[:, None] if X.ndim == 1 else X
        B, lt = self._logB(X), np.log(self.transmat_ + 1e-300)
        T, k = B.shape
        delta, psi = np.zeros((T, k)), np.zeros((T, k), int)
        delta[0] = np.log(self.startprob_ + 1e-300) + B[0]
        for t in range(1, T):
            m = delta[t - 1][:, None] + lt
            psi[t], delta[t] = m.argmax(0), m.max(0) + B[t]
        path = np.zeros(T, int)
        path[-1] = delta[-1].argmax()
        for t in range(T - 2, -1, -1):
            path[t] = psi[t + 1][path[t + 1]]
        return out(path)

    def sample(self, n, seed=None):
        r = rng_of(seed)
        s = r.choice(self._n_components, p=self.startprob_)
        xs, ss = [], []
        for _ in range(n):
            xs.append(r.multivariate_normal(self.means_[s], self.covars_[s]))
            ss.append(s)
            s = r.choice(self._n_components, p=self.transmat_[s])
        return out(np.array(xs)), out(np.array(ss))


# ----------------------------------------------------------------------------- outliers
class LocalOutlierFactor(Estimator):
    _params = ("contamination",)

    def __init__(self, n_neighbors=20):
        self._n_neighbors, self._contamination = n_neighbors, 0.1

    def _lof(self, Q, exclude_self):
        D = np.sqrt(pairwise_sq_dists(Q, self.X_))
        k = min(self._n_neighbors, len(self.X_) - 1)
        idx = np.argsort(D, 1)[:, (1 if exclude_self else 0):k + (1 if exclude_self else 0)]
        d = np.take_along_axis(D, idx, 1)
        reach = np.maximum(d, self._kdist[idx])
        lrd = 1.0 / np.maximum(reach.mean(1), 1e-12)
        return (self._lrd[idx].mean(1) / lrd) if hasattr(self, "_lrd") else lrd, idx, lrd

    def fit(self, X, y=None):
        self.X_ = to_np(X)
        D = np.sqrt(pairwise_sq_dists(self.X_, self.X_))
        k = min(self._n_neighbors, len(self.X_) - 1)
        self._kdist = np.sort(D, 1)[:, k]
        _, idx, lrd = self._lof(self.X_, True)
        self._lrd = lrd
        self.negative_outlier_factor_ = -(lrd[idx].mean(1) / lrd)
        self.offset_ = np.quantile(self.negative_outlier_factor_, self._contamination)
        return self

    def fit_predict(self, X, y=None):
        self.fit(X)
        return out(np.where(self.negative_outlier_factor_ < self.offset_, -1.0, 1.0))

    def score_samples(self, X):
        return out(-self._lof(to_np(X), False)[0])

    def predict(self, X):
        return out(np.where(to_np(self.score_samples(X)) < self.offset_, -1.0, 1.0))


class OneClassSVM(Estimator):
    """nu-one-class SVM in the dual: min 1/2 a'Ka, 0 <= a <= 1/(nu n), sum a = 1 (projected gradient)."""
    _params = ("nu", "gamma", "kernel", "max_iter")

    def __init__(self):
        from .linear import Kernel
        self._nu, self._gamma, self._kernel, self._max_iter = 0.1, None, Kernel.rbf(), 500

    def fit(self, X, y=None):
        self.X_ = to_np(X)
        if self._gamma is not None:
            self._kernel.gamma = self._gamma
        K = self._kernel.compute(self.X_)
        n = len(K)
        ub = 1.0 / (self._nu * n)
        a = np.full(n, 1.0 / n)
        lr = 1.0 / max(np.linalg.norm(K, 2), 1e-12)
        for _ in range(self._max_iter):
            a = a - lr * (K @ a)
            lo, hi = a.min() - ub, a.max()           # project on {0 <= a <= ub, sum a = 1} by bisection on the shift
            for _ in range(50):
                mid = (lo + hi) / 2
                if np.clip(a - mid, 0, ub).sum() > 1:
                    lo = mid
                else:
                    hi = mid
            a = np.clip(a - (lo + hi) / 2, 0, ub)
        self.dual_coef_ = a
        sv = (a > 1e-8) & (a < ub - 1e-8)
        f = K @ a
        self.rho_ = f[sv].mean() if sv.any() else np.quantile(f, self._nu)
        return self

    def decision_function(self, X):
        return out(self._kernel.compute(to_np(X), self.X_) @ self.dual_coef_ - self.rho_)

    def predict(self, X):
        return out(np.where(to_np(self.decision_function(X)) >= 0, 1.0, -1.0))


class EllipticEnvelope(Estimator):
    """Robust covariance by concentration steps on the half of the points with the smallest Mahalanobis distance."""
    _params = ("contamination", "support_fraction", "seed")

    def __init__(self):
        self._contamination, self._support_fraction, self._seed = 0.1, None, 0

    def fit(self, X, y=None):
        X = to_np(X)
        n, d = X.shape
        h = int((self._support_fraction or (n + d + 1) / (2 * n)) * n)
        idx = rng_of(self._seed).choice(n, h, replace=False)
        for _ in range(30):
            mu, S = X[idx].mean(0), np.cov(X[idx].T).reshape(d, d) + 1e-9 * np.eye(d)
            md = (((X - mu) @ np.linalg.inv(S)) * (X - mu)).sum(1)
            nidx = np.argsort(md)[:h]
            if set(nidx) == set(idx):
                break
            idx = nidx
        self.location_, self.covariance_ = mu, S
        self._inv = np.linalg.inv(S)
        self.threshold_ = np.quantile(self.mahalanobis(X).numpy(), 1 - self._contamination)
        return self

    def mahalanobis(self, X):
        Xc = to_np(X) - self.location_
        return out(((Xc @ self._inv) * Xc).sum(1))

    def decision_function(self, X):
        return out(self.threshold_ - to_np(self.mahalanobis(X)))

    def predict(self, X):
        return out(np.where(to_np(self.mahalanobis(X)) <= self.threshold_, 1.0, -1.0))
