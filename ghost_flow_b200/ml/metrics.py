"""Classification, regression and clustering metrics as free functions (ghostflow-ml/src/metrics.rs,
metrics_advanced.rs). All return Python floats (or numpy arrays / dicts where the result is not a scalar)."""
from __future__ import annotations

import numpy as np

from ._base import pairwise_sq_dists, to_np


def accuracy_score(y_true, y_pred):
    return float((to_np(y_true) == to_np(y_pred)).mean())


def confusion_matrix(y_true, y_pred, labels=None):
    yt, yp = to_np(y_true), to_np(y_pred)
    labels = np.unique(np.concatenate((yt, yp))) if labels is None else np.asarray(labels)
    m = np.zeros((len(labels), len(labels)), int)
    for i, a in enumerate(labels):
        for j, b in enumerate(labels):
            m[i, j] = int(((yt == a) & (yp == b)).sum())
    return m


def _prf(y_true, y_pred, average):
    yt, yp = to_np(y_true), to_np(y_pred)
    labels = np.unique(np.concatenate((yt, yp)))
    if average == "binary":
        labels = np.array([labels.max()])
    tp = np.array([((yt == c) & (yp == c)).sum() for c in labels], float)
    fp = np.array([((yt != c) & (yp == c)).sum() for c in labels], float)
    fn = np.array([((yt == c) & (yp != c)).sum() for c in labels], float)
    if average == "micro":
        tp, fp, fn = tp.sum(keepdims=True), fp.sum(keepdims=True), fn.sum(keepdims=True)
    p = tp / np.maximum(tp + fp, 1e-300)
    r = tp / np.maximum(tp + fn, 1e-300)
    f = 2 * p * r / np.maximum(p + r, 1e-300)
    if average == "weighted":
        w = np.array([(yt == c).sum() for c in labels], float)
        w /= w.sum()
        return float((p * w).sum()), float((r * w).sum()), float((f * w).sum())
    return float(p.mean()), float(r.mean()), float(f.mean())


def precision_score(y_true, y_pred, average="binary"):
    return _prf(y_true, y_pred, average)[0]


def recall_score(y_true, y_pred, average="binary"):
    return _prf(y_true, y_pred, average)[1]


def f1_score(y_true, y_pred, average="binary"):
    return _prf(y_true, y_pred, average)[2]


def roc_auc_score(y_true, y_score):
    yt, s = to_np(y_true), to_np(y_score)
    pos = yt == yt.max()
    order = np.argsort(s)
    ranks = np.empty(len(s))
    ranks[order] = np.arange(1, len(s) + 1)
    for v in np.unique(s):                       # average ranks of ties
        m = s == v
        if m.sum() > 1:
            ranks[m] = ranks[m].mean()
    npos, nneg = pos.sum(), (~pos).sum()
    return float((ranks[pos].sum() - npos * (npos + 1) / 2) / max(1, npos * nneg))


def classification_report(y_true, y_pred) -> dict:
    yt, yp = to_np(y_true), to_np(y_pred)
    rep = {}
    for c in np.unique(yt):
        tp = ((yt == c) & (yp == c)).sum()
        p = tp / max(1, (yp == c).sum())
        r = tp / max(1, (yt == c).sum())
        rep[float(c)] = {"precision": float(p), "recall": float(r), "f1": float(2 * p * r / max(p + r, 1e-300)),
                         "support": int((yt == c).sum())}
    rep["accuracy"] = accuracy_score(yt, yp)
    return rep


def mean_squared_error(y_true, y_pred):
    return float(((to_np(y_true) - to_np(y_pred)) ** 2).mean())


def root_mean_squared_error(y_true, y_pred):
    return float(np.sqrt(mean_squared_error(y_true, y_pred)))


def mean_absolute_error(y_true, y_pred):
    return float(np.abs(to_np(y_true) - to_np(y_pred)).mean())


def r2_score(y_true, y_pred):
    yt, yp = to_np(y_true), to_np(y_pred)
    return float(1 - ((yt - yp) ** 2).sum() / max(((yt - yt.mean()) ** 2).sum(), 1e-300))


def mean_absolute_percentage_error(y_true, y_pred):
    yt, yp = to_np(y_true), to_np(y_pred)
    return float((np.abs(yt - yp) / np.maximum(np.abs(yt), 1e-12)).mean())


def explained_variance_score(y_true, y_pred):
    yt, yp = to_np(y_true), to_np(y_pred)
    return float(1 - (yt - yp).var() / max(yt.var(), 1e-300))


mse, rmse, mae, r2, mape = (mean_squared_error, root_mean_squared_error, mean_absolute_error, r2_score,
                            mean_absolute_percentage_error)


def log_loss(y_true, p, eps=1e-15):
    yt, p = to_np(y_true), np.clip(to_np(p), eps, 1 - eps)
    if p.ndim == 2:
        return log_loss_multiclass(yt, p, eps)
    return float(-(yt * np.log(p) + (1 - yt) * np.log(1 - p)).mean())


def log_loss_multiclass(y_true, P, eps=1e-15):
    yt, P = to_np(y_true).astype(int), np.clip(to_np(P), eps, 1.0)
    P = P / P.sum(1, keepdims=True)
    return float(-np.log(P[np.arange(len(yt)), yt]).mean())


def hinge_loss(y_true, decision):
    y = np.where(to_np(y_true) > 0, 1.0, -1.0)
    return float(np.maximum(0, 1 - y * to_np(decision)).mean())


def squared_hinge_loss(y_true, decision):
    y = np.where(to_np(y_true) > 0, 1.0, -1.0)
    return float((np.maximum(0, 1 - y * to_np(decision)) ** 2).mean())


def cohen_kappa_score(a, b):
    m = confusion_matrix(a, b).astype(float)
    n = m.sum()
    po = np.trace(m) / n
    pe = (m.sum(0) * m.sum(1)).sum() / n ** 2
    return float((po - pe) / max(1 - pe, 1e-300))


def matthews_corrcoef(y_true, y_pred):
    m = confusion_matrix(y_true, y_pred).astype(float)
    t, p, c, s = m.sum(1), m.sum(0), np.trace(m), m.sum()
    den = np.sqrt((s ** 2 - (p ** 2).sum()) * (s ** 2 - (t ** 2).sum()))
    return float((c * s - (t * p).sum()) / den) if den > 0 else 0.0


def _contingency(a, b):
    ua, ia = np.unique(to_np(a), return_inverse=True)
    ub, ib = np.unique(to_np(b), return_inverse=True)
    m = np.zeros((len(ua), len(ub)))
    np.add.at(m, (ia, ib), 1)
    return m


def adjusted_rand_score(a, b):
    m = _contingency(a, b)
    comb = lambda x: x * (x - 1) / 2  # noqa: E731
    s, sa, sb, n = comb(m).sum(), comb(m.sum(1)).sum(), comb(m.sum(0)).sum(), comb(m.sum())
    exp = sa * sb / max(n, 1e-300)
    den = 0.5 * (sa + sb) - exp
    return float((s - exp) / den) if den != 0 else 1.0


def normalized_mutual_info_score(a, b):
    m = _contingency(a, b)
    p = m / m.sum()
    pa, pb = p.sum(1, keepdims=True), p.sum(0, keepdims=True)
    nz = p > 0
    mi = (p[nz] * np.log(p[nz] / (pa @ pb)[nz])).sum()
    ha = -(pa[pa > 0] * np.log(pa[pa > 0])).sum()
    hb = -(pb[pb > 0] * np.log(pb[pb > 0])).sum()
    return float(mi / max(np.sqrt(ha * hb), 1e-300)) if ha > 0 and hb > 0 else 1.0


def fowlkes_mallows_score(a, b):
    m = _contingency(a, b)
    tk = (m ** 2).sum() - m.sum()
    pk = (m.sum(0) ** 2).sum() - m.sum()
    qk = (m.sum(1) ** 2).sum() - m.sum()
    return float(tk / np.sqrt(pk * qk)) if pk > 0 and qk > 0 else 0.0


def silhouette_score(X, labels):
    X, l = to_np(X), to_np(labels)
    D = np.sqrt(pairwise_sq_dists(X, X))
    cl = np.unique(l)
    s = np.zeros(len(X))
    for i in range(len(X)):
        same = l == l[i]
        a = D[i, same].sum() / max(1, same.sum() - 1)
        b = min(D[i, l == c].mean() for c in cl if c != l[i]) if len(cl) > 1 else 0.0
        s[i] = (b - a) / max(a, b, 1e-300) if same.sum() > 1 else 0.0
    return float(s.mean())


def davies_bouldin_score(X, labels):
    X, l = to_np(X), to_np(labels)
    cl = np.unique(l)
    cen = np.stack([X[l == c].mean(0) for c in cl])
    sc = np.array([np.sqrt(((X[l == c] - cen[i]) ** 2).sum(1)).mean() for i, c in enumerate(cl)])
    M = np.sqrt(pairwise_sq_dists(cen, cen))
    np.fill_diagonal(M, np.inf)
    return float(np.mean([np.max((sc[i] + sc) / M[i]) for i in range(len(cl))]))


def calinski_harabasz_score(X, labels):
    X, l = to_np(X), to_np(labels)
    cl = np.unique(l)
    n, k = len(X), len(cl)
    mean = X.mean(0)
    b = sum((l == c).sum() * ((X[l == c].mean(0) - mean) ** 2).sum() for c in cl)
    w = sum(((X[l == c] - X[l == c].mean(0)) ** 2).sum() for c in cl)
    return float(b / max(w, 1e-300) * (n - k) / max(1, k - 1))
