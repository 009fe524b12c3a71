"""Forecasting and time-series diagnostics (ghostflow-ml/src/time_series.rs, time_series_extended.rs)."""
from __future__ import annotations

import numpy as np

from ._base import Estimator, out, to_np


class SimpleExponentialSmoothing(Estimator):
    def __init__(self, alpha=0.3):
        self._alpha = alpha

    def fit(self, y):
        y = to_np(y)
        l = y[0]
        self.fitted_ = [l]
        for v in y[1:]:
            l = self._alpha * v + (1 - self._alpha) * l
            self.fitted_.append(l)
        self.level_ = l
        return self

    def forecast(self, steps=1):
        return out(np.full(steps, self.level_))

    predict = forecast


class HoltLinear(Estimator):
    def __init__(self, alpha=0.3, beta=0.1):
        self._alpha, self._beta = alpha, beta

    def fit(self, y):
        y = to_np(y)
        l, b = y[0], y[1] - y[0]
        for v in y[1:]:
            pl = l
            l = self._alpha * v + (1 - self._alpha) * (l + b)
            b = self._beta * (l - pl) + (1 - self._beta) * b
        self.level_, self.trend_ = l, b
        return self

    def forecast(self, steps=1):
        return out(self.level_ + self.trend_ * np.arange(1, steps + 1))

    predict = forecast


class HoltWinters(Estimator):
    _params = ("alpha", "beta", "gamma", "seasonal")

    def __init__(self, seasonal_periods=12):
        self._m, self._alpha, self._beta, self._gamma, self._seasonal = seasonal_periods, 0.3, 0.1, 0.1, "additive"

    def fit(self, y):
        y, m = to_np(y), self._m
        mult = self._seasonal == "multiplicative"
        l = y[:m].mean()
        b = (y[m:2 * m].mean() - y[:m].mean()) / m if len(y) >= 2 * m else 0.0
        s = list(y[:m] / l if mult else y[:m] - l)
        for t, v in enumerate(y):
            st = s[t % m]
            pl = l
            l = self._alpha * (v / st if mult else v - st) + (1 - self._alpha) * (l + b)
            b = self._beta * (l - pl) + (1 - self._beta) * b
            s[t % m] = self._gamma * (v / l if mult else v - l) + (1 - self._gamma) * st
        self.level_, self.trend_, self.season_, self._n = l, b, s, len(y)
        return self

    def forecast(self, steps=1):
        h = np.arange(1, steps + 1)
        seas = np.array([self.season_[(self._n + i - 1) % self._m] for i in h])
        base = self.level_ + self.trend_ * h
        return out(base * seas if self._seasonal == "multiplicative" else base + seas)

    predict = forecast


class MovingAverage(Estimator):
    def __init__(self, window=3):
        self._window = window

    def fit(self, y):
        self.y_ = to_np(y)
        return self

    def transform(self, y=None):
        y = self.y_ if y is None else to_np(y)
        c = np.cumsum(np.insert(y, 0, 0.0))
        return out((c[self._window:] - c[:-self._window]) / self._window)

    def forecast(self, steps=1):
        hist = list(self.y_)
        res = []
        for _ in range(steps):
            res.append(np.mean(hist[-self._window:]))
            hist.append(res[-1])
        return out(res)

    predict = forecast


class EWMA(Estimator):
    def __init__(self, span=10):
        self._span = span

    def fit(self, y):
        self.y_ = to_np(y)
        return self

    def transform(self, y=None):
        y = self.y_ if y is None else to_np(y)
        a = 2.0 / (self._span + 1)
        res, s = [], y[0]
        for v in y:
            s = a * v + (1 - a) * s
            res.append(s)
        return out(res)

    def forecast(self, steps=1):
        return out(np.full(steps, to_np(self.transform())[-1]))

    predict = forecast


def _difference(y, d, lag=1):
    for _ in range(d):
        y = y[lag:] - y[:-lag]
    return y


def _invertible(theta):
    """Shrinks moving-average coefficients into the region where the residual recursion is stable."""
    a = np.abs(theta).sum()
    return theta * (0.95 / a) if a >= 0.95 else theta


class ARIMA(Estimator):
    """ARIMA(p, d, q) by conditional sum of squares: AR part from least squares, MA part refined on the residuals
    (Hannan-Rissanen), forecasts integrated back."""

    def __init__(self, p=1, d=0, q=0):
        self._p, self._d, self._q = p, d, q

    def _fit_arma(self, z):
        p, q = self._p, self._q
        mu = z.mean()
        zc = z - mu
        m = max(p + q, 1) + 3
        if q > 0:                                   # long AR to estimate innovations
            L = min(len(zc) // 3, max(m, 10))
            A = np.stack([zc[L - i - 1:len(zc) - i - 1] for i in range(L)], 1)
            phi_long = np.linalg.lstsq(A, zc[L:], rcond=None)[0]
            e = np.concatenate((np.zeros(L), zc[L:] - A @ phi_long))
        else:
            e = np.zeros_like(zc)
        s = max(p, q)
        cols = [zc[s - i - 1:len(zc) - i - 1] for i in range(p)] + [e[s - j - 1:len(zc) - j - 1] for j in range(q)]
        if cols:
            A = np.stack(cols, 1)
            coef = np.linalg.lstsq(A, zc[s:], rcond=None)[0]
        else:
            coef = np.zeros(0)
        self.mu_, self.ar_, self.ma_ = mu, coef[:p], _invertible(coef[p:])
        res = np.zeros_like(zc)
        for t in range(len(zc)):
            pred = sum(self.ar_[i] * zc[t - i - 1] for i in range(p) if t - i - 1 >= 0) + \
                   sum(self.ma_[j] * res[t - j - 1] for j in range(q) if t - j - 1 >= 0)
            res[t] = zc[t] - pred
        self.resid_, self.sigma2_ = res, float(res.var())

    def fit(self, y):
        self.y_ = to_np(y)
        self.z_ = _difference(self.y_, self._d)
        self._fit_arma(self.z_)
        return self

    def _forecast_z(self, steps):
        zc, res = list(self.z_ - self.mu_), list(self.resid_)
        fc = []
        for _ in range(steps):
            v = sum(self.ar_[i] * zc[-i - 1] for i in range(self._p) if len(zc) > i) + \
                sum(self.ma_[j] * res[-j - 1] for j in range(self._q) if len(res) > j)
            zc.append(v)
            res.append(0.0)
            fc.append(v + self.mu_)
        return np.array(fc)

    def forecast(self, steps=1):
        f = self._forecast_z(steps)
        tails = [self.y_]
        for _ in range(self._d - 1):
            tails.append(_difference(tails[-1], 1))
        for lvl in reversed(tails[:self._d]):
            f = lvl[-1] + np.cumsum(f)
        return out(f)

    predict = forecast

    def aic(self):
        n = len(self.z_)
        return float(n * np.log(max(self.sigma2_, 1e-300)) + 2 * (self._p + self._q + 1))


class SARIMA(ARIMA):
    """Seasonal differencing D times at lag ``period`` plus seasonal AR/MA lags folded into one ARMA regression."""

    def __init__(self, p=1, d=0, q=0, P=0, D=0, Q=0, period=12):
        super().__init__(p, d, q)
        self._P, self._D, self._Q, self._period = P, D, Q, period

    def fit(self, y):
        self.y_ = to_np(y)
        s = self._period
        zs = _difference(self.y_, self._D, s)
        self._after_seasonal = zs
        z = _difference(zs, self._d)
        self.z_ = z
        mu = z.mean()
        zc = z - mu
        ar_lags = list(range(1, self._p + 1)) + [s * k for k in range(1, self._P + 1)]
        ma_lags = list(range(1, self._q + 1)) + [s * k for k in range(1, self._Q + 1)]
        L = min(len(zc) // 3, max(2 * s, 10)) if ma_lags else 0
        if ma_lags:
            A = np.stack([zc[L - i - 1:len(zc) - i - 1] for i in range(L)], 1)
            e = np.concatenate((np.zeros(L), zc[L:] - A @ np.linalg.lstsq(A, zc[L:], rcond=None)[0]))
        else:
            e = np.zeros_like(zc)
        m = max(ar_lags + ma_lags + [0])
        cols = [zc[m - l:len(zc) - l] for l in ar_lags] + [e[m - l:len(zc) - l] for l in ma_lags]
        coef = np.linalg.lstsq(np.stack(cols, 1), zc[m:], rcond=None)[0] if cols else np.zeros(0)
        self.mu_, self._ar_lags, self._ma_lags = mu, ar_lags, ma_lags
        self.ar_, self.ma_ = coef[:len(ar_lags)], _invertible(coef[len(ar_lags):])
        res = np.zeros_like(zc)
        for t in range(len(zc)):
            pred = sum(c * zc[t - l] for c, l in zip(self.ar_, ar_lags) if t - l >= 0) + \
                   sum(c * res[t - l] for c, l in zip(self.ma_, ma_lags) if t - l >= 0)
            res[t] = zc[t] - pred
        self.resid_, self.sigma2_ = res, float(res.var())
        return self

    def _forecast_z(self, steps):
        zc, res = list(self.z_ - self.mu_), list(self.resid_)
        fc = []
        for _ in range(steps):
            v = sum(c * zc[-l] for c, l in zip(self.ar_, self._ar_lags) if len(zc) >= l) + \
                sum(c * res[-l] for c, l in zip(self.ma_, self._ma_lags) if len(res) >= l)
            zc.append(v)
            res.append(0.0)
            fc.append(v + self.mu_)
        return np.array(fc)

    def forecast(self, steps=1):
        f = self._forecast_z(steps)
        tails = [self._after_seasonal]
        for _ in range(self._d - 1):
            tails.append(_difference(tails[-1], 1))
        for lvl in reversed(tails[:self._d]):
            f = lvl[-1] + np.cumsum(f)
        s = self._period
        hist = list(self.y_)
        for _ in range(self._D):                         # undo one seasonal difference (D > 1 is rare)
            res = []
            for i, v in enumerate(f):
                res.append(v + (hist[len(hist) - s + i] if i < s else res[i - s]))
            f = np.array(res)
        return out(f)

    predict = forecast


class STLDecomposition(Estimator):
    """Seasonal-trend decomposition: centred moving-average trend, period-wise seasonal means of the detrended
    series (centred to sum to zero), remainder; two refinement passes."""
    _params = ("robust",)

    def __init__(self, period=12):
        self._period, self._robust = period, False

    def fit(self, y):
        y, m = to_np(y), self._period
        seasonal = np.zeros_like(y)
        for _ in range(2):
            d = y - seasonal
            k = m if m % 2 else m + 1
            pad = np.pad(d, (k // 2, k // 2), mode="edge")
            w = np.ones(k)
            if m % 2 == 0:
                w[0] = w[-1] = 0.5
            trend = np.convolve(pad, w / w.sum(), mode="valid")
            det = y - trend
            agg = np.median if self._robust else np.mean
            means = np.array([agg(det[i::m]) for i in range(m)])
            means -= means.mean()
            seasonal = np.tile(means, len(y) // m + 1)[:len(y)]
        self.trend_, self.seasonal_, self.resid_ = trend, seasonal, y - trend - seasonal
        return self

    def components(self):
        return out(self.trend_), out(self.seasonal_), out(self.resid_)


def acf(y, nlags=20):
    y = to_np(y) - to_np(y).mean()
    den = (y * y).sum()
    return out([1.0] + [float((y[k:] * y[:-k]).sum() / den) for k in range(1, nlags + 1)])


def pacf(y, nlags=20):
    r = to_np(acf(y, nlags))
    res = [1.0]
    phi_prev = np.zeros(0)
    for k in range(1, nlags + 1):                       # Durbin-Levinson
        num = r[k] - (phi_prev * r[k - 1:0:-1][:len(phi_prev)]).sum() if k > 1 else r[1]
        den = 1 - (phi_prev * r[1:k]).sum() if k > 1 else 1.0
        pk = num / den
        phi_prev = np.concatenate((phi_prev - pk * phi_prev[::-1], [pk]))
        res.append(float(pk))
    return out(res)


def adf_test(y, max_lag=None):
    """Augmented Dickey-Fuller with a constant. Returns (t statistic, approximate p-value, used lag)."""
    y = to_np(y)
    n = len(y)
    lag = int(max_lag if max_lag is not None else np.floor(12 * (n / 100) ** 0.25))
    lag = min(lag, n // 2 - 2)
    dy = np.diff(y)
    rows = len(dy) - lag
    cols = [y[lag:-1], np.ones(rows)] + [dy[lag - i:len(dy) - i] for i in range(1, lag + 1)]
    A = np.stack(cols, 1)
    t = dy[lag:]
    beta, *_ = np.linalg.lstsq(A, t, rcond=None)
    resid = t - A @ beta
    s2 = resid @ resid / max(1, rows - A.shape[1])
    se = np.sqrt(s2 * np.linalg.inv(A.T @ A)[0, 0])
    stat = beta[0] / se
    # MacKinnon (constant, no trend) critical values for interpolation of a rough p-value
    crit = [(-3.43, 0.01), (-2.86, 0.05), (-2.57, 0.10), (-1.94, 0.30), (-0.5, 0.90)]
    p = float(np.interp(stat, [c for c, _ in crit], [v for _, v in crit], left=0.001, right=0.99))
    return float(stat), p, lag
