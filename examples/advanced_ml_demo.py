"""Classical ML tour: boosting, mixtures, HMM, CRF, feature engineering and hyper-parameter search
(the contents of the reference's examples/advanced_ml_demo.rs and v0_3_0_complete_demo.rs)."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import ghost_flow_b200.ml as ml  # noqa: E402


def main():
    r = np.random.default_rng(0)
    X = r.standard_normal((300, 6))
    y = ((X[:, 0] > 0) ^ (X[:, 1] > 0)).astype(float)
    Xtr, Xte, ytr, yte = ml.train_test_split(X, y, 0.25, seed=0)
    for m in (ml.XGBoostClassifier(30).max_depth(3).learning_rate(0.3), ml.LightGBMClassifier(30).num_leaves(15),
              ml.RandomForestClassifier(30).max_depth(8)):
        print(type(m).__name__, "test accuracy", round(m.fit(Xtr, ytr).score(Xte, yte), 3))
    blobs = np.vstack([r.standard_normal((80, 2)) * 0.5 + c for c in ([0, 0], [4, 4], [0, 5])])
    gmm = ml.GaussianMixture(3).fit(blobs)
    print("GMM BIC", round(gmm.bic(blobs), 1), "weights", np.round(gmm.weights_, 2))
    seq = np.concatenate([r.normal(0, 1, 100), r.normal(5, 1, 100)])[:, None]
    print("HMM states", ml.GaussianHMM(2, 1).fit(seq).predict(seq).numpy()[[0, 99, 100, 199]])
    seqs = [r.standard_normal((15, 3)) for _ in range(20)]
    labs = [(s[:, 0] > 0).astype(float) for s in seqs]
    crf = ml.LinearChainCRF(2, 3).max_iter(40).fit(seqs, labs)
    print("CRF token accuracy", float((crf.predict(seqs[0]).numpy() == labs[0]).mean()))
    feats = ml.PolynomialFeatures(2).fit_transform(ml.StandardScaler().fit_transform(X))
    print("polynomial features", feats.shape)
    space = ml.ParameterSpace().add_float("alpha", 1e-3, 10.0, log=True)
    best, score = ml.BayesianOptimization(space, 12).optimize(
        lambda p: ml.cross_val_score(ml.Ridge(p["alpha"]), X, X @ np.arange(6.0) + 0.1 * r.standard_normal(300), 3).mean())
    print("Bayesian search: alpha", round(best["alpha"], 4), "cv R2", round(score, 4))


if __name__ == "__main__":
    main()
