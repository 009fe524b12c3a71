"""Classical-ML package: every estimator family on small synthetic problems with known structure."""
import numpy as np
import pytest

import ghost_flow_b200.ml as ml

R = np.random.default_rng(0)
X = R.standard_normal((240, 5))
W = np.array([1.0, -2.0, 0.0, 0.0, 3.0])
Y_REG = X @ W + 0.5 + 0.01 * R.standard_normal(240)
Y_BIN = (X[:, 0] + X[:, 1] > 0).astype(float)
Y_XOR = ((X[:, 0] > 0) ^ (X[:, 1] > 0)).astype(float)
Y_3 = np.digitize(X[:, 0] + X[:, 2], [-0.7, 0.7]).astype(float)
BLOBS = np.vstack([R.standard_normal((50, 2)) * 0.4 + c for c in ([0, 0], [4, 4], [0, 5])])
BLOB_Y = np.repeat([0, 1, 2], 50)


def test_every_name_of_the_reference_inventory_exists():
    names = """DecisionTreeClassifier DecisionTreeRegressor RandomForestClassifier RandomForestRegressor
    GradientBoostingClassifier GradientBoostingRegressor AdaBoostClassifier BaggingClassifier ExtraTreesClassifier
    VotingClassifier IsolationForest StackingRegressor StackingClassifier LinearMeta LogisticMeta XGBoostClassifier
    XGBoostRegressor LightGBMClassifier LinearRegression Ridge Lasso ElasticNet LogisticRegression SGDClassifier
    SGDRegressor RidgeClassifier HuberRegressor RANSACRegressor TheilSenRegressor QuantileRegressor
    PassiveAggressiveRegressor SVC SVR KernelRidge KernelPCA Nystrom KNeighborsClassifier KNeighborsRegressor GaussianNB
    MultinomialNB BernoulliNB ComplementNB BayesianRidge ARDRegression LinearDiscriminantAnalysis
    QuadraticDiscriminantAnalysis GaussianProcessRegressor GaussianProcessClassifier GaussianMixture
    BayesianGaussianMixture GaussianHMM LinearChainCRF Perceptron MLPClassifier MLPRegressor RBFNetwork RBFClassifier
    KMeans DBSCAN AgglomerativeClustering SpectralClustering MeanShift MiniBatchKMeans AffinityPropagation OPTICS BIRCH
    HDBSCAN PCA SVD NMF FactorAnalysis FastICA SparsePCA DictionaryLearning IncrementalPCA MiniBatchSparsePCA TSNE MDS
    Isomap LocallyLinearEmbedding LocalOutlierFactor OneClassSVM EllipticEnvelope VarianceThreshold SelectKBest RFE
    PolynomialFeatures FeatureHasher TargetEncoder OneHotEncoder SplineTransformer PowerTransformer QuantileTransformer
    StandardScaler MinMaxScaler Normalizer LabelEncoder RobustScaler MaxAbsScaler OrdinalEncoder KBinsDiscretizer
    Binarizer KFold StratifiedKFold LeaveOneOut TimeSeriesSplit RandomizedSearchCV GroupKFold RepeatedKFold
    StratifiedShuffleSplit BayesianOptimization RandomSearch GridSearch Hyperband BOHB IsotonicRegression PlattScaling
    CalibratedClassifier LabelPropagation LabelSpreading SelfTrainingClassifier OneVsRestClassifier OneVsOneClassifier
    OutputCodeClassifier ClassifierChain RandomOverSampler RandomUnderSampler SMOTE BorderlineSMOTE ADASYN
    SimpleExponentialSmoothing HoltLinear HoltWinters ARIMA MovingAverage EWMA SARIMA STLDecomposition WordTokenizer
    CharTokenizer BPETokenizer TfidfVectorizer Word2Vec ImageAugmentation ImageNormalization ImageResize ImageCrop
    RandomCrop ColorJitter DARTS ENAS ProgressiveNAS HardwareAwareNAS AutoML MetaLearner DistributedConfig
    DataParallelTrainer DistributedDataLoader GradientCompression RingAllReduce DistributedOptimizer GPUContext GPUTensor
    GPUOps GPUMemoryManager AutoMixedPrecision train_test_split cross_val_score parameter_grid accuracy_score
    f1_score roc_auc_score confusion_matrix r2_score silhouette_score adjusted_rand_score acf pacf adf_test""".split()
    missing = [n for n in names if not hasattr(ml, n)]
    assert not missing, missing


@pytest.mark.parametrize("make", [
    lambda: ml.LinearRegression(), lambda: ml.Ridge(0.1), lambda: ml.Lasso(0.01), lambda: ml.ElasticNet(0.01, 0.5),
    lambda: ml.SGDRegressor(), lambda: ml.HuberRegressor(), lambda: ml.RANSACRegressor(), lambda: ml.TheilSenRegressor(),
    lambda: ml.QuantileRegressor(0.5), lambda: ml.PassiveAggressiveRegressor(), lambda: ml.BayesianRidge(),
    lambda: ml.ARDRegression(), lambda: ml.KernelRidge().alpha(0.05), lambda: ml.SVR().c(10.0),
    lambda: ml.GaussianProcessRegressor().alpha(1e-2), lambda: ml.XGBoostRegressor(30).max_depth(3),
    lambda: ml.GradientBoostingRegressor(40), lambda: ml.RandomForestRegressor(15), lambda: ml.MLPRegressor([32]).max_iter(150).learning_rate(5e-3),
    lambda: ml.RBFNetwork(40)])
def test_regressors_fit_a_linear_target(make):
    m = make().fit(X, Y_REG)
    assert m.score(X, Y_REG) > 0.9


def test_linear_models_recover_the_coefficients():
    assert np.allclose(ml.LinearRegression().fit(X, Y_REG).coef_, W, atol=0.01)
    lasso = ml.Lasso(0.05).fit(X, Y_REG)
    assert abs(lasso.coef_[2]) < 1e-6 and abs(lasso.coef_[3]) < 1e-6          # sparsity on the null features
    _, std = ml.BayesianRidge().fit(X, Y_REG).predict_with_std(X[:5])
    assert (std.numpy() > 0).all()


@pytest.mark.parametrize("make", [
    lambda: ml.LogisticRegression(), lambda: ml.SGDClassifier(), lambda: ml.RidgeClassifier(), lambda: ml.Perceptron(),
    lambda: ml.SVC(), lambda: ml.KNeighborsClassifier(5), lambda: ml.GaussianNB(), lambda: ml.LinearDiscriminantAnalysis(),
    lambda: ml.QuadraticDiscriminantAnalysis(), lambda: ml.GaussianProcessClassifier(), lambda: ml.DecisionTreeClassifier().max_depth(5),
    lambda: ml.RandomForestClassifier(15), lambda: ml.ExtraTreesClassifier(15), lambda: ml.BaggingClassifier(8),
    lambda: ml.GradientBoostingClassifier(15), lambda: ml.XGBoostClassifier(15).max_depth(3), lambda: ml.LightGBMClassifier(15),
    lambda: ml.AdaBoostClassifier(25).max_depth(2), lambda: ml.MLPClassifier([32]).max_iter(100).learning_rate(5e-3),
    lambda: ml.RBFClassifier(30), lambda: ml.OneVsRestClassifier(), lambda: ml.OneVsOneClassifier()])
def test_classifiers_on_linearly_separable_and_three_class_data(make):
    assert make().fit(X, Y_BIN).score(X, Y_BIN) > 0.9
    assert make().fit(X, Y_3).score(X, Y_3) > 0.55      # the middle class is not linearly separable one-vs-rest


def test_trees_solve_xor_and_report_importances():
    t = ml.DecisionTreeClassifier().fit(X, Y_XOR)
    assert t.score(X, Y_XOR) > 0.95
    imp = ml.RandomForestClassifier(20).fit(X, Y_XOR).feature_importances().numpy()
    assert imp[:2].sum() > 0.5 and imp[:2].min() > imp[2:].max()
    vote = ml.VotingClassifier(ml.VotingType.Soft).add_estimator(ml.DecisionTreeClassifier()).add_estimator(ml.GaussianNB())
    assert vote.fit(X, Y_XOR).score(X, Y_XOR) > 0.9
    stack = ml.StackingClassifier().add_estimator(ml.DecisionTreeClassifier()).add_estimator(ml.GaussianNB())
    assert stack.fit(X, Y_XOR).score(X, Y_XOR) > 0.9


@pytest.mark.parametrize("make", [
    lambda: ml.KMeans(3), lambda: ml.MiniBatchKMeans(3), lambda: ml.DBSCAN(0.6, 4), lambda: ml.AgglomerativeClustering(3),
    lambda: ml.SpectralClustering(3), lambda: ml.MeanShift(), lambda: ml.AffinityPropagation().preference(-50),
    lambda: ml.BIRCH().threshold(0.8), lambda: ml.HDBSCAN(8), lambda: ml.GaussianMixture(3), lambda: ml.OPTICS(5)])
def test_clusterers_find_three_blobs(make):
    labels = make().fit_predict(BLOBS).numpy()
    assert ml.adjusted_rand_score(BLOB_Y, labels) > 0.8


def test_mixture_hmm_and_outliers():
    g = ml.GaussianMixture(3).fit(BLOBS)
    assert g.bic(BLOBS) < ml.GaussianMixture(1).fit(BLOBS).bic(BLOBS)
    seq = np.concatenate([R.normal(0, 1, 80), R.normal(6, 1, 80)])[:, None]
    path = ml.GaussianHMM(2, 1).fit(seq).predict(seq).numpy()
    assert (path[:80] == path[0]).mean() > 0.95 and (path[80:] == path[-1]).mean() > 0.95 and path[0] != path[-1]
    out = np.vstack((BLOBS, [[12.0, -12.0]]))
    assert ml.LocalOutlierFactor(10).fit_predict(out).numpy()[-1] == -1
    assert ml.IsolationForest(50).contamination(0.01).fit(out).predict(out).numpy()[-1] == -1
    assert ml.EllipticEnvelope().fit(BLOBS).predict(np.array([[30.0, -30.0]])).numpy()[0] == -1
    assert ml.OneClassSVM().fit(BLOBS).predict(np.array([[30.0, -30.0]])).numpy()[0] == -1


def test_decompositions_and_manifolds():
    Z = R.standard_normal((150, 3)) @ R.standard_normal((3, 8)) + 0.01 * R.standard_normal((150, 8))
    p = ml.PCA(3).fit(Z)
    assert p.explained_variance_ratio_.sum() > 0.999
    assert np.abs(p.inverse_transform(p.transform(Z)).numpy() - Z).max() < 0.1
    ip = ml.IncrementalPCA(3).batch_size(50).fit(Z)
    assert np.abs(np.abs((ip.components_ @ p.components_.T).diagonal()) - 1).max() < 1e-3
    assert ml.NMF(3).fit(np.abs(Z)).reconstruction_err_ < np.linalg.norm(np.abs(Z)) * 0.5
    S = np.stack([np.sin(np.linspace(0, 20, 400)), np.sign(np.cos(np.linspace(0, 31, 400)))], 1)
    rec = ml.FastICA(2).fit_transform(S @ np.array([[1, 0.5], [0.3, 1]])).numpy()
    assert (np.abs(np.corrcoef(rec.T, S.T)[:2, 2:]).max(1) > 0.95).all()
    for m in (ml.MDS(2), ml.Isomap(2), ml.LocallyLinearEmbedding(2).n_neighbors(10), ml.TSNE(2).n_iter(250).perplexity(20)):
        assert ml.silhouette_score(m.fit_transform(BLOBS).numpy(), BLOB_Y) > 0.5
    for m in (ml.SVD(3), ml.FactorAnalysis(3), ml.SparsePCA(2), ml.DictionaryLearning(4).alpha(0.1), ml.KernelPCA(2), ml.Nystrom(10)):
        assert m.fit_transform(Z).shape[0] == 150


def test_preprocessing_round_trips_and_selection():
    for sc in (ml.StandardScaler(), ml.MinMaxScaler(), ml.RobustScaler(), ml.MaxAbsScaler()):
        assert np.allclose(sc.inverse_transform(sc.fit_transform(X)).numpy(), X, atol=1e-5)
    assert np.allclose(ml.Normalizer("l2").transform(X).numpy().__pow__(2).sum(1), 1, atol=1e-5)
    cat = R.integers(0, 4, (50, 2)).astype(float)
    oh = ml.OneHotEncoder().fit(cat)
    assert np.array_equal(oh.inverse_transform(oh.transform(cat)).numpy(), cat)
    assert ml.PolynomialFeatures(2).fit_transform(X).shape == [240, 21]
    assert ml.SelectKBest(2, ml.ScoreFunction.FRegression).fit(X, Y_REG).get_support()[[1, 4]].all()
    assert ml.RFE(3).fit(X, Y_REG).get_support()[[0, 1, 4]].all()
    assert ml.KBinsDiscretizer(4).fit_transform(X).numpy().max() == 3
    assert abs(ml.PowerTransformer().fit_transform(np.exp(X)).numpy().mean()) < 1e-5
    assert ml.QuantileTransformer().fit_transform(X).numpy().min() >= 0


def test_metrics_known_values():
    y, p = np.array([0, 1, 1, 0, 1, 0.0]), np.array([0, 1, 0, 0, 1, 1.0])
    assert ml.accuracy_score(y, p) == pytest.approx(4 / 6)
    assert ml.f1_score(y, p) == pytest.approx(2 / 3)
    assert ml.roc_auc_score(y, [0.1, 0.9, 0.4, 0.2, 0.8, 0.6]) == pytest.approx(8 / 9)
    assert ml.matthews_corrcoef(y, p) == pytest.approx(1 / 3)
    assert ml.confusion_matrix(y, p).tolist() == [[2, 1], [1, 2]]
    assert ml.r2_score([1, 2, 3.0], [1, 2, 3.0]) == 1.0
    assert ml.adjusted_rand_score([0, 0, 1, 1], [1, 1, 0, 0]) == 1.0
    assert ml.normalized_mutual_info_score([0, 0, 1, 1], [1, 1, 0, 0]) == pytest.approx(1.0)
    assert ml.log_loss([1, 0], [0.9, 0.1]) == pytest.approx(-np.log(0.9))


def test_model_selection_and_search():
    assert sorted(np.concatenate([te for _, te in ml.KFold(4).split(X)])) == list(range(240))
    for tr, te in ml.StratifiedKFold(3).split(X, Y_BIN):
        assert abs(Y_BIN[te].mean() - Y_BIN.mean()) < 0.05
    assert ml.cross_val_score(ml.LogisticRegression(), X, Y_BIN, 3).mean() > 0.9
    gs = ml.model_selection.GridSearchCV(ml.Ridge(1.0), {"alpha": [0.01, 100.0]}).fit(X, Y_REG)
    assert gs.best_params_["alpha"] == 0.01
    sp = ml.ParameterSpace().add_float("x", -2, 2).add_float("y", -2, 2)
    best, val = ml.BayesianOptimization(sp, 25).optimize(lambda p: -(p["x"] - 1) ** 2 - (p["y"] + 0.5) ** 2)
    assert val > -0.1
    assert ml.Hyperband(sp, 9).optimize(lambda p, b: -(p["x"] - 1) ** 2)[1] > -1.0


def test_semi_supervised_calibration_resampling():
    ys = Y_BIN.copy()
    ys[40:] = -1
    assert (ml.LabelSpreading().gamma(0.5).fit(X, ys).transduction_ == Y_BIN).mean() > 0.8
    assert ml.SelfTrainingClassifier(ml.GaussianNB()).fit(X, ys).score(X, Y_BIN) > 0.85
    assert ml.CalibratedClassifier(ml.GaussianNB(), "isotonic").fit(X, Y_BIN).score(X, Y_BIN) > 0.9
    iso = ml.IsotonicRegression().fit(np.arange(6.0), np.array([1, 3, 2, 4, 6, 5.0]))
    assert np.all(np.diff(iso.predict(np.arange(6.0)).numpy()) >= 0)
    yi = (X[:, 0] > 1.2).astype(float)
    for s in (ml.RandomOverSampler(), ml.SMOTE(), ml.BorderlineSMOTE(), ml.ADASYN()):
        _, yr = s.fit_resample(X, yi)
        counts = np.bincount(yr.numpy().astype(int))
        assert counts[0] == counts[1]


def test_time_series_text_vision():
    t = np.arange(120)
    y = 10 + 0.1 * t + 3 * np.sin(2 * np.pi * t / 12)
    truth = 10 + 0.1 * np.arange(120, 126) + 3 * np.sin(2 * np.pi * np.arange(120, 126) / 12)
    assert np.abs(ml.HoltWinters(12).fit(y).forecast(6).numpy() - truth).mean() < 0.5
    assert np.abs(ml.SARIMA(1, 0, 0, 1, 1, 0, 12).fit(y).forecast(6).numpy() - truth).mean() < 0.5
    assert np.isfinite(ml.ARIMA(2, 1, 1).fit(y).forecast(6).numpy()).all()
    assert np.abs(ml.STLDecomposition(12).fit(y).resid_).mean() < 0.3
    assert ml.adf_test(R.standard_normal(200), max_lag=1)[1] < 0.05
    docs = ["the cat sat on the mat", "the dog sat on the log", "cats and dogs"]
    w = ml.WordTokenizer().fit(docs)
    assert w.decode(w.encode("the cat sat")) == "the cat sat"
    b = ml.BPETokenizer(40).fit(docs)
    assert b.decode(b.encode("the cat")) == "the cat"
    assert ml.TfidfVectorizer().fit_transform(docs).shape == [3, 10]
    img = R.random((3, 32, 32))
    assert ml.ImageResize(16, 16).transform(img).shape == [3, 16, 16]
    assert ml.RandomCrop(8, 8).transform(img).shape == [3, 8, 8]


def test_nas_automl_and_distributed_helpers():
    ev = lambda c: -abs(c.cost() - 20)  # noqa: E731
    assert ml.DARTS(3, 2).search(ev, 30)[1] > -10
    assert ml.ENAS(4).search(ev, 5)[1] > -15
    am = ml.AutoML(ml.AutoMLConfig(time_budget_s=20, models=[ml.ModelType.Linear, ml.ModelType.NaiveBayes])).fit(X, Y_BIN)
    assert am.best_model().score > 0.9 and len(am.leaderboard()) >= 2
    res = ml.RingAllReduce(3).all_reduce([[1, 2, 3, 4.0], [10, 20, 30, 40.0], [100, 200, 300, 400.0]])
    assert all(np.allclose(v.numpy(), [37, 74, 111, 148]) for v in res)
    gc = ml.GradientCompression(ml.CompressionMethod.TopK, 0.25)
    g = np.array([0.1, -5, 0.2, 3, 0.05, 0.01, 1, -0.3])
    assert np.count_nonzero(gc.decompress(gc.compress(g))) == 2
    assert ml.DistributedDataLoader(4, 3, 2).shard_bounds(20) == (12, 20)
    amp = ml.AutoMixedPrecision(init_scale=1024.0)
    assert amp.update(True) is False and amp.scale == 512.0
