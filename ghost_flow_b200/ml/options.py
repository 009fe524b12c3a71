"""Option enums of the reference's estimators (ghostflow-ml: preprocessing_extended.rs, calibration.rs, manifold.rs,
clustering_*.rs, linear_sgd.rs, model_selection_extended.rs, ...). The estimators of this package take their options
as strings through the fluent setters; every setter also accepts the enum member, whose value is that string. Only
options that an estimator here really distinguishes are listed."""
from __future__ import annotations

import enum


class _Opt(str, enum.Enum):
    def __str__(self):
        return self.value


class BinStrategy(_Opt):
    Uniform = "uniform"
    Quantile = "quantile"
    KMeans = "kmeans"


class BinEncode(_Opt):
    Ordinal = "ordinal"
    OneHot = "onehot"


class Norm(_Opt):
    L1 = "l1"
    L2 = "l2"
    Max = "max"


class CalibrationMethod(_Opt):
    Sigmoid = "sigmoid"
    Isotonic = "isotonic"


class LPKernel(_Opt):
    RBF = "rbf"
    KNN = "knn"


class PerceptronPenalty(_Opt):
    L1 = "l1"
    L2 = "l2"
    ElasticNet = "elasticnet"


class PowerMethod(_Opt):
    YeoJohnson = "yeo-johnson"
    BoxCox = "box-cox"


class SGDRegressorLoss(_Opt):
    SquaredError = "squared_error"
    Huber = "huber"
    EpsilonInsensitive = "epsilon_insensitive"


class Scoring(_Opt):
    Accuracy = "accuracy"
    F1 = "f1"
    Precision = "precision"
    Recall = "recall"
    R2 = "r2"
    NegMSE = "neg_mse"
    NegMAE = "neg_mae"


class SeasonalType(_Opt):
    Additive = "additive"
    Multiplicative = "multiplicative"


class TSNEMetric(_Opt):
    Euclidean = "euclidean"
    Cosine = "cosine"
    Manhattan = "manhattan"


OPTICSMetric = TSNEMetric


class SpectralAffinity(_Opt):
    RBF = "rbf"
    NearestNeighbors = "nearest_neighbors"


class MiniBatchInit(_Opt):
    Random = "random"
    KMeansPlusPlus = "k-means++"


class OutputDistribution(_Opt):
    Uniform = "uniform"
    Normal = "normal"


def option_value(v):
    """The string behind an option: enum members give their value, anything else is returned as it is."""
    return v.value if isinstance(v, enum.Enum) else v
