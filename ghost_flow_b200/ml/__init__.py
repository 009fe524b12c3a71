"""Classical machine learning with the reference's estimator names (ghostflow-ml/src/lib.rs re-exports): an
sklearn-shaped API on :class:`ghost_flow_b200.Tensor`. Host code (numpy/scipy), deliberately off the GPU hot path.

Sub-modules: ``preprocessing`` (scalers, encoders, feature engineering/selection), ``metrics``, ``model_selection``
(splitters, search, Bayesian optimisation, Hyperband/BOHB), ``linear`` (linear/SGD/robust/Bayesian/kernel/SVM/
neighbours/naive Bayes/discriminant analysis/Gaussian processes), ``tree`` (trees, forests, boosting, stacking),
``cluster`` (clustering, mixtures, HMM, outlier detection), ``decomposition`` (PCA family, manifold learning),
``neural`` (MLP, RBF networks, CRF, calibration, semi-supervised, multi-class, re-sampling), ``timeseries``,
``text_vision``, ``automl`` (NAS, AutoML, ml-level distributed helpers, device façade).
"""
from . import (automl, cluster, decomposition, linear, metrics, model_selection, neural, preprocessing, text_vision,
               timeseries, tree)
from .automl import *  # noqa: F401,F403
from .cluster import *  # noqa: F401,F403
from .decomposition import *  # noqa: F401,F403
from .linear import *  # noqa: F401,F403
from .metrics import *  # noqa: F401,F403
from .model_selection import *  # noqa: F401,F403
from .neural import *  # noqa: F401,F403
from .preprocessing import *  # noqa: F401,F403
from .text_vision import *  # noqa: F401,F403
from .timeseries import *  # noqa: F401,F403
from .tree import *  # noqa: F401,F403

# two reference files define a class of the same name; the later module wins above, the other stays reachable
from .preprocessing import PolynomialFeatures, OneHotEncoder, TargetEncoder  # noqa: F401,E402

gpu = automl          # ghostflow-ml/src/gpu.rs names live in ``automl`` (GPUContext, GPUTensor, GPUOps, ...)
distributed = automl  # ghostflow-ml/src/distributed.rs names likewise (DataParallelTrainer, RingAllReduce, ...)

from . import options  # noqa: E402,F401
from .options import *  # noqa: E402,F401,F403
