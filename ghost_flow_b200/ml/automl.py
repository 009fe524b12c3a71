"""Architecture search, AutoML, the ml-level distributed helpers and device façade (ghostflow-ml/src/nas.rs,
automl.rs, distributed.rs, gpu.rs)."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field

import numpy as np
import torch

from ._base import Estimator, out, rng_of, softmax, to_np


# ----------------------------------------------------------------------------- NAS
class Operation(enum.Enum):
    Conv3x3 = "conv3x3"
    Conv5x5 = "conv5x5"
    SepConv3x3 = "sep_conv3x3"
    DilConv3x3 = "dil_conv3x3"
    MaxPool3x3 = "max_pool3x3"
    AvgPool3x3 = "avg_pool3x3"
    SkipConnect = "skip"
    Zero = "zero"

    def cost(self) -> float:
        """Relative multiply-accumulate cost per position and channel pair."""
        return {"conv3x3": 9.0, "conv5x5": 25.0, "sep_conv3x3": 2.0, "dil_conv3x3": 2.0, "max_pool3x3": 0.1,
                "avg_pool3x3": 0.1, "skip": 0.0, "zero": 0.0}[self.value]

    def build(self, channels: int) -> torch.nn.Module:
        nn, c = torch.nn, channels
        v = self.value
        if v == "conv3x3":
            return nn.Sequential(nn.Conv2d(c, c, 3, padding=1, bias=False), nn.BatchNorm2d(c), nn.ReLU())
        if v == "conv5x5":
            return nn.Sequential(nn.Conv2d(c, c, 5, padding=2, bias=False), nn.BatchNorm2d(c), nn.ReLU())
        if v == "sep_conv3x3":
            return nn.Sequential(nn.Conv2d(c, c, 3, padding=1, groups=c, bias=False), nn.Conv2d(c, c, 1, bias=False),
                                 nn.BatchNorm2d(c), nn.ReLU())
        if v == "dil_conv3x3":
            return nn.Sequential(nn.Conv2d(c, c, 3, padding=2, dilation=2, groups=c, bias=False),
                                 nn.Conv2d(c, c, 1, bias=False), nn.BatchNorm2d(c), nn.ReLU())
        if v == "max_pool3x3":
            return nn.MaxPool2d(3, 1, 1)
        if v == "avg_pool3x3":
            return nn.AvgPool2d(3, 1, 1)
        if v == "skip":
            return nn.Identity()
        return _Zero()


class _Zero(torch.nn.Module):
    def forward(self, x):
        return x * 0


@dataclass
class Cell:
    """A DAG: node i (>= 2) sums ``ops[(j, i)]`` applied to earlier nodes j; the output concatenates/averages nodes."""
    num_nodes: int
    edges: dict = field(default_factory=dict)        # (src, dst) -> Operation

    def cost(self):
        return sum(op.cost() for op in self.edges.values())

    def build(self, channels):
        return _CellModule(self, channels)


class _CellModule(torch.nn.Module):
    def __init__(self, cell, channels):
        super().__init__()
        self.cell = cell
        self.ops = torch.nn.ModuleDict({f"{s}_{d}": op.build(channels) for (s, d), op in cell.edges.items()})

    def forward(self, x):
        nodes = [x, x]
        for d in range(2, self.cell.num_nodes + 2):
            ins = [self.ops[f"{s}_{d}"](nodes[s]) for (s, dd) in self.cell.edges if dd == d]
            nodes.append(sum(ins) if ins else torch.zeros_like(x))
        return sum(nodes[2:]) / max(1, self.cell.num_nodes)


_CANDIDATES = [o for o in Operation]


class DARTS(Estimator):
    """Continuous relaxation: one softmax over operations per edge; ``derive`` keeps the strongest non-zero
    operation on the two strongest incoming edges of every node."""
    _params = ("arch_learning_rate", "seed")

    def __init__(self, num_nodes=4, num_cells=8):
        self._num_nodes, self._num_cells, self._arch_learning_rate, self._seed = num_nodes, num_cells, 3e-3, 0
        r = rng_of(self._seed)
        self.edges = [(s, d) for d in range(2, num_nodes + 2) for s in range(d)]
        self.alphas = {e: 1e-3 * r.standard_normal(len(_CANDIDATES)) for e in self.edges}

    def architecture_weights(self):
        return {e: softmax(a[None])[0] for e, a in self.alphas.items()}

    def update(self, grads: dict):
        """One gradient step on the architecture parameters (``grads``: edge -> d loss / d alpha)."""
        for e, g in grads.items():
            self.alphas[e] -= self._arch_learning_rate * np.asarray(g)

    def search(self, evaluate, steps=50, eps=0.5):
        """Zeroth-order search when only a black-box score is available: perturb alphas, keep improvements."""
        r = rng_of(self._seed)
        best = evaluate(self.derive())
        for _ in range(steps):
            e = self.edges[int(r.integers(len(self.edges)))]
            old = self.alphas[e].copy()
            self.alphas[e] = old + eps * r.standard_normal(len(old))
            s = evaluate(self.derive())
            if s > best:
                best = s
            else:
                self.alphas[e] = old
        return self.derive(), best

    def derive(self) -> Cell:
        w = self.architecture_weights()
        zero = _CANDIDATES.index(Operation.Zero)
        cell = Cell(self._num_nodes)
        for d in range(2, self._num_nodes + 2):
            cands = []
            for s in range(d):
                p = w[(s, d)].copy()
                p[zero] = -1
                cands.append((p.max(), s, _CANDIDATES[int(p.argmax())]))
            for _, s, op in sorted(cands, key=lambda t: -t[0])[:2]:
                cell.edges[(s, d)] = op
        return cell


class ENAS(Estimator):
    """Controller with per-decision categorical logits trained by REINFORCE with a moving-average baseline."""
    _params = ("num_nodes", "learning_rate", "seed")

    def __init__(self, num_samples=10):
        self._num_samples, self._num_nodes, self._learning_rate, self._seed = num_samples, 4, 0.1, 0
        self._rng = rng_of(self._seed)
        self.logits_src = {d: np.zeros(d) for d in range(2, self._num_nodes + 2)}
        self.logits_op = {d: np.zeros(len(_CANDIDATES)) for d in range(2, self._num_nodes + 2)}
        self.baseline = None

    def sample(self):
        cell, trace = Cell(self._num_nodes), []
        for d in range(2, self._num_nodes + 2):
            ps, po = softmax(self.logits_src[d][None])[0], softmax(self.logits_op[d][None])[0]
            s, o = int(self._rng.choice(len(ps), p=ps)), int(self._rng.choice(len(po), p=po))
            cell.edges[(s, d)] = _CANDIDATES[o]
            trace.append((d, s, o, ps, po))
        return cell, trace

    def search(self, evaluate, iterations=20):
        best = (None, -np.inf)
        for _ in range(iterations):
            batch = [self.sample() for _ in range(self._num_samples)]
            rewards = [float(evaluate(c)) for c, _ in batch]
            self.baseline = np.mean(rewards) if self.baseline is None else 0.9 * self.baseline + 0.1 * np.mean(rewards)
            for (c, trace), rwd in zip(batch, rewards):
                if rwd > best[1]:
                    best = (c, rwd)
                adv = rwd - self.baseline
                for d, s, o, ps, po in trace:
                    gs, go = -ps, -po
                    gs[s] += 1
                    go[o] += 1
                    self.logits_src[d] += self._learning_rate * adv * gs
                    self.logits_op[d] += self._learning_rate * adv * go
        return best


class ProgressiveNAS(Estimator):
    """Grows cells one node at a time, keeping the ``beam`` best partial cells within the complexity budget."""
    _params = ("beam", "max_nodes")

    def __init__(self, complexity_budget=100.0):
        self._complexity_budget, self._beam, self._max_nodes = complexity_budget, 4, 4

    def search(self, evaluate):
        beam = [Cell(0)]
        best = (None, -np.inf)
        for n in range(1, self._max_nodes + 1):
            cands = []
            for c in beam:
                d = n + 1
                for s in range(d):
                    for op in _CANDIDATES:
                        if op is Operation.Zero:
                            continue
                        nc = Cell(n, dict(c.edges))
                        nc.edges[(s, d)] = op
                        if nc.cost() <= self._complexity_budget:
                            cands.append(nc)
            scored = sorted(((float(evaluate(c)), i, c) for i, c in enumerate(cands)), key=lambda t: -t[0])
            if not scored:
                break
            beam = [c for _, _, c in scored[:self._beam]]
            if scored[0][0] > best[1]:
                best = (scored[0][2], scored[0][0])
        return best


class HardwareAwareNAS(Estimator):
    """Random search with the score penalised by the latency estimate exceeding the target:
    score = accuracy * min(1, target / latency) ** penalty."""
    _params = ("penalty", "num_nodes", "seed", "channels", "resolution")

    _THROUGHPUT = {"cpu": 5e10, "gpu": 2e13, "b200": 1e15, "mobile": 5e9, "edge": 1e9}

    def __init__(self, target_hardware="b200", target_latency=1.0):
        self._target_hardware, self._target_latency = str(target_hardware).lower(), target_latency
        self._penalty, self._num_nodes, self._seed, self._channels, self._resolution = 1.0, 4, 0, 64, 32

    def estimate_latency(self, cell: Cell) -> float:
        """Milliseconds for one cell on the target: MACs / sustained throughput of that class of device."""
        macs = cell.cost() * self._channels ** 2 * self._resolution ** 2
        return 1e3 * 2 * macs / self._THROUGHPUT.get(self._target_hardware, 1e12)

    def search(self, evaluate, iterations=50):
        r = rng_of(self._seed)
        best = (None, -np.inf)
        for _ in range(iterations):
            c = Cell(self._num_nodes)
            for d in range(2, self._num_nodes + 2):
                for s in r.choice(d, min(2, d), replace=False):
                    c.edges[(int(s), d)] = _CANDIDATES[int(r.integers(len(_CANDIDATES) - 1))]
            lat = self.estimate_latency(c)
            score = float(evaluate(c)) * min(1.0, self._target_latency / max(lat, 1e-12)) ** self._penalty
            if score > best[1]:
                best = (c, score)
        return best


# ----------------------------------------------------------------------------- AutoML
class TaskType(enum.Enum):
    Classification = "classification"
    Regression = "regression"


class OptimizationMetric(enum.Enum):
    Accuracy = "accuracy"
    F1 = "f1"
    RocAuc = "roc_auc"
    R2 = "r2"
    MSE = "mse"


class ModelType(enum.Enum):
    Linear = "linear"
    Tree = "tree"
    RandomForest = "random_forest"
    GradientBoosting = "gradient_boosting"
    KNN = "knn"
    NaiveBayes = "naive_bayes"
    SVM = "svm"
    MLP = "mlp"


@dataclass
class AutoMLConfig:
    task: TaskType = TaskType.Classification
    metric: OptimizationMetric | None = None
    time_budget_s: float = 60.0
    cv_folds: int = 3
    models: list | None = None
    seed: int = 0


@dataclass
class TrainedModel:
    model_type: ModelType
    params: dict
    score: float
    fit_time_s: float
    estimator: object = None


def _candidates(task, seed):
    from . import linear as L, neural as N, tree as T
    if task is TaskType.Classification:
        return [(ModelType.Linear, L.LogisticRegression, [{}, {"c": 0.1}, {"c": 10.0}]),
                (ModelType.NaiveBayes, L.GaussianNB, [{}]),
                (ModelType.KNN, lambda: L.KNeighborsClassifier(5), [{}, {"n_neighbors": 3}, {"n_neighbors": 11}]),
                (ModelType.Tree, T.DecisionTreeClassifier, [{"max_depth": 4}, {"max_depth": 8}]),
                (ModelType.RandomForest, lambda: T.RandomForestClassifier(30), [{"max_depth": 6}, {"max_depth": None}]),
                (ModelType.GradientBoosting, lambda: T.XGBoostClassifier(30), [{"max_depth": 3}, {"max_depth": 5, "learning_rate": 0.1}]),
                (ModelType.SVM, L.SVC, [{"c": 1.0}]),
                (ModelType.MLP, lambda: N.MLPClassifier([32]), [{"max_iter": 60, "learning_rate": 5e-3}])]
    return [(ModelType.Linear, lambda: L.Ridge(1.0), [{"alpha": 0.01}, {"alpha": 1.0}, {"alpha": 10.0}]),
            (ModelType.KNN, lambda: L.KNeighborsRegressor(5), [{}, {"n_neighbors": 3}]),
            (ModelType.Tree, T.DecisionTreeRegressor, [{"max_depth": 4}, {"max_depth": 8}]),
            (ModelType.RandomForest, lambda: T.RandomForestRegressor(30), [{"max_depth": 6}, {"max_depth": None}]),
            (ModelType.GradientBoosting, lambda: T.XGBoostRegressor(40), [{"max_depth": 3}, {"max_depth": 5, "learning_rate": 0.1}]),
            (ModelType.SVM, L.SVR, [{"c": 10.0}]),
            (ModelType.MLP, lambda: N.MLPRegressor([32]), [{"max_iter": 80, "learning_rate": 5e-3}])]


class MetaLearner:
    """Meta-features of a dataset and a warm-start ordering of model families from them."""

    def extract_meta_features(self, X, y) -> dict:
        X, y = to_np(X), to_np(y)
        n, d = X.shape
        cl = np.unique(y)
        corr = np.nan_to_num(np.corrcoef(X.T)) if d > 1 else np.ones((1, 1))
        return {"n_samples": n, "n_features": d, "n_classes": len(cl) if len(cl) < max(20, n // 10) else 0,
                "class_imbalance": float(np.bincount(np.unique(y, return_inverse=True)[1]).max() / n) if len(cl) < n // 2 else 0.0,
                "mean_abs_correlation": float(np.abs(corr[np.triu_indices(d, 1)]).mean()) if d > 1 else 0.0,
                "mean_skewness": float(np.abs(((X - X.mean(0)) ** 3).mean(0) / (X.std(0) ** 3 + 1e-12)).mean()),
                "dimensionality": d / n}

    def recommend(self, meta: dict) -> list:
        order = [ModelType.GradientBoosting, ModelType.RandomForest, ModelType.Linear, ModelType.KNN, ModelType.Tree,
                 ModelType.SVM, ModelType.NaiveBayes, ModelType.MLP]
        if meta["dimensionality"] > 0.5 or meta["n_samples"] < 100:
            order.remove(ModelType.Linear)
            order.insert(0, ModelType.Linear)
        if meta["n_samples"] > 5000:
            order.remove(ModelType.SVM)
            order.append(ModelType.SVM)
        return order


class AutoML:
    def __init__(self, config: AutoMLConfig | None = None):
        self.config = config or AutoMLConfig()
        self.leaderboard_: list[TrainedModel] = []

    def _metric(self):
        from . import metrics as M
        m = self.config.metric or (OptimizationMetric.Accuracy if self.config.task is TaskType.Classification
                                   else OptimizationMetric.R2)
        return {"accuracy": M.accuracy_score, "f1": lambda a, b: M.f1_score(a, b, "macro"), "roc_auc": M.roc_auc_score,
                "r2": M.r2_score, "mse": lambda a, b: -M.mean_squared_error(a, b)}[m.value]

    def fit(self, X, y):
        from .model_selection import KFold, StratifiedKFold, cross_val_score
        start = time.monotonic()
        order = MetaLearner().recommend(MetaLearner().extract_meta_features(X, y))
        cands = sorted(_candidates(self.config.task, self.config.seed), key=lambda c: order.index(c[0]))
        if self.config.models:
            cands = [c for c in cands if c[0] in self.config.models]
        cv = (StratifiedKFold if self.config.task is TaskType.Classification else KFold)(self.config.cv_folds, True, self.config.seed)
        metric = self._metric()
        for mt, ctor, grid in cands:
            for params in grid:
                if time.monotonic() - start > self.config.time_budget_s and self.leaderboard_:
                    break
                t0 = time.monotonic()
                try:
                    s = float(cross_val_score(ctor().set(**params), X, y, cv, metric).mean())
                except Exception:
                    continue
                self.leaderboard_.append(TrainedModel(mt, params, s, time.monotonic() - t0))
        self.leaderboard_.sort(key=lambda m: -m.score)
        top = self.leaderboard_[0]
        ctor = next(c[1] for c in cands if c[0] is top.model_type)
        top.estimator = ctor().set(**top.params).fit(X, y)
        return self

    def leaderboard(self):
        return list(self.leaderboard_)

    def best_model(self) -> TrainedModel:
        return self.leaderboard_[0]

    def predict(self, X):
        return self.best_model().estimator.predict(X)


# ----------------------------------------------------------------------------- distributed helpers (ml level)
class CommunicationBackend(enum.Enum):
    Threads = "threads"
    Processes = "processes"
    MPI = "mpi"
    NCCL = "nccl"


class DistributedStrategy(enum.Enum):
    DataParallel = "data_parallel"
    ModelParallel = "model_parallel"


@dataclass
class DistributedConfig:
    world_size: int = 1
    rank: int = 0
    backend: CommunicationBackend = CommunicationBackend.Processes
    strategy: DistributedStrategy = DistributedStrategy.DataParallel


def _dist():
    import torch.distributed as dist
    return dist if dist.is_available() and dist.is_initialized() else None


class DataParallelTrainer:
    """Gradient averaging over the ranks of the current process group (all-reduce); without one, over the
    worker gradients passed in (the reference's thread mode)."""

    def __init__(self, config: DistributedConfig):
        self.config = config

    def all_reduce(self, grads):
        """``grads``: list of per-layer arrays (this rank's) -> mean over ranks."""
        d = _dist()
        res = []
        for g in grads:
            t = torch.as_tensor(to_np(g, np.float32)).clone()
            if d is not None:
                d.all_reduce(t)
                t /= d.get_world_size()
            res.append(t.numpy())
        return res

    def sync_gradients(self, worker_grads):
        """``worker_grads``: [workers][layers] arrays held by one process -> their mean, then all-reduced."""
        mean = [np.mean([to_np(w[l]) for w in worker_grads], 0) for l in range(len(worker_grads[0]))]
        return self.all_reduce(mean)

    sync_gradients_threads = sync_gradients_processes = sync_gradients_mpi = sync_gradients

    def broadcast_parameters(self, params, src=0):
        d = _dist()
        res = []
        for p in params:
            t = torch.as_tensor(to_np(p, np.float32)).clone()
            if d is not None:
                d.broadcast(t, src)
            res.append(t.numpy())
        return res


class DistributedDataLoader:
    """Rank-contiguous shards (the last rank takes the remainder), batches of ``batch_size`` inside the shard."""

    def __init__(self, batch_size, world_size=1, rank=0):
        self.batch_size, self.world_size, self.rank = batch_size, world_size, rank

    def shard_bounds(self, n):
        per = n // self.world_size
        lo = self.rank * per
        return lo, n if self.rank == self.world_size - 1 else lo + per

    def batches(self, X, y=None):
        Xn = to_np(X)
        lo, hi = self.shard_bounds(len(Xn))
        for s in range(lo, hi, self.batch_size):
            e = min(hi, s + self.batch_size)
            yield (out(Xn[s:e]), out(to_np(y)[s:e])) if y is not None else out(Xn[s:e])

    def num_batches(self, n):
        lo, hi = self.shard_bounds(n)
        return -(-(hi - lo) // self.batch_size)


class CompressionMethod(enum.Enum):
    TopK = "topk"
    RandomK = "randomk"
    Quantization = "quantization"
    Null = "none"


class GradientCompression:
    """Sparsification (top-k / random-k with the kept fraction ``ratio``) or 8-bit linear quantisation; ``compress``
    returns what would cross the wire, ``decompress`` rebuilds a dense gradient. The residual that was not sent
    is kept and added to the next gradient (error feedback)."""

    def __init__(self, method=CompressionMethod.TopK, ratio=0.1, seed=0):
        self.method, self.ratio, self._rng, self._residual = method, ratio, rng_of(seed), {}

    def compress(self, grad, key=0):
        g = to_np(grad).ravel() + self._residual.get(key, 0.0)
        m = getattr(self.method, "value", self.method)
        k = max(1, int(len(g) * self.ratio))
        if m == "topk":
            idx = np.argpartition(np.abs(g), -k)[-k:]
            payload = ("sparse", idx, g[idx], len(g))
        elif m == "randomk":
            idx = self._rng.choice(len(g), k, replace=False)
            payload = ("sparse", idx, g[idx] / self.ratio * (k / len(g)) / (k / len(g)), len(g))
        elif m == "quantization":
            lo, hi = g.min(), g.max()
            q = np.round((g - lo) / max(hi - lo, 1e-12) * 255).astype(np.uint8)
            payload = ("q8", q, (lo, hi), len(g))
        else:
            payload = ("dense", g.copy(), None, len(g))
        self._residual[key] = g - self.decompress(payload).ravel()
        return payload

    def decompress(self, payload, shape=None):
        kind, a, b, n = payload
        if kind == "sparse":
            d = np.zeros(n)
            d[a] = b
        elif kind == "q8":
            d = a.astype(np.float64) / 255 * (b[1] - b[0]) + b[0]
        else:
            d = a
        return d.reshape(shape) if shape is not None else d

    def compression_ratio(self, payload):
        kind, a, b, n = payload
        sent = {"sparse": len(a) * 8 if kind == "sparse" else 0, "q8": n + 8, "dense": n * 4}[kind]
        return n * 4 / max(1, sent)


class RingAllReduce:
    """Reduce-scatter then all-gather around a ring of ``world_size`` participants. ``all_reduce(chunks)`` takes
    every participant's vector ([world, n]) and returns the element-wise mean each of them ends up with, following
    the ring schedule step by step (the reference's version replaces a layer by the mean of its own elements)."""

    def __init__(self, world_size, rank=0):
        self.world_size, self.rank = world_size, rank

    def all_reduce(self, data, average=True):
        D = np.array([to_np(d).ravel() for d in data], dtype=np.float64)
        w, n = D.shape
        assert w == self.world_size
        bounds = np.linspace(0, n, w + 1).astype(int)
        seg = lambda i: slice(bounds[i % w], bounds[i % w + 1])  # noqa: E731
        for step in range(w - 1):                    # reduce-scatter
            sends = [(r, (r - step) % w, D[r, seg(r - step)].copy()) for r in range(w)]
            for r, s, buf in sends:
                D[(r + 1) % w, seg(s)] += buf
        for step in range(w - 1):                    # all-gather
            sends = [(r, (r + 1 - step) % w, D[r, seg(r + 1 - step)].copy()) for r in range(w)]
            for r, s, buf in sends:
                D[(r + 1) % w, seg(s)] = buf
        if average:
            D /= w
        return [out(d) for d in D]


class DistributedOptimizer:
    """Wraps an optimizer ``step(params, grads)`` so that gradients are averaged over ranks (optionally compressed)
    before it runs."""

    def __init__(self, optimizer, config: DistributedConfig, compression: GradientCompression | None = None):
        self.optimizer, self.config, self.compression = optimizer, config, compression
        self.trainer = DataParallelTrainer(config)

    def step(self, params, grads):
        if self.compression is not None:
            grads = [self.compression.decompress(self.compression.compress(g, i), np.shape(to_np(g))) for i, g in enumerate(grads)]
        grads = self.trainer.all_reduce(grads)
        return self.optimizer.step(params, grads) if hasattr(self.optimizer, "step") else self.optimizer(params, grads)


# ----------------------------------------------------------------------------- device façade (ml level)
class DeviceType(enum.Enum):
    CPU = "cpu"
    CUDA = "cuda"
    OpenCL = "opencl"
    Metal = "metal"
    Vulkan = "vulkan"


@dataclass
class DeviceInfo:
    device_type: DeviceType
    name: str
    total_memory: int
    compute_capability: tuple


class GPUContext:
    def __init__(self, device=0):
        self.device_index = device
        self.device = torch.device("cuda", device) if self.is_cuda_available() else torch.device("cpu")

    @staticmethod
    def is_cuda_available() -> bool:
        return torch.cuda.is_available()

    def info(self) -> DeviceInfo:
        if self.device.type == "cuda":
            p = torch.cuda.get_device_properties(self.device)
            return DeviceInfo(DeviceType.CUDA, p.name, p.total_memory, (p.major, p.minor))
        return DeviceInfo(DeviceType.CPU, "cpu", 0, (0, 0))

    def synchronize(self):
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)


class GPUTensor:
    """Data that really lives on the context's device (the reference keeps a host Vec)."""

    def __init__(self, data, dims, context: GPUContext):
        self.context = context
        self.t = torch.as_tensor(to_np(data, np.float32)).reshape(tuple(dims)).to(context.device)

    @property
    def dims(self):
        return tuple(self.t.shape)

    def to_host(self):
        return out(self.t.detach().cpu().numpy())


class GPUOps:
    def __init__(self, context: GPUContext):
        self.context = context

    def _wrap(self, t):
        g = GPUTensor.__new__(GPUTensor)
        g.context, g.t = self.context, t
        return g

    def matmul(self, a: GPUTensor, b: GPUTensor):
        from ..ops.gemm import matmul
        return self._wrap(matmul(a.t, b.t))

    def conv2d(self, x: GPUTensor, w: GPUTensor, stride=1, padding=0):
        return self._wrap(torch.nn.functional.conv2d(x.t, w.t, stride=stride, padding=padding))

    def batch_norm(self, x: GPUTensor, mean, var, gamma=None, beta=None, eps=1e-5):
        sh = (1, -1, 1, 1)
        m, v = (torch.as_tensor(to_np(a, np.float32), device=x.t.device).view(sh) for a in (mean, var))
        y = (x.t - m) / torch.sqrt(v + eps)
        if gamma is not None:
            y = y * torch.as_tensor(to_np(gamma, np.float32), device=x.t.device).view(sh)
        if beta is not None:
            y = y + torch.as_tensor(to_np(beta, np.float32), device=x.t.device).view(sh)
        return self._wrap(y)

    def max_pool2d(self, x: GPUTensor, kernel=2, stride=None):
        return self._wrap(torch.nn.functional.max_pool2d(x.t, kernel, stride or kernel))

    def relu(self, x: GPUTensor):
        return self._wrap(torch.relu(x.t))


class GPUMemoryManager:
    def __init__(self, context: GPUContext):
        self.context = context
        self.allocations: dict[int, int] = {}
        self._peak = 0

    def allocate(self, nbytes: int):
        t = torch.empty(nbytes, dtype=torch.uint8, device=self.context.device)
        self.allocations[t.data_ptr()] = nbytes
        self._peak = max(self._peak, self.allocated_bytes())
        return t

    def allocated_memory(self) -> int:
        """Bytes currently handed out (ghostflow-ml/src/gpu.rs:451-462)."""
        return self.allocated_bytes()

    def peak_memory(self) -> int:
        return self._peak

    def free(self, t):
        self.allocations.pop(t.data_ptr(), None)

    def allocated_bytes(self):
        return sum(self.allocations.values())

    def memory_info(self):
        if self.context.device.type == "cuda":
            return torch.cuda.mem_get_info(self.context.device)
        return (0, 0)


class AutoMixedPrecision:
    """Dynamic loss scaling: halve on overflow, double after ``growth_interval`` clean steps."""

    def __init__(self, init_scale=65536.0, growth_factor=2.0, backoff_factor=0.5, growth_interval=2000):
        self.scale, self.growth_factor, self.backoff_factor, self.growth_interval = init_scale, growth_factor, backoff_factor, growth_interval
        self._good = 0
        self.enabled = True

    def scale_loss(self, loss):
        return loss * self.scale if self.enabled else loss

    def unscale(self, grads):
        return [to_np(g) / self.scale for g in grads]

    def has_overflow(self, grads) -> bool:
        return any(not np.isfinite(to_np(g)).all() for g in grads)

    def update(self, overflow: bool) -> bool:
        """Returns True if the optimizer step should be applied."""
        if overflow:
            self.scale *= self.backoff_factor
            self._good = 0
            return False
        self._good += 1
        if self._good >= self.growth_interval:
            self.scale *= self.growth_factor
            self._good = 0
        return True
