"""Federated learning, differential privacy and adversarial robustness utilities with the reference's names.

* ``FederatedClient / FederatedServer / AggregationStrategy / SecureAggregation`` (ghostflow-nn/src/federated.rs:84-380)
* ``DPConfig / PrivacyAccountant / DPSGDOptimizer / PATEEnsemble / LocalDP`` (differential_privacy.rs:17-330)
* ``AttackConfig / AdversarialAttack(fgsm, pgd, cw, deepfool) / AdversarialTrainer / RandomizedSmoothing``
  (adversarial.rs:15-380). Unlike the reference's attacks, which estimate gradients without autograd, these
  differentiate through the model.
"""
from __future__ import annotations

import copy
import enum
import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F


# =========================================================================== federated
class AggregationStrategy(enum.Enum):
    FedAvg = "fedavg"
    FedProx = "fedprox"
    FedAdam = "fedadam"
    Median = "median"
    TrimmedMean = "trimmed_mean"


class FederatedClient:
    def __init__(self, client_id: int, model, num_samples: int = 1, lr: float = 0.01, mu: float = 0.0):
        self.client_id, self.model, self.num_samples, self.lr, self.mu = client_id, model, num_samples, lr, mu

    def set_weights(self, state: dict):
        self.model.load_state_dict(state)

    def get_weights(self) -> dict:
        return {k: v.detach().clone() for k, v in self.model.state_dict().items()}

    def local_train(self, batches, loss_fn, epochs: int = 1) -> dict:
        """SGD on the client's data; with ``mu > 0`` adds the FedProx proximal term. Returns the weight delta."""
        start = self.get_weights()
        params = [p for p in self.model.parameters() if p.requires_grad]
        names = [n for n, p in self.model.named_parameters() if p.requires_grad]
        for _ in range(epochs):
            for x, y in batches:
                loss = loss_fn(self.model(x), y)
                if self.mu > 0:
                    loss = loss + 0.5 * self.mu * sum((p - start[n]).pow(2).sum() for n, p in zip(names, params))
                grads = torch.autograd.grad(loss, params)
                with torch.no_grad():
                    for p, g in zip(params, grads):
                        p -= self.lr * g
        end = self.get_weights()
        return {k: end[k] - start[k] for k in end if end[k].is_floating_point()}


class SecureAggregation:
    """Pairwise additive masks that cancel in the sum: the server only ever sees masked updates."""

    def __init__(self, num_clients: int, seed: int = 0):
        self.num_clients, self.seed = num_clients, seed

    def mask(self, client_id: int, update: dict) -> dict:
        out = {}
        for k, v in update.items():
            m = torch.zeros_like(v)
            for other in range(self.num_clients):
                if other == client_id:
                    continue
                lo, hi = min(client_id, other), max(client_id, other)
                g = torch.Generator().manual_seed(hash((self.seed, lo, hi, k)) & 0x7FFFFFFF)
                r = torch.randn(v.shape, generator=g).to(v.dtype)
                m += r if client_id == lo else -r
            out[k] = v + m
        return out


class FederatedServer:
    def __init__(self, model, strategy: AggregationStrategy = AggregationStrategy.FedAvg, server_lr: float = 1.0,
                 client_fraction: float = 1.0, trim_ratio: float = 0.1):
        self.model, self.strategy, self.server_lr = model, strategy, server_lr
        self.client_fraction, self.trim_ratio = client_fraction, trim_ratio
        self.round = 0
        self._m, self._v = {}, {}

    def select_clients(self, clients, generator=None):
        k = max(1, int(round(self.client_fraction * len(clients))))
        idx = torch.randperm(len(clients), generator=generator)[:k].tolist()
        return [clients[i] for i in idx]

    def aggregate(self, updates: list, weights: list | None = None) -> dict:
        """Combines client deltas and applies them to the global model."""
        n = len(updates)
        w = torch.tensor(weights or [1.0] * n, dtype=torch.float32)
        w = w / w.sum()
        agg = {}
        for k in updates[0]:
            stack = torch.stack([u[k].float() for u in updates])
            if self.strategy == AggregationStrategy.Median:
                agg[k] = stack.median(0).values
            elif self.strategy == AggregationStrategy.TrimmedMean:
                t = int(self.trim_ratio * n)
                s = stack.sort(0).values
                agg[k] = s[t:n - t].mean(0) if n - 2 * t > 0 else s.mean(0)
            else:
                agg[k] = (stack * w.view(-1, *[1] * (stack.dim() - 1))).sum(0)
        state = self.model.state_dict()
        self.round += 1
        for k, d in agg.items():
            if self.strategy == AggregationStrategy.FedAdam:
                m = self._m.setdefault(k, torch.zeros_like(d))
                v = self._v.setdefault(k, torch.zeros_like(d))
                m.mul_(0.9).add_(d, alpha=0.1)
                v.mul_(0.99).addcmul_(d, d, value=0.01)
                d = m / (v.sqrt() + 1e-3)
            state[k] = state[k] + (self.server_lr * d).to(state[k].dtype)
        self.model.load_state_dict(state)
        return agg

    def run_round(self, clients, batches_of, loss_fn, secure: SecureAggregation | None = None):
        chosen = self.select_clients(clients)
        global_w = {k: v.clone() for k, v in self.model.state_dict().items()}
        ups, ws = [], []
        for c in chosen:
            c.set_weights(global_w)
            u = c.local_train(batches_of(c), loss_fn)
            ups.append(secure.mask(c.client_id, u) if secure and len(chosen) == secure.num_clients else u)
            ws.append(c.num_samples)
        if secure and len(chosen) == secure.num_clients:
            ws = None  # masks only cancel in the unweighted sum
        return self.aggregate(ups, ws)


# =========================================================================== differential privacy
@dataclass
class DPConfig:
    epsilon: float = 1.0
    delta: float = 1e-5
    max_grad_norm: float = 1.0
    noise_multiplier: float = 1.1
    batch_size: int = 256
    dataset_size: int = 60000


class PrivacyAccountant:
    """Moments-style bound: eps(T) ~= q * sqrt(T * 2 ln(1/delta)) / sigma (strong composition of subsampled
    Gaussian mechanisms)."""

    def __init__(self, config: DPConfig):
        self.config = config
        self.steps = 0

    def step(self):
        self.steps += 1

    def get_epsilon(self) -> float:
        c = self.config
        q = c.batch_size / c.dataset_size
        return q * math.sqrt(max(self.steps, 0) * 2.0 * math.log(1.0 / c.delta)) / c.noise_multiplier

    def is_budget_exhausted(self) -> bool:
        return self.get_epsilon() >= self.config.epsilon

    def remaining_budget(self) -> float:
        return max(0.0, self.config.epsilon - self.get_epsilon())


class DPSGDOptimizer:
    """Per-sample clipping + Gaussian noise around any optimizer (``process_gradients`` then ``step``)."""

    def __init__(self, optimizer, config: DPConfig | None = None, generator=None):
        self.optimizer, self.config = optimizer, config or DPConfig()
        self.accountant = PrivacyAccountant(self.config)
        self.generator = generator

    def clip_gradients(self, per_sample_grads: list):
        """per_sample_grads: list over parameters of ``[B, ...]`` tensors. Returns clipped copies."""
        B = per_sample_grads[0].shape[0]
        norms = torch.sqrt(sum(g.reshape(B, -1).float().pow(2).sum(1) for g in per_sample_grads))
        scale = (self.config.max_grad_norm / (norms + 1e-6)).clamp(max=1.0)
        return [g * scale.view(B, *[1] * (g.dim() - 1)).to(g.dtype) for g in per_sample_grads]

    def add_noise(self, summed: list):
        std = self.config.noise_multiplier * self.config.max_grad_norm
        return [g + torch.randn(g.shape, generator=self.generator, device=g.device if self.generator is None else "cpu"
                                ).to(g.device, g.dtype) * std for g in summed]

    def process_gradients(self, per_sample_grads: list):
        B = per_sample_grads[0].shape[0]
        clipped = self.clip_gradients(per_sample_grads)
        noisy = self.add_noise([g.sum(0) for g in clipped])
        return [g / B for g in noisy]

    def step(self, per_sample_grads: list | None = None):
        if per_sample_grads is not None:
            for p, g in zip(self.optimizer.parameters(), self.process_gradients(per_sample_grads)):
                p.grad = g.to(p.dtype)
        self.optimizer.step()
        self.accountant.step()

    def should_stop(self) -> bool:
        return self.accountant.is_budget_exhausted()


class PATEEnsemble:
    """Noisy-argmax aggregation of teacher votes."""

    def __init__(self, num_teachers: int, num_classes: int, noise_scale: float = 1.0, generator=None):
        self.num_teachers, self.num_classes, self.noise_scale, self.generator = num_teachers, num_classes, noise_scale, generator

    def aggregate(self, teacher_preds: torch.Tensor) -> torch.Tensor:
        """teacher_preds ``[teachers, samples]`` of class ids -> noisy majority labels ``[samples]``."""
        votes = F.one_hot(teacher_preds.long(), self.num_classes).sum(0).float()
        u = torch.rand(votes.shape, generator=self.generator).clamp(1e-9, 1 - 1e-9) - 0.5
        lap = -self.noise_scale * torch.sign(u) * torch.log1p(-2 * u.abs())
        return (votes + lap).argmax(-1)


class LocalDP:
    """Randomised response / Laplace mechanism applied on the client."""

    def __init__(self, epsilon: float, generator=None):
        self.epsilon, self.generator = epsilon, generator

    def randomized_response(self, bits: torch.Tensor) -> torch.Tensor:
        p = math.exp(self.epsilon) / (math.exp(self.epsilon) + 1)
        keep = torch.rand(bits.shape, generator=self.generator) < p
        return torch.where(keep, bits, 1 - bits)

    def laplace(self, x: torch.Tensor, sensitivity: float = 1.0) -> torch.Tensor:
        u = torch.rand(x.shape, generator=self.generator).clamp(1e-9, 1 - 1e-9) - 0.5
        return x - (sensitivity / self.epsilon) * torch.sign(u) * torch.log1p(-2 * u.abs())


# =========================================================================== adversarial
class AttackType(enum.Enum):
    FGSM = "fgsm"
    PGD = "pgd"
    CW = "cw"
    DeepFool = "deepfool"


@dataclass
class AttackConfig:
    attack_type: AttackType = AttackType.PGD
    epsilon: float = 0.3
    num_iterations: int = 40
    step_size: float = 0.01
    random_init: bool = True
    clip_min: float = 0.0
    clip_max: float = 1.0


class AdversarialAttack:
    def __init__(self, config: AttackConfig | None = None):
        self.config = config or AttackConfig()

    def _grad(self, model, x, y):
        x = x.detach().clone().requires_grad_(True)
        loss = F.cross_entropy(model(x).float(), y.long())
        return torch.autograd.grad(loss, x)[0]

    def fgsm(self, model, x, y):
        c = self.config
        return (x + c.epsilon * self._grad(model, x, y).sign()).clamp(c.clip_min, c.clip_max).detach()

    def pgd(self, model, x, y):
        c = self.config
        adv = x.clone()
        if c.random_init:
            adv = (adv + torch.empty_like(adv).uniform_(-c.epsilon, c.epsilon)).clamp(c.clip_min, c.clip_max)
        for _ in range(c.num_iterations):
            adv = adv + c.step_size * self._grad(model, adv, y).sign()
            adv = torch.min(torch.max(adv, x - c.epsilon), x + c.epsilon).clamp(c.clip_min, c.clip_max)
        return adv.detach()

    def cw(self, model, x, y, confidence: float = 0.0, c_const: float = 1.0, lr: float = 0.01):
        cfg = self.config
        w = torch.atanh((2 * (x - cfg.clip_min) / (cfg.clip_max - cfg.clip_min) - 1).clamp(-0.999, 0.999))
        w = w.detach().requires_grad_(True)
        opt = torch.optim.Adam([w], lr=lr)
        for _ in range(cfg.num_iterations):
            adv = (torch.tanh(w) + 1) / 2 * (cfg.clip_max - cfg.clip_min) + cfg.clip_min
            logits = model(adv).float()
            real = logits.gather(1, y.long()[:, None]).squeeze(1)
            other = logits.masked_fill(F.one_hot(y.long(), logits.shape[1]).bool(), float("-inf")).amax(1)
            loss = ((adv - x).flatten(1).pow(2).sum(1) + c_const * (real - other + confidence).clamp(min=0)).sum()
            opt.zero_grad()
            loss.backward()
            opt.step()
        return ((torch.tanh(w) + 1) / 2 * (cfg.clip_max - cfg.clip_min) + cfg.clip_min).detach()

    def deepfool(self, model, x, y, overshoot: float = 0.02):
        cfg = self.config
        adv = x.clone()
        for _ in range(cfg.num_iterations):
            a = adv.detach().clone().requires_grad_(True)
            logits = model(a).float()
            if bool((logits.argmax(1) != y).all()):
                break
            real = logits.gather(1, y.long()[:, None]).squeeze(1)
            best = None
            for k in range(logits.shape[1]):
                diff = logits[:, k] - real
                g = torch.autograd.grad(diff.sum(), a, retain_graph=True)[0]
                dist = diff.abs() / g.flatten(1).norm(dim=1).clamp(min=1e-8)
                dist = torch.where(y == k, torch.full_like(dist, float("inf")), dist)
                step = (dist + 1e-4)[:, *[None] * (x.dim() - 1)] * g / g.flatten(1).norm(dim=1).clamp(min=1e-8)[
                    :, *[None] * (x.dim() - 1)]
                if best is None:
                    best = (dist, step)
                else:
                    m = dist < best[0]
                    best = (torch.where(m, dist, best[0]), torch.where(m[:, *[None] * (x.dim() - 1)], step, best[1]))
            still = (logits.argmax(1) == y)[:, *[None] * (x.dim() - 1)]
            adv = torch.where(still, adv + (1 + overshoot) * best[1], adv).clamp(cfg.clip_min, cfg.clip_max)
        return adv.detach()

    def generate(self, model, x, y):
        return {AttackType.FGSM: self.fgsm, AttackType.PGD: self.pgd, AttackType.CW: self.cw,
                AttackType.DeepFool: self.deepfool}[self.config.attack_type](model, x, y)


@dataclass
class AdversarialTrainingConfig:
    attack: AttackConfig = None
    adversarial_ratio: float = 0.5
    label_smoothing: float = 0.1


class AdversarialTrainer:
    def __init__(self, model, optimizer, config: AdversarialTrainingConfig | None = None):
        self.model, self.optimizer = model, optimizer
        self.config = config or AdversarialTrainingConfig()
        self.attack = AdversarialAttack(self.config.attack or AttackConfig(num_iterations=5))

    def train_step(self, x, y) -> float:
        n_adv = int(self.config.adversarial_ratio * x.shape[0])
        if n_adv:
            x = torch.cat((self.attack.generate(self.model, x[:n_adv], y[:n_adv]), x[n_adv:]))
        loss = F.cross_entropy(self.model(x).float(), y.long(), label_smoothing=self.config.label_smoothing)
        self.optimizer.zero_grad()
        loss.backward()
        self.optimizer.step()
        return float(loss)


class RandomizedSmoothing:
    def __init__(self, model, sigma: float = 0.25, num_samples: int = 100, generator=None):
        self.model, self.sigma, self.num_samples, self.generator = model, sigma, num_samples, generator

    @torch.no_grad()
    def _counts(self, x, num_classes):
        counts = torch.zeros(x.shape[0], num_classes)
        for _ in range(self.num_samples):
            noise = torch.randn(x.shape, generator=self.generator).to(x.device, x.dtype) * self.sigma
            pred = self.model(x + noise).argmax(1).cpu()
            counts[torch.arange(x.shape[0]), pred] += 1
        return counts

    def predict(self, x, num_classes: int):
        return self._counts(x, num_classes).argmax(1)

    def certify(self, x, num_classes: int):
        """(predicted class, certified L2 radius sigma * Phi^-1(p_lower)); radius 0 when abstaining."""
        counts = self._counts(x, num_classes)
        top = counts.argmax(1)
        p = (counts.max(1).values / self.num_samples).clamp(max=1 - 1e-6)
        p_low = (p - 1.96 * torch.sqrt(p * (1 - p) / self.num_samples)).clamp(min=0.0)
        radius = torch.where(p_low > 0.5, self.sigma * torch.special.ndtri(p_low.double()).float(),
                             torch.zeros_like(p_low))
        return top, radius


class DifferentialPrivacy:
    """Clip-and-noise for federated updates (ghostflow-nn/src/federated.rs:311-380): every client update is clipped
    to ``clip_norm`` in global L2 norm and Gaussian noise of standard deviation ``noise_multiplier * clip_norm`` is
    added to the aggregate."""

    def __init__(self, clip_norm: float = 1.0, noise_multiplier: float = 1.0, seed: int = 0):
        self.clip_norm, self.noise_multiplier = clip_norm, noise_multiplier
        self._gen = torch.Generator().manual_seed(seed)

    def clip_update(self, update: dict) -> dict:
        total = torch.sqrt(sum((v.float() ** 2).sum() for v in update.values()))
        scale = min(1.0, self.clip_norm / max(float(total), 1e-12))
        return {k: v * scale for k, v in update.items()}

    def add_noise(self, aggregate: dict, num_clients: int = 1) -> dict:
        std = self.noise_multiplier * self.clip_norm / max(1, num_clients)
        return {k: v + torch.randn(v.shape, generator=self._gen).to(v.device, v.dtype) * std for k, v in aggregate.items()}

    def privatize(self, updates: list) -> dict:
        clipped = [self.clip_update(u) for u in updates]
        mean = {k: sum(u[k] for u in clipped) / len(clipped) for k in clipped[0]}
        return self.add_noise(mean, len(clipped))
