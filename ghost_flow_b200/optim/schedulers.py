"""Learning-rate schedulers (ghostflow-optim/src/scheduler.rs:12-222). Like the reference's, each scheduler
owns its optimizer (``optimizer()`` / ``optimizer_mut()``); ``step()`` advances the schedule and writes the
new rate into the optimizer."""
from __future__ import annotations

import math


class _Scheduler:
    def __init__(self, optimizer):
        self._opt = optimizer
        self.base_lr = optimizer.get_lr()
        self.current_step = 0

    def optimizer(self):
        return self._opt

    optimizer_mut = optimizer

    def get_lr(self) -> float:
        return self._opt.get_lr()

    def _lr_at(self, step: int) -> float:
        raise NotImplementedError

    def step(self) -> float:
        self.current_step += 1
        lr = self._lr_at(self.current_step)
        self._opt.set_lr(lr)
        return lr

    def state_dict(self):
        return {k: v for k, v in self.__dict__.items() if k != "_opt"}

    def load_state_dict(self, sd):
        self.__dict__.update(sd)
        self._opt.set_lr(self._lr_at(self.current_step) if self.current_step else self.base_lr)


LRScheduler = _Scheduler     # the reference's trait name (ghostflow-optim/src/scheduler.rs:6-9): step() and get_lr()


class StepLR(_Scheduler):
    def __init__(self, optimizer, step_size: int, gamma: float = 0.1):
        super().__init__(optimizer)
        self.step_size, self.gamma = step_size, gamma

    def _lr_at(self, step):
        return self.base_lr * self.gamma ** (step // self.step_size)


class ExponentialLR(_Scheduler):
    def __init__(self, optimizer, gamma: float):
        super().__init__(optimizer)
        self.gamma = gamma

    def _lr_at(self, step):
        return self.base_lr * self.gamma ** step


class CosineAnnealingLR(_Scheduler):
    """Cosine from the base rate to ``eta_min`` with period ``t_max`` (the schedule restarts: ``t = step % t_max``)."""

    def __init__(self, optimizer, t_max: int, eta_min: float = 0.0):
        super().__init__(optimizer)
        self.t_max, self.eta_min = t_max, eta_min

    def _lr_at(self, step):
        t = step % self.t_max
        return self.eta_min + (self.base_lr - self.eta_min) * (1 + math.cos(math.pi * t / self.t_max)) / 2


class LinearWarmup(_Scheduler):
    """Linear ramp from ``start_factor * base`` to the base rate over ``warmup_steps``, then constant."""

    def __init__(self, optimizer, warmup_steps: int, start_factor: float = 0.0):
        super().__init__(optimizer)
        self.warmup_steps, self.start_factor = warmup_steps, start_factor

    def _lr_at(self, step):
        if step >= self.warmup_steps:
            return self.base_lr
        f = self.start_factor + (1 - self.start_factor) * step / max(1, self.warmup_steps)
        return self.base_lr * f


class WarmupCosine(_Scheduler):
    """Linear warm-up followed by one cosine decay to ``min_ratio * base`` (the usual LLM schedule)."""

    def __init__(self, optimizer, warmup_steps: int, total_steps: int, min_ratio: float = 0.1):
        super().__init__(optimizer)
        self.warmup_steps, self.total_steps, self.min_ratio = warmup_steps, total_steps, min_ratio

    def _lr_at(self, step):
        if step < self.warmup_steps:
            return self.base_lr * step / max(1, self.warmup_steps)
        p = min(1.0, (step - self.warmup_steps) / max(1, self.total_steps - self.warmup_steps))
        return self.base_lr * (self.min_ratio + (1 - self.min_ratio) * 0.5 * (1 + math.cos(math.pi * p)))


class ReduceLROnPlateau(_Scheduler):
    """Multiplies the rate by ``factor`` after ``patience`` calls of ``step_with_loss`` without improvement."""

    def __init__(self, optimizer, factor: float = 0.1, patience: int = 10, min_lr: float = 0.0,
                 threshold: float = 1e-4, mode: str = "min"):
        super().__init__(optimizer)
        self.factor, self.patience, self.min_lr, self.threshold, self.mode = factor, patience, min_lr, threshold, mode
        self.best = math.inf if mode == "min" else -math.inf
        self.bad = 0

    def step_with_loss(self, loss: float) -> float:
        loss = float(loss)
        better = loss < self.best - self.threshold if self.mode == "min" else loss > self.best + self.threshold
        if better:
            self.best, self.bad = loss, 0
        else:
            self.bad += 1
            if self.bad > self.patience:
                self._opt.set_lr(max(self.min_lr, self._opt.get_lr() * self.factor))
                self.bad = 0
        return self._opt.get_lr()

    def step(self, loss=None):
        return self.step_with_loss(loss if loss is not None else self.best)

    def _lr_at(self, step):
        return self._opt.get_lr()
