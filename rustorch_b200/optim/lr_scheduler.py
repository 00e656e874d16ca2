"""Learning-rate schedulers (src/optim/lr_scheduler.rs:9-579).

Each scheduler owns a reference to its optimizer (any object with ``param_groups`` or with
``learning_rate() / set_learning_rate()``, so the fused flat optimizers work too) and exposes
``step()``, ``get_lr()``, ``get_last_lr()``, ``state_dict()``.
"""
from __future__ import annotations

import enum
import math
from typing import List, Optional, Sequence


def _get_lr(opt) -> float:
    if hasattr(opt, "learning_rate") and callable(opt.learning_rate):
        return float(opt.learning_rate())
    return float(opt.param_groups[0]["lr"])


def _set_lr(opt, lr: float) -> None:
    if hasattr(opt, "set_learning_rate"):
        opt.set_learning_rate(lr)
    else:
        for g in opt.param_groups:
            g["lr"] = lr


class LRScheduler:
    def __init__(self, optimizer):
        self.optimizer = optimizer
        self.base_lr = _get_lr(optimizer)
        self.last_epoch = 0
        self._last_lr = self.base_lr

    def compute_lr(self, epoch: int) -> float:
        raise NotImplementedError

    def step(self) -> float:
        self.last_epoch += 1
        self._last_lr = self.compute_lr(self.last_epoch)
        _set_lr(self.optimizer, self._last_lr)
        return self._last_lr

    def get_lr(self) -> float:
        return self._last_lr

    def get_last_lr(self) -> List[float]:
        return [self._last_lr]

    def state_dict(self) -> dict:
        return {k: v for k, v in self.__dict__.items() if k != "optimizer" and not callable(v)}

    def load_state_dict(self, sd: dict) -> None:
        self.__dict__.update(sd)
        _set_lr(self.optimizer, self._last_lr)


class StepLR(LRScheduler):
    """``lr = base * gamma ** (epoch // step_size)`` (:37-66)."""

    def __init__(self, optimizer, step_size: int, gamma: float = 0.1):
        super().__init__(optimizer)
        self.step_size, self.gamma = step_size, gamma

    def compute_lr(self, epoch):
        return self.base_lr * self.gamma ** (epoch // self.step_size)


class ExponentialLR(LRScheduler):
    def __init__(self, optimizer, gamma: float):
        super().__init__(optimizer)
        self.gamma = gamma

    def compute_lr(self, epoch):
        return self.base_lr * self.gamma ** epoch


class CosineAnnealingLR(LRScheduler):
    """``eta_min + (base - eta_min) * (1 + cos(pi * epoch / t_max)) / 2`` (:129-140)."""

    def __init__(self, optimizer, t_max: int, eta_min: float = 0.0):
        super().__init__(optimizer)
        self.t_max, self.eta_min = t_max, eta_min

    def compute_lr(self, epoch):
        return self.eta_min + (self.base_lr - self.eta_min) * (1 + math.cos(math.pi * epoch / self.t_max)) / 2


class MultiStepLR(LRScheduler):
    def __init__(self, optimizer, milestones: Sequence[int], gamma: float = 0.1):
        super().__init__(optimizer)
        self.milestones, self.gamma = sorted(milestones), gamma

    def compute_lr(self, epoch):
        return self.base_lr * self.gamma ** sum(1 for m in self.milestones if epoch >= m)


class WarmupScheduler(LRScheduler):
    """Linear ramp from the optimizer's lr to ``target_lr`` over ``warmup_epochs`` (:371)."""

    def __init__(self, optimizer, target_lr: float, warmup_epochs: int):
        super().__init__(optimizer)
        self.target_lr, self.warmup_epochs = target_lr, max(1, warmup_epochs)

    def compute_lr(self, epoch):
        if epoch >= self.warmup_epochs:
            return self.target_lr
        return self.base_lr + (self.target_lr - self.base_lr) * epoch / self.warmup_epochs


class AnnealStrategy(enum.Enum):
    """Cosine or linear annealing of ``OneCycleLR`` (src/optim/lr_scheduler.rs:428-436)."""

    COS = "cos"
    LINEAR = "linear"


class OneCycleLR(LRScheduler):
    """``(opt, max_lr, total_steps, pct_start=0.3, anneal=Cos)``: ramp from max_lr/25 to max_lr, then anneal
    to max_lr/25/1e4 (:428-436)."""

    def __init__(self, optimizer, max_lr: float, total_steps: int, pct_start: float = 0.3,
                 anneal_strategy: AnnealStrategy = AnnealStrategy.COS, div_factor: float = 25.0,
                 final_div_factor: float = 1e4):
        super().__init__(optimizer)
        self.max_lr, self.total_steps, self.pct_start = max_lr, total_steps, pct_start
        self.anneal = anneal_strategy
        self.initial_lr = max_lr / div_factor
        self.min_lr = self.initial_lr / final_div_factor
        self._last_lr = self.initial_lr
        _set_lr(optimizer, self.initial_lr)

    def _interp(self, a, b, t):
        if self.anneal is AnnealStrategy.COS or str(self.anneal).lower().endswith("cos"):
            return b + (a - b) * (1 + math.cos(math.pi * t)) / 2
        return a + (b - a) * t

    def compute_lr(self, epoch):
        up = max(1.0, self.pct_start * self.total_steps)
        if epoch <= up:
            return self._interp(self.initial_lr, self.max_lr, epoch / up)
        t = min(1.0, (epoch - up) / max(1.0, self.total_steps - up))
        return self._interp(self.max_lr, self.min_lr, t)


class PolynomialLR(LRScheduler):
    """``(opt, total_epochs, power=1, min_lr=0)`` (:497-520)."""

    def __init__(self, optimizer, total_epochs: int, power: float = 1.0, min_lr: float = 0.0):
        super().__init__(optimizer)
        self.total_epochs, self.power, self.min_lr = total_epochs, power, min_lr

    def compute_lr(self, epoch):
        t = min(epoch, self.total_epochs) / self.total_epochs
        return (self.base_lr - self.min_lr) * (1 - t) ** self.power + self.min_lr


class PlateauMode(enum.Enum):
    """Whether ``ReduceLROnPlateau`` watches a metric that should fall or rise."""

    MIN = "min"
    MAX = "max"


class ThresholdMode(enum.Enum):
    """Relative or absolute improvement threshold of ``ReduceLROnPlateau``."""

    REL = "rel"
    ABS = "abs"


class ReduceLROnPlateau(LRScheduler):
    """``(opt, mode, factor=0.1, patience=10, threshold=1e-4, threshold_mode=Rel, cooldown=0, min_lr=0, eps=1e-8)``
    with ``step_with_metric(value)`` (:222-240)."""

    def __init__(self, optimizer, mode: PlateauMode = PlateauMode.MIN, factor: float = 0.1, patience: int = 10,
                 threshold: float = 1e-4, threshold_mode: ThresholdMode = ThresholdMode.REL, cooldown: int = 0,
                 min_lr: float = 0.0, eps: float = 1e-8):
        super().__init__(optimizer)
        self.mode = PlateauMode(mode) if not isinstance(mode, PlateauMode) else mode
        self.threshold_mode = ThresholdMode(threshold_mode) if not isinstance(threshold_mode, ThresholdMode) else threshold_mode
        self.factor, self.patience, self.threshold = factor, patience, threshold
        self.cooldown, self.min_lr, self.eps = cooldown, min_lr, eps
        self.best: Optional[float] = None
        self.num_bad, self.cooldown_counter = 0, 0

    def _better(self, v: float) -> bool:
        if self.best is None:
            return True
        if self.mode is PlateauMode.MIN:
            thr = self.best * (1 - self.threshold) if self.threshold_mode is ThresholdMode.REL else self.best - self.threshold
            return v < thr
        thr = self.best * (1 + self.threshold) if self.threshold_mode is ThresholdMode.REL else self.best + self.threshold
        return v > thr

    def step_with_metric(self, value: float) -> float:
        self.last_epoch += 1
        if self._better(value):
            self.best, self.num_bad = value, 0
        else:
            self.num_bad += 1
        if self.cooldown_counter > 0:
            self.cooldown_counter -= 1
            self.num_bad = 0
        if self.num_bad > self.patience:
            new = max(self._last_lr * self.factor, self.min_lr)
            if self._last_lr - new > self.eps:
                self._last_lr = new
                _set_lr(self.optimizer, new)
            self.cooldown_counter, self.num_bad = self.cooldown, 0
        return self._last_lr

    def step(self, metric: Optional[float] = None) -> float:
        if metric is None:
            raise ValueError("ReduceLROnPlateau.step needs the monitored metric")
        return self.step_with_metric(metric)
