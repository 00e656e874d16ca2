"""Optimizer utilities: gradient clipping, convergence metrics, stability guards, a factory with
suggested hyper-parameters and the optimizer throughput benchmark (src/optim/utils.rs:10-671,
src/optim/benchmarks.rs:13-348)."""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional

import torch


def clip_grad_norm(parameters: Iterable[torch.Tensor], max_norm: float, norm_type: float = 2.0) -> float:
    ps = [p for p in parameters if p.grad is not None]
    if not ps:
        return 0.0
    return float(torch.nn.utils.clip_grad_norm_(ps, max_norm, norm_type))


def clip_grad_value(parameters: Iterable[torch.Tensor], clip_value: float) -> None:
    torch.nn.utils.clip_grad_value_([p for p in parameters if p.grad is not None], clip_value)


def grad_norm(parameters: Iterable[torch.Tensor], norm_type: float = 2.0) -> float:
    gs = [p.grad.detach().float().norm(norm_type) for p in parameters if p.grad is not None]
    return float(torch.stack(gs).norm(norm_type)) if gs else 0.0


@dataclass
class StabilityConfig:
    max_grad_norm: Optional[float] = None
    max_grad_value: Optional[float] = None
    skip_nonfinite: bool = True
    eps: float = 1e-8

    def apply(self, parameters: List[torch.Tensor]) -> bool:
        """Clip as configured; returns False if the step should be skipped (non-finite gradients)."""
        if self.skip_nonfinite:
            for p in parameters:
                if p.grad is not None and not bool(torch.isfinite(p.grad).all()):
                    return False
        if self.max_grad_value is not None:
            clip_grad_value(parameters, self.max_grad_value)
        if self.max_grad_norm is not None:
            clip_grad_norm(parameters, self.max_grad_norm)
        return True


@dataclass
class OptimizerMetrics:
    """Rolling loss / gradient-norm history with convergence detection."""
    window: int = 10
    tolerance: float = 1e-6
    losses: List[float] = field(default_factory=list)
    grad_norms: List[float] = field(default_factory=list)

    def record(self, loss: float, gnorm: float = 0.0) -> None:
        self.losses.append(float(loss))
        self.grad_norms.append(float(gnorm))

    def has_converged(self) -> bool:
        if len(self.losses) < self.window + 1:
            return False
        recent = self.losses[-self.window:]
        return max(recent) - min(recent) < self.tolerance

    def is_diverging(self) -> bool:
        return bool(self.losses) and (not math.isfinite(self.losses[-1]) or
                                      (len(self.losses) > self.window and self.losses[-1] > 10 * min(self.losses)))

    def improvement_rate(self) -> float:
        if len(self.losses) < 2:
            return 0.0
        n = min(self.window, len(self.losses) - 1)
        return (self.losses[-n - 1] - self.losses[-1]) / n


class OptimizerFactory:
    """Create optimizers by name and suggest starting hyper-parameters for a problem type."""

    @staticmethod
    def create(name: str, params, **kw):
        from . import optimizers as O
        table = {"sgd": O.SGD, "adam": O.Adam, "adamw": O.AdamW, "rmsprop": O.RMSprop, "adagrad": O.AdaGrad,
                 "nadam": O.NAdam, "radam": O.RAdam, "adamax": O.Adamax, "adabound": O.AdaBound, "lamb": O.LAMB,
                 "lbfgs": O.LBFGS}
        key = name.lower()
        if key not in table:
            raise ValueError(f"unknown optimizer '{name}'")
        return table[key](params, **kw)

    @staticmethod
    def suggest_parameters(model_type: str, dataset_size: int = 10000) -> Dict[str, object]:
        t = model_type.lower()
        if t in ("transformer", "nlp", "gpt", "bert", "llm"):
            return {"optimizer": "adamw", "lr": 6e-4 if dataset_size > 1e6 else 3e-4, "betas": (0.9, 0.95),
                    "weight_decay": 0.1, "warmup_steps": 2000}
        if t in ("cnn", "vision", "resnet"):
            return {"optimizer": "sgd", "lr": 0.1, "momentum": 0.9, "weight_decay": 1e-4, "nesterov": False}
        if t in ("rnn", "lstm", "gru"):
            return {"optimizer": "adam", "lr": 1e-3, "clip_grad_norm": 1.0}
        if t in ("large_batch", "lamb"):
            return {"optimizer": "lamb", "lr": 2e-3, "weight_decay": 0.01}
        return {"optimizer": "adam", "lr": 1e-3}


class OptimizerBenchmark:
    """Steps-per-second of optimizers on a synthetic parameter set — the measurement behind the
    reference's published Adamax / RAdam / NAdam numbers (README.md:298-302)."""

    def __init__(self, n_params: int = 10, param_size: int = 1000, steps: int = 1000, device="cpu"):
        self.n_params, self.param_size, self.steps, self.device = n_params, param_size, steps, device

    def run(self, name: str, **kw) -> Dict[str, float]:
        ps = [torch.nn.Parameter(torch.randn(self.param_size, device=self.device)) for _ in range(self.n_params)]
        for p in ps:
            p.grad = torch.randn_like(p)
        opt = OptimizerFactory.create(name, ps, **kw)
        for _ in range(10):
            opt.step()
        if torch.device(self.device).type == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(self.steps):
            opt.step()
        if torch.device(self.device).type == "cuda":
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        return {"optimizer": name, "steps_per_s": self.steps / dt, "us_per_step": dt / self.steps * 1e6}

    def run_adam_comparison(self) -> List[Dict[str, float]]:
        return [self.run(n) for n in ("adam", "adamw", "adamax", "radam", "nadam")]
