"""Validated tensor / variable helpers (src/nn/safe_ops.rs:13-263)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Sequence

import torch


@dataclass
class TensorStats:
    """Summary of a tensor's values (src/nn/safe_ops.rs:236-270); also indexable by field name."""
    min: float
    max: float
    mean: float
    variance: float
    count: int
    nan_count: int = 0
    inf_count: int = 0

    def std_dev(self) -> float:
        return math.sqrt(self.variance) if self.variance >= 0 else float("nan")

    def is_reasonable(self) -> bool:
        return not (math.isinf(self.min) or math.isinf(self.max) or math.isnan(self.mean) or math.isnan(self.variance)) \
            and self.variance >= 0

    def __getitem__(self, key: str):
        if key == "std":
            return self.std_dev()
        if key == "numel":
            return self.count
        return getattr(self, key)


class SafeOps:
    @staticmethod
    def create_variable(data: Sequence[float], shape: Sequence[int], requires_grad: bool = False) -> torch.Tensor:
        n = 1
        for s in shape:
            if s < 0:
                raise ValueError("negative dimension")
            n *= s
        if n != len(data):
            raise ValueError(f"shape {tuple(shape)} needs {n} values, got {len(data)}")
        t = torch.tensor(list(data), dtype=torch.float32).reshape(tuple(shape))
        SafeOps.validate_finite(t)
        return t.requires_grad_(requires_grad)

    @staticmethod
    def validate_finite(t: torch.Tensor) -> None:
        if not bool(torch.isfinite(t).all()):
            raise ValueError("tensor contains NaN or Inf")

    @staticmethod
    def is_finite(t: torch.Tensor) -> bool:
        return bool(torch.isfinite(t).all())

    @staticmethod
    def get_stats(t: torch.Tensor) -> TensorStats:
        if t.numel() == 0:
            raise ValueError("Empty tensor")
        f = t.detach().float()
        return TensorStats(float(f.min()), float(f.max()), float(f.mean()), float(f.var(unbiased=False)), f.numel(),
                           int(torch.isnan(f).sum()), int(torch.isinf(f).sum()))

    @staticmethod
    def reshape(t: torch.Tensor, shape: Sequence[int]) -> torch.Tensor:
        if int(torch.tensor(shape).prod()) != t.numel():
            raise ValueError(f"cannot reshape {tuple(t.shape)} to {tuple(shape)}")
        return t.reshape(tuple(shape))

    @staticmethod
    def apply_function(t: torch.Tensor, fn) -> torch.Tensor:
        out = fn(t)
        SafeOps.validate_finite(out)
        return out

    @staticmethod
    def relu(t: torch.Tensor) -> torch.Tensor:
        return torch.relu(t)
