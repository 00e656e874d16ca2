"""Validated tensor / variable helpers (src/nn/safe_ops.rs:13-263)."""
from __future__ import annotations

from typing import Dict, Sequence

import torch


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
    def get_stats(t: torch.Tensor) -> Dict[str, float]:
        f = t.detach().float()
        return {"mean": float(f.mean()), "std": float(f.std(unbiased=False)), "min": float(f.min()),
                "max": float(f.max()), "numel": f.numel(),
                "nan_count": int(torch.isnan(f).sum()), "inf_count": int(torch.isinf(f).sum())}

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
