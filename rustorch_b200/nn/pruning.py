"""Weight pruning: magnitude / random / structured masks with schedules (src/nn/pruning.rs:30-591)."""
from __future__ import annotations

import enum
from typing import Dict, Iterable, Optional, Tuple

import torch
import torch.nn as nn


class PruningMethod(enum.Enum):
    MAGNITUDE = "magnitude"
    RANDOM = "random"
    STRUCTURED = "structured"  # whole output rows/channels by L2 norm


class PruningSchedule(enum.Enum):
    ONE_SHOT = "one_shot"
    GRADUAL = "gradual"          # linear ramp to the target sparsity
    POLYNOMIAL = "polynomial"    # cubic ramp (Zhu & Gupta)


class Pruner:
    def __init__(self, method: PruningMethod = PruningMethod.MAGNITUDE, sparsity: float = 0.5,
                 schedule: PruningSchedule = PruningSchedule.ONE_SHOT, total_steps: int = 1, seed: int = 0):
        if not 0.0 <= sparsity < 1.0:
            raise ValueError("sparsity must be in [0, 1)")
        self.method, self.target, self.schedule, self.total_steps = method, sparsity, schedule, max(1, total_steps)
        self.step_count = 0
        self.masks: Dict[str, torch.Tensor] = {}
        self._gen = torch.Generator().manual_seed(seed)

    def current_sparsity(self) -> float:
        if self.schedule is PruningSchedule.ONE_SHOT:
            return self.target
        t = min(1.0, self.step_count / self.total_steps)
        if self.schedule is PruningSchedule.GRADUAL:
            return self.target * t
        return self.target * (1.0 - (1.0 - t) ** 3)

    def compute_mask(self, w: torch.Tensor, sparsity: Optional[float] = None) -> torch.Tensor:
        s = self.current_sparsity() if sparsity is None else sparsity
        if s <= 0:
            return torch.ones_like(w, dtype=torch.bool)
        if self.method is PruningMethod.RANDOM:
            r = torch.rand(w.shape, generator=self._gen).to(w.device)
            return r >= s
        if self.method is PruningMethod.STRUCTURED and w.dim() >= 2:
            norms = w.detach().float().flatten(1).norm(dim=1)
            k = int(s * norms.numel())
            if k == 0:
                return torch.ones_like(w, dtype=torch.bool)
            thr = norms.kthvalue(k).values
            keep = norms > thr
            return keep.view(-1, *([1] * (w.dim() - 1))).expand_as(w).clone()
        flat = w.detach().abs().float().flatten()
        k = int(s * flat.numel())
        if k == 0:
            return torch.ones_like(w, dtype=torch.bool)
        thr = flat.kthvalue(k).values
        return w.detach().abs().float() > thr

    def prune(self, named_parameters: Iterable[Tuple[str, nn.Parameter]], only_weights: bool = True) -> Dict[str, float]:
        """Update masks for the current schedule step and zero the pruned weights in place."""
        self.step_count += 1
        out = {}
        for name, p in named_parameters:
            if only_weights and p.dim() < 2:
                continue
            mask = self.compute_mask(p.data)
            if name in self.masks:
                mask &= self.masks[name]      # once pruned, stays pruned
            self.masks[name] = mask
            with torch.no_grad():
                p.mul_(mask.to(p.dtype))
            out[name] = 1.0 - float(mask.float().mean())
        return out

    def apply_masks(self, named_parameters) -> None:
        """Re-apply stored masks (call after every optimizer step)."""
        with torch.no_grad():
            for name, p in named_parameters:
                m = self.masks.get(name)
                if m is not None:
                    p.mul_(m.to(p.dtype))

    def sparsity_report(self) -> Dict[str, float]:
        return {k: 1.0 - float(m.float().mean()) for k, m in self.masks.items()}
