"""Weight pruning: importance criteria, mask structures (unstructured, output channels, input filters, n:m blocks),
sparsity schedules, lottery-ticket rewinding and a module wrapper (src/nn/pruning.rs:30-640).

Masks are computed with tensor operations on the device that holds the weights (one ``kthvalue`` / ``topk`` per
tensor), not with host loops.  The gradient and Taylor criteria use the parameter's ``.grad`` when it is there
(the reference substitutes the weight magnitude, src/nn/pruning.rs:252-261); without a gradient they fall back to the
same substitutes.  The n:m block structure (2:4 in particular) is the pattern the sparse tensor-core path wants.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn


class PruningMethod(enum.Enum):
    """Importance criterion of the pruner (src/nn/pruning.rs:30-47); ``MAGNITUDE`` is ``L1_NORM``."""

    L1_NORM = "l1"               # |w|
    L2_NORM = "l2"               # w^2
    RANDOM = "random"
    GRADIENT = "gradient"        # |dL/dw|  (|w| without a gradient)
    TAYLOR = "taylor"            # |w * dL/dw|  (w^2 without a gradient)
    STRUCTURED = "structured"    # whole output rows / channels by L2 norm (shorthand for L2 + CHANNEL structure)
    MAGNITUDE = "l1"             # alias of L1_NORM


class PruningStructure:
    """Which groups of weights share one decision (src/nn/pruning.rs:51-73)."""

    def __init__(self, kind: str, n: int = 0, m: int = 0):
        if kind not in ("unstructured", "channel", "filter", "block"):
            raise ValueError(f"unknown pruning structure {kind!r}")
        if kind == "block" and not 0 < n <= m:
            raise ValueError("n:m sparsity needs 0 < n <= m")
        self.kind, self.n, self.m = kind, int(n), int(m)

    @classmethod
    def block(cls, n: int, m: int) -> "PruningStructure":
        """Keep the ``n`` most important weights of every ``m`` consecutive ones."""
        return cls("block", n, m)

    def __eq__(self, other):
        return isinstance(other, PruningStructure) and (self.kind, self.n, self.m) == (other.kind, other.n, other.m)

    def __hash__(self):
        return hash((self.kind, self.n, self.m))

    def __repr__(self):
        return f"PruningStructure.block({self.n}, {self.m})" if self.kind == "block" else f"PruningStructure.{self.kind.upper()}"


PruningStructure.UNSTRUCTURED = PruningStructure("unstructured")
PruningStructure.CHANNEL = PruningStructure("channel")      # output channels (dim 0)
PruningStructure.FILTER = PruningStructure("filter")        # input channels (dim 1)


class PruningSchedule:
    """Sparsity as a function of the epoch counter (src/nn/pruning.rs:76-113, 393-439).

    ``ONE_SHOT`` gives the target at once.  ``linear`` / ``polynomial`` / ``exponential`` are zero before
    ``start_epoch``, the target from ``end_epoch`` on, and ``target * f(progress)`` in between with ``f`` the identity,
    ``progress ** power`` or ``1 - exp(-5 progress)``.  ``GRADUAL`` and ``POLYNOMIAL`` are step-counted forms that take
    their length from the pruner's ``total_steps``: a linear ramp, and the cubic ramp ``1 - (1 - t)^3``."""

    def __init__(self, kind: str, start_epoch: int = 0, end_epoch: int = 0, power: float = 1.0):
        self.kind, self.start_epoch, self.end_epoch, self.power = kind, int(start_epoch), int(end_epoch), float(power)

    @classmethod
    def one_shot(cls) -> "PruningSchedule":
        return cls.ONE_SHOT

    @classmethod
    def linear(cls, start_epoch: int, end_epoch: int) -> "PruningSchedule":
        return cls("linear", start_epoch, end_epoch)

    @classmethod
    def polynomial(cls, start_epoch: int, end_epoch: int, power: float = 3.0) -> "PruningSchedule":
        return cls("polynomial", start_epoch, end_epoch, power)

    @classmethod
    def exponential(cls, start_epoch: int, end_epoch: int) -> "PruningSchedule":
        return cls("exponential", start_epoch, end_epoch)

    def fraction(self, epoch: int, total_steps: int = 1) -> float:
        """Share of the target sparsity that applies at ``epoch``."""
        if self.kind == "one_shot":
            return 1.0
        if self.kind in ("gradual", "cubic"):
            t = min(1.0, epoch / max(1, total_steps))
            return t if self.kind == "gradual" else 1.0 - (1.0 - t) ** 3
        if epoch < self.start_epoch:
            return 0.0
        if epoch >= self.end_epoch:
            return 1.0
        t = (epoch - self.start_epoch) / (self.end_epoch - self.start_epoch)
        if self.kind == "linear":
            return t
        if self.kind == "polynomial":
            return t ** self.power
        return 1.0 - math.exp(-5.0 * t)

    def __repr__(self):
        return f"PruningSchedule({self.kind!r}, {self.start_epoch}, {self.end_epoch}, {self.power})"


PruningSchedule.ONE_SHOT = PruningSchedule("one_shot")
PruningSchedule.GRADUAL = PruningSchedule("gradual")
PruningSchedule.POLYNOMIAL = PruningSchedule("cubic")


@dataclass
class PruningMask:
    """Boolean keep-mask of one tensor with its counts (src/nn/pruning.rs:118-162)."""
    mask: torch.Tensor

    def __post_init__(self):
        self.mask = self.mask.to(torch.bool)
        self.total_count = self.mask.numel()
        self.pruned_count = self.total_count - int(self.mask.sum())
        self.sparsity = self.pruned_count / max(1, self.total_count)

    def compression_ratio(self) -> float:
        return 1.0 / (1.0 - self.sparsity) if self.sparsity < 1.0 else float("inf")

    def remaining_params(self) -> int:
        return self.total_count - self.pruned_count

    def apply(self, t: torch.Tensor) -> torch.Tensor:
        return t * self.mask.to(device=t.device, dtype=t.dtype)


def _keep_above_kth(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Keep-mask that drops the ``k`` lowest scores (ties at the threshold are dropped with it)."""
    if k <= 0:
        return torch.ones_like(scores, dtype=torch.bool)
    flat = scores.flatten()
    if k >= flat.numel():
        return torch.zeros_like(scores, dtype=torch.bool)
    return scores > flat.kthvalue(k).values


class Pruner:
    """Computes and remembers pruning masks per named tensor.

    ``Pruner(method, sparsity, schedule, total_steps, seed, structure)``; the reference's argument order
    ``(method, structure, target_sparsity, schedule)`` is accepted too (src/nn/pruning.rs:206-231)."""

    def __init__(self, method: PruningMethod = PruningMethod.L1_NORM, sparsity=0.5,
                 schedule=PruningSchedule.ONE_SHOT, total_steps=1, seed: int = 0,
                 structure: Optional[PruningStructure] = None):
        if isinstance(sparsity, PruningStructure):           # (method, structure, target_sparsity, schedule)
            structure, sparsity, schedule = sparsity, schedule, (total_steps if isinstance(total_steps, PruningSchedule)
                                                                 else PruningSchedule.ONE_SHOT)
            total_steps = 1
        if not 0.0 <= float(sparsity) < 1.0:
            raise ValueError("sparsity must be in [0, 1)")
        if structure is None:
            structure = PruningStructure.CHANNEL if method is PruningMethod.STRUCTURED else PruningStructure.UNSTRUCTURED
        self.method, self.structure, self.target, self.schedule = method, structure, float(sparsity), schedule
        self.total_steps = max(1, int(total_steps))
        self.step_count = 0                                  # the epoch counter of the schedule
        self.masks: Dict[str, torch.Tensor] = {}
        self.original_weights: Dict[str, torch.Tensor] = {}
        self._gen = torch.Generator().manual_seed(seed)

    # ---- schedule
    @property
    def current_epoch(self) -> int:
        return self.step_count

    def step_epoch(self) -> None:
        self.step_count += 1

    def current_sparsity(self) -> float:
        return self.target * self.schedule.fraction(self.step_count, self.total_steps)

    get_current_sparsity = current_sparsity

    # ---- scores and masks
    def importance_scores(self, w: torch.Tensor, grad: Optional[torch.Tensor] = None) -> torch.Tensor:
        wf = w.detach().float()
        m = self.method
        if m is PruningMethod.RANDOM:
            return torch.rand(w.shape, generator=self._gen).to(w.device)
        if m is PruningMethod.GRADIENT:
            return grad.detach().float().abs() if grad is not None else wf.abs()
        if m is PruningMethod.TAYLOR:
            return (wf * grad.detach().float()).abs() if grad is not None else wf * wf
        if m in (PruningMethod.L2_NORM, PruningMethod.STRUCTURED):
            return wf * wf
        return wf.abs()

    def create_mask(self, scores: torch.Tensor, sparsity: float) -> torch.Tensor:
        st = self.structure
        if st.kind == "block":
            n, m = st.n, st.m
            flat = scores.flatten()
            full = flat.numel() // m * m
            keep = torch.ones_like(flat, dtype=torch.bool)   # an incomplete last block is kept whole
            if full and n < m:
                blocks = flat[:full].view(-1, m)
                top = blocks.topk(n, dim=1).indices
                kb = torch.zeros_like(blocks, dtype=torch.bool)
                kb.scatter_(1, top, True)
                keep[:full] = kb.flatten()
            tail = flat.numel() - full
            if tail > n:                                     # a ragged tail longer than n keeps its n best
                kt = torch.zeros(tail, dtype=torch.bool, device=flat.device)
                kt[flat[full:].topk(n).indices] = True
                keep[full:] = kt
            return keep.view(scores.shape)
        if sparsity <= 0:
            return torch.ones_like(scores, dtype=torch.bool)
        if st.kind in ("channel", "filter") and scores.dim() >= 2:
            dim = 0 if st.kind == "channel" else 1
            other = [d for d in range(scores.dim()) if d != dim]
            # the scores are non-negative; the group score is their root sum of squares
            g = (scores * scores).sum(dim=other).sqrt() if self.method not in (PruningMethod.L2_NORM, PruningMethod.STRUCTURED) \
                else scores.sum(dim=other).sqrt()
            keep = _keep_above_kth(g, int(sparsity * g.numel()))
            shape = [1] * scores.dim()
            shape[dim] = -1
            return keep.view(shape).expand_as(scores).clone()
        return _keep_above_kth(scores, int(sparsity * scores.numel()))

    def compute_mask(self, w: torch.Tensor, sparsity: Optional[float] = None, grad: Optional[torch.Tensor] = None) -> torch.Tensor:
        s = self.current_sparsity() if sparsity is None else float(sparsity)
        if self.method is PruningMethod.RANDOM and self.structure.kind == "unstructured":
            if s <= 0:
                return torch.ones_like(w, dtype=torch.bool)
            return self.importance_scores(w) >= s            # each weight dropped with probability s
        return self.create_mask(self.importance_scores(w, grad), s)

    # ---- the reference's tensor / module entry points
    def prune_tensor(self, tensor: torch.Tensor, layer_name: str, grad: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Returns the masked tensor, records the mask under ``layer_name`` and, the first time a name is seen, a copy
        of the unpruned weights for lottery-ticket rewinding."""
        if layer_name not in self.original_weights:
            self.original_weights[layer_name] = tensor.detach().clone()
        mask = self.compute_mask(tensor, grad=grad)
        self.masks[layer_name] = mask
        return tensor.detach() * mask.to(tensor.dtype)

    def prune_module(self, module: nn.Module, layer_prefix: str = "") -> List[torch.Tensor]:
        """Masked copies of all parameters of ``module``, named ``<prefix>_<index>`` as the reference names them."""
        return [self.prune_tensor(p.data, f"{layer_prefix}_{i}", p.grad) for i, p in enumerate(module.parameters())]

    def reset_to_original_weights(self, layer_name: str) -> Optional[torch.Tensor]:
        w = self.original_weights.get(layer_name)
        return None if w is None else w.clone()

    def rewind(self, named_parameters: Iterable[Tuple[str, nn.Parameter]]) -> None:
        """Lottery ticket: put the surviving weights back to their first-seen values, keep the pruned ones at zero."""
        with torch.no_grad():
            for name, p in named_parameters:
                w0, m = self.original_weights.get(name), self.masks.get(name)
                if w0 is not None:
                    p.copy_(w0 if m is None else w0 * m.to(w0.dtype))

    def get_statistics(self) -> Dict[str, float]:
        return {k: 1.0 - float(m.float().mean()) for k, m in self.masks.items()}

    sparsity_report = get_statistics

    def get_global_sparsity(self) -> float:
        total = sum(m.numel() for m in self.masks.values())
        if total == 0:
            return 0.0
        return sum(m.numel() - int(m.sum()) for m in self.masks.values()) / total

    def get_mask(self, layer_name: str) -> Optional[PruningMask]:
        m = self.masks.get(layer_name)
        return None if m is None else PruningMask(m)

    def clear_masks(self) -> None:
        self.masks.clear()

    # ---- in-place training-loop form
    def prune(self, named_parameters: Iterable[Tuple[str, nn.Parameter]], only_weights: bool = True) -> Dict[str, float]:
        """Advance the schedule by one step, update the masks and zero the pruned weights in place."""
        self.step_count += 1
        out = {}
        for name, p in named_parameters:
            if only_weights and p.dim() < 2:
                continue
            if name not in self.original_weights:
                self.original_weights[name] = p.detach().clone()
            mask = self.compute_mask(p.data, grad=p.grad)
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


class PruningAwareModule(nn.Module):
    """Wraps a module and a pruner: while pruning is enabled every forward pass in training mode re-applies the
    masks, so optimizer steps cannot revive pruned weights; ``step_epoch`` advances the schedule and recomputes the
    masks (src/nn/pruning.rs:529-640)."""

    def __init__(self, module: nn.Module, pruner: Pruner):
        super().__init__()
        self.module, self.pruner = module, pruner
        self.pruning_enabled = False

    def enable_pruning(self) -> None:
        self.pruning_enabled = True
        self._update_masks()

    def disable_pruning(self) -> None:
        self.pruning_enabled = False

    def _named(self):
        return [(n, p) for n, p in self.module.named_parameters() if p.dim() >= 2]

    def _update_masks(self) -> None:
        with torch.no_grad():
            for name, p in self._named():
                if name not in self.pruner.original_weights:
                    self.pruner.original_weights[name] = p.detach().clone()
                mask = self.pruner.compute_mask(p.data, grad=p.grad)
                if name in self.pruner.masks:
                    mask &= self.pruner.masks[name]
                self.pruner.masks[name] = mask
                p.mul_(mask.to(p.dtype))

    def step_epoch(self) -> None:
        self.pruner.step_epoch()
        if self.pruning_enabled:
            self._update_masks()

    def get_statistics(self) -> Dict[str, float]:
        return self.pruner.get_statistics()

    def forward(self, *args, **kw):
        if self.pruning_enabled and self.training:
            self.pruner.apply_masks(self._named())
        return self.module(*args, **kw)
