"""Loss functions and modules with the reference's names and arguments (src/nn/loss.rs).

The reference's ``CrossEntropyLoss`` recurses forever (:58-69,98-106), ``nll_loss`` forwards to it and
``binary_cross_entropy`` / ``huber_loss`` are placeholders (:176-206); the semantics here are
PyTorch's.  ``reduction`` strings are ``"mean" | "sum" | "none"``.
"""
from __future__ import annotations

import enum
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


class Reduction(enum.Enum):
    """``mean`` / ``sum`` / ``none`` reduction of a loss (src/nn/loss.rs:26-69)."""

    NONE = "none"
    MEAN = "mean"
    SUM = "sum"


def _red(r) -> str:
    return r.value if isinstance(r, Reduction) else str(r).lower()


def _apply(x: torch.Tensor, reduction) -> torch.Tensor:
    r = _red(reduction)
    if r == "mean":
        return x.mean()
    if r == "sum":
        return x.sum()
    return x


# ----------------------------------------------------------------- functional
def mse_loss(input, target, reduction="mean"):
    return F.mse_loss(input, target, reduction=_red(reduction))


def _class_targets(input, target):
    """Class indices held in a floating tensor (the binding has one tensor type, so its targets are floats) become
    ``long``; a floating target of the logits' own shape is a distribution over classes and stays as it is."""
    if isinstance(target, torch.Tensor) and target.is_floating_point() and target.dim() == input.dim() - 1:
        return target.long()
    return target


def cross_entropy(input, target, weight=None, ignore_index: int = -100, reduction="mean", label_smoothing: float = 0.0):
    target = _class_targets(input, target)
    return F.cross_entropy(input, target, weight, ignore_index=ignore_index, reduction=_red(reduction),
                           label_smoothing=label_smoothing)


cross_entropy_loss = cross_entropy


def nll_loss(input, target, weight=None, ignore_index: int = -100, reduction="mean"):
    return F.nll_loss(input, _class_targets(input, target), weight, ignore_index=ignore_index, reduction=_red(reduction))


def binary_cross_entropy(input, target, weight=None, reduction="mean"):
    return F.binary_cross_entropy(input, target, weight, reduction=_red(reduction))


def binary_cross_entropy_with_logits(input, target, weight=None, pos_weight=None, reduction="mean"):
    return F.binary_cross_entropy_with_logits(input, target, weight, pos_weight=pos_weight, reduction=_red(reduction))


def huber_loss(input, target, delta: float = 1.0, reduction="mean"):
    return F.huber_loss(input, target, reduction=_red(reduction), delta=delta)


def l1_loss(input, target, reduction="mean"):
    return F.l1_loss(input, target, reduction=_red(reduction))


def smooth_l1_loss(input, target, beta: float = 1.0, reduction="mean"):
    return F.smooth_l1_loss(input, target, reduction=_red(reduction), beta=beta)


def kl_div(input, target, reduction="mean", log_target: bool = False):
    r = _red(reduction)
    return F.kl_div(input, target, reduction="batchmean" if r == "batchmean" else r, log_target=log_target)


def focal_loss(input, target, alpha: float = 0.25, gamma: float = 2.0, reduction="mean"):
    """Multi-class focal loss on logits ``[N, C]`` with class targets ``[N]``."""
    logp = F.log_softmax(input, dim=-1)
    logpt = logp.gather(-1, target.long().unsqueeze(-1)).squeeze(-1)
    pt = logpt.exp()
    return _apply(-alpha * (1 - pt).pow(gamma) * logpt, reduction)


def triplet_margin_loss(anchor, positive, negative, margin: float = 1.0, p: float = 2.0, swap: bool = False,
                        reduction="mean"):
    return F.triplet_margin_loss(anchor, positive, negative, margin=margin, p=p, swap=swap, reduction=_red(reduction))


def margin_ranking_loss(x1, x2, target, margin: float = 0.0, reduction="mean"):
    return F.margin_ranking_loss(x1, x2, target, margin=margin, reduction=_red(reduction))


def cosine_embedding_loss(x1, x2, target, margin: float = 0.0, reduction="mean"):
    return F.cosine_embedding_loss(x1, x2, target, margin=margin, reduction=_red(reduction))


# -------------------------------------------------------------------- modules
class _Loss(nn.Module):
    def __init__(self, reduction="mean"):
        super().__init__()
        self.reduction = _red(reduction)


class MSELoss(_Loss):
    def forward(self, input, target):
        return mse_loss(input, target, self.reduction)


class L1Loss(_Loss):
    def forward(self, input, target):
        return l1_loss(input, target, self.reduction)


class HuberLoss(_Loss):
    def __init__(self, delta: float = 1.0, reduction="mean"):
        super().__init__(reduction)
        self.delta = delta

    def forward(self, input, target):
        return huber_loss(input, target, self.delta, self.reduction)


class CrossEntropyLoss(_Loss):
    """``CrossEntropyLoss()``: logits ``[N, C]`` (or ``[N, C, ...]``) and class indices."""

    def __init__(self, weight=None, ignore_index: int = -100, reduction="mean", label_smoothing: float = 0.0):
        super().__init__(reduction)
        self.register_buffer("weight", weight)
        self.ignore_index, self.label_smoothing = ignore_index, label_smoothing

    def forward(self, input, target):
        return cross_entropy(input, target, self.weight, self.ignore_index, self.reduction, self.label_smoothing)


class NLLLoss(_Loss):
    def __init__(self, weight=None, ignore_index: int = -100, reduction="mean"):
        super().__init__(reduction)
        self.register_buffer("weight", weight)
        self.ignore_index = ignore_index

    def forward(self, input, target):
        return nll_loss(input, target.long(), self.weight, self.ignore_index, self.reduction)


class BCELoss(_Loss):
    def forward(self, input, target):
        return binary_cross_entropy(input, target, reduction=self.reduction)


class BCEWithLogitsLoss(_Loss):
    """``(weight, pos_weight, reduction)`` (src/nn/loss.rs:634-640)."""

    def __init__(self, weight=None, pos_weight=None, reduction="mean"):
        super().__init__(reduction)
        self.register_buffer("weight", weight)
        self.register_buffer("pos_weight", pos_weight)

    def forward(self, input, target):
        return binary_cross_entropy_with_logits(input, target, self.weight, self.pos_weight, self.reduction)


class FocalLoss(_Loss):
    """``(alpha, gamma)`` (src/nn/loss.rs:236)."""

    def __init__(self, alpha: float = 0.25, gamma: float = 2.0, reduction="mean"):
        super().__init__(reduction)
        self.alpha, self.gamma = alpha, gamma

    def forward(self, input, target):
        return focal_loss(input, target, self.alpha, self.gamma, self.reduction)


class TripletLoss(_Loss):
    """``(margin)`` with Euclidean distance (src/nn/loss.rs:313)."""

    def __init__(self, margin: float = 1.0, reduction="mean"):
        super().__init__(reduction)
        self.margin = margin

    def forward(self, anchor, positive, negative):
        return triplet_margin_loss(anchor, positive, negative, self.margin, reduction=self.reduction)


class TripletMarginLoss(_Loss):
    """``(margin=1, p=2, swap=False, reduction)`` (src/nn/loss.rs:1054-1062)."""

    def __init__(self, margin: float = 1.0, p: float = 2.0, swap: bool = False, reduction="mean"):
        super().__init__(reduction)
        self.margin, self.p, self.swap = margin, p, swap

    def forward(self, anchor, positive, negative):
        return triplet_margin_loss(anchor, positive, negative, self.margin, self.p, self.swap, self.reduction)


class KLDivLoss(_Loss):
    def __init__(self, reduction="mean", log_target: bool = False):
        super().__init__(reduction)
        self.log_target = log_target

    def forward(self, input, target):
        return kl_div(input, target, self.reduction, self.log_target)


class MarginRankingLoss(_Loss):
    def __init__(self, margin: float = 0.0, reduction="mean"):
        super().__init__(reduction)
        self.margin = margin

    def forward(self, x1, x2, target):
        return margin_ranking_loss(x1, x2, target, self.margin, self.reduction)


class CosineEmbeddingLoss(_Loss):
    def __init__(self, margin: float = 0.0, reduction="mean"):
        super().__init__(reduction)
        self.margin = margin

    def forward(self, x1, x2, target):
        return cosine_embedding_loss(x1, x2, target, self.margin, self.reduction)


from .._interop import accept_wrappers as _accept_wrappers  # noqa: E402

_accept_wrappers(globals())       # forward() of the layers above also takes this package's Tensor / Variable
