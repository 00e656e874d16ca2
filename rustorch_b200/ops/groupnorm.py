"""GroupNorm / InstanceNorm on the native slab kernel (csrc/norm/groupnorm.cu); PyTorch elsewhere.

The reference computes both with host loops (src/nn/normalization.rs:343-520, src/nn/instance_norm.rs:148-330).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native

_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def supported(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in _DTYPES and x.dim() >= 2 and x.numel() > 0 and _native.available()


def _f32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else t.detach().float().contiguous()


class GroupNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, groups: int, eps: float):
        C = _native.load(required=True)
        xc = x.contiguous()
        y = torch.empty_like(xc)
        slabs = xc.shape[0] * groups
        mean = torch.empty(slabs, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        g32 = _f32(weight)
        C.groupnorm(xc, y, None, g32, _f32(bias), mean, rstd, None, None, groups, eps)
        ctx.save_for_backward(xc, g32 if g32 is not None else torch.empty(0, device=x.device), mean, rstd)
        ctx.groups, ctx.eps = groups, eps
        ctx.affine = (weight is not None, bias is not None)
        ctx.wdtype = weight.dtype if weight is not None else None
        ctx.bdtype = bias.dtype if bias is not None else None
        return y

    @staticmethod
    def backward(ctx, dy):
        C = _native.load(required=True)
        xc, g32, mean, rstd = ctx.saved_tensors
        has_w, has_b = ctx.affine
        dyc = dy.contiguous()
        dx = torch.empty_like(xc)
        ch = xc.shape[1]
        dgamma = torch.zeros(ch, dtype=torch.float32, device=xc.device) if has_w else None
        dbeta = torch.zeros(ch, dtype=torch.float32, device=xc.device) if has_b else None
        C.groupnorm(xc, dx, dyc, g32 if has_w else None, None, mean, rstd, dgamma, dbeta, ctx.groups, ctx.eps)
        return (dx, dgamma.to(ctx.wdtype) if has_w else None, dbeta.to(ctx.bdtype) if has_b else None, None, None)


def group_norm(x: torch.Tensor, num_groups: int, weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
               eps: float = 1e-5) -> torch.Tensor:
    if supported(x) and x.shape[1] % num_groups == 0:
        return GroupNormFn.apply(x, weight, bias, num_groups, eps)
    return torch.nn.functional.group_norm(x, num_groups, weight, bias, eps)


def instance_norm(x: torch.Tensor, weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                  eps: float = 1e-5) -> torch.Tensor:
    """Per-sample, per-channel statistics: GroupNorm with one channel per group."""
    if supported(x):
        return GroupNormFn.apply(x, weight, bias, x.shape[1], eps)
    return torch.nn.functional.instance_norm(x, None, None, weight, bias, True, 0.0, eps)
