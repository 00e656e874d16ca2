"""BatchNorm on the native kernels (training + inference, optional fused residual add and ReLU), with autograd.

The kernels work on a channels-last matrix ``[pixels, C]``.  An NCHW tensor is brought to
``torch.channels_last`` first (a no-op when the network already runs channels-last, which is the layout the
convolution kernels want as well); ``[N, C]`` inputs are already in that form.  Semantics follow
src/nn/batchnorm.rs:120-330 (biased variance for normalisation, unbiased for the running estimate).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native


def _to_matrix(x: torch.Tensor):
    """-> (x2 [M, C] contiguous view/copy, restore(y2) -> tensor shaped like x)."""
    if x.dim() == 2:
        xc = x.contiguous()
        return xc, lambda y: y
    C = x.shape[1]
    perm = (0,) + tuple(range(2, x.dim())) + (1,)
    inv = (0, x.dim() - 1) + tuple(range(1, x.dim() - 1))
    xl = x.permute(perm).contiguous()                 # free when x is channels-last already
    shape = xl.shape
    return xl.view(-1, C), lambda y: y.view(shape).permute(inv)


class BatchNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, running_mean, running_var, residual, training: bool, momentum: float, eps: float,
                relu: bool):
        C_ = _native.load(required=True)
        x2, restore = _to_matrix(x)
        r2 = _to_matrix(residual)[0] if residual is not None else None
        C = x2.shape[1]
        y2 = torch.empty_like(x2)
        scratch = torch.empty(2, C, dtype=torch.float32, device=x.device)
        g = gamma.float().contiguous() if gamma is not None else None
        b = beta.float().contiguous() if beta is not None else None
        save_mean = torch.empty(C, dtype=torch.float32, device=x.device) if training else None
        save_rstd = torch.empty(C, dtype=torch.float32, device=x.device) if training else None
        C_.batchnorm_fwd(x2, r2, y2, g, b, running_mean, running_var, save_mean, save_rstd, scratch, eps, momentum, relu,
                         training)
        if training:
            ctx.save_for_backward(x2, y2 if relu else None, g, save_mean, save_rstd)
        else:
            rstd = torch.rsqrt(running_var.float() + eps)
            ctx.save_for_backward(x2, y2 if relu else None, g, running_mean.float(), rstd)
        ctx.restore, ctx.training = restore, training
        ctx.has_res = residual is not None
        ctx.param_dtypes = (gamma.dtype if gamma is not None else None, beta.dtype if beta is not None else None)
        return restore(y2)

    @staticmethod
    def backward(ctx, dy):
        C_ = _native.load(required=True)
        x2, y_relu, g, mean, rstd = ctx.saved_tensors
        dy2, _ = _to_matrix(dy)
        C = x2.shape[1]
        dx2 = torch.empty_like(x2)
        dres2 = torch.empty_like(x2) if ctx.has_res else None
        scratch = torch.empty(2, C, dtype=torch.float32, device=x2.device)
        if ctx.training:
            C_.batchnorm_bwd(x2, dy2, y_relu, dx2, dres2, g, mean, rstd, scratch)
        else:
            # inference-mode statistics are constants: dx = gamma * rstd * dy
            C_.batchnorm_bwd(x2, dy2, y_relu, dx2, dres2, g, mean, rstd, scratch)
            gd = dres2 if dres2 is not None else (dy2 if y_relu is None else dy2 * (y_relu > 0))
            dx2 = (gd.float() * (rstd * (g if g is not None else 1.0))).to(x2.dtype)
        gdt, bdt = ctx.param_dtypes
        dgamma = scratch[1].to(gdt) if gdt is not None else None
        dbeta = scratch[0].to(bdt) if bdt is not None else None
        return (ctx.restore(dx2), dgamma, dbeta, None, None, ctx.restore(dres2) if dres2 is not None else None,
                None, None, None, None)


def supported(x: torch.Tensor) -> bool:
    if not (x.is_cuda and x.dtype in (torch.float32, torch.bfloat16, torch.float16) and x.dim() >= 2 and _native.available()):
        return False
    return x.shape[1] % (4 if x.dtype == torch.float32 else 8) == 0 and x.numel() > 0


def batch_norm(x: torch.Tensor, running_mean: Optional[torch.Tensor], running_var: Optional[torch.Tensor],
               weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, training: bool = False,
               momentum: float = 0.1, eps: float = 1e-5, residual: Optional[torch.Tensor] = None, relu: bool = False
               ) -> torch.Tensor:
    """``relu((batch_norm(x) + residual))`` with the last two optional; native on CUDA, PyTorch elsewhere."""
    use_batch = training or running_mean is None
    if supported(x) and (running_mean is None or running_mean.dtype == torch.float32):
        return BatchNormFn.apply(x, weight, bias, running_mean, running_var, residual, use_batch, momentum, eps, relu)
    y = torch.nn.functional.batch_norm(x, running_mean, running_var, weight, bias, use_batch, momentum, eps)
    if residual is not None:
        y = y + residual
    return torch.relu(y) if relu else y
