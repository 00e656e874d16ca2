"""Python entry points of the hand-written sm_100a kernels (thin wrappers over ``_C``).

Each function allocates its outputs with torch and launches on torch's current stream.
Shapes/dtypes are validated in C++ (csrc/bindings.cpp).  Reference parity notes live in the
kernel sources; the reference's own GPU dispatch is src/gpu/matrix_ops.rs:274-632.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _native

EPI_NONE, EPI_GELU_DUAL, EPI_DGELU, EPI_RESIDUAL = 0, 1, 2, 3
OPT_ADAMW, OPT_ADAM, OPT_SGD = 0, 1, 2


def _C():
    return _native.load(required=True)


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
         bias: Optional[torch.Tensor] = None, aux: Optional[torch.Tensor] = None,
         epilogue: int = EPI_NONE, alpha: float = 1.0, accumulate: bool = False,
         split_k: int = 1, block_n: int = 0, alpha_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[b,m,n] = alpha * sum_k A[b,m,k] B[b,n,k]`` (+ epilogue) on tcgen05.

    ``a`` is ``[.., M, K]`` (``a_mn=False``) or ``[.., K, M]`` (``a_mn=True``); ``b`` is
    ``[.., N, K]`` or ``[.., K, N]`` likewise.  Rank 2 or 3; last dim contiguous.  ``alpha_dev`` is an optional
    one-element fp32 CUDA tensor multiplied into ``alpha`` on the device (no host read).
    """
    M = a.shape[-1] if a_mn else a.shape[-2]
    N = b.shape[-1] if b_mn else b.shape[-2]
    if out is None:
        shape = (*a.shape[:-2], M, N)
        out = (torch.zeros if accumulate else torch.empty)(shape, dtype=out_dtype, device=a.device)
    _C().gemm(a, a_mn, b, b_mn, out, bias, aux, epilogue, float(alpha), accumulate, split_k, block_n, alpha_dev)
    return out


def attention_fwd(q, k, v, causal: bool, scale: Optional[float] = None):
    """q [B,Tq,H,D], k/v [B,Tk,Hkv,D] (strided views allowed) -> (o [B,Tq,H,D], lse [B,H,Tq])."""
    B, Tq, H, D = q.shape
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    o = torch.empty((B, Tq, H, D), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, H, Tq), dtype=torch.float32, device=q.device)
    _C().attn_fwd(q, k, v, o, lse, causal, float(scale))
    return o, lse


def attention_bwd(q, k, v, o, d_o, lse, causal: bool, scale: Optional[float] = None,
                  dq=None, dk=None, dv=None):
    B, Tq, H, D = q.shape
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    if dq is None:
        dq = torch.empty(q.shape, dtype=torch.bfloat16, device=q.device)
    if dk is None:
        dk = torch.empty(k.shape, dtype=torch.bfloat16, device=q.device)
    if dv is None:
        dv = torch.empty(v.shape, dtype=torch.bfloat16, device=q.device)
    delta = torch.empty((B, H, Tq), dtype=torch.float32, device=q.device)
    if d_o.stride() != o.stride():
        d_o = d_o.contiguous() if o.is_contiguous() else d_o.clone(memory_format=torch.preserve_format)
    # 64-wide heads: fp32 accumulation buffer for dQ, which turns the backward into one kernel over the tile pairs
    dq_acc = torch.empty((B, Tq, H, D), dtype=torch.float32, device=q.device) if D == 64 else None
    _C().attn_bwd(q, k, v, o, d_o, lse, delta, dq, dk, dv, causal, float(scale), dq_acc)
    return dq, dk, dv


def layer_norm_fwd(x, gamma, beta, eps: float):
    y = torch.empty_like(x)
    rows = x.numel() // gamma.numel()
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    _C().norm_fwd(x, gamma, beta, y, mean, rstd, float(eps), False)
    return y, mean, rstd


def layer_norm_bwd(dy, x, gamma, mean, rstd, dgamma, dbeta, dres=None, reduce_stream: int = 0):
    """``reduce_stream``: raw handle of a CUDA stream that takes the second stage (partial sums -> dgamma / dbeta),
    ordered after the first by an event; 0 keeps both stages on the current stream."""
    dx = torch.empty_like(x)
    partial = _C().norm_bwd(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, False, int(reduce_stream))
    if reduce_stream:
        return dx, partial          # the caller keeps the partial sums alive until it has joined the side stream
    return dx


def rms_norm_fwd(x, gamma, eps: float):
    y = torch.empty_like(x)
    rows = x.numel() // gamma.numel()
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    _C().norm_fwd(x, gamma, None, y, None, rstd, float(eps), True)
    return y, rstd


def rms_norm_bwd(dy, x, gamma, rstd, dgamma, dres=None, reduce_stream: int = 0):
    dx = torch.empty_like(x)
    partial = _C().norm_bwd(dy, x, gamma, None, rstd, dres, dx, dgamma, None, True, int(reduce_stream))
    if reduce_stream:
        return dx, partial
    return dx


def embedding_fwd(idx, wte, wpe=None, T: int = 1):
    out = torch.empty((*idx.shape, wte.shape[1]), dtype=torch.bfloat16, device=idx.device)
    _C().embedding_fwd(idx.contiguous(), wte, wpe, out, int(T))
    return out


def embedding_bwd(idx, dout, dwte, dwpe, T: int, vocab: int):
    _C().embedding_bwd(idx.contiguous(), dout.contiguous(), dwte, dwpe, int(T), int(vocab))


def cross_entropy_(logits, targets, vocab: int, grad_scale: float, ignore_index: int = -100):
    """In place: logits <- d(sum of row losses * grad_scale)/d(logits).  Returns per-row losses."""
    loss = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
    _C().cross_entropy(logits, targets.contiguous(), loss, int(vocab), float(grad_scale),
                       int(ignore_index))
    return loss


def colsum_accum(x2d, out_f32):
    _C().colsum_accum(x2d, out_f32)


def reduce_all(x, mode: str = "sum"):
    modes = {"sum": 0, "sumsq": 1, "max": 2, "min": 3}
    init = {"sum": 0.0, "sumsq": 0.0, "max": float("-inf"), "min": float("inf")}[mode]
    out = torch.full((1,), init, dtype=torch.float32, device=x.device)
    _C().reduce_all(x.contiguous(), modes[mode], out)
    return out


def fused_optim_step(master, grad, m, v, param_lp, *, mode: int, lr: float, beta1: float = 0.9,
                     beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.0,
                     bias_corr1: float = 1.0, bias_corr2: float = 1.0, grad_scale: float = 1.0,
                     zero_grad: bool = True, nesterov: bool = False, first_step: bool = False):
    _C().fused_optim_step(master, grad, m, v, param_lp, mode, lr, beta1, beta2, eps, weight_decay,
                          bias_corr1, bias_corr2, grad_scale, zero_grad, nesterov, first_step)
