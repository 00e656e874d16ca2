"""Elementwise arithmetic, activations, row softmax and row reductions on the native kernels, with autograd.

On a CUDA tensor (fp32 / bf16 / fp16, contiguous) every function here launches the kernels of
``csrc/elementwise``; anything else (CPU, integer types, broadcasting shapes) takes the PyTorch
expression of the same math, which is also the oracle of the tests.  Mirrors the reference's GPU
elementwise / activation / reduction traits (src/gpu/activation_ops.rs:22-845, reduction_ops.rs:20-450,
src/gpu/cuda_kernels.rs:70-330).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from .. import _native

BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3, "max": 4, "min": 5, "pow": 6}
UNARY = {"relu": 0, "sigmoid": 1, "tanh": 2, "gelu": 3, "gelu_tanh": 3, "gelu_erf": 4, "silu": 5, "swish": 5, "elu": 6,
         "leaky_relu": 7, "selu": 8, "mish": 9, "softplus": 10, "hardtanh": 11, "relu6": 12, "hardsigmoid": 13,
         "hardswish": 14, "exp": 15, "log": 16, "sqrt": 17, "rsqrt": 18, "neg": 19, "abs": 20, "square": 21, "sin": 22,
         "cos": 23, "scale_shift": 24, "reciprocal": 25}
_FLOATS = (torch.float32, torch.bfloat16, torch.float16)


def _torch_unary(name: str, x: torch.Tensor, p0: float, p1: float) -> torch.Tensor:
    return {
        "relu": lambda: F.relu(x), "sigmoid": lambda: torch.sigmoid(x), "tanh": lambda: torch.tanh(x),
        "gelu": lambda: F.gelu(x, approximate="tanh"), "gelu_tanh": lambda: F.gelu(x, approximate="tanh"),
        "gelu_erf": lambda: F.gelu(x), "silu": lambda: F.silu(x), "swish": lambda: F.silu(x),
        "elu": lambda: F.elu(x, p0), "leaky_relu": lambda: F.leaky_relu(x, p0), "selu": lambda: F.selu(x),
        "mish": lambda: F.mish(x), "softplus": lambda: F.softplus(x, p0, p1), "hardtanh": lambda: F.hardtanh(x, p0, p1),
        "relu6": lambda: F.relu6(x), "hardsigmoid": lambda: F.hardsigmoid(x), "hardswish": lambda: F.hardswish(x),
        "exp": lambda: torch.exp(x), "log": lambda: torch.log(x), "sqrt": lambda: torch.sqrt(x),
        "rsqrt": lambda: torch.rsqrt(x), "neg": lambda: -x, "abs": lambda: x.abs(), "square": lambda: x * x,
        "sin": lambda: torch.sin(x), "cos": lambda: torch.cos(x), "scale_shift": lambda: x * p0 + p1,
        "reciprocal": lambda: 1.0 / x,
    }[name]()


_DEFAULTS = {"elu": (1.0, 0.0), "leaky_relu": (0.01, 0.0), "softplus": (1.0, 20.0), "hardtanh": (-1.0, 1.0),
             "scale_shift": (1.0, 0.0)}


def _on_device(*ts: torch.Tensor) -> bool:
    return all(t.is_cuda and t.dtype in _FLOATS for t in ts) and _native.available()


class _Unary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, op: int, p0: float, p1: float):
        xc = x.contiguous()
        out = torch.empty_like(xc)
        _native.load(required=True).ew_unary(op, xc, None, out, p0, p1)
        ctx.save_for_backward(xc)
        ctx.args = (op, p0, p1)
        return out

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        op, p0, p1 = ctx.args
        dx = torch.empty_like(x)
        _native.load(required=True).ew_unary(op, x, dy.contiguous(), dx, p0, p1)
        return dx, None, None, None


def unary(name: str, x: torch.Tensor, p0: Optional[float] = None, p1: Optional[float] = None) -> torch.Tensor:
    d0, d1 = _DEFAULTS.get(name, (0.0, 0.0))
    p0 = d0 if p0 is None else float(p0)
    p1 = d1 if p1 is None else float(p1)
    if _on_device(x):
        return _Unary.apply(x, UNARY[name], p0, p1)
    return _torch_unary(name, x, p0, p1)


class _Binary(torch.autograd.Function):
    """Same-shape tensors or tensor-scalar.  Backward is expressed with the same kernels."""

    @staticmethod
    def forward(ctx, a, b, op: int, alpha: float):
        C = _native.load(required=True)
        ac = a.contiguous()
        out = torch.empty_like(ac)
        if isinstance(b, torch.Tensor):
            bc = b.contiguous()
            C.ew_binary(op, ac, bc, out, 0.0, alpha, 0)
            ctx.save_for_backward(ac, bc)
            ctx.scalar = None
        else:
            C.ew_binary(op, ac, None, out, float(b), alpha, 1)
            ctx.save_for_backward(ac)
            ctx.scalar = float(b)
        ctx.op, ctx.alpha = op, alpha
        return out

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous()
        op, alpha = ctx.op, ctx.alpha
        if ctx.scalar is None:
            a, b = ctx.saved_tensors
        else:
            (a,), b = ctx.saved_tensors, ctx.scalar
        need_b = ctx.scalar is None and ctx.needs_input_grad[1]
        da = db = None
        if op == 0:      # a + alpha b
            da, db = dy, (dy * alpha if need_b else None)
        elif op == 1:
            da, db = dy, (dy * -alpha if need_b else None)
        elif op == 2:
            da, db = binary("mul", dy, b), (binary("mul", dy, a) if need_b else None)
        elif op == 3:
            da = binary("div", dy, b)
            db = -binary("div", binary("mul", da, a), b) if need_b else None
        elif op in (4, 5):
            mask = (a >= b) if op == 4 else (a <= b)
            da, db = dy * mask, (dy * ~mask if need_b else None)
        else:            # pow
            da = dy * b * torch.pow(a, b - 1)
            db = dy * torch.pow(a, b) * torch.log(a) if need_b else None
        return da, db, None, None


def binary(name: str, a: torch.Tensor, b, alpha: float = 1.0) -> torch.Tensor:
    same = isinstance(b, torch.Tensor) and b.shape == a.shape and b.dtype == a.dtype
    if _on_device(a) and (same and _on_device(b) or isinstance(b, (int, float))):
        return _Binary.apply(a, b, BINARY[name], float(alpha))
    return {"add": lambda: torch.add(a, b, alpha=alpha), "sub": lambda: torch.sub(a, b, alpha=alpha), "mul": lambda: a * b,
            "div": lambda: a / b, "max": lambda: torch.maximum(a, torch.as_tensor(b, dtype=a.dtype, device=a.device)),
            "min": lambda: torch.minimum(a, torch.as_tensor(b, dtype=a.dtype, device=a.device)),
            "pow": lambda: torch.pow(a, b)}[name]()


def add(a, b, alpha: float = 1.0): return binary("add", a, b, alpha)
def sub(a, b, alpha: float = 1.0): return binary("sub", a, b, alpha)
def mul(a, b): return binary("mul", a, b)
def div(a, b): return binary("div", a, b)


class _Softmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, log_mode: bool):
        y = torch.empty_like(x2)
        _native.load(required=True).softmax_rows(x2, None, y, log_mode)
        ctx.save_for_backward(y)
        ctx.log_mode = log_mode
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        dx = torch.empty_like(y)
        _native.load(required=True).softmax_rows(y, dy.contiguous(), dx, ctx.log_mode)
        return dx, None


def _softmax(x: torch.Tensor, dim: int, log_mode: bool) -> torch.Tensor:
    if _on_device(x) and x.dim() >= 1:
        d = dim % x.dim()
        xt = x.movedim(d, -1) if d != x.dim() - 1 else x
        xc = xt.contiguous()
        y = _Softmax.apply(xc.view(-1, xc.shape[-1]), log_mode).view(xc.shape)
        return y.movedim(-1, d) if d != x.dim() - 1 else y
    return F.log_softmax(x, dim) if log_mode else F.softmax(x, dim)


def softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    return _softmax(x, dim, False)


def log_softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    return _softmax(x, dim, True)


_RMODES = {"sum": 0, "mean": 1, "max": 2, "min": 3, "var": 4}


def reduce_last(x: torch.Tensor, mode: str, unbiased: bool = True) -> torch.Tensor:
    """Reduction over the last dim; fp32 result.  (No autograd: used by statistics and validation code.)"""
    if _on_device(x) and x.dim() >= 1 and not x.requires_grad:
        xc = x.contiguous()
        out = torch.empty(xc.shape[:-1].numel(), dtype=torch.float32, device=x.device)
        _native.load(required=True).reduce_rows(xc.view(-1, xc.shape[-1]), out, _RMODES[mode], 1.0 if unbiased else 0.0)
        return out.view(xc.shape[:-1])
    xf = x.float()
    return {"sum": lambda: xf.sum(-1), "mean": lambda: xf.mean(-1), "max": lambda: xf.max(-1).values,
            "min": lambda: xf.min(-1).values, "var": lambda: xf.var(-1, unbiased=unbiased)}[mode]()
