"""Pooling and dropout on the native kernels (csrc/nn/pool_dropout.cu).

Pooling works on channels-last storage: an NCHW tensor in ``torch.channels_last`` memory format is passed to the kernel
as the ``[N, H, W, C]`` array it already is (other inputs are converted once).  Max pooling records the window position
of each maximum in one byte, which is all the backward pass reads besides ``dy``.  Dropout draws its bits from
Philox4x32-10 keyed by ``(seed, offset)``; backward regenerates them, so no mask tensor exists.  On CPU, for dtypes or
channel counts the kernels do not take, and for windows they do not cover (dilation, ceil mode) the functions fall
back to PyTorch.  Reference: src/nn/pool2d.rs:34-330, src/nn/adaptive_pool.rs:47-260, src/nn/dropout.rs:63-176.
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch
import torch.nn.functional as F

from .. import _native

IntOrPair = Union[int, Tuple[int, int]]
_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def _pair(v) -> Tuple[int, int]:
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


def supported(x: torch.Tensor, kernel: Tuple[int, int]) -> bool:
    if not (x.is_cuda and x.dim() == 4 and x.dtype in _DTYPES and _native.available()):
        return False
    vec = 4 if x.dtype == torch.float32 else 8
    return x.shape[1] % vec == 0 and kernel[0] * kernel[1] <= 255 and x.numel() > 0


def _nhwc(x: torch.Tensor) -> torch.Tensor:
    """[N, H, W, C] contiguous view (a copy only if the tensor is not channels-last already)."""
    return x.permute(0, 2, 3, 1).contiguous()


class _Pool2d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, is_max, k, s, p):
        C = _native.load(required=True)
        xh = _nhwc(x)
        N, H, W, Ch = xh.shape
        OH, OW = (H + 2 * p[0] - k[0]) // s[0] + 1, (W + 2 * p[1] - k[1]) // s[1] + 1
        y = torch.empty((N, OH, OW, Ch), dtype=x.dtype, device=x.device)
        idx = torch.empty((N, OH, OW, Ch), dtype=torch.uint8, device=x.device) if is_max else None
        C.pool2d(xh, y, idx, is_max, False, k[0], k[1], s[0], s[1], p[0], p[1])
        ctx.geom = (is_max, k, s, p, (N, H, W, Ch))
        if is_max:
            ctx.save_for_backward(idx)
        return y.permute(0, 3, 1, 2)                       # NCHW view of channels-last storage

    @staticmethod
    def backward(ctx, dy):
        is_max, k, s, p, shape = ctx.geom
        C = _native.load(required=True)
        dyh = _nhwc(dy)
        dx = torch.empty(shape, dtype=dy.dtype, device=dy.device)
        idx = ctx.saved_tensors[0] if is_max else None
        C.pool2d(dx, dyh, idx, is_max, True, k[0], k[1], s[0], s[1], p[0], p[1])
        return dx.permute(0, 3, 1, 2), None, None, None, None


def max_pool2d(x: torch.Tensor, kernel_size: IntOrPair, stride: Optional[IntOrPair] = None, padding: IntOrPair = 0) -> torch.Tensor:
    k = _pair(kernel_size)
    s = _pair(stride) if stride is not None else k
    p = _pair(padding)
    if supported(x, k):
        return _Pool2d.apply(x, True, k, s, p)
    return F.max_pool2d(x, k, s, p)


def avg_pool2d(x: torch.Tensor, kernel_size: IntOrPair, stride: Optional[IntOrPair] = None, padding: IntOrPair = 0) -> torch.Tensor:
    k = _pair(kernel_size)
    s = _pair(stride) if stride is not None else k
    p = _pair(padding)
    if supported(x, k):
        return _Pool2d.apply(x, False, k, s, p)
    return F.avg_pool2d(x, k, s, p)


def adaptive_avg_pool2d(x: torch.Tensor, output_size: IntOrPair) -> torch.Tensor:
    """Native when the output divides the input evenly (global pooling included): a plain average pool then."""
    if not isinstance(output_size, int) and any(v is None for v in output_size):
        return F.adaptive_avg_pool2d(x, output_size)
    o = _pair(output_size)
    if x.dim() == 4 and x.shape[2] % o[0] == 0 and x.shape[3] % o[1] == 0:
        k = (x.shape[2] // o[0], x.shape[3] // o[1])
        if supported(x, k):
            return _Pool2d.apply(x, False, k, k, (0, 0))
    return F.adaptive_avg_pool2d(x, o)


def adaptive_max_pool2d(x: torch.Tensor, output_size: IntOrPair) -> torch.Tensor:
    if not isinstance(output_size, int) and any(v is None for v in output_size):
        return F.adaptive_max_pool2d(x, output_size)
    o = _pair(output_size)
    if x.dim() == 4 and x.shape[2] % o[0] == 0 and x.shape[3] % o[1] == 0:
        k = (x.shape[2] // o[0], x.shape[3] // o[1])
        if supported(x, k):
            return _Pool2d.apply(x, True, k, k, (0, 0))
    return F.adaptive_max_pool2d(x, o)


# ------------------------------------------------------------------------------------------------ dropout
_offsets = {}


def _next_offset(device: torch.device, numel: int) -> Tuple[int, int]:
    """(seed, offset) for the next dropout call on a device: the seed follows ``torch.manual_seed``, the offset
    advances by one per call (the element index is the Philox counter, the offset is part of the counter word)."""
    seed = torch.initial_seed() & 0x7FFFFFFFFFFFFFFF
    key = (device.index, seed)
    off = _offsets.get(key, 0)
    _offsets[key] = off + 1
    return seed, off


def _dense(x: torch.Tensor) -> bool:
    """Memory is one gap-free block (any dimension order that PyTorch names a memory format)."""
    if x.is_contiguous():
        return True
    if x.dim() == 4:
        return x.is_contiguous(memory_format=torch.channels_last)
    if x.dim() == 5:
        return x.is_contiguous(memory_format=torch.channels_last_3d)
    return False


class _Dropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed, offset):
        C = _native.load(required=True)
        xc = x if _dense(x) else x.contiguous()   # the mask is indexed by memory offset
        y = torch.empty_like(xc)
        C.dropout(xc, y, p, seed, offset)
        ctx.args = (p, seed, offset, y.stride())
        return y

    @staticmethod
    def backward(ctx, dy):
        p, seed, offset, strides = ctx.args
        C = _native.load(required=True)
        dyc = dy if dy.stride() == strides else torch.empty_strided(dy.shape, strides, dtype=dy.dtype, device=dy.device).copy_(dy)
        dx = torch.empty_like(dyc)
        C.dropout(dyc, dx, p, seed, offset)
        return dx, None, None, None


def dropout(x: torch.Tensor, p: float = 0.5, training: bool = True, inplace: bool = False) -> torch.Tensor:
    if not training or p == 0.0:
        return x
    if p >= 1.0:
        return x.mul_(0.0) if inplace else torch.zeros_like(x)
    vec = 4 if x.dtype == torch.float32 else 8
    if x.is_cuda and not inplace and x.dtype in _DTYPES and x.numel() % vec == 0 and x.numel() > 0 and _native.available():
        seed, off = _next_offset(x.device, x.numel())
        return _Dropout.apply(x, float(p), seed, off)
    return F.dropout(x, p, True, inplace)
