"""Neural-network layers with RusTorch's constructor signatures and defaults.

``Module`` is ``torch.nn.Module`` (``forward / parameters / train / eval`` as in the reference's
trait, src/nn/mod.rs:50-147).  Each layer cites the reference definition whose argument order and
defaults it keeps.  Every layer is differentiable (the reference's conv / norm / activation
layers return variables with no ``grad_fn``, e.g. src/nn/conv2d.rs:263-267).  On CUDA with bf16
tensors Linear / LayerNorm / RMSNorm / attention run on the hand-written sm_100a kernels.
"""
from __future__ import annotations

import math
import os
from typing import List, Optional, Sequence, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import fused
from .conv_base import Validator

# fp32 CUDA Linear layers run on the tcgen05 GEMM as three bf16 products (RUSTORCH_FP32_LINEAR=library: cuBLAS SGEMM)
_FP32_NATIVE = os.environ.get("RUSTORCH_FP32_LINEAR", "native") != "library"

Module = nn.Module
Parameter = nn.Parameter
IntOrPair = Union[int, Tuple[int, int]]


def _native(x: torch.Tensor, *params: Optional[torch.Tensor]) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16
            and all(p is None or p.dtype == torch.bfloat16 for p in params))


class Sequential(nn.Sequential):
    """``add_module / get_module / len`` container (src/nn/mod.rs:90-147)."""

    def add(self, module: nn.Module) -> "Sequential":
        self.add_module(str(len(self)), module)
        return self

    def get_module(self, index: int) -> nn.Module:
        return self[index]

    def len(self) -> int:
        return len(self)


class Linear(nn.Module):
    """``Linear(input_size, output_size, bias=True)``: ``y = x W^T + b`` with weight ``[out, in]``.

    Weight AND bias are drawn from ``N(0, sqrt(2 / in))`` as in the reference
    (src/nn/linear.rs:72-115); ``new_no_bias`` is ``bias=False``.
    """

    def __init__(self, input_size: int, output_size: int, bias: Optional[bool] = True, device=None, dtype=None):
        super().__init__()
        if int(input_size) <= 0 or int(output_size) <= 0:
            raise ValueError("Linear: input_size and output_size must be positive")
        self.input_size, self.output_size = input_size, output_size
        std = math.sqrt(2.0 / input_size)
        kw = dict(device=device, dtype=dtype)
        self.weight = nn.Parameter(torch.empty(output_size, input_size, **kw).normal_(0, std))
        self.bias = nn.Parameter(torch.empty(output_size, **kw).normal_(0, std)) if bias is not False else None

    in_features = property(lambda self: self.input_size)
    out_features = property(lambda self: self.output_size)

    @classmethod
    def new_no_bias(cls, input_size: int, output_size: int, **kw) -> "Linear":
        return cls(input_size, output_size, bias=False, **kw)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.input_size % 8 == 0 and self.output_size % 8 == 0 and x.is_cuda:
            if _native(x, self.weight, self.bias):
                return fused.LinearFn.apply(x, self.weight, self.bias)
            if x.dtype == torch.float16 and self.weight.dtype == torch.float16 and fused.K._native.available():
                return fused.LinearF16Fn.apply(x, self.weight, self.bias)      # fp16 operands, fp32 accumulation
            if (x.dtype == torch.float32 and self.weight.dtype == torch.float32 and _FP32_NATIVE
                    and fused.K._native.available()):
                return fused.LinearF32Fn.apply(x, self.weight, self.bias)      # three bf16 GEMMs, fp32 accumulation
        return F.linear(x, self.weight, self.bias)


class _ConvNd(nn.Module):
    _fn = None
    _nd = 2

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 bias=True, device=None, dtype=None):
        super().__init__()
        nd = self._nd
        tup = lambda v: tuple(v) if isinstance(v, (tuple, list)) else (v,) * nd  # noqa: E731
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding, self.dilation = tup(kernel_size), tup(stride), tup(padding), tup(dilation)
        self.groups = groups
        Validator.validate_conv_params(in_channels, out_channels, self.kernel_size, self.stride, self.padding, self.dilation, groups)
        fan_in = in_channels // groups * math.prod(self.kernel_size)
        kw = dict(device=device, dtype=dtype)
        # Kaiming normal, std = sqrt(2 / fan_in) (src/nn/conv2d.rs:77-130)
        self.weight = nn.Parameter(torch.empty(out_channels, in_channels // groups, *self.kernel_size, **kw)
                                   .normal_(0, math.sqrt(2.0 / fan_in)))
        self.bias = nn.Parameter(torch.zeros(out_channels, **kw)) if bias else None

    def forward(self, x):
        return type(self)._fn(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups)

    def output_size(self, *spatial: int) -> Tuple[int, ...]:
        """``(H + 2p - d(k-1) - 1)/s + 1`` per spatial dim (src/nn/conv2d.rs:134-139)."""
        return tuple((n + 2 * p - d * (k - 1) - 1) // s + 1
                     for n, k, s, p, d in zip(spatial, self.kernel_size, self.stride, self.padding, self.dilation))


class Conv1d(_ConvNd):
    """``(in, out, kernel, stride=1, padding=0, dilation=1, groups=1, bias=True)`` (src/nn/conv1d.rs:121-135)."""
    _fn, _nd = staticmethod(F.conv1d), 1

    def forward(self, x):
        """bf16 CUDA layers with Cin, Cout multiples of 64 run as one-row images on the implicit-GEMM kernels."""
        from ..ops.conv import conv1d
        return conv1d(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups)


class Conv2d(_ConvNd):
    """``(in, out, kernel(h,w), stride=(1,1), padding=(0,0), bias=True)`` weight ``[oc, ic, kh, kw]`` (src/nn/conv2d.rs:77-88)."""
    _fn, _nd = staticmethod(F.conv2d), 2

    def __init__(self, in_channels, out_channels, kernel_size, stride=(1, 1), padding=(0, 0), bias=True,
                 dilation=1, groups=1, device=None, dtype=None):
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias, device, dtype)

    def forward(self, x):
        """bf16 CUDA layers with Cin, Cout multiples of 64 run on the implicit-GEMM tcgen05 kernels; others on the library."""
        from ..ops.conv import conv2d
        return conv2d(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups)


class Conv3d(_ConvNd):
    """``(in, out, kernel(d,h,w), stride, padding, dilation, groups, bias)`` (src/nn/conv3d.rs:74-90)."""
    _fn, _nd = staticmethod(F.conv3d), 3

    def forward(self, x):
        """bf16 CUDA tensors: patch gather + tcgen05 GEMM per group (+ patch scatter backward), csrc/conv/unfold_nd.cu."""
        from ..ops.conv_nd import conv_nd
        return conv_nd(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups)


class _ConvTransposeNd(nn.Module):
    _fn = None
    _nd = 2

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, output_padding=0, dilation=1,
                 groups=1, bias=True, device=None, dtype=None):
        super().__init__()
        nd = self._nd
        tup = lambda v: tuple(v) if isinstance(v, (tuple, list)) else (v,) * nd  # noqa: E731
        self.in_channels, self.out_channels, self.groups = in_channels, out_channels, groups
        self.kernel_size, self.stride, self.padding = tup(kernel_size), tup(stride), tup(padding)
        self.output_padding, self.dilation = tup(output_padding), tup(dilation)
        Validator.validate_conv_params(in_channels, out_channels, self.kernel_size, self.stride, self.padding, self.dilation, groups)
        if any(op >= max(st, d) for op, st, d in zip(self.output_padding, self.stride, self.dilation)):
            raise ValueError("Output padding must be smaller than either stride or dilation")
        fan_in = in_channels * math.prod(self.kernel_size)
        kw = dict(device=device, dtype=dtype)
        self.weight = nn.Parameter(torch.empty(in_channels, out_channels // groups, *self.kernel_size, **kw)
                                   .normal_(0, math.sqrt(2.0 / fan_in)))
        self.bias = nn.Parameter(torch.zeros(out_channels, **kw)) if bias else None

    def forward(self, x):
        """bf16 CUDA tensors: GEMM + patch scatter (the input-gradient form of a convolution), csrc/conv/unfold_nd.cu."""
        from ..ops.conv_nd import conv_transpose_nd
        return conv_transpose_nd(x, self.weight, self.bias, self.stride, self.padding, self.output_padding, self.groups, self.dilation)


class ConvTranspose1d(_ConvTransposeNd):
    """Transposed 1-D convolution: GEMM + patch scatter (src/nn/conv_transpose.rs)."""

    _fn, _nd = staticmethod(F.conv_transpose1d), 1


class ConvTranspose2d(_ConvTransposeNd):
    """``(in, out, kernel, stride, padding, output_padding, dilation, groups, bias)`` (src/nn/conv_transpose.rs:81-96)."""
    _fn, _nd = staticmethod(F.conv_transpose2d), 2

    def forward(self, x):
        """bf16 CUDA layers with Cin, Cout multiples of 64 run as the input-gradient form of the implicit-GEMM kernels."""
        from ..ops.conv import conv_transpose2d
        return conv_transpose2d(x, self.weight, self.bias, self.stride, self.padding, self.output_padding, self.groups, self.dilation)

    @classmethod
    def upsample_2x(cls, channels: int, **kw) -> "ConvTranspose2d":
        return cls(channels, channels, 4, stride=2, padding=1, **kw)

    @classmethod
    def upsample_4x(cls, channels: int, **kw) -> "ConvTranspose2d":
        return cls(channels, channels, 8, stride=4, padding=2, **kw)


class ConvTranspose3d(_ConvTransposeNd):
    """Transposed 3-D convolution: GEMM + patch scatter (src/nn/conv_transpose_3d.rs)."""

    _fn, _nd = staticmethod(F.conv_transpose3d), 3


class _BatchNorm(nn.modules.batchnorm._BatchNorm):
    """``(num_features, eps=1e-5, momentum=0.1, affine=True)``; gamma=1, beta=0; ``is_training()``,
    ``running_mean()/running_var()`` accessors (src/nn/batchnorm.rs:77-92,454-470)."""

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1, affine: bool = True,
                 track_running_stats: bool = True, device=None, dtype=None):
        super().__init__(num_features, eps, momentum, affine, track_running_stats, device=device, dtype=dtype)

    def forward(self, x, residual=None, relu: bool = False):
        """``relu(bn(x) + residual)`` when the optional arguments are given (the ResNet block tail, fused)."""
        self._check_input_dim(x)
        from ..ops.batchnorm import batch_norm
        momentum = 0.0 if self.momentum is None else self.momentum
        if self.training and self.track_running_stats and self.num_batches_tracked is not None:
            self.num_batches_tracked.add_(1)
            if self.momentum is None:
                momentum = 1.0 / float(self.num_batches_tracked)
        if self.running_mean is not None and self.running_mean.dtype != torch.float32 and x.is_cuda:
            # ``model.to(bf16)`` also casts the buffers; the statistics are kept (and updated by the kernel) in fp32
            self.running_mean = self.running_mean.float()
            self.running_var = self.running_var.float()
        rm = self.running_mean if (not self.training or self.track_running_stats) else None
        rv = self.running_var if (not self.training or self.track_running_stats) else None
        return batch_norm(x, rm, rv, self.weight, self.bias, self.training or rm is None, momentum, self.eps, residual, relu)

    def is_training(self) -> bool:
        return self.training

    def get_running_mean(self) -> torch.Tensor:
        return self.running_mean

    def get_running_var(self) -> torch.Tensor:
        return self.running_var


class BatchNorm1d(_BatchNorm):
    """Batch normalisation over ``[N, C]`` or ``[N, C, L]`` (src/nn/batchnorm.rs:77-92)."""

    def _check_input_dim(self, x):
        if x.dim() not in (2, 3):
            raise ValueError(f"expected 2D or 3D input (got {x.dim()}D)")


class BatchNorm2d(_BatchNorm):
    """Batch normalisation over ``[N, C, H, W]``; channels-last CUDA kernels for statistics, apply and backward (src/nn/batchnorm.rs)."""

    def _check_input_dim(self, x):
        if x.dim() != 4:
            raise ValueError(f"expected 4D input (got {x.dim()}D)")


class LayerNorm(nn.Module):
    """``(normalized_shape, eps=1e-5, elementwise_affine=True)`` (src/nn/normalization.rs:59-99)."""

    def __init__(self, normalized_shape: Union[int, Sequence[int]], eps: float = 1e-5,
                 elementwise_affine: bool = True, device=None, dtype=None):
        super().__init__()
        self.normalized_shape = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
        self.eps = eps
        kw = dict(device=device, dtype=dtype)
        if elementwise_affine:
            self.weight = nn.Parameter(torch.ones(self.normalized_shape, **kw))
            self.bias = nn.Parameter(torch.zeros(self.normalized_shape, **kw))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)

    def forward(self, x):
        n = math.prod(self.normalized_shape)
        if self.weight is not None and _native(x, self.weight, self.bias) and n % 8 == 0 and x.is_contiguous():
            return fused.LayerNormFn.apply(x, self.weight.reshape(-1), self.bias.reshape(-1), self.eps)
        return F.layer_norm(x, self.normalized_shape, self.weight, self.bias, self.eps)


class RMSNorm(nn.Module):
    """``x / sqrt(mean(x^2) + eps) * weight``, **eps default 1e-8**, weight = 1 (src/nn/normalization.rs:587-608,652-701)."""

    def __init__(self, normalized_shape: Union[int, Sequence[int]], eps: float = 1e-8, device=None, dtype=None):
        super().__init__()
        self.normalized_shape = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(self.normalized_shape, device=device, dtype=dtype))

    def forward(self, x):
        n = math.prod(self.normalized_shape)
        if _native(x, self.weight) and n % 8 == 0 and x.is_contiguous():
            return fused.RMSNormFn.apply(x, self.weight.reshape(-1), self.eps)
        dims = tuple(range(-len(self.normalized_shape), 0))
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(dims, keepdim=True) + self.eps)
        return (y * self.weight.float()).to(x.dtype)


class GroupNorm(nn.GroupNorm):
    """``(num_groups, num_channels, eps=1e-5, affine=True)`` (src/nn/normalization.rs:343-350); one CTA per
    (sample, group) slab on CUDA."""

    def forward(self, x):
        from ..ops.groupnorm import group_norm
        return group_norm(x, self.num_groups, self.weight, self.bias, self.eps)


class _InstanceNormNative:
    """Batch statistics on the slab kernel; layers that track running statistics (or evaluate with them) keep
    PyTorch's path."""

    def forward(self, x):
        if self.track_running_stats or x.dim() != self._rank:
            return super().forward(x)
        from ..ops.groupnorm import instance_norm
        return instance_norm(x, self.weight, self.bias, self.eps)


class InstanceNorm1d(_InstanceNormNative, nn.InstanceNorm1d):
    """``(num_features, eps=1e-5, momentum=0.1, affine, track_running_stats)`` (src/nn/instance_norm.rs:148-156)."""
    _rank = 3


class InstanceNorm2d(_InstanceNormNative, nn.InstanceNorm2d):
    """Instance normalisation over ``[N, C, H, W]`` (src/nn/instance_norm.rs:148-156)."""

    _rank = 4


class InstanceNorm3d(_InstanceNormNative, nn.InstanceNorm3d):
    """Instance normalisation over ``[N, C, D, H, W]`` (src/nn/instance_norm.rs)."""

    _rank = 5


from ..ops import pool as _pool  # noqa: E402


class Dropout(nn.Module):
    """``(p, inplace)``: training zeroes with probability p and scales by 1/(1-p); eval is identity
    (src/nn/dropout.rs:63,105-176)."""

    def __init__(self, p: float = 0.5, inplace: bool = False):
        super().__init__()
        if not 0.0 <= p <= 1.0:
            raise ValueError("dropout probability must be in [0, 1]")
        self.p, self.inplace = p, inplace

    def is_training(self) -> bool:
        return self.training

    def forward(self, x):
        return _pool.dropout(x, self.p, self.training, self.inplace)      # Philox kernel on CUDA, no mask tensor


class AlphaDropout(nn.AlphaDropout):
    """Dropout that keeps the self-normalising property of SELU networks (src/nn/dropout.rs:290-420)."""


Identity = nn.Identity


def dropout(x, p: float = 0.5, training: bool = True):
    return _pool.dropout(x, p, training)


class Flatten(nn.Flatten):
    """``Flatten(start_dim=1, end_dim=-1)`` (python/src/lib.rs)."""


class Embedding(nn.Module):
    """``(vocab_size, embedding_dim, padding_idx, max_norm, freeze)``: init ``N(0, 1/sqrt(dim))``,
    padding row zero, ``requires_grad = not freeze`` (src/nn/embedding.rs:63-112)."""

    def __init__(self, vocab_size: int, embedding_dim: int, padding_idx: Optional[int] = None,
                 max_norm: Optional[float] = None, freeze: bool = False, device=None, dtype=None):
        super().__init__()
        self.vocab_size, self.embedding_dim = vocab_size, embedding_dim
        self.padding_idx, self.max_norm = padding_idx, max_norm
        w = torch.empty(vocab_size, embedding_dim, device=device, dtype=dtype).normal_(0, 1.0 / math.sqrt(embedding_dim))
        if padding_idx is not None:
            w[padding_idx] = 0
        self.weight = nn.Parameter(w, requires_grad=not freeze)

    num_embeddings = property(lambda self: self.vocab_size)

    def forward(self, idx: torch.Tensor) -> torch.Tensor:
        return F.embedding(idx.long(), self.weight, self.padding_idx, self.max_norm)


class PositionalEmbedding(nn.Module):
    """Learned positions ``(max_length, dim)`` added to the input (src/nn/embedding.rs:297)."""

    def __init__(self, max_length: int, embedding_dim: int, device=None, dtype=None):
        super().__init__()
        self.max_length = max_length
        self.weight = nn.Parameter(torch.empty(max_length, embedding_dim, device=device, dtype=dtype)
                                   .normal_(0, 1.0 / math.sqrt(embedding_dim)))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        T = x.shape[-2]
        if T > self.max_length:
            raise ValueError(f"sequence length {T} exceeds max_length {self.max_length}")
        return x + self.weight[:T]


def sinusoidal_table(max_len: int, dim: int) -> torch.Tensor:
    pos = torch.arange(max_len, dtype=torch.float32).unsqueeze(1)
    div = torch.exp(torch.arange(0, dim, 2, dtype=torch.float32) * (-math.log(10000.0) / dim))
    pe = torch.zeros(max_len, dim)
    pe[:, 0::2] = torch.sin(pos * div)
    pe[:, 1::2] = torch.cos(pos * div)[:, : dim // 2]
    return pe


class SinusoidalPositionalEncoding(nn.Module):
    """Fixed sin/cos table ``(max_length, dim)`` (src/nn/embedding.rs:498)."""

    def __init__(self, max_length: int, embedding_dim: int):
        super().__init__()
        self.register_buffer("pe", sinusoidal_table(max_length, embedding_dim), persistent=False)

    def forward(self, x):
        return x + self.pe[: x.shape[-2]].to(x.dtype)


class PositionalEncoding(nn.Module):
    """``(d_model, max_len=5000)`` (+ dropout) (src/nn/transformer_phase6.rs:680-681)."""

    def __init__(self, d_model: int, max_len: int = 5000, dropout: float = 0.0):
        super().__init__()
        self.register_buffer("pe", sinusoidal_table(max_len, d_model), persistent=False)
        self.drop = nn.Dropout(dropout)

    def forward(self, x):
        return self.drop(x + self.pe[: x.shape[-2]].to(x.dtype))


# ------------------------------------------------------------------------ pooling
class MaxPool2d(nn.MaxPool2d):
    """``(kernel, stride=kernel, padding=(0,0))`` (src/nn/pool2d.rs:34-40)."""

    def __init__(self, kernel_size: IntOrPair, stride: Optional[IntOrPair] = None, padding: IntOrPair = 0):
        Validator.validate_pool_params(kernel_size, stride, padding)
        super().__init__(kernel_size, stride, padding)

    def forward(self, x):
        return _pool.max_pool2d(x, self.kernel_size, self.stride, self.padding)   # channels-last kernel on CUDA


class AvgPool2d(nn.AvgPool2d):
    def __init__(self, kernel_size: IntOrPair, stride: Optional[IntOrPair] = None, padding: IntOrPair = 0):
        Validator.validate_pool_params(kernel_size, stride, padding)
        super().__init__(kernel_size, stride, padding)

    def forward(self, x):
        return _pool.avg_pool2d(x, self.kernel_size, self.stride, self.padding)


class AdaptiveAvgPool2d(nn.AdaptiveAvgPool2d):
    """``(output_size)`` / ``global()`` (src/nn/adaptive_pool.rs:47,64)."""

    @classmethod
    def global_pool(cls) -> "AdaptiveAvgPool2d":
        return cls((1, 1))

    def forward(self, x):
        return _pool.adaptive_avg_pool2d(x, self.output_size)


class AdaptiveMaxPool2d(nn.AdaptiveMaxPool2d):
    @classmethod
    def global_pool(cls) -> "AdaptiveMaxPool2d":
        return cls((1, 1))

    def forward(self, x):
        return _pool.adaptive_max_pool2d(x, self.output_size)


# -------------------------------------------------------------------- activations
# On CUDA floating tensors these launch the native elementwise / softmax kernels (forward and backward);
# elsewhere they are the PyTorch expression of the same function.
from ..ops import elementwise as _ew  # noqa: E402


def relu(x):
    return _ew.unary("relu", x)


def sigmoid(x):
    return _ew.unary("sigmoid", x)


def tanh(x):
    return _ew.unary("tanh", x)


def leaky_relu(x, negative_slope: float = 0.01):
    return _ew.unary("leaky_relu", x, negative_slope)


def softmax(x, dim: int = -1):
    """Row-wise softmax over ``dim`` (the reference's attention normalises over the whole
    tensor by mistake, src/nn/attention.rs:362-384)."""
    return _ew.softmax(x, dim)


def log_softmax(x, dim: int = -1):
    return _ew.log_softmax(x, dim)


def gelu(x):
    """tanh approximation, as the reference (src/nn/activation.rs:206-217)."""
    return _ew.unary("gelu_tanh", x)


def swish(x):
    return _ew.unary("silu", x)


silu = swish


def elu(x, alpha: float = 1.0):
    return _ew.unary("elu", x, alpha)


def selu(x):
    return _ew.unary("selu", x)


def mish(x):
    return _ew.unary("mish", x)


def hardswish(x):
    return _ew.unary("hardswish", x)


def softplus(x, beta: float = 1.0, threshold: float = 20.0):
    return _ew.unary("softplus", x, beta, threshold)


def relu6(x):
    return _ew.unary("relu6", x)


def hardsigmoid(x):
    return _ew.unary("hardsigmoid", x)


def glu(x, dim: int = -1):
    return F.glu(x, dim)


def swiglu(x, dim: int = -1):
    """``swish(a) * b`` with ``[a, b] = split(x)`` (src/nn/activation.rs:378-419)."""
    a, b = x.chunk(2, dim)
    return F.silu(a) * b


def geglu(x, dim: int = -1):
    a, b = x.chunk(2, dim)
    return F.gelu(a, approximate="tanh") * b


def reglu(x, dim: int = -1):
    a, b = x.chunk(2, dim)
    return F.relu(a) * b


class ReLU(nn.ReLU):
    def forward(self, x):
        return relu(x)


class Sigmoid(nn.Sigmoid):
    def forward(self, x):
        return sigmoid(x)


class Tanh(nn.Tanh):
    def forward(self, x):
        return tanh(x)


class LeakyReLU(nn.LeakyReLU):
    def forward(self, x):
        return leaky_relu(x, self.negative_slope)


class Softmax(nn.Softmax):
    def __init__(self, dim: int = -1):
        super().__init__(dim)

    def forward(self, x):
        return softmax(x, self.dim)


class LogSoftmax(nn.LogSoftmax):
    def __init__(self, dim: int = -1):
        super().__init__(dim)

    def forward(self, x):
        return log_softmax(x, self.dim)


class GELU(nn.Module):
    def forward(self, x):
        return gelu(x)


class Swish(nn.SiLU):
    def forward(self, x):
        return swish(x)


class GLU(nn.GLU):
    """Gated linear unit: first half of ``dim`` times the sigmoid of the second half (src/nn/activation.rs)."""


class ELU(nn.ELU):
    def forward(self, x):
        return elu(x, self.alpha)


class SELU(nn.SELU):
    def forward(self, x):
        return selu(x)


class Mish(nn.Mish):
    def forward(self, x):
        return mish(x)


class Hardswish(nn.Hardswish):
    def forward(self, x):
        return hardswish(x)


class Softplus(nn.Softplus):
    def forward(self, x):
        return softplus(x, self.beta, self.threshold)


from .._interop import accept_wrappers as _accept_wrappers  # noqa: E402

_accept_wrappers(globals())       # forward() of the layers above also takes this package's Tensor / Variable
