"""Shared pieces of the convolution and pooling layers: parameter validation, output-size arithmetic and weight
initialisation (src/nn/conv_base.rs:103-375).  The layer constructors in ``layers.py`` call :class:`Validator`, so a
bad configuration fails when the layer is built, with the reference's messages, rather than at the first forward."""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch


def _seq(v) -> Tuple[int, ...]:
    return tuple(int(x) for x in v) if isinstance(v, (tuple, list)) else (int(v),)


class Validator:
    @staticmethod
    def validate_conv_params(in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1,
                             groups: int = 1) -> None:
        if in_channels <= 0 or out_channels <= 0:
            raise ValueError("Input and output channels must be positive")
        if groups <= 0:
            raise ValueError("Groups must be positive")
        if in_channels % groups:
            raise ValueError("Input channels must be divisible by groups")
        if out_channels % groups:
            raise ValueError("Output channels must be divisible by groups")
        if any(k <= 0 for k in _seq(kernel_size)):
            raise ValueError("Kernel size must be positive")
        if any(s <= 0 for s in _seq(stride)):
            raise ValueError("Stride must be positive")
        if any(d <= 0 for d in _seq(dilation)):
            raise ValueError("Dilation must be positive")
        named = isinstance(padding, str) or (isinstance(padding, (tuple, list)) and any(isinstance(p, str) for p in padding))
        if not named and any(p < 0 for p in _seq(padding)):
            raise ValueError("Padding must not be negative")

    @staticmethod
    def validate_pool_params(kernel_size, stride=None, padding=0) -> None:
        if any(k <= 0 for k in _seq(kernel_size)):
            raise ValueError("Kernel size must be positive")
        if stride is not None and any(s <= 0 for s in _seq(stride)):
            raise ValueError("Stride must be positive")
        ks, ps = _seq(kernel_size), _seq(padding)
        if len(ps) == 1:
            ps = ps * len(ks)
        if any(p < 0 or 2 * p > k for k, p in zip(ks, ps)):
            raise ValueError("Padding must be at most half of the kernel size")

    @staticmethod
    def validate_adaptive_output_size(output_size) -> None:
        if any(s is not None and s <= 0 for s in (output_size if isinstance(output_size, (tuple, list)) else (output_size,))):
            raise ValueError("Output size must be positive")


class ConvOps:
    @staticmethod
    def calc_output_size_1d(input_size: int, kernel_size: int, stride: int = 1, padding: int = 0, dilation: int = 1) -> int:
        span = input_size + 2 * padding - dilation * (kernel_size - 1) - 1
        if span < 0:
            raise ValueError(f"kernel extent {dilation * (kernel_size - 1) + 1} exceeds the padded input {input_size + 2 * padding}")
        return span // stride + 1

    @staticmethod
    def calc_output_size_2d(input_size, kernel_size, stride=(1, 1), padding=(0, 0), dilation=(1, 1)) -> Tuple[int, int]:
        return tuple(ConvOps.calc_output_size_1d(i, k, s, p, d)
                     for i, k, s, p, d in zip(input_size, kernel_size, stride, padding, dilation))

    @staticmethod
    def calc_output_size_3d(input_size, kernel_size, stride=(1, 1, 1), padding=(0, 0, 0), dilation=(1, 1, 1)) -> Tuple[int, int, int]:
        return tuple(ConvOps.calc_output_size_1d(i, k, s, p, d)
                     for i, k, s, p, d in zip(input_size, kernel_size, stride, padding, dilation))

    @staticmethod
    def calc_transposed_output_size_1d(input_size: int, kernel_size: int, stride: int = 1, padding: int = 0,
                                       output_padding: int = 0, dilation: int = 1) -> int:
        return (input_size - 1) * stride - 2 * padding + dilation * (kernel_size - 1) + output_padding + 1

    @staticmethod
    def init_conv_params(input_size: int, output_size: int, kernel_size, groups: int = 1, use_bias: bool = True,
                         device=None, dtype=None, generator: Optional[torch.Generator] = None):
        """``(weight [out, in / groups, *kernel], bias or None)``: normal weights with standard deviation
        ``sqrt(6 / fan_in)`` and a zero bias, the reference's rule (src/nn/conv_base.rs:215-262)."""
        ks = _seq(kernel_size)
        Validator.validate_conv_params(input_size, output_size, ks, groups=groups)
        fan_in = (input_size // groups) * math.prod(ks)
        w = torch.empty(output_size, input_size // groups, *ks, device=device, dtype=dtype)
        w.normal_(0.0, math.sqrt(6.0 / fan_in), generator=generator)
        w.requires_grad_(True)
        b = torch.zeros(output_size, device=device, dtype=dtype, requires_grad=True) if use_bias else None
        return w, b


def collect_conv_parameters(weight: torch.Tensor, bias: Optional[torch.Tensor]) -> Sequence[torch.Tensor]:
    return [weight] if bias is None else [weight, bias]
