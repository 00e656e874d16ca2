"""``rustorch.nn.functional``: the stateless forms of the layers (python/python/rustorch/nn.py:444-464 names ``relu``,
``mse_loss`` and ``cross_entropy``; the rest follow the layer set of this package).  Activations, softmax, dropout and
pooling run this package's CUDA kernels on GPU tensors; every function takes ``torch.Tensor``, ``Tensor`` or
``Variable`` arguments and answers in kind."""
from __future__ import annotations

import functools

import torch.nn.functional as _F

from .._interop import call_unwrapped
from ..ops import pool as _pool
from .layers import (dropout, elu, geglu, gelu, glu, hardsigmoid, hardswish, leaky_relu, log_softmax, mish, reglu, relu, relu6, selu,  # noqa: F401
                     sigmoid, softmax, softplus, swiglu, swish, tanh)
from .loss import (binary_cross_entropy, binary_cross_entropy_with_logits, cosine_embedding_loss, cross_entropy, focal_loss,  # noqa: F401
                   huber_loss, kl_div, l1_loss, margin_ranking_loss, mse_loss, nll_loss, smooth_l1_loss, triplet_margin_loss)

silu = swish


def _wrapped(fn):
    """Accept this package's wrappers around a function whose body reaches kernels through ``autograd.Function``."""
    @functools.wraps(fn)
    def call(*args, **kwargs):
        return call_unwrapped(fn, args, kwargs)
    return call


for _n in ("dropout", "elu", "geglu", "gelu", "glu", "hardsigmoid", "hardswish", "leaky_relu", "log_softmax", "mish", "reglu", "relu", "relu6",
           "selu", "sigmoid", "softmax", "softplus", "swiglu", "swish", "silu", "tanh", "binary_cross_entropy",
           "binary_cross_entropy_with_logits", "cosine_embedding_loss", "cross_entropy", "focal_loss", "huber_loss", "kl_div", "l1_loss",
           "margin_ranking_loss", "mse_loss", "nll_loss", "smooth_l1_loss", "triplet_margin_loss"):
    globals()[_n] = _wrapped(globals()[_n])


@_wrapped
def linear(input, weight, bias=None):
    return _F.linear(input, weight, bias)


@_wrapped
def max_pool2d(input, kernel_size, stride=None, padding=0):
    return _pool.max_pool2d(input, kernel_size, stride if stride is not None else kernel_size, padding)


@_wrapped
def avg_pool2d(input, kernel_size, stride=None, padding=0):
    return _pool.avg_pool2d(input, kernel_size, stride if stride is not None else kernel_size, padding)


@_wrapped
def adaptive_avg_pool2d(input, output_size):
    return _pool.adaptive_avg_pool2d(input, output_size)


@_wrapped
def layer_norm(input, normalized_shape, weight=None, bias=None, eps: float = 1e-5):
    return _F.layer_norm(input, tuple(normalized_shape) if not isinstance(normalized_shape, int) else (normalized_shape,), weight, bias, eps)


@_wrapped
def embedding(input, weight, padding_idx=None):
    return _F.embedding(input.long(), weight, padding_idx)


@_wrapped
def conv2d(input, weight, bias=None, stride=1, padding=0, dilation=1, groups=1):
    return _F.conv2d(input, weight, bias, stride, padding, dilation, groups)


@_wrapped
def one_hot(input, num_classes: int = -1):
    return _F.one_hot(input.long(), num_classes)


@_wrapped
def normalize(input, p: float = 2.0, dim: int = 1, eps: float = 1e-12):
    return _F.normalize(input, p, dim, eps)


@_wrapped
def scaled_dot_product_attention(query, key, value, attn_mask=None, dropout_p: float = 0.0, is_causal: bool = False):
    return _F.scaled_dot_product_attention(query, key, value, attn_mask, dropout_p, is_causal)
