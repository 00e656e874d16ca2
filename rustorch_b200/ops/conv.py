"""Conv2d on the implicit-GEMM tcgen05 kernels (csrc/conv/conv2d_igemm.cu), with autograd.

Tensors are channels-last: an NCHW tensor in ``torch.channels_last`` memory format IS an NHWC array, and a weight
``[Cout, Cin, KH, KW]`` in channels-last format IS ``[Cout, KH, KW, Cin]``, so the kernels read both without copies.
Forward and the weight gradient always use the native kernels when the layer qualifies (Cin % 64 == 0, Cout % 8 == 0,
groups 1, dilation 1, square stride / padding); the input gradient does for stride 1 (it is the forward kernel on ``dy``
with the filter rotated and its channel axes swapped) and falls back to the library for strided layers.
Layers these kernels do not cover (groups, dilation, other channel counts) go to :mod:`rustorch_b200.ops.conv_nd`
(patch gather + tcgen05 GEMM + patch scatter).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from .. import _native


def _all_one(v) -> bool:
    return v == 1 if isinstance(v, int) else all(int(e) == 1 for e in v)


def supported(x: torch.Tensor, weight: torch.Tensor, stride, padding, dilation=1, groups: int = 1) -> bool:
    s = stride if isinstance(stride, int) else stride[0]
    p = padding if isinstance(padding, int) else padding[0]
    if not (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 4 and _native.available()):
        return False
    if groups != 1 or not _all_one(dilation):
        return False
    if not isinstance(stride, int) and stride[0] != stride[1]:
        return False
    if isinstance(padding, str) or isinstance(p, str):
        return False
    Cout, Cin, KH, KW = weight.shape
    return Cin % 64 == 0 and Cout % 64 == 0 and KH <= 7 and KW <= 7 and 1 <= s <= 4


def _nhwc(t: torch.Tensor) -> torch.Tensor:
    """NCHW-shaped tensor -> contiguous [N, H, W, C] view (copy only if it was not channels-last)."""
    return t.permute(0, 2, 3, 1).contiguous()


def _pads(padding) -> tuple:
    return (padding, padding) if isinstance(padding, int) else (int(padding[0]), int(padding[-1]))


def _strided_dgrad(C, dyh: torch.Tensor, wh: torch.Tensor, xshape, stride: int, pad_h: int, pad_w: Optional[int] = None
                   ) -> Optional[torch.Tensor]:
    """Input gradient of a strided convolution as ``stride^2`` stride-1 convolutions of ``dy``, one per parity class
    of the input pixels: class ``(ph, pw)`` only receives the taps with ``kh = ph + pad (mod stride)`` (same for kw),
    and its pixels form a dense grid, so the forward kernel computes it with a sub-filter and scatters the results to
    every ``stride``-th pixel of ``dx``.  Classes without taps (1x1 kernels) stay zero.  ``None``: geometry not covered."""
    N, H, W, Cin = xshape
    Cout, KH, KW, _ = wh.shape
    pad_w = pad_h if pad_w is None else pad_w

    def taps(ph: int, K: int, pad: int):
        ks = [k for k in range(K) if (ph + pad - k) % stride == 0]
        offs = [(ph + pad - k) // stride for k in ks]            # dy index = y + off, descending k -> ascending off
        return ks[::-1], offs[::-1]

    plans = []
    for ph in range(stride):
        khs, offh = taps(ph, KH, pad_h)
        for pw in range(stride):
            kws, offw = taps(pw, KW, pad_w)
            rows, cols = -(-(H - ph) // stride), -(-(W - pw) // stride)
            if rows <= 0 or cols <= 0 or not khs or not kws:
                plans.append(None)
                continue
            # a stride-1 correlation needs consecutive offsets starting at -pad' with pad' >= 0, the same for h and w
            if offh != list(range(offh[0], offh[0] + len(offh))) or offw != list(range(offw[0], offw[0] + len(offw))):
                return None
            if offh[0] > 0 or offw[0] > 0:
                return None
            plans.append((ph, pw, khs, kws, -offh[0], -offw[0], rows, cols))
    full = all(pl is not None for pl in plans)
    dx = (torch.empty if full else torch.zeros)((N, H, W, Cin), dtype=torch.bfloat16, device=dyh.device)
    for pl in plans:
        if pl is None:
            continue
        ph, pw, khs, kws, p2h, p2w, rows, cols = pl
        # sub-filter [Cin][n_h][n_w][Cout]: the contraction runs over the layer's output channels
        sub = wh[:, khs][:, :, kws].permute(3, 1, 2, 0).contiguous()
        C.conv2d_fwd_scatter(dyh, sub, dx, p2w, rows, cols, stride, ph, pw, pad_h=p2h)
    return dx


class Conv2dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, stride: int, pad):
        C = _native.load(required=True)
        xh, wh = _nhwc(x), _nhwc(weight)                       # [N,H,W,Cin], [Cout,KH,KW,Cin]
        N, H, W, _ = xh.shape
        Cout, KH, KW, _ = wh.shape
        pad_h, pad_w = _pads(pad)
        OH, OW = (H + 2 * pad_h - KH) // stride + 1, (W + 2 * pad_w - KW) // stride + 1
        out = torch.empty(N, OH, OW, Cout, dtype=torch.bfloat16, device=x.device)
        C.conv2d_fwd(xh, wh, out, bias, stride, pad_w, pad_h=pad_h)
        ctx.save_for_backward(xh, wh)
        ctx.geom = (stride, pad, bias is not None, tuple(x.shape))
        # flat-parameter training keeps conv filters in [Cout, KH, KW, Cin] order: dW accumulates straight into the fp32 buffer
        ctx.main_grad = weight.main_grad if getattr(weight, "_flat_ohwi", False) and hasattr(weight, "main_grad") else None
        return out.permute(0, 3, 1, 2)                          # NCHW shape, channels-last memory

    @staticmethod
    def backward(ctx, dy):
        C = _native.load(required=True)
        xh, wh = ctx.saved_tensors
        stride, pad, has_bias, xshape = ctx.geom
        pad_h, pad_w = _pads(pad)
        dyh = _nhwc(dy)
        Cout, KH, KW, Cin = wh.shape
        dx = dw = db = None
        if ctx.needs_input_grad[1] and ctx.main_grad is not None:
            C.conv2d_wgrad(xh, dyh, ctx.main_grad.view(Cout, KH, KW, Cin), stride, pad_w, pad_h=pad_h)
        elif ctx.needs_input_grad[1]:
            dwf = torch.zeros(Cout, KH, KW, Cin, dtype=torch.float32, device=dyh.device)
            C.conv2d_wgrad(xh, dyh, dwf, stride, pad_w, pad_h=pad_h)
            dw = dwf.to(torch.bfloat16).permute(0, 3, 1, 2)    # back to [Cout, Cin, KH, KW] (channels-last memory)
        if ctx.needs_input_grad[0]:
            if stride == 1 and KH - 1 - pad_h >= 0 and KW - 1 - pad_w >= 0:
                # full correlation of dy with the rotated filter: w'[ci][kh][kw][co] = w[co][KH-1-kh][KW-1-kw][ci]
                wr = wh.flip(1, 2).permute(3, 1, 2, 0).contiguous()
                dxh = torch.empty(xh.shape, dtype=torch.bfloat16, device=dyh.device)
                C.conv2d_fwd(dyh, wr, dxh, None, 1, KW - 1 - pad_w, pad_h=KH - 1 - pad_h)
                dx = dxh.permute(0, 3, 1, 2)
            else:
                dxh = _strided_dgrad(C, dyh, wh, xh.shape, stride, pad_h, pad_w)
                dx = dxh.permute(0, 3, 1, 2) if dxh is not None else \
                    torch.nn.grad.conv2d_input(xshape, wh.permute(0, 3, 1, 2), dy, stride, (pad_h, pad_w))
        if has_bias and ctx.needs_input_grad[2]:
            db = dyh.float().sum((0, 1, 2)).to(torch.bfloat16)
        return dx, dw, db, None, None


def im2col_supported(x: torch.Tensor, weight: torch.Tensor, stride, padding, dilation=1, groups: int = 1) -> bool:
    """Few input channels (a network's stem): patch matrix + tcgen05 GEMM.  The input must not need a gradient."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 4 and _native.available()):
        return False
    if x.requires_grad or groups != 1 or not _all_one(dilation):
        return False
    if not isinstance(stride, int) and stride[0] != stride[1] or not isinstance(padding, int) and padding[0] != padding[1]:
        return False
    if isinstance(padding if isinstance(padding, int) else padding[0], str):
        return False
    Cout, Cin, KH, KW = weight.shape
    return Cin % 64 != 0 and Cin * KH * KW <= 512 and Cout % 8 == 0


class Im2colConv2dFn(torch.autograd.Function):
    """``y = col(x) @ W^T`` with ``col`` written once by csrc/conv/im2col.cu and kept for the weight gradient
    ``dW = dy^T @ col`` (both products on the tcgen05 GEMM; the second in its weight-gradient layout with split-K)."""

    @staticmethod
    def forward(ctx, x, weight, bias, stride: int, pad: int):
        from . import kernels as K
        C = _native.load(required=True)
        xh, wh = _nhwc(x), _nhwc(weight)                       # [N,H,W,Cin], [Cout,KH,KW,Cin]
        N, H, W, Cin = xh.shape
        Cout, KH, KW, _ = wh.shape
        OH, OW = (H + 2 * pad - KH) // stride + 1, (W + 2 * pad - KW) // stride + 1
        k_real = KH * KW * Cin
        k_pad = -(-k_real // 64) * 64
        col = torch.empty(N * OH * OW, k_pad, dtype=torch.bfloat16, device=x.device)
        C.im2col_nhwc(xh, col, KH, KW, stride, pad)
        w2 = torch.zeros(Cout, k_pad, dtype=torch.bfloat16, device=x.device)
        w2[:, :k_real] = wh.reshape(Cout, k_real)
        out = K.gemm(col, w2, bias=bias)                       # [N*OH*OW, Cout] = NHWC output
        ctx.save_for_backward(col)
        ctx.geom = (Cout, KH, KW, Cin, k_real, bias is not None)
        return out.view(N, OH, OW, Cout).permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dy):
        from . import kernels as K
        (col,) = ctx.saved_tensors
        Cout, KH, KW, Cin, k_real, has_bias = ctx.geom
        dy2 = _nhwc(dy).reshape(-1, Cout)
        dw = db = None
        if ctx.needs_input_grad[1]:
            dwf = torch.zeros(Cout, col.shape[1], dtype=torch.float32, device=dy.device)
            K.gemm(dy2, col, a_mn=True, b_mn=True, out=dwf, accumulate=True,
                   split_k=torch.cuda.get_device_properties(dy2.device).multi_processor_count)
            dw = dwf[:, :k_real].reshape(Cout, KH, KW, Cin).to(torch.bfloat16).permute(0, 3, 1, 2)
        if has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(torch.bfloat16)
        return None, dw, db, None, None


def conv2d(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, stride=1, padding=0, dilation=1,
           groups: int = 1) -> torch.Tensor:
    if im2col_supported(x, weight, stride, padding, dilation, groups):
        s = stride if isinstance(stride, int) else stride[0]
        p = padding if isinstance(padding, int) else padding[0]
        return Im2colConv2dFn.apply(x, weight, bias, s, p)
    if supported(x, weight, stride, padding, dilation, groups):
        s = stride if isinstance(stride, int) else stride[0]
        return Conv2dFn.apply(x, weight, bias, s, _pads(padding))
    from .conv_nd import conv_nd      # groups, dilation, other channel counts: unfold + tcgen05 GEMM (library on the CPU)
    return conv_nd(x, weight, bias, stride, padding, dilation, groups)


def _one(v) -> int:
    return v if isinstance(v, int) else int(v[0])


def conv1d(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, stride=1, padding=0, dilation=1,
           groups: int = 1) -> torch.Tensor:
    """``[N, C, L]`` convolution as a one-row image on the 2-D kernels (padding along the length only)."""
    if (x.dim() == 3 and not isinstance(padding, str) and _all_one(dilation) and groups == 1 and _one(stride) <= 4
            and supported(x.unsqueeze(2), weight.unsqueeze(2), _one(stride), (0, _one(padding)))):
        y = Conv2dFn.apply(x.unsqueeze(2), weight.unsqueeze(2), bias, _one(stride), (0, _one(padding)))
        return y.squeeze(2)
    from .conv_nd import conv_nd
    return conv_nd(x, weight, bias, stride, padding, dilation, groups)


class ConvTranspose2dFn(torch.autograd.Function):
    """Transposed convolution = the input gradient of the convolution with the same weight: forward runs the (strided)
    dgrad path, the gradient with respect to the input is a plain forward convolution of ``dy``, the weight gradient is
    the convolution's weight gradient with the roles of input and output swapped."""

    @staticmethod
    def forward(ctx, x, weight, stride: int, pad: int, out_pad: int):
        C = _native.load(required=True)
        xh = _nhwc(x)                                           # [N,H,W,Cin]: the "dy" of the underlying convolution
        wh = _nhwc(weight)                                      # weight [Cin, Cout, KH, KW] -> [Cin, KH, KW, Cout]
        N, H, W, Cin = xh.shape
        _, KH, KW, Cout = wh.shape
        OH, OW = (H - 1) * stride - 2 * pad + KH + out_pad, (W - 1) * stride - 2 * pad + KW + out_pad
        if stride == 1:
            wr = wh.flip(1, 2).permute(3, 1, 2, 0).contiguous()
            out = torch.empty(N, OH, OW, Cout, dtype=torch.bfloat16, device=x.device)
            C.conv2d_fwd(xh, wr, out, None, 1, KW - 1 - pad, pad_h=KH - 1 - pad)
        else:
            out = _strided_dgrad(C, xh, wh, (N, OH, OW, Cout), stride, pad)
            if out is None:
                raise RuntimeError("conv_transpose2d: geometry not covered by the native path")
        ctx.save_for_backward(xh, wh)
        ctx.geom = (stride, pad)
        return out.permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dy):
        C = _native.load(required=True)
        xh, wh = ctx.saved_tensors
        stride, pad = ctx.geom
        dyh = _nhwc(dy)                                         # [N,OH,OW,Cout]: the input of the underlying convolution
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dxh = torch.empty(xh.shape, dtype=torch.bfloat16, device=dyh.device)
            C.conv2d_fwd(dyh, wh, dxh, None, stride, pad)
            dx = dxh.permute(0, 3, 1, 2)
        if ctx.needs_input_grad[1]:
            dwf = torch.zeros(wh.shape, dtype=torch.float32, device=dyh.device)
            C.conv2d_wgrad(dyh, xh, dwf, stride, pad)
            dw = dwf.to(torch.bfloat16).permute(0, 3, 1, 2)
        return dx, dw, None, None, None


def conv_transpose2d_supported(x, weight, stride, padding, output_padding, dilation, groups) -> bool:
    if not (x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and _native.available()):
        return False
    s, p, op = _pads(stride), _pads(padding), _pads(output_padding)
    if s[0] != s[1] or p[0] != p[1] or op[0] != op[1] or not _all_one(dilation) or groups != 1 or not 1 <= s[0] <= 4:
        return False
    Cin, Cout, KH, KW = weight.shape
    if Cin % 64 or Cout % 64 or KH > 7 or KW > 7 or KH - 1 - p[0] < 0 or KW - 1 - p[0] < 0 or op[0] >= s[0]:
        return False
    return KH >= s[0] and KW >= s[0]                 # every parity class of the output sees at least one tap


def conv_transpose2d(x, weight, bias=None, stride=1, padding=0, output_padding=0, groups: int = 1, dilation=1) -> torch.Tensor:
    if conv_transpose2d_supported(x, weight, stride, padding, output_padding, dilation, groups):
        try:
            y = ConvTranspose2dFn.apply(x, weight, _one(stride), _one(padding), _one(output_padding))
            return y if bias is None else y + bias.view(1, -1, 1, 1)
        except RuntimeError as e:
            if "not covered" not in str(e):
                raise
    from .conv_nd import conv_transpose_nd
    return conv_transpose_nd(x, weight, bias, stride, padding, output_padding, groups, dilation)
