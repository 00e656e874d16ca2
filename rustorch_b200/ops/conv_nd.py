"""Convolutions the implicit-GEMM conv2d kernels do not cover (Conv3d, grouped and dilated Conv1d / Conv2d / Conv3d,
ConvTranspose1d / 2d-with-groups / 3d) on this package's own kernels: a patch gather (``unfold_nd``), one tcgen05 GEMM
per group (batched over the groups) and, for input gradients and transposed convolutions, a patch scatter
(``fold_nd``) - csrc/conv/unfold_nd.cu + csrc/gemm/gemm_tcgen05.cu.

    conv        : col = unfold(x)            y  = col W^T (+ bias)
      d weight  :                            dW = dy^T col              (fp32 accumulation)
      d input   : dcol = dy W                dx = fold(dcol)
    transposed  : col = x W (W: [Cin, Cout_g * taps])   y = fold(col) (+ bias)   -- the input gradient of a convolution
      d weight  : dW = x^T unfold(dy)        d input : dx = unfold(dy) W^T

Everything runs on channels-last bf16 tensors; ``conv_nd`` / ``conv_transpose_nd`` accept the usual ``[N, C, *spatial]``
tensors of 1 to 3 spatial dimensions and return the same.  CPU tensors and other dtypes take ``torch.nn.functional``
(which is also the oracle of the tests).  Reference: a scalar conv3d kernel with groups and dilation
(src/gpu/cuda_kernels.cu:133-198) and host loops in src/nn/conv3d.rs:74-237, src/nn/conv_transpose_3d.rs,
src/nn/conv1d.rs:121-135.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import _native
from . import kernels as K


def _triple(v, nd: int, fill: int) -> Tuple[int, int, int]:
    """Geometry of an nd-dimensional convolution as (depth, height, width) with neutral values in front."""
    t = (int(v),) * nd if isinstance(v, int) else tuple(int(e) for e in v)
    assert len(t) == nd, f"expected {nd} values, got {t}"
    return (fill,) * (3 - nd) + t


def native_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and _native.available() and 3 <= x.dim() <= 5


def _to_cl(x: torch.Tensor) -> torch.Tensor:
    """[N, C, *sp] -> contiguous channels-last [N, D, H, W, C] (singleton leading spatial dims for 1-D / 2-D)."""
    nd = x.dim() - 2
    x5 = x.reshape(x.shape[0], x.shape[1], *([1] * (3 - nd)), *x.shape[2:])
    return x5.permute(0, 2, 3, 4, 1).contiguous()


def _from_cl(y: torch.Tensor, nd: int) -> torch.Tensor:
    """[N, D, H, W, C] -> [N, C, *sp] (a channels-last view, no copy)."""
    y = y.permute(0, 4, 1, 2, 3)
    return y.reshape(y.shape[0], y.shape[1], *y.shape[5 - nd:])


def _out_size(inp: Sequence[int], k, s, p, d) -> Tuple[int, int, int]:
    return tuple((inp[i] + 2 * p[i] - d[i] * (k[i] - 1) - 1) // s[i] + 1 for i in range(3))


def _k_pad(k: int) -> int:
    return -(-k // 8) * 8


def _unfold(x_cl: torch.Tensor, out_sp, kernel, stride, pad, dil, groups: int) -> torch.Tensor:
    N, _, _, _, C = x_cl.shape
    M = N * out_sp[0] * out_sp[1] * out_sp[2]
    kk = kernel[0] * kernel[1] * kernel[2] * (C // groups)
    col = torch.empty((groups, M, _k_pad(kk)), dtype=torch.bfloat16, device=x_cl.device)
    _native.load(required=True).unfold_nd(x_cl, col, list(out_sp), list(kernel), list(stride), list(pad), list(dil), groups, False)
    return col


def _fold(col: torch.Tensor, in_shape_cl, out_sp, kernel, stride, pad, dil, groups: int) -> torch.Tensor:
    x = torch.empty(in_shape_cl, dtype=torch.bfloat16, device=col.device)
    _native.load(required=True).unfold_nd(x, col, list(out_sp), list(kernel), list(stride), list(pad), list(dil), groups, True)
    return x


def _w_matrix(w: torch.Tensor, groups: int) -> torch.Tensor:
    """Conv weight [Cout, Cg, *k] -> [groups, pad8(Cout_g), k_pad] with the patch order (taps major, channel minor) of
    unfold.  Rows and columns are zero-padded to multiples of 8 so that every TMA row of the GEMM is 16-byte aligned."""
    Cout, Cg = w.shape[0], w.shape[1]
    taps = w[0, 0].numel()
    co = Cout // groups
    wm = w.reshape(Cout, Cg, taps).permute(0, 2, 1).reshape(groups, co, taps * Cg)
    kp, cp = _k_pad(taps * Cg), _k_pad(co)
    if kp != taps * Cg or cp != co:
        wm = F.pad(wm, (0, kp - taps * Cg, 0, cp - co))
    return wm.contiguous()


def _w_matrix_grad(dwm: torch.Tensor, w_shape, groups: int) -> torch.Tensor:
    Cout, Cg = w_shape[0], w_shape[1]
    taps = 1
    for e in w_shape[2:]:
        taps *= e
    co = Cout // groups
    return dwm[:, :co, :taps * Cg].reshape(Cout, taps, Cg).permute(0, 2, 1).reshape(w_shape)


def _group_cols(y_g: torch.Tensor, n_real: int) -> torch.Tensor:
    """[groups, M, pad8(n)] -> [M, groups * n]."""
    G, M, _ = y_g.shape
    y_g = y_g[:, :, :n_real]
    return y_g[0] if G == 1 else y_g.permute(1, 0, 2).reshape(M, G * n_real)


def _split_cols(y: torch.Tensor, groups: int) -> torch.Tensor:
    """[M, groups * n] -> contiguous [groups, M, pad8(n)] (zero columns appended)."""
    M, C = y.shape
    n = C // groups
    y_g = y.view(1, M, C) if groups == 1 else y.view(M, groups, n).permute(1, 0, 2)
    if n % 8:
        y_g = F.pad(y_g, (0, _k_pad(n) - n))
    return y_g.contiguous()


class ConvNdFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, stride, pad, dil, groups: int):
        nd = x.dim() - 2
        kernel = _triple(tuple(w.shape[2:]), nd, 1)
        x_cl = _to_cl(x)
        out_sp = _out_size(x_cl.shape[1:4], kernel, stride, pad, dil)
        col = _unfold(x_cl, out_sp, kernel, stride, pad, dil, groups)           # [G, M, kp]
        wm = _w_matrix(w, groups)                                               # [G, Cout_g, kp]
        y_g = K.gemm(col, wm)                                                   # [G, M, Cout_g]
        y = _group_cols(y_g, w.shape[0] // groups)
        if bias is not None:
            y = y + bias.to(y.dtype)
        N = x.shape[0]
        y_cl = y.reshape(N, *out_sp, w.shape[0])
        ctx.save_for_backward(col, wm, w)
        ctx.geom = (x_cl.shape, out_sp, kernel, stride, pad, dil, groups, nd, bias is not None)
        return _from_cl(y_cl, nd)

    @staticmethod
    def backward(ctx, dy):
        col, wm, w = ctx.saved_tensors
        x_shape_cl, out_sp, kernel, stride, pad, dil, groups, nd, has_bias = ctx.geom
        Cout = w.shape[0]
        dy2 = _to_cl(dy).reshape(-1, Cout)                                      # [M, Cout]
        dy_g = _split_cols(dy2, groups)                                         # [G, M, Cout_g]
        dx = dw = db = None
        if ctx.needs_input_grad[1]:
            dwm = K.gemm(dy_g, col, a_mn=True, b_mn=True, out_dtype=torch.float32, accumulate=True)   # [G, Cout_g, kp]
            dw = _w_matrix_grad(dwm, w.shape, groups).to(w.dtype)
        if has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(w.dtype)
        if ctx.needs_input_grad[0]:
            dcol = K.gemm(dy_g, wm, b_mn=True)                                  # [G, M, kp]
            dx_cl = _fold(dcol, tuple(x_shape_cl), out_sp, kernel, stride, pad, dil, groups)
            dx = _from_cl(dx_cl, nd)
        return dx, dw, db, None, None, None, None


class ConvTransposeNdFn(torch.autograd.Function):
    """``w``: [Cin, Cout_g, *k] as in ``torch.nn.ConvTranspose*``."""

    @staticmethod
    def forward(ctx, x, w, bias, stride, pad, out_pad, dil, groups: int):
        nd = x.dim() - 2
        kernel = _triple(tuple(w.shape[2:]), nd, 1)
        Cin, Cout_g = w.shape[0], w.shape[1]
        Cout = Cout_g * groups
        x_cl = _to_cl(x)                                                         # the "dy" of the equivalent convolution
        in_sp = tuple(x_cl.shape[1:4])
        out_sp = tuple((in_sp[i] - 1) * stride[i] - 2 * pad[i] + dil[i] * (kernel[i] - 1) + out_pad[i] + 1 for i in range(3))
        # equivalent convolution: weight [Cin, Cout_g, *k] maps Cout -> Cin; its patch matrix is [G, Cin_g, taps * Cout_g]
        wm = _w_matrix(w, groups)                                                # [G, Cin_g, kp]
        x_g = _split_cols(x_cl.reshape(-1, Cin), groups)                         # [G, M, Cin_g]
        col = K.gemm(x_g, wm, b_mn=True)                                         # [G, M, kp]
        N = x.shape[0]
        y_cl = _fold(col, (N, *out_sp, Cout), in_sp, kernel, stride, pad, dil, groups)
        if bias is not None:
            y_cl = y_cl + bias.to(y_cl.dtype)
        ctx.save_for_backward(x_g, wm, w)
        ctx.geom = (in_sp, out_sp, kernel, stride, pad, dil, groups, nd, bias is not None, Cout)
        return _from_cl(y_cl, nd)

    @staticmethod
    def backward(ctx, dy):
        x_g, wm, w = ctx.saved_tensors
        in_sp, out_sp, kernel, stride, pad, dil, groups, nd, has_bias, Cout = ctx.geom
        dy_cl = _to_cl(dy)                                                       # [N, *out_sp, Cout]
        col = _unfold(dy_cl, in_sp, kernel, stride, pad, dil, groups)            # [G, M, kp]: patches of dy at every input position
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx_g = K.gemm(col, wm)                                               # [G, M, Cin_g]
            N = dy.shape[0]
            dx_cl = _group_cols(dx_g, w.shape[0] // groups).reshape(N, *in_sp, w.shape[0])
            dx = _from_cl(dx_cl, nd)
        if ctx.needs_input_grad[1]:
            dwm = K.gemm(x_g, col, a_mn=True, b_mn=True, out_dtype=torch.float32, accumulate=True)    # [G, Cin_g, kp]
            dw = _w_matrix_grad(dwm, w.shape, groups).to(w.dtype)
        if has_bias and ctx.needs_input_grad[2]:
            db = dy_cl.reshape(-1, Cout).float().sum(0).to(w.dtype)
        return dx, dw, db, None, None, None, None, None


def conv_nd(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, stride=1, padding=0, dilation=1,
            groups: int = 1) -> torch.Tensor:
    """1-3 D convolution; bf16 CUDA tensors run on unfold + tcgen05 GEMM, everything else on ``torch.nn.functional``."""
    nd = x.dim() - 2
    if native_ok(x, w) and not isinstance(padding, str):
        return ConvNdFn.apply(x, w, bias, _triple(stride, nd, 1), _triple(padding, nd, 0), _triple(dilation, nd, 1), int(groups))
    return (F.conv1d, F.conv2d, F.conv3d)[nd - 1](x, w, bias, stride, padding, dilation, groups)


def conv_transpose_nd(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, stride=1, padding=0,
                      output_padding=0, groups: int = 1, dilation=1) -> torch.Tensor:
    nd = x.dim() - 2
    if native_ok(x, w):
        return ConvTransposeNdFn.apply(x, w, bias, _triple(stride, nd, 1), _triple(padding, nd, 0), _triple(output_padding, nd, 0),
                                       _triple(dilation, nd, 1), int(groups))
    return (F.conv_transpose1d, F.conv_transpose2d, F.conv_transpose3d)[nd - 1](x, w, bias, stride, padding, output_padding, groups, dilation)
