"""Whole-sequence RNN / LSTM / GRU passes of one layer and one direction as autograd Functions.

Forward: the input projection of ALL time steps is one GEMM (``[T*B, In] x W_ih^T``); every step is then one
recurrent GEMM (``h W_hh^T`` with the step's input projection added in the GEMM epilogue) and one fused gate kernel
(csrc/nn/rnn_amp_sparse.cu).  Backward walks the steps in reverse with one gate-backward kernel and one GEMM per
step (``dh_{t-1} = dgates_t W_hh``, the output gradient of step t-1 added in the epilogue) and finishes with ONE
weight-gradient GEMM per weight over the stacked steps (``dW_hh = dGates^T H_prev``, ``dW_ih = dGates^T X``), one
column sum per bias and one GEMM for ``dX``.  On bf16 CUDA tensors every GEMM is the tcgen05 kernel
(csrc/gemm/gemm_tcgen05.cu); other dtypes and CPU tensors evaluate the same schedule with torch matmuls, which is
also how the CPU tests check the schedule against ``torch.nn.LSTM / GRU / RNN``.

Gate order ``[i, f, g, o]`` (LSTM) and ``[r, z, n]`` (GRU), as in the reference (src/nn/lstm_cell.rs:84-126,
src/nn/gru_cell.rs, src/nn/rnn.rs:451-462) and in PyTorch, so state dicts are interchangeable.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native
from . import elementwise as E
from . import kernels as K
from . import rnn as G


def _native_ok(*ts: torch.Tensor) -> bool:
    """bf16 CUDA tensors whose inner sizes keep every TMA row 16-byte aligned."""
    return (_native.available() and all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts)
            and all(t.shape[-1] % 8 == 0 for t in ts))


def _mm_nt(a, w, bias=None, residual=None, out=None):
    """``a @ w^T (+ bias) (+ residual)``; a [M, K], w [N, K]; written into ``out`` when given."""
    if _native_ok(a, w) and (bias is None or bias.dtype == torch.bfloat16):
        a = a.contiguous()
        if residual is not None:
            return K.gemm(a, w, bias=bias, aux=residual.contiguous(), epilogue=K.EPI_RESIDUAL, out=out)
        return K.gemm(a, w, bias=bias, out=out)
    res = a @ w.t()
    if bias is not None:
        res = res + bias
    if residual is not None:
        res = res + residual
    if out is not None:
        out.copy_(res)
        return out
    return res


def _mm_nn(a, w, residual=None):
    """``a @ w (+ residual)``; a [M, N], w [N, K] (the input-gradient product, w read as stored)."""
    if _native_ok(a, w):
        a = a.contiguous()
        if residual is not None:
            return K.gemm(a, w, b_mn=True, aux=residual.contiguous(), epilogue=K.EPI_RESIDUAL)
        return K.gemm(a, w, b_mn=True)
    out = a @ w
    return out + residual if residual is not None else out


def _wgrad(dy2d, x2d, like):
    """``dy2d^T @ x2d`` in fp32, returned in the dtype of ``like``."""
    if _native_ok(dy2d, x2d):
        g = K.gemm(dy2d.contiguous(), x2d.contiguous(), a_mn=True, b_mn=True, out_dtype=torch.float32, accumulate=True)
        return g.to(like.dtype)
    acc = torch.float64 if dy2d.dtype == torch.float64 else torch.float32
    return (dy2d.to(acc).t() @ x2d.to(acc)).to(like.dtype)


def _colsum(dy2d, like):
    if dy2d.is_cuda and dy2d.dtype == torch.bfloat16 and _native.available() and dy2d.shape[1] % 8 == 0:
        out = torch.zeros(dy2d.shape[1], dtype=torch.float32, device=dy2d.device)
        K.colsum_accum(dy2d.contiguous(), out)
        return out.to(like.dtype)
    return dy2d.to(torch.float64 if dy2d.dtype == torch.float64 else torch.float32).sum(0).to(like.dtype)


def _zeros_like_h(x, B, H):
    return torch.zeros(B, H, dtype=x.dtype, device=x.device)


def _stack_prev(h0, h_all):
    """[h0, h_1 .. h_{T-1}] as one [T*B, H] matrix: row block t holds the state that ENTERED step t."""
    return torch.cat([h0.unsqueeze(0), h_all[:-1]], 0).reshape(-1, h0.shape[-1])


def _order(T: int, reverse: bool):
    return range(T - 1, -1, -1) if reverse else range(T)


class LSTMSeqFn(torch.autograd.Function):
    """x [T, B, In], h0 / c0 [B, H] -> (out [T, B, H], h_T, c_T).  ``reverse`` walks the sequence backwards in time."""

    @staticmethod
    def forward(ctx, x, h0, c0, w_ih, w_hh, b_ih, b_hh, reverse: bool):
        T, B, _ = x.shape
        H = w_hh.shape[1]
        x2 = x.reshape(T * B, -1)
        bias = None
        if b_ih is not None:
            bias = b_ih + b_hh if b_hh is not None else b_ih
        gi = _mm_nt(x2, w_ih, bias).view(T, B, 4 * H)
        use_kernel = G.on_device(gi, c0)
        out = torch.empty(T, B, H, dtype=x.dtype, device=x.device)
        act = torch.empty(T, B, 4 * H, dtype=x.dtype, device=x.device)     # activated gates of every step
        c_all = torch.empty(T, B, H, dtype=x.dtype, device=x.device)
        h, c = h0.contiguous(), c0.contiguous()
        C = _native.load(required=True) if use_kernel else None
        for t in _order(T, reverse):
            gates = _mm_nt(h, w_hh, None, gi[t], out=act[t])       # pre-activations land in the step's slot
            if use_kernel:
                C.lstm_gates_fwd(act[t], c, out[t], c_all[t])      # ... and are activated in place
            else:
                i, f, g, o = gates.clone().chunk(4, 1)
                a = torch.cat([torch.sigmoid(i), torch.sigmoid(f), torch.tanh(g), torch.sigmoid(o)], 1)
                act[t].copy_(a)
                i, f, g, o = a.chunk(4, 1)
                c_all[t].copy_(f * c + i * g)
                out[t].copy_(o * torch.tanh(c_all[t]))
            h, c = out[t], c_all[t]
        ctx.save_for_backward(x, h0, c0, w_ih, w_hh, out, act, c_all)
        ctx.meta = (reverse, b_ih is not None, b_hh is not None, use_kernel)
        last = 0 if reverse else T - 1
        return out, out[last].clone(), c_all[last].clone()

    @staticmethod
    def backward(ctx, d_out, d_hT, d_cT):
        x, h0, c0, w_ih, w_hh, out, act, c_all = ctx.saved_tensors
        reverse, has_bih, has_bhh, use_kernel = ctx.meta
        T, B, H = out.shape
        d_out = d_out.contiguous() if d_out is not None else torch.zeros_like(out)
        dgates = torch.empty_like(act)
        C = _native.load(required=True) if use_kernel else None
        steps = list(_order(T, reverse))[::-1]                    # last processed step first
        dh = d_out[steps[0]] if d_hT is None else E.add(d_out[steps[0]], d_hT.to(d_out.dtype))
        dc = d_cT.contiguous().to(d_out.dtype) if d_cT is not None else _zeros_like_h(x, B, H)
        c0 = c0.contiguous()
        for n, t in enumerate(steps):
            nxt = steps[n + 1] if n + 1 < T else None
            c_in = c_all[nxt] if nxt is not None else c0          # cell state that entered step t
            if use_kernel:
                dc_new = torch.empty_like(dc)
                C.lstm_gates_bwd(act[t], c_in, c_all[t], dh.contiguous(), dc.contiguous(), dgates[t], dc_new)
                dc = dc_new
            else:
                i, f, g, o = act[t].chunk(4, 1)
                tc = torch.tanh(c_all[t])
                dct = dc + dh * o * (1 - tc * tc)
                dgates[t].copy_(torch.cat([dct * g * i * (1 - i), dct * c_in * f * (1 - f), dct * i * (1 - g * g),
                                           dh * tc * o * (1 - o)], 1))
                dc = dct * f
            # gradient that reaches the previous step's h: through W_hh, plus that step's own output gradient
            dh = _mm_nn(dgates[t], w_hh, d_out[nxt] if nxt is not None else None)
        dg2 = dgates.view(T * B, 4 * H)
        if reverse:
            h_prev = torch.cat([out[1:], h0.unsqueeze(0)], 0).reshape(T * B, H)
        else:
            h_prev = _stack_prev(h0, out)
        x2 = x.reshape(T * B, -1)
        d_whh = _wgrad(dg2, h_prev, w_hh)
        d_wih = _wgrad(dg2, x2, w_ih)
        db = _colsum(dg2, w_ih) if (has_bih or has_bhh) else None
        dx = _mm_nn(dg2, w_ih).view(x.shape) if ctx.needs_input_grad[0] else None
        return dx, dh, dc, d_wih, d_whh, (db if has_bih else None), (db if has_bhh else None), None


class GRUSeqFn(torch.autograd.Function):
    """x [T, B, In], h0 [B, H] -> (out [T, B, H], h_T)."""

    @staticmethod
    def forward(ctx, x, h0, w_ih, w_hh, b_ih, b_hh, reverse: bool):
        T, B, _ = x.shape
        H = w_hh.shape[1]
        gi = _mm_nt(x.reshape(T * B, -1), w_ih, b_ih).view(T, B, 3 * H)
        use_kernel = G.on_device(gi, h0)
        out = torch.empty(T, B, H, dtype=x.dtype, device=x.device)
        save = torch.empty(T, B, 4 * H, dtype=x.dtype, device=x.device)    # r, z, n, (W_hn h + b_hn) of every step
        h = h0.contiguous()
        C = _native.load(required=True) if use_kernel else None
        for t in _order(T, reverse):
            gh = _mm_nt(h, w_hh, b_hh)
            if use_kernel:
                C.gru_gates_fwd(gi[t].contiguous(), gh, h.contiguous(), out[t], save[t])
            else:
                ir, iz, in_ = gi[t].chunk(3, 1)
                hr, hz, hn = gh.chunk(3, 1)
                r, z = torch.sigmoid(ir + hr), torch.sigmoid(iz + hz)
                n = torch.tanh(in_ + r * hn)
                save[t].copy_(torch.cat([r, z, n, hn], 1))
                out[t].copy_((1 - z) * n + z * h)
            h = out[t]
        ctx.save_for_backward(x, h0, w_ih, w_hh, out, save)
        ctx.meta = (reverse, b_ih is not None, b_hh is not None, use_kernel)
        return out, out[0 if reverse else T - 1].clone()

    @staticmethod
    def backward(ctx, d_out, d_hT):
        x, h0, w_ih, w_hh, out, save = ctx.saved_tensors
        reverse, has_bih, has_bhh, use_kernel = ctx.meta
        T, B, H = out.shape
        d_out = d_out.contiguous() if d_out is not None else torch.zeros_like(out)
        dgi = torch.empty(T, B, 3 * H, dtype=x.dtype, device=x.device)
        dgh = torch.empty_like(dgi)
        C = _native.load(required=True) if use_kernel else None
        steps = list(_order(T, reverse))[::-1]
        dh = d_out[steps[0]] if d_hT is None else E.add(d_out[steps[0]], d_hT.to(d_out.dtype))
        for n, t in enumerate(steps):
            nxt = steps[n + 1] if n + 1 < T else None
            h_in = out[nxt] if nxt is not None else h0
            if use_kernel:
                dh_direct = torch.empty_like(h0)
                C.gru_gates_bwd(save[t], h_in.contiguous(), dh.contiguous(), dgi[t], dgh[t], dh_direct)
            else:
                r, z, nn_, hn = save[t].chunk(4, 1)
                dn = dh * (1 - z) * (1 - nn_ * nn_)
                dz = dh * (h_in - nn_) * z * (1 - z)
                dr = dn * hn * r * (1 - r)
                dgi[t].copy_(torch.cat([dr, dz, dn], 1))
                dgh[t].copy_(torch.cat([dr, dz, dn * r], 1))
                dh_direct = dh * z
            carry = dh_direct if nxt is None else E.add(dh_direct, d_out[nxt])
            dh = _mm_nn(dgh[t], w_hh, carry)
        dgi2, dgh2 = dgi.view(T * B, 3 * H), dgh.view(T * B, 3 * H)
        if reverse:
            h_prev = torch.cat([out[1:], h0.unsqueeze(0)], 0).reshape(T * B, H)
        else:
            h_prev = _stack_prev(h0, out)
        d_whh = _wgrad(dgh2, h_prev, w_hh)
        d_wih = _wgrad(dgi2, x.reshape(T * B, -1), w_ih)
        d_bih = _colsum(dgi2, w_ih) if has_bih else None
        d_bhh = _colsum(dgh2, w_ih) if has_bhh else None
        dx = _mm_nn(dgi2, w_ih).view(x.shape) if ctx.needs_input_grad[0] else None
        return dx, dh, d_wih, d_whh, d_bih, d_bhh, None


class RNNSeqFn(torch.autograd.Function):
    """Elman RNN: ``h_t = act(x_t W_ih^T + b_ih + h_{t-1} W_hh^T + b_hh)`` with ``act`` = tanh or relu."""

    @staticmethod
    def forward(ctx, x, h0, w_ih, w_hh, b_ih, b_hh, reverse: bool, nonlinearity: str):
        T, B, _ = x.shape
        H = w_hh.shape[1]
        bias = None
        if b_ih is not None:
            bias = b_ih + b_hh if b_hh is not None else b_ih
        gi = _mm_nt(x.reshape(T * B, -1), w_ih, bias).view(T, B, H)
        out = torch.empty(T, B, H, dtype=x.dtype, device=x.device)
        h = h0.contiguous()
        for t in _order(T, reverse):
            pre = _mm_nt(h, w_hh, None, gi[t])
            out[t].copy_(E.unary(nonlinearity, pre))
            h = out[t]
        ctx.save_for_backward(x, h0, w_ih, w_hh, out)
        ctx.meta = (reverse, b_ih is not None, b_hh is not None, nonlinearity)
        return out, out[0 if reverse else T - 1].clone()

    @staticmethod
    def backward(ctx, d_out, d_hT):
        x, h0, w_ih, w_hh, out = ctx.saved_tensors
        reverse, has_bih, has_bhh, nonlinearity = ctx.meta
        T, B, H = out.shape
        d_out = d_out.contiguous() if d_out is not None else torch.zeros_like(out)
        dpre = torch.empty_like(out)
        steps = list(_order(T, reverse))[::-1]
        dh = d_out[steps[0]] if d_hT is None else E.add(d_out[steps[0]], d_hT.to(d_out.dtype))
        for n, t in enumerate(steps):
            y = out[t]
            deriv = (1 - y * y) if nonlinearity == "tanh" else (y > 0).to(y.dtype)     # both derivatives in terms of the output
            dpre[t].copy_(E.mul(dh.contiguous(), deriv.contiguous()))
            nxt = steps[n + 1] if n + 1 < T else None
            dh = _mm_nn(dpre[t], w_hh, d_out[nxt] if nxt is not None else None)
        dp2 = dpre.view(T * B, H)
        if reverse:
            h_prev = torch.cat([out[1:], h0.unsqueeze(0)], 0).reshape(T * B, H)
        else:
            h_prev = _stack_prev(h0, out)
        d_whh = _wgrad(dp2, h_prev, w_hh)
        d_wih = _wgrad(dp2, x.reshape(T * B, -1), w_ih)
        db = _colsum(dp2, w_ih) if (has_bih or has_bhh) else None
        dx = _mm_nn(dp2, w_ih).view(x.shape) if ctx.needs_input_grad[0] else None
        return dx, dh, d_wih, d_whh, (db if has_bih else None), (db if has_bhh else None), None, None


def lstm_layer(x, h0, c0, w_ih, w_hh, b_ih, b_hh, reverse: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return LSTMSeqFn.apply(x, h0, c0, w_ih, w_hh, b_ih, b_hh, reverse)


def gru_layer(x, h0, w_ih, w_hh, b_ih, b_hh, reverse: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    return GRUSeqFn.apply(x, h0, w_ih, w_hh, b_ih, b_hh, reverse)


def rnn_layer(x, h0, w_ih, w_hh, b_ih, b_hh, reverse: bool = False, nonlinearity: str = "tanh") -> Tuple[torch.Tensor, torch.Tensor]:
    return RNNSeqFn.apply(x, h0, w_ih, w_hh, b_ih, b_hh, reverse, nonlinearity)
