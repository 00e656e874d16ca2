"""Fused gate arithmetic of LSTM / GRU cells (csrc/nn/rnn_amp_sparse.cu).

The two projections of a cell (``x W_ih^T + b_ih`` and ``h W_hh^T + b_hh``) are GEMMs; everything after them - four
(three) activations and the state update - is one kernel forward and one backward instead of a dozen elementwise ops.
Gate order ``[i, f, g, o]`` for LSTM and ``[r, z, n]`` for GRU, as in the reference (src/nn/lstm_cell.rs:84-126,
src/nn/gru_cell.rs) and in PyTorch.
"""
from __future__ import annotations

from typing import Tuple

import torch

from .. import _native

_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def on_device(*ts: torch.Tensor) -> bool:
    return all(t.is_cuda and t.dtype in _DTYPES for t in ts) and len({t.dtype for t in ts}) == 1 and _native.available()


class _LstmGates(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gates, c):
        C = _native.load(required=True)
        act = gates.contiguous().clone()                   # becomes the activated gates
        c = c.contiguous()
        h_new, c_new = torch.empty_like(c), torch.empty_like(c)
        C.lstm_gates_fwd(act, c, h_new, c_new)
        ctx.save_for_backward(act, c, c_new)
        return h_new, c_new

    @staticmethod
    def backward(ctx, dh, dc_new):
        act, c, c_new = ctx.saved_tensors
        C = _native.load(required=True)
        dgates, dc = torch.empty_like(act), torch.empty_like(c)
        C.lstm_gates_bwd(act, c, c_new, dh.contiguous() if dh is not None else None,
                         dc_new.contiguous() if dc_new is not None else None, dgates, dc)
        return dgates, dc


class _GruGates(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gi, gh, h):
        C = _native.load(required=True)
        gi, gh, h = gi.contiguous(), gh.contiguous(), h.contiguous()
        h_new = torch.empty_like(h)
        save = torch.empty((h.shape[0], 4 * h.shape[1]), dtype=h.dtype, device=h.device)
        C.gru_gates_fwd(gi, gh, h, h_new, save)
        ctx.save_for_backward(save, h)
        return h_new

    @staticmethod
    def backward(ctx, dh_new):
        save, h = ctx.saved_tensors
        C = _native.load(required=True)
        B, H = h.shape
        dgi = torch.empty((B, 3 * H), dtype=h.dtype, device=h.device)
        dgh, dh = torch.empty_like(dgi), torch.empty_like(h)
        C.gru_gates_bwd(save, h, dh_new.contiguous(), dgi, dgh, dh)
        return dgi, dgh, dh


def lstm_gates(gates: torch.Tensor, c: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``gates [B, 4H]`` (pre-activation, order i f g o), ``c [B, H]`` -> ``(h', c')``."""
    if on_device(gates, c):
        return _LstmGates.apply(gates, c)
    i, f, g, o = gates.chunk(4, 1)
    c_new = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
    return torch.sigmoid(o) * torch.tanh(c_new), c_new


def gru_gates(gi: torch.Tensor, gh: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
    """``gi = x W_ih^T + b_ih``, ``gh = h W_hh^T + b_hh`` (both ``[B, 3H]``, order r z n) -> ``h'``."""
    if on_device(gi, gh, h):
        return _GruGates.apply(gi, gh, h)
    ir, iz, in_ = gi.chunk(3, 1)
    hr, hz, hn = gh.chunk(3, 1)
    r, z = torch.sigmoid(ir + hr), torch.sigmoid(iz + hz)
    n = torch.tanh(in_ + r * hn)
    return (1 - z) * n + z * h
