"""Recurrent layers: ``RNNCell/RNN``, ``LSTMCell/LSTM``, ``GRUCell/GRU``.

Constructor order ``(input_size, hidden_size, num_layers=1, bias=True, batch_first=False, dropout=0.0,
bidirectional=False)`` and the LSTM gate order ``[i, f, g, o]`` follow the reference
(src/nn/rnn.rs:451-462, src/nn/lstm_layer.rs:56-92, src/nn/lstm_cell.rs:84-126,
src/nn/gru_layer.rs:56-68).  Cells: ``forward(x, state=None)``; LSTM state is ``(h, c)``.

The whole-sequence layers are this package's own modules (not ``torch.nn.LSTM`` subclasses, so no cuDNN): each
layer and direction is one :mod:`rustorch_b200.ops.rnn_seq` Function: one GEMM projects the inputs of all time
steps, each step is one recurrent GEMM plus one fused gate kernel, and the backward pass ends in one weight-gradient
GEMM per weight over the stacked steps.  Parameter names (``weight_ih_l0``, ``weight_hh_l0_reverse``, ...) and
layouts are PyTorch's, so state dicts load both ways.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import rnn as _rnn_ops
from ..ops import rnn_seq as _seq


def _linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
    """``x W^T + b``: the tcgen05 GEMM (with autograd) for bf16 CUDA operands, ``F.linear`` otherwise."""
    if _seq._native_ok(x, w) and (b is None or b.dtype == torch.bfloat16):
        from .fused import LinearFn
        return LinearFn.apply(x, w, b)
    return F.linear(x, w, b)


class RNNCell(nn.RNNCell):
    """Elman cell ``h' = act(W_ih x + b_ih + W_hh h + b_hh)`` (src/nn/rnn.rs)."""

    def __init__(self, input_size: int, hidden_size: int, bias: bool = True, nonlinearity: str = "tanh", **kw):
        super().__init__(input_size, hidden_size, bias, nonlinearity, **kw)


class LSTMCell(nn.LSTMCell):
    """``forward(x, (h, c) | None) -> (h, c)``; weights stacked ``[i, f, g, o]``."""

    def forward(self, x: torch.Tensor, state: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        if x.dim() != 2:
            return super().forward(x, state)
        if state is None:
            z = torch.zeros(x.shape[0], self.hidden_size, dtype=x.dtype, device=x.device)
            state = (z, z)
        h, c = state
        gates = _linear(x, self.weight_ih, self.bias_ih) + _linear(h, self.weight_hh, self.bias_hh)
        return _rnn_ops.lstm_gates(gates, c)          # one fused kernel on CUDA


class GRUCell(nn.GRUCell):
    def forward(self, x: torch.Tensor, h: Optional[torch.Tensor] = None):
        if x.dim() != 2:
            return super().forward(x, h)
        if h is None:
            h = torch.zeros(x.shape[0], self.hidden_size, dtype=x.dtype, device=x.device)
        return _rnn_ops.gru_gates(_linear(x, self.weight_ih, self.bias_ih), _linear(h, self.weight_hh, self.bias_hh), h)


class _RecurrentBase(nn.Module):
    """Multi-layer, optionally bidirectional recurrent stack over :mod:`rustorch_b200.ops.rnn_seq`."""

    _GATES = 1
    mode = "RNN"

    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, bias: bool = True, batch_first: bool = False,
                 dropout: float = 0.0, bidirectional: bool = False, device=None, dtype=None):
        super().__init__()
        if num_layers < 1 or hidden_size < 1:
            raise ValueError("num_layers and hidden_size must be positive")
        if not 0.0 <= dropout <= 1.0:
            raise ValueError("dropout must be in [0, 1]")
        self.input_size, self.hidden_size, self.num_layers = input_size, hidden_size, num_layers
        self.bias, self.batch_first, self.dropout, self.bidirectional = bias, batch_first, float(dropout), bidirectional
        kw = {"device": device, "dtype": dtype}
        dirs = 2 if bidirectional else 1
        g = self._GATES * hidden_size
        self._flat_names: List[List[str]] = []
        for layer in range(num_layers):
            in_l = input_size if layer == 0 else hidden_size * dirs
            for d in range(dirs):
                sfx = f"_l{layer}" + ("_reverse" if d == 1 else "")
                names = [f"weight_ih{sfx}", f"weight_hh{sfx}"]
                self.register_parameter(names[0], nn.Parameter(torch.empty(g, in_l, **kw)))
                self.register_parameter(names[1], nn.Parameter(torch.empty(g, hidden_size, **kw)))
                if bias:
                    names += [f"bias_ih{sfx}", f"bias_hh{sfx}"]
                    self.register_parameter(names[2], nn.Parameter(torch.empty(g, **kw)))
                    self.register_parameter(names[3], nn.Parameter(torch.empty(g, **kw)))
                self._flat_names.append(names)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        k = 1.0 / math.sqrt(self.hidden_size)
        for p in self.parameters():
            nn.init.uniform_(p, -k, k)

    def init_hidden(self, batch: int, device=None, dtype=None):
        n = self.num_layers * (2 if self.bidirectional else 1)
        p = next(self.parameters())
        return torch.zeros(n, batch, self.hidden_size, device=device or p.device, dtype=dtype or p.dtype)

    def _params_of(self, layer: int, d: int):
        names = self._flat_names[layer * (2 if self.bidirectional else 1) + d]
        ps = [getattr(self, n) for n in names]
        return ps + [None, None] if not self.bias else ps

    # one layer, one direction: returns (out [T, B, H], final states...)
    def _run(self, x, state, params, reverse):
        raise NotImplementedError

    def _split_state(self, hx, batch, x):
        raise NotImplementedError

    def forward(self, x: torch.Tensor, hx=None):
        unbatched = x.dim() == 2
        if unbatched:
            x = x.unsqueeze(1)
        elif self.batch_first:
            x = x.transpose(0, 1)
        x = x.contiguous()
        T, B, _ = x.shape
        dirs = 2 if self.bidirectional else 1
        states = self._split_state(hx, B, x, unbatched)
        finals = []
        inp = x
        for layer in range(self.num_layers):
            outs = []
            for d in range(dirs):
                idx = layer * dirs + d
                res = self._run(inp, tuple(s[idx] for s in states), self._params_of(layer, d), d == 1)
                outs.append(res[0])
                finals.append(res[1:])
            inp = outs[0] if dirs == 1 else torch.cat(outs, 2)
            if self.dropout > 0 and self.training and layer + 1 < self.num_layers:
                inp = F.dropout(inp, self.dropout, True)
        out = inp
        if unbatched:
            out = out.squeeze(1)
        elif self.batch_first:
            out = out.transpose(0, 1)
        stacked = tuple(torch.stack([f[k] for f in finals], 0) for k in range(len(finals[0])))
        if unbatched:
            stacked = tuple(s.squeeze(1) for s in stacked)
        return out, (stacked if len(stacked) > 1 else stacked[0])

    def extra_repr(self) -> str:
        return (f"{self.input_size}, {self.hidden_size}, num_layers={self.num_layers}, bias={self.bias}, "
                f"batch_first={self.batch_first}, dropout={self.dropout}, bidirectional={self.bidirectional}")

    def flatten_parameters(self) -> None:
        """Kept for API parity with ``torch.nn`` recurrent modules; the weights need no repacking here."""


class RNN(_RecurrentBase):
    """Elman RNN with ``tanh`` or ``relu`` (src/nn/rnn.rs:451-462)."""

    _GATES = 1
    mode = "RNN_TANH"

    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, bias: bool = True,
                 batch_first: bool = False, dropout: float = 0.0, bidirectional: bool = False,
                 nonlinearity: str = "tanh", **kw):
        if nonlinearity not in ("tanh", "relu"):
            raise ValueError("nonlinearity must be 'tanh' or 'relu'")
        self.nonlinearity = nonlinearity
        super().__init__(input_size, hidden_size, num_layers, bias, batch_first, dropout, bidirectional, **kw)

    def _split_state(self, hx, batch, x, unbatched=False):
        if hx is None:
            hx = self.init_hidden(batch, x.device, x.dtype)
        elif unbatched:
            hx = hx.unsqueeze(1)
        return (hx,)

    def _run(self, x, state, params, reverse):
        w_ih, w_hh, b_ih, b_hh = params
        return _seq.rnn_layer(x, state[0], w_ih, w_hh, b_ih, b_hh, reverse, self.nonlinearity)


class LSTM(_RecurrentBase):
    """``forward(x, (h0, c0) | None) -> (out, (h_n, c_n))`` (src/nn/lstm_layer.rs:56-92)."""

    _GATES = 4
    mode = "LSTM"

    def init_state(self, batch: int, device=None, dtype=None):
        h = self.init_hidden(batch, device, dtype)
        return h, torch.zeros_like(h)

    def _split_state(self, hx, batch, x, unbatched=False):
        if hx is None:
            return self.init_state(batch, x.device, x.dtype)
        h, c = hx
        if unbatched:
            h, c = h.unsqueeze(1), c.unsqueeze(1)
        return h, c

    def _run(self, x, state, params, reverse):
        w_ih, w_hh, b_ih, b_hh = params
        return _seq.lstm_layer(x, state[0], state[1], w_ih, w_hh, b_ih, b_hh, reverse)


class GRU(_RecurrentBase):
    """``forward(x, h0 | None) -> (out, h_n)``, gate order ``[r, z, n]`` (src/nn/gru_layer.rs:56-68)."""

    _GATES = 3
    mode = "GRU"

    def _split_state(self, hx, batch, x, unbatched=False):
        if hx is None:
            hx = self.init_hidden(batch, x.device, x.dtype)
        elif unbatched:
            hx = hx.unsqueeze(1)
        return (hx,)

    def _run(self, x, state, params, reverse):
        w_ih, w_hh, b_ih, b_hh = params
        return _seq.gru_layer(x, state[0], w_ih, w_hh, b_ih, b_hh, reverse)


from .._interop import accept_wrappers as _accept_wrappers  # noqa: E402

_accept_wrappers(globals())       # forward() of the layers above also takes this package's Tensor / Variable
