"""Recurrent layers: ``RNNCell/RNN``, ``LSTMCell/LSTM``, ``GRUCell/GRU``.

Constructor order ``(input_size, hidden_size, num_layers=1, bias=True, batch_first=False, dropout=0.0,
bidirectional=False)`` and the LSTM gate order ``[i, f, g, o]`` follow the reference
(src/nn/rnn.rs:451-462, src/nn/lstm_layer.rs:56-92, src/nn/lstm_cell.rs:84-126,
src/nn/gru_layer.rs:56-68).  Cells: ``forward(x, state=None)``; LSTM state is ``(h, c)``.
Each time step is one GEMM per operand plus fused gate pointwise math; the whole sequence
runs on torch's (cuDNN) kernels when on CUDA, which keep the same gate order.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import rnn as _rnn_ops


class RNNCell(nn.RNNCell):
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
        gates = F.linear(x, self.weight_ih, self.bias_ih) + F.linear(h, self.weight_hh, self.bias_hh)
        return _rnn_ops.lstm_gates(gates, c)          # one fused kernel on CUDA


class GRUCell(nn.GRUCell):
    def forward(self, x: torch.Tensor, h: Optional[torch.Tensor] = None):
        if x.dim() != 2:
            return super().forward(x, h)
        if h is None:
            h = torch.zeros(x.shape[0], self.hidden_size, dtype=x.dtype, device=x.device)
        return _rnn_ops.gru_gates(F.linear(x, self.weight_ih, self.bias_ih), F.linear(h, self.weight_hh, self.bias_hh), h)


class _Recurrent:
    def init_hidden(self, batch: int, device=None, dtype=None):
        n = self.num_layers * (2 if self.bidirectional else 1)
        return torch.zeros(n, batch, self.hidden_size, device=device, dtype=dtype)


class RNN(nn.RNN, _Recurrent):
    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, bias: bool = True,
                 batch_first: bool = False, dropout: float = 0.0, bidirectional: bool = False,
                 nonlinearity: str = "tanh", **kw):
        super().__init__(input_size, hidden_size, num_layers, nonlinearity=nonlinearity, bias=bias,
                         batch_first=batch_first, dropout=dropout, bidirectional=bidirectional, **kw)


class LSTM(nn.LSTM, _Recurrent):
    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, bias: bool = True,
                 batch_first: bool = False, dropout: float = 0.0, bidirectional: bool = False, **kw):
        super().__init__(input_size, hidden_size, num_layers, bias=bias, batch_first=batch_first,
                         dropout=dropout, bidirectional=bidirectional, **kw)

    def init_state(self, batch: int, device=None, dtype=None):
        h = self.init_hidden(batch, device, dtype)
        return h, torch.zeros_like(h)


class GRU(nn.GRU, _Recurrent):
    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, bias: bool = True,
                 batch_first: bool = False, dropout: float = 0.0, bidirectional: bool = False, **kw):
        super().__init__(input_size, hidden_size, num_layers, bias=bias, batch_first=batch_first,
                         dropout=dropout, bidirectional=bidirectional, **kw)
