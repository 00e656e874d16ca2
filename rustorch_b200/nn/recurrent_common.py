"""Shared pieces of the recurrent layers (src/nn/recurrent_common.rs:13-450): the per-cell configuration, weight
initialisation, gate slicing and the time-step / stacking helpers of the multi-layer loops.  The whole-sequence
layers in ``rnn.py`` do their input projections as one GEMM over all steps and only keep the recurrent product and
the fused gate kernel inside the time loop; these helpers are the reference-shaped view of the same arithmetic."""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch


@dataclass
class RecurrentConfig:
    input_size: int
    hidden_size: int
    num_gates: int
    bias: bool = True
    training: bool = True

    @classmethod
    def rnn(cls, input_size: int, hidden_size: int, bias: bool = True) -> "RecurrentConfig":
        return cls(input_size, hidden_size, 1, bias)

    @classmethod
    def gru(cls, input_size: int, hidden_size: int, bias: bool = True) -> "RecurrentConfig":
        return cls(input_size, hidden_size, 3, bias)

    @classmethod
    def lstm(cls, input_size: int, hidden_size: int, bias: bool = True) -> "RecurrentConfig":
        return cls(input_size, hidden_size, 4, bias)

    @property
    def gate_rows(self) -> int:
        return self.num_gates * self.hidden_size


class TrainingMode(enum.Enum):
    TRAINING = "training"
    EVALUATION = "evaluation"

    @property
    def is_training(self) -> bool:
        return self is TrainingMode.TRAINING


class RecurrentOps:
    """Cell-level arithmetic.  ``lstm_step`` / ``gru_step`` run the fused gate kernels on CUDA."""

    @staticmethod
    def init_weights(config: RecurrentConfig, device=None, dtype=None, generator=None) -> Tuple[torch.Tensor, torch.Tensor]:
        """``(w_ih [gates * H, I], w_hh [gates * H, H])``, uniform in ``+-1/sqrt(H)``."""
        k = 1.0 / math.sqrt(config.hidden_size)
        w_ih = torch.empty(config.gate_rows, config.input_size, device=device, dtype=dtype).uniform_(-k, k, generator=generator)
        w_hh = torch.empty(config.gate_rows, config.hidden_size, device=device, dtype=dtype).uniform_(-k, k, generator=generator)
        return w_ih.requires_grad_(True), w_hh.requires_grad_(True)

    @staticmethod
    def init_bias(config: RecurrentConfig, device=None, dtype=None) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        """Zero biases; for an LSTM the forget-gate slice of ``b_ih`` starts at one (gate order i, f, g, o)."""
        if not config.bias:
            return None, None
        b_ih = torch.zeros(config.gate_rows, device=device, dtype=dtype)
        b_hh = torch.zeros(config.gate_rows, device=device, dtype=dtype)
        if config.num_gates == 4:
            b_ih[config.hidden_size:2 * config.hidden_size] = 1.0
        return b_ih.requires_grad_(True), b_hh.requires_grad_(True)

    @staticmethod
    def linear_transform(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        return torch.nn.functional.linear(x, weight, bias)

    matmul_variables = staticmethod(torch.matmul)
    add_variables = staticmethod(torch.add)
    multiply_variables = staticmethod(torch.mul)
    sigmoid = staticmethod(torch.sigmoid)
    tanh = staticmethod(torch.tanh)

    @staticmethod
    def subtract_from_scalar(scalar: float, x: torch.Tensor) -> torch.Tensor:
        return scalar - x

    @staticmethod
    def transpose_variable(x: torch.Tensor) -> torch.Tensor:
        return x.transpose(-1, -2)

    @staticmethod
    def slice_gates(gates: torch.Tensor, gate_idx: int, hidden_size: int) -> torch.Tensor:
        if (gate_idx + 1) * hidden_size > gates.shape[-1]:
            raise IndexError(f"gate {gate_idx} of width {hidden_size} is outside {gates.shape[-1]} columns")
        return gates[..., gate_idx * hidden_size:(gate_idx + 1) * hidden_size]

    @staticmethod
    def zero_hidden_state(batch_size: int, hidden_size: int, device=None, dtype=None) -> torch.Tensor:
        return torch.zeros(batch_size, hidden_size, device=device, dtype=dtype)

    # ---- layer-level helpers
    @staticmethod
    def init_state(num_layers: int, batch: int, hidden: int, bidirectional: bool = False, device=None, dtype=None) -> torch.Tensor:
        return torch.zeros(num_layers * (2 if bidirectional else 1), batch, hidden, device=device, dtype=dtype)

    @staticmethod
    def to_time_major(x: torch.Tensor, batch_first: bool) -> torch.Tensor:
        return x.transpose(0, 1) if batch_first else x

    @staticmethod
    def reverse_sequence(x: torch.Tensor) -> torch.Tensor:
        return x.flip(0)

    @staticmethod
    def lstm_step(gates: torch.Tensor, c: torch.Tensor):
        from ..ops import rnn
        return rnn.lstm_gates(gates, c)

    @staticmethod
    def gru_step(gi: torch.Tensor, gh: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        from ..ops import rnn
        return rnn.gru_gates(gi, gh, h)

    @staticmethod
    def run_cell(cell, x: torch.Tensor, state=None, reverse: bool = False):
        """Unrolls a cell over a time-major sequence; returns (outputs [T, B, H], last state)."""
        steps = range(x.shape[0] - 1, -1, -1) if reverse else range(x.shape[0])
        outs = [None] * x.shape[0]
        for t in steps:
            state = cell(x[t], state)
            outs[t] = state[0] if isinstance(state, tuple) else state
        return torch.stack(outs, 0), state


def collect_recurrent_parameters(weight_ih, weight_hh, bias_ih=None, bias_hh=None) -> List[torch.Tensor]:
    return [p for p in (weight_ih, weight_hh, bias_ih, bias_hh) if p is not None]


class MultiLayerUtils:
    @staticmethod
    def get_timestep_input(x: torch.Tensor, t: int, batch_first: bool) -> torch.Tensor:
        """``[B, I]`` slice of step ``t`` from ``[B, T, I]`` (batch first) or ``[T, B, I]``."""
        T = x.shape[1] if batch_first else x.shape[0]
        if not 0 <= t < T:
            raise IndexError(f"time step {t} outside a sequence of {T}")
        return x[:, t] if batch_first else x[t]

    @staticmethod
    def stack_outputs(outputs: Sequence[torch.Tensor], batch_first: bool) -> torch.Tensor:
        if not outputs:
            raise ValueError("no outputs to stack")
        return torch.stack(list(outputs), dim=1 if batch_first else 0)

    @staticmethod
    def stack_hidden_states(states: Sequence[torch.Tensor]) -> torch.Tensor:
        """``[num_layers * directions, B, H]`` from per-layer ``[B, H]`` states."""
        if not states:
            raise ValueError("no hidden states to stack")
        return torch.stack(list(states), dim=0)
