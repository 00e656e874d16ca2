"""nn-level tensor quantisation: int8 / int4, symmetric / asymmetric (src/nn/quantization.rs:22-447)."""
from __future__ import annotations

import enum
from dataclasses import dataclass

import torch


class QuantizationType(enum.Enum):
    INT8_SYMMETRIC = "int8_sym"
    INT8_ASYMMETRIC = "int8_asym"
    INT4_SYMMETRIC = "int4_sym"
    INT4_ASYMMETRIC = "int4_asym"


@dataclass
class QuantizedTensor:
    data: torch.Tensor      # int8 storage (int4 values occupy the low nibble range)
    scale: float
    zero_point: int
    qtype: QuantizationType
    shape: tuple

    def dequantize(self) -> torch.Tensor:
        return (self.data.float() - self.zero_point) * self.scale

    def size_bytes(self) -> int:
        bits = 4 if "int4" in self.qtype.value else 8
        return (self.data.numel() * bits + 7) // 8


class Quantizer:
    def __init__(self, qtype: QuantizationType = QuantizationType.INT8_SYMMETRIC):
        self.qtype = qtype

    def _range(self):
        bits = 4 if "int4" in self.qtype.value else 8
        sym = self.qtype.value.endswith("_sym")
        if sym:
            return -(2 ** (bits - 1) - 1), 2 ** (bits - 1) - 1, True
        return -(2 ** (bits - 1)), 2 ** (bits - 1) - 1, False

    def quantize(self, x: torch.Tensor) -> QuantizedTensor:
        qmin, qmax, sym = self._range()
        xf = x.detach().float()
        if sym:
            amax = float(xf.abs().max().clamp_min(1e-12))
            scale, zp = amax / qmax, 0
        else:
            lo, hi = float(xf.min()), float(xf.max())
            scale = max((hi - lo) / (qmax - qmin), 1e-12)
            zp = int(round(qmin - lo / scale))
        q = torch.clamp(torch.round(xf / scale) + zp, qmin, qmax).to(torch.int8)
        return QuantizedTensor(q, scale, zp, self.qtype, tuple(x.shape))

    def dequantize(self, q: QuantizedTensor) -> torch.Tensor:
        return q.dequantize()

    def quantization_error(self, x: torch.Tensor) -> float:
        return float((self.quantize(x).dequantize() - x.float()).abs().max())
