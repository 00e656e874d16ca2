"""nn-level tensor quantisation: int8 / int4 / fp16, symmetric / asymmetric, calibration modes, a parameter cache
per layer and a quantisation-aware-training wrapper (src/nn/quantization.rs:22-447).

All arithmetic is tensor arithmetic on the device that holds the data.  Two things go beyond the reference: the
entropy calibration really searches the clipping threshold that minimises the KL divergence between the value
histogram and its quantised form (the reference falls back to min / max there, src/nn/quantization.rs:203-213), and
the fake quantisation of :class:`QuantizationAwareModule` passes gradients straight through inside the clipping
range (the reference rebuilds the variable and so cuts the graph, src/nn/quantization.rs:351-366).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Dict, List, Optional, Union

import torch
import torch.nn as nn


class QuantizationType(enum.Enum):
    INT8 = "int8"
    INT4 = "int4"
    FLOAT16 = "float16"
    DYNAMIC = "dynamic"                  # int8 with parameters taken from each tensor as it comes
    INT8_SYMMETRIC = "int8_sym"
    INT8_ASYMMETRIC = "int8_asym"
    INT4_SYMMETRIC = "int4_sym"
    INT4_ASYMMETRIC = "int4_asym"

    @property
    def bits(self) -> int:
        return 16 if self is QuantizationType.FLOAT16 else (4 if "int4" in self.value else 8)


class CalibrationMode:
    """How the clipping range is chosen: ``MIN_MAX``, ``percentile(p)`` (the central share ``p`` of the sorted
    values) or ``ENTROPY`` (KL-minimising threshold)."""

    def __init__(self, kind: str, p: float = 1.0):
        self.kind, self.p = kind, float(p)

    @classmethod
    def percentile(cls, p: float) -> "CalibrationMode":
        if not 0.0 < p <= 1.0:
            raise ValueError("percentile share must be in (0, 1]")
        return cls("percentile", p)

    def __eq__(self, other):
        return isinstance(other, CalibrationMode) and (self.kind, self.p) == (other.kind, other.p)

    def __hash__(self):
        return hash((self.kind, self.p))

    def __repr__(self):
        return f"CalibrationMode.percentile({self.p})" if self.kind == "percentile" else f"CalibrationMode.{self.kind.upper()}"


CalibrationMode.MIN_MAX = CalibrationMode("min_max")
CalibrationMode.ENTROPY = CalibrationMode("entropy")


@dataclass
class QuantizationParams:
    scale: float
    zero_point: int
    qmin: int
    qmax: int
    qtype: QuantizationType

    @classmethod
    def int8_symmetric(cls, scale: float) -> "QuantizationParams":
        return cls(float(scale), 0, -128, 127, QuantizationType.INT8)

    @classmethod
    def int8_asymmetric(cls, scale: float, zero_point: int) -> "QuantizationParams":
        return cls(float(scale), int(zero_point), -128, 127, QuantizationType.INT8)

    @classmethod
    def int4_symmetric(cls, scale: float) -> "QuantizationParams":
        return cls(float(scale), 0, -8, 7, QuantizationType.INT4)

    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        return torch.clamp(torch.round(x.float() / self.scale) + self.zero_point, self.qmin, self.qmax)

    def fake_quantize(self, x: torch.Tensor) -> torch.Tensor:
        """Quantise-dequantise with a straight-through gradient inside ``[qmin, qmax]`` and zero outside."""
        q = x / self.scale + self.zero_point
        inside = ((q >= self.qmin) & (q <= self.qmax)).to(x.dtype)
        y = ((self.quantize(x.detach()) - self.zero_point) * self.scale).to(x.dtype)
        return y + (x - x.detach()) * inside


class QuantizedTensor:
    """Integer codes (int8 storage; int4 codes use the low range; fp16 keeps half floats) + their parameters.
    ``QuantizedTensor(data, shape, params)`` or the older ``(data, scale, zero_point, qtype, shape)``."""

    def __init__(self, data: torch.Tensor, *args):
        if len(args) == 2 and isinstance(args[1], QuantizationParams):
            shape, params = args
        elif len(args) == 4:
            scale, zp, qtype, shape = args
            bits = qtype.bits
            params = QuantizationParams(float(scale), int(zp), -(2 ** (bits - 1)), 2 ** (bits - 1) - 1, qtype)
        else:
            raise TypeError("QuantizedTensor(data, shape, params)")
        self.data, self.shape, self.params = data, tuple(shape), params

    scale = property(lambda self: self.params.scale)
    zero_point = property(lambda self: self.params.zero_point)
    qtype = property(lambda self: self.params.qtype)

    def dequantize(self) -> torch.Tensor:
        if self.params.qtype is QuantizationType.FLOAT16:
            return self.data.float().view(self.shape)
        return ((self.data.float() - self.params.zero_point) * self.params.scale).view(self.shape)

    def compression_ratio(self) -> float:
        return 32.0 / self.params.qtype.bits

    def memory_bytes(self) -> int:
        return (self.data.numel() * self.params.qtype.bits + 7) // 8

    size_bytes = memory_bytes


def _entropy_threshold(x: torch.Tensor, levels: int, bins: int = 2048) -> float:
    """Clipping threshold of ``|x|`` that minimises KL(histogram || histogram quantised to ``levels`` bins)."""
    a = x.detach().abs().float().flatten()
    amax = float(a.max())
    if amax == 0.0 or a.numel() < 2 * levels:
        return amax
    hist = torch.histc(a, bins=bins, min=0.0, max=amax).double()
    best, best_kl = amax, float("inf")
    for i in range(levels, bins + 1, max(1, bins // 128)):
        p = hist[:i].clone()
        p[i - 1] += hist[i:].sum()                           # the clipped tail lands in the last bin
        if p.sum() == 0:
            continue
        # merge the i bins into `levels` groups, then spread each group evenly over its non-empty bins
        edges = torch.linspace(0, i, levels + 1).round().long()
        q = torch.zeros(i, dtype=torch.float64)
        src = hist[:i]
        for g in range(levels):
            lo, hi = int(edges[g]), int(edges[g + 1])
            if hi <= lo:
                continue
            seg = src[lo:hi]
            nz = seg > 0
            if nz.any():
                q[lo:hi][nz] = seg.sum() / nz.sum()
        pn, qn = p / p.sum(), q / q.sum().clamp_min(1e-300)
        m = pn > 0
        kl = float((pn[m] * (pn[m] / qn[m].clamp_min(1e-12)).log()).sum())
        if kl < best_kl:
            best_kl, best = kl, amax * i / bins
    return best


class Quantizer:
    """``Quantizer(calibration_mode, symmetric)`` as in the reference, or ``Quantizer(qtype)`` for a fixed type with
    min / max calibration; parameters computed for a named layer are cached and reused."""

    def __init__(self, mode: Union[CalibrationMode, QuantizationType] = QuantizationType.INT8_SYMMETRIC, symmetric: bool = True):
        if isinstance(mode, QuantizationType):
            self.qtype, self.calibration_mode = mode, CalibrationMode.MIN_MAX
            self.symmetric = not mode.value.endswith("_asym")
        else:
            self.qtype, self.calibration_mode, self.symmetric = QuantizationType.INT8, mode, bool(symmetric)
        self.param_cache: Dict[str, QuantizationParams] = {}

    # ---- parameters
    def _clip_range(self, x: torch.Tensor, bits: int):
        xf = x.detach().float().flatten()
        cm = self.calibration_mode
        if cm.kind == "percentile" and xf.numel() > 1:
            s = xf.sort().values
            low = int((1.0 - cm.p) * 0.5 * s.numel())
            return float(s[low]), float(s[s.numel() - 1 - low])
        if cm.kind == "entropy":
            t = _entropy_threshold(xf, 2 ** (bits - 1))
            return max(float(xf.min()), -t), min(float(xf.max()), t)
        return float(xf.min()), float(xf.max())

    def compute_quantization_params(self, x: torch.Tensor, qtype: Optional[QuantizationType] = None) -> QuantizationParams:
        qtype = qtype or self.qtype
        if qtype is QuantizationType.FLOAT16:
            return QuantizationParams(1.0, 0, 0, 0, qtype)
        bits = qtype.bits
        sym = self.symmetric if qtype in (QuantizationType.INT8, QuantizationType.DYNAMIC) else not qtype.value.endswith("_asym")
        lo, hi = self._clip_range(x, bits)
        if sym:
            qmax = 2 ** (bits - 1) - 1
            # the reference's parameter objects carry the full two's-complement range; the scale maps |x|max to qmax
            qmin = -(2 ** (bits - 1)) if qtype in (QuantizationType.INT8, QuantizationType.INT4, QuantizationType.DYNAMIC) else -qmax
            return QuantizationParams(max(abs(lo), abs(hi), 1e-12) / qmax, 0, qmin, qmax, qtype)
        qmin, qmax = -(2 ** (bits - 1)), 2 ** (bits - 1) - 1
        scale = max((hi - lo) / (qmax - qmin), 1e-12)
        return QuantizationParams(scale, int(round(qmin - lo / scale)), qmin, qmax, qtype)

    # ---- tensors and modules
    def quantize_tensor(self, x: torch.Tensor, qtype: Optional[QuantizationType] = None, layer_name: Optional[str] = None) -> QuantizedTensor:
        qtype = qtype or self.qtype
        if layer_name is not None and qtype is not QuantizationType.DYNAMIC:
            params = self.param_cache.get(layer_name)
            if params is None or params.qtype is not qtype:
                params = self.param_cache[layer_name] = self.compute_quantization_params(x, qtype)
        else:
            params = self.compute_quantization_params(x, qtype)
        if qtype is QuantizationType.FLOAT16:
            return QuantizedTensor(x.detach().to(torch.float16), tuple(x.shape), params)
        return QuantizedTensor(params.quantize(x.detach()).to(torch.int8), tuple(x.shape), params)

    def quantize(self, x: torch.Tensor) -> QuantizedTensor:
        return self.quantize_tensor(x)

    def quantize_module(self, module: nn.Module, qtype: Optional[QuantizationType] = None, layer_name: str = "") -> List[QuantizedTensor]:
        """All parameters of ``module``, cached under ``<layer_name>_<index>``."""
        return [self.quantize_tensor(p.data, qtype, f"{layer_name}_{i}") for i, p in enumerate(module.parameters())]

    def dequantize(self, q: QuantizedTensor) -> torch.Tensor:
        return q.dequantize()

    def quantization_error(self, x: torch.Tensor) -> float:
        return float((self.quantize(x).dequantize() - x.float()).abs().max())

    def clear_cache(self) -> None:
        self.param_cache.clear()

    def get_statistics(self) -> Dict[str, QuantizationParams]:
        return dict(self.param_cache)


class QuantizationAwareModule(nn.Module):
    """Wraps a module for quantisation-aware training: while enabled, the input (and, with ``weights=True``, every
    matrix parameter) passes through quantise-dequantise with a straight-through gradient.  Input parameters come
    from ``set_qparams("input", …)`` or from a running min / max observed in training mode."""

    def __init__(self, module: nn.Module, qtype: QuantizationType = QuantizationType.INT8, symmetric: bool = True,
                 weights: bool = False, momentum: float = 0.1):
        super().__init__()
        self.module = module
        self.qparams: Dict[str, QuantizationParams] = {}
        self.qat_enabled, self.fake_quantize = False, True
        self.qtype, self.weights, self.momentum = qtype, weights, momentum
        self._quantizer = Quantizer(CalibrationMode.MIN_MAX, symmetric)
        self._observed: Optional[List[float]] = None
        self._fixed = set()

    def enable_qat(self) -> None:
        self.qat_enabled = True

    def disable_qat(self) -> None:
        self.qat_enabled = False

    def set_fake_quantize(self, enabled: bool) -> None:
        self.fake_quantize = bool(enabled)

    def set_qparams(self, layer_name: str, params: QuantizationParams) -> None:
        self.qparams[layer_name] = params
        self._fixed.add(layer_name)

    def _observe(self, x: torch.Tensor) -> None:
        lo, hi = float(x.detach().min()), float(x.detach().max())
        if self._observed is None:
            self._observed = [lo, hi]
        else:
            m = self.momentum
            self._observed = [(1 - m) * self._observed[0] + m * lo, (1 - m) * self._observed[1] + m * hi]
        rng = torch.tensor(self._observed)
        self.qparams["input"] = self._quantizer.compute_quantization_params(rng, self.qtype)

    def apply_fake_quantization(self, x: torch.Tensor, layer_name: str) -> torch.Tensor:
        if not (self.qat_enabled and self.fake_quantize):
            return x
        if layer_name == "input" and "input" not in self._fixed and self.training:
            self._observe(x)
        p = self.qparams.get(layer_name)
        return x if p is None else p.fake_quantize(x)

    def forward(self, x, *args, **kw):
        x = self.apply_fake_quantization(x, "input")
        if not (self.weights and self.qat_enabled and self.fake_quantize):
            return self.module(x, *args, **kw)
        named = [(n, p) for n, p in self.module.named_parameters() if p.dim() >= 2]
        fq = {n: self._quantizer.compute_quantization_params(p, self.qtype).fake_quantize(p) for n, p in named}
        return torch.func.functional_call(self.module, fq, (x, *args), kw)
