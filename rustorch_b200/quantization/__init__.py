"""Integer quantization: schemes, quantized tensors (int8 / int4), observers and static calibration, quantized
ops, and quantization-aware training (src/quantization/types.rs:14-380, schemes.rs:12-340,
calibration.rs:15-520, operations.rs:12-480, qat.rs:19-560).

Tensors stay on their device.  ``qmatmul`` / ``qlinear`` multiply int8 operands with int32 accumulation through
``torch._int_mm`` on CUDA (tensor-core IMMA) when shapes allow and an exact integer matmul otherwise; the
GGUF block formats used by the LLM runtime live in ``rustorch_b200.llm.quant``.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Dict, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


class QuantizationType(Enum):
    INT8 = "int8"
    UINT8 = "uint8"
    INT4 = "int4"

    def bits(self) -> int:
        return 4 if self is QuantizationType.INT4 else 8

    def range(self) -> Tuple[int, int]:
        return {"int8": (-128, 127), "uint8": (0, 255), "int4": (-8, 7)}[self.value]


class QuantizationScheme(Enum):
    SYMMETRIC = "symmetric"
    ASYMMETRIC = "asymmetric"
    PER_CHANNEL_SYMMETRIC = "per_channel_symmetric"
    PER_CHANNEL_ASYMMETRIC = "per_channel_asymmetric"

    def compute_params(self, data: torch.Tensor, qtype: QuantizationType = QuantizationType.INT8, axis: int = 0):
        if self in (QuantizationScheme.SYMMETRIC, QuantizationScheme.ASYMMETRIC):
            return QuantParamCalculator.compute(data.min(), data.max(), qtype, self is QuantizationScheme.SYMMETRIC)
        red = [d for d in range(data.dim()) if d != axis % data.dim()]
        return QuantParamCalculator.compute(data.amin(red), data.amax(red), qtype, self is QuantizationScheme.PER_CHANNEL_SYMMETRIC)


class CalibrationMethod(Enum):
    MINMAX = "minmax"
    PERCENTILE = "percentile"
    ENTROPY = "entropy"

    def compute_range(self, data: torch.Tensor, percentile: float = 99.99) -> Tuple[torch.Tensor, torch.Tensor]:
        f = data.detach().float().reshape(-1)
        if self is CalibrationMethod.MINMAX:
            return f.min(), f.max()
        if self is CalibrationMethod.PERCENTILE:
            q = torch.tensor([1 - percentile / 100, percentile / 100], device=f.device)
            if f.numel() > 1_000_000:
                f = f[torch.randint(0, f.numel(), (1_000_000,), device=f.device)]
            lo, hi = torch.quantile(f, q)
            return lo, hi
        return _entropy_range(f)


def _entropy_range(f: torch.Tensor, bins: int = 2048, levels: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """KL-divergence calibration: pick the clipping threshold whose ``levels``-bin quantisation of |x| diverges
    least from the full histogram."""
    a = f.abs()
    mx = float(a.max()) or 1.0
    hist = torch.histc(a, bins=bins, min=0.0, max=mx).double().cpu()
    best, best_t = float("inf"), mx
    for i in range(levels, bins + 1, 16):
        p = hist[:i].clone()
        p[i - 1] += hist[i:].sum()
        if p.sum() == 0:
            continue
        chunks = p.reshape(levels, -1) if i % levels == 0 else None
        if chunks is None:
            idx = (torch.arange(i) * levels // i)
            qsum = torch.zeros(levels, dtype=torch.double).index_add_(0, idx, p)
            cnt = torch.zeros(levels, dtype=torch.double).index_add_(0, idx, (p > 0).double())
            q = (qsum / cnt.clamp_min(1))[idx] * (p > 0)
        else:
            cnt = (chunks > 0).sum(1, keepdim=True).clamp_min(1)
            q = ((chunks.sum(1, keepdim=True) / cnt) * (chunks > 0)).reshape(-1)
        pn, qn = p / p.sum(), q / q.sum().clamp_min(1e-30)
        m = pn > 0
        kl = float((pn[m] * (pn[m] / qn[m].clamp_min(1e-30)).log()).sum())
        if kl < best:
            best, best_t = kl, mx * i / bins
    t = torch.tensor(best_t, device=f.device)
    return -t, t


class QuantParamCalculator:
    @staticmethod
    def compute(lo: torch.Tensor, hi: torch.Tensor, qtype: QuantizationType, symmetric: bool):
        """-> ``(scale, zero_point)`` tensors (0-dim, or per channel)."""
        qmin, qmax = qtype.range()
        lo, hi = lo.float().clamp_max(0), hi.float().clamp_min(0)
        if symmetric:
            bound = torch.maximum(lo.abs(), hi.abs())
            scale = (bound / (qmax if qmin < 0 else (qmax - qmin) / 2)).clamp_min(1e-12)
            zp = torch.zeros_like(scale, dtype=torch.int32) if qmin < 0 else torch.full_like(scale, (qmax + 1) // 2, dtype=torch.int32)
        else:
            scale = ((hi - lo) / (qmax - qmin)).clamp_min(1e-12)
            zp = (qmin - torch.round(lo / scale)).clamp(qmin, qmax).to(torch.int32)
        return scale, zp

    @staticmethod
    def symmetric(data: torch.Tensor, bits: int = 8):
        return QuantParamCalculator.compute(data.min(), data.max(), QuantizationType.INT4 if bits == 4 else QuantizationType.INT8, True)

    @staticmethod
    def asymmetric(data: torch.Tensor, bits: int = 8):
        return QuantParamCalculator.compute(data.min(), data.max(), QuantizationType.INT4 if bits == 4 else QuantizationType.INT8, False)

    @staticmethod
    def per_channel(data: torch.Tensor, axis: int = 0, bits: int = 8, symmetric: bool = True):
        red = [d for d in range(data.dim()) if d != axis % data.dim()]
        return QuantParamCalculator.compute(data.amin(red), data.amax(red), QuantizationType.INT4 if bits == 4 else QuantizationType.INT8, symmetric)


@dataclass
class QuantizationConfig:
    qtype: QuantizationType = QuantizationType.INT8
    scheme: QuantizationScheme = QuantizationScheme.SYMMETRIC
    calibration: CalibrationMethod = CalibrationMethod.MINMAX
    per_channel_axis: int = 0


class QuantizedTensor:
    """Integer codes (int8 storage; int4 values occupy [-8, 7]) + scale / zero point (scalar or per channel)."""

    def __init__(self, data: torch.Tensor, scale: torch.Tensor, zero_point: torch.Tensor, qtype: QuantizationType = QuantizationType.INT8,
                 axis: Optional[int] = None):
        self.data, self.scale, self.zero_point, self.qtype, self.axis = data, scale, zero_point, qtype, axis

    @property
    def shape(self):
        return self.data.shape

    def numel(self) -> int:
        return self.data.numel()

    def ndim(self) -> int:
        return self.data.dim()

    @property
    def device(self):
        return self.data.device

    def _bshape(self):
        if self.axis is None or self.scale.dim() == 0:
            return ()
        s = [1] * self.data.dim()
        s[self.axis % self.data.dim()] = -1
        return s

    def dequantize(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        bs = self._bshape()
        sc, zp = (self.scale.view(bs), self.zero_point.view(bs)) if bs else (self.scale, self.zero_point)
        return ((self.data.to(torch.int32) - zp).float() * sc).to(dtype)

    def to(self, device) -> "QuantizedTensor":
        return QuantizedTensor(self.data.to(device), self.scale.to(device), self.zero_point.to(device), self.qtype, self.axis)

    to_device = to

    def quantization_params(self):
        return self.scale, self.zero_point

    def is_compatible_with(self, other: "QuantizedTensor") -> bool:
        return (self.qtype is other.qtype and self.scale.shape == other.scale.shape and bool(torch.allclose(self.scale, other.scale))
                and bool(torch.equal(self.zero_point, other.zero_point)))

    def reshape(self, *shape) -> "QuantizedTensor":
        if self.axis is not None and self.scale.dim() > 0:
            raise ValueError("cannot reshape a per-channel quantized tensor")
        return QuantizedTensor(self.data.reshape(*shape), self.scale, self.zero_point, self.qtype, None)

    def pack_int4(self) -> torch.Tensor:
        """Two int4 codes per byte (low nibble first)."""
        if self.qtype is not QuantizationType.INT4:
            raise ValueError("pack_int4 needs an INT4 tensor")
        flat = (self.data.reshape(-1).to(torch.int16) & 0xF).to(torch.uint8)
        if flat.numel() % 2:
            flat = torch.cat([flat, flat.new_zeros(1)])
        return flat[0::2] | (flat[1::2] << 4)

    @staticmethod
    def unpack_int4(packed: torch.Tensor, numel: int) -> torch.Tensor:
        lo, hi = (packed & 0xF).to(torch.int8), (packed >> 4).to(torch.int8)
        both = torch.stack([lo, hi], 1).reshape(-1)[:numel]
        return torch.where(both > 7, both - 16, both)


def quantize(x: torch.Tensor, scale: torch.Tensor, zero_point: torch.Tensor, qtype: QuantizationType = QuantizationType.INT8,
             axis: Optional[int] = None) -> QuantizedTensor:
    qmin, qmax = qtype.range()
    q = QuantizedTensor(x, scale, zero_point, qtype, axis)
    bs = q._bshape()
    sc, zp = (scale.view(bs), zero_point.view(bs)) if bs else (scale, zero_point)
    codes = (torch.round(x.float() / sc) + zp).clamp(qmin, qmax)
    q.data = codes.to(torch.uint8 if qtype is QuantizationType.UINT8 else torch.int8)
    return q


def quantize_tensor(x: torch.Tensor, config: Optional[QuantizationConfig] = None) -> QuantizedTensor:
    """The ``TensorQuantization::quantize`` entry point: compute parameters from the data and encode."""
    c = config or QuantizationConfig()
    per_ch = c.scheme in (QuantizationScheme.PER_CHANNEL_SYMMETRIC, QuantizationScheme.PER_CHANNEL_ASYMMETRIC)
    scale, zp = c.scheme.compute_params(x.detach(), c.qtype, c.per_channel_axis)
    return quantize(x.detach(), scale, zp, c.qtype, c.per_channel_axis if per_ch else None)


# ------------------------------------------------------------------------------ observers
class Observer:
    def observe(self, x: torch.Tensor) -> None:
        raise NotImplementedError

    def get_range(self) -> Tuple[torch.Tensor, torch.Tensor]:
        raise NotImplementedError

    def reset(self) -> None:
        raise NotImplementedError

    def compute_params(self, qtype=QuantizationType.INT8, symmetric: bool = True):
        lo, hi = self.get_range()
        return QuantParamCalculator.compute(lo, hi, qtype, symmetric)


class MinMaxObserver(Observer):
    """Running min / max, optionally smoothed with an exponential moving average."""

    def __init__(self, averaging: Optional[float] = None):
        self.averaging = averaging
        self.reset()

    def reset(self):
        self.lo = self.hi = None
        self.count = 0

    def observe(self, x):
        lo, hi = x.detach().float().min(), x.detach().float().max()
        if self.lo is None:
            self.lo, self.hi = lo, hi
        elif self.averaging is None:
            self.lo, self.hi = torch.minimum(self.lo, lo), torch.maximum(self.hi, hi)
        else:
            a = self.averaging
            self.lo, self.hi = self.lo * (1 - a) + lo * a, self.hi * (1 - a) + hi * a
        self.count += 1

    def get_range(self):
        if self.lo is None:
            raise RuntimeError("observer has seen no data")
        return self.lo, self.hi


class HistogramObserver(Observer):
    """Histogram over a growing symmetric range; ``compute_optimal_range`` clips at quantiles."""

    def __init__(self, bins: int = 2048):
        self.bins = bins
        self.reset()

    def reset(self):
        self.hist, self.bound = None, 0.0

    def observe(self, x):
        f = x.detach().float().reshape(-1)
        b = float(f.abs().max())
        if self.hist is None or b > self.bound:
            new_bound = max(b, self.bound * 2 if self.hist is not None else b) or 1.0
            new = torch.zeros(self.bins, dtype=torch.float64)
            if self.hist is not None:       # re-bin the old counts into the wider range
                centers = (torch.arange(self.bins) + 0.5) / self.bins * 2 * self.bound - self.bound
                idx = ((centers + new_bound) / (2 * new_bound) * self.bins).long().clamp(0, self.bins - 1)
                new.index_add_(0, idx, self.hist)
            self.hist, self.bound = new, new_bound
        self.hist += torch.histc(f, bins=self.bins, min=-self.bound, max=self.bound).double().cpu()

    def compute_optimal_range(self, target_quantiles: Tuple[float, float] = (0.0001, 0.9999)):
        if self.hist is None:
            raise RuntimeError("observer has seen no data")
        cdf = torch.cumsum(self.hist, 0) / self.hist.sum()
        lo_i = int(torch.searchsorted(cdf, torch.tensor(target_quantiles[0], dtype=torch.float64)))
        hi_i = int(torch.searchsorted(cdf, torch.tensor(target_quantiles[1], dtype=torch.float64)))
        w = 2 * self.bound / self.bins
        return torch.tensor(-self.bound + lo_i * w), torch.tensor(-self.bound + (hi_i + 1) * w)

    def get_range(self):
        return self.compute_optimal_range()


class StaticQuantizer:
    """Named observers -> calibrated ``(scale, zero_point)`` per tensor."""

    def __init__(self, qtype: QuantizationType = QuantizationType.INT8):
        self.qtype = qtype
        self.observers: Dict[str, Observer] = {}
        self.params: Dict[str, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.method = CalibrationMethod.MINMAX

    def with_calibration_method(self, method: CalibrationMethod) -> "StaticQuantizer":
        self.method = method
        return self

    def add_observer(self, name: str, observer: Optional[Observer] = None) -> None:
        self.observers[name] = observer or (MinMaxObserver() if self.method is CalibrationMethod.MINMAX else HistogramObserver())

    def observe(self, name: str, data: torch.Tensor) -> None:
        if name not in self.observers:
            self.add_observer(name)
        self.observers[name].observe(data)

    def calibrate(self, scheme: QuantizationScheme = QuantizationScheme.SYMMETRIC) -> None:
        sym = scheme in (QuantizationScheme.SYMMETRIC, QuantizationScheme.PER_CHANNEL_SYMMETRIC)
        self.params = {k: o.compute_params(self.qtype, sym) for k, o in self.observers.items()}

    def get_params(self, name: str):
        return self.params.get(name)

    def quantize(self, name: str, data: torch.Tensor) -> QuantizedTensor:
        if name not in self.params:
            raise KeyError(f"'{name}' has not been calibrated")
        s, z = self.params[name]
        return quantize(data, s.to(data.device), z.to(data.device), self.qtype)

    def is_calibrated(self) -> bool:
        return bool(self.params) and set(self.params) == set(self.observers)

    def reset(self) -> None:
        for o in self.observers.values():
            o.reset()
        self.params = {}


def calibrate_batch(quantizer: StaticQuantizer, batches: Sequence[Dict[str, torch.Tensor]], scheme=QuantizationScheme.SYMMETRIC) -> None:
    for b in batches:
        for k, v in b.items():
            quantizer.observe(k, v)
    quantizer.calibrate(scheme)


# ------------------------------------------------------------------------------ quantized ops
def _requant(acc: torch.Tensor, scale: float, out_scale: torch.Tensor, out_zp: torch.Tensor, qtype: QuantizationType) -> QuantizedTensor:
    return quantize(acc.float() * scale, out_scale, out_zp, qtype)


def _native_i8():
    from .. import _native
    return _native.load(required=False)


def int8_gemm(a: torch.Tensor, b_nk: torch.Tensor, row_scale: Optional[torch.Tensor] = None,
              col_scale: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [M, K] (int8) . b_nk [N, K]^T (int8)`` on the tcgen05 integer tensor cores (csrc/quant/gemm_i8_tcgen05.cu).

    Without scales the int32 accumulator is returned; with ``row_scale`` (1 or M values) and ``col_scale`` (1 or N
    values) the kernel's epilogue returns fp32 ``acc * row_scale * col_scale (+ bias)``.  K is zero-padded to a
    multiple of 16 (zeros add nothing to the sum).  CPU tensors take an exact integer matmul.
    """
    C = _native_i8() if a.is_cuda else None
    if C is None:
        acc = a.to(torch.int32) @ b_nk.to(torch.int32).t()
        if row_scale is None:
            return acc
        y = acc.float() * row_scale.reshape(-1, 1) * col_scale.reshape(1, -1)
        return y + bias if bias is not None else y
    K = a.shape[1]
    if K % 16 or a.stride(0) % 16 or b_nk.stride(0) % 16 or a.stride(1) != 1 or b_nk.stride(1) != 1:
        pad = -K % 16
        a = F.pad(a, (0, pad)).contiguous()
        b_nk = F.pad(b_nk, (0, pad)).contiguous()
    if row_scale is None:
        out = torch.empty(a.shape[0], b_nk.shape[0], dtype=torch.int32, device=a.device)
        C.gemm_i8(a, b_nk, out)
        return out
    out = torch.empty(a.shape[0], b_nk.shape[0], dtype=torch.float32, device=a.device)
    f = lambda t: t.detach().to(device=a.device, dtype=torch.float32).reshape(-1).contiguous()  # noqa: E731
    C.gemm_i8(a, b_nk, out, f(row_scale), f(col_scale), None if bias is None else f(bias))
    return out


def _int_mm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """int8 [M, K] @ int8 [K, N] -> int32: the native tcgen05 int8 GEMM on CUDA, an exact integer matmul on the CPU."""
    if a.is_cuda and _native_i8() is not None:
        return int8_gemm(a.contiguous(), b.t().contiguous())
    if a.is_cuda:                         # exact: |codes| <= 128, K < 2^24 / 2^14
        return (a.float() @ b.float()).round().to(torch.int32) if a.shape[1] <= 1024 else (a.double() @ b.double()).round().to(torch.int32)
    return a.to(torch.int32) @ b.to(torch.int32)


class QuantizedOps:
    @staticmethod
    def qadd(a: QuantizedTensor, b: QuantizedTensor, out_scale=None, out_zp=None) -> QuantizedTensor:
        r = a.dequantize() + b.dequantize()
        if out_scale is None:
            out_scale, out_zp = QuantParamCalculator.compute(r.min(), r.max(), a.qtype, True)
        return quantize(r, out_scale, out_zp, a.qtype)

    @staticmethod
    def qmul(a: QuantizedTensor, b: QuantizedTensor, out_scale=None, out_zp=None) -> QuantizedTensor:
        prod = (a.data.to(torch.int32) - a.zero_point) * (b.data.to(torch.int32) - b.zero_point)
        r = prod.float() * (a.scale * b.scale)
        if out_scale is None:
            out_scale, out_zp = QuantParamCalculator.compute(r.min(), r.max(), a.qtype, True)
        return quantize(r, out_scale, out_zp, a.qtype)

    @staticmethod
    def qmatmul_int32(a: QuantizedTensor, b: QuantizedTensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """-> (int32 accumulator with zero points removed, fp32 scale of one accumulator unit)."""
        if a.axis is not None or b.axis is not None:
            raise ValueError("qmatmul expects per-tensor parameters (use qlinear for per-channel weights)")
        K = a.data.shape[-1]
        acc = _int_mm(a.data.reshape(-1, K).to(torch.int8), b.data.to(torch.int8))
        if int(a.zero_point) or int(b.zero_point):        # (A - za)(B - zb) = AB - za ΣB - zb ΣA + K za zb
            za, zb = int(a.zero_point), int(b.zero_point)
            acc = (acc - za * b.data.to(torch.int32).sum(0, keepdim=True) - zb * a.data.reshape(-1, K).to(torch.int32).sum(1, keepdim=True)
                   + K * za * zb)
        return acc.reshape(*a.data.shape[:-1], b.data.shape[-1]), a.scale * b.scale

    @staticmethod
    def qmatmul(a: QuantizedTensor, b: QuantizedTensor, out_scale=None, out_zp=None) -> QuantizedTensor:
        acc, s = QuantizedOps.qmatmul_int32(a, b)
        r = acc.float() * s
        if out_scale is None:
            out_scale, out_zp = QuantParamCalculator.compute(r.min(), r.max(), a.qtype, True)
        return quantize(r, out_scale, out_zp, a.qtype)

    @staticmethod
    def qrelu(a: QuantizedTensor) -> QuantizedTensor:
        zp = a.zero_point.to(a.data.dtype) if a.zero_point.dim() == 0 else a.zero_point.view(a._bshape()).to(a.data.dtype)
        return QuantizedTensor(torch.maximum(a.data, zp.expand_as(a.data)), a.scale, a.zero_point, a.qtype, a.axis)

    @staticmethod
    def qconv2d(x: QuantizedTensor, w: QuantizedTensor, bias: Optional[torch.Tensor] = None, stride=1, padding=0) -> torch.Tensor:
        """Quantised convolution as an int8 GEMM over the unfolded patches: codes are centred by their zero points,
        multiplied on the integer tensor cores (CUDA) or exactly on the CPU, and scaled back to fp32 in the epilogue.
        Falls back to the dequantised convolution for per-channel activations or codes that do not fit int8 once
        centred."""
        st = (stride, stride) if isinstance(stride, int) else tuple(stride)
        pd = (padding, padding) if isinstance(padding, int) else tuple(padding)
        per_tensor_x = x.axis is None and x.scale.numel() == 1
        w_sym = (w.zero_point.numel() == 1 and int(w.zero_point) == 0) or (w.zero_point.numel() > 1 and not bool(w.zero_point.any()))
        if x.data.dim() != 4 or not per_tensor_x or not w_sym or (w.axis not in (None, 0)):
            return F.conv2d(x.dequantize(), w.dequantize(), bias, st, pd)
        xc = x.data.to(torch.int32) - x.zero_point.to(torch.int32)
        if int(xc.min()) < -128 or int(xc.max()) > 127:
            return F.conv2d(x.dequantize(), w.dequantize(), bias, st, pd)
        N, Cin, H, W = x.data.shape
        Cout, _, KH, KW = w.data.shape
        OH, OW = (H + 2 * pd[0] - KH) // st[0] + 1, (W + 2 * pd[1] - KW) // st[1] + 1
        cols = F.unfold(xc.float(), (KH, KW), padding=pd, stride=st)                 # [N, Cin*KH*KW, OH*OW] (zero = centred zero point)
        a = cols.transpose(1, 2).reshape(N * OH * OW, Cin * KH * KW).to(torch.int8).contiguous()
        wk = w.data.reshape(Cout, -1).to(torch.int8).contiguous()
        y = int8_gemm(a, wk, x.scale.reshape(-1)[:1], w.scale.reshape(-1) if w.scale.numel() > 1 else w.scale.reshape(-1)[:1], bias)
        return y.reshape(N, OH, OW, Cout).permute(0, 3, 1, 2).contiguous()


class DequantizeOps:
    @staticmethod
    def dequantize(q: QuantizedTensor, dtype=torch.float32) -> torch.Tensor:
        return q.dequantize(dtype)


def qlinear(x: QuantizedTensor, w: QuantizedTensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x [.., K]`` (per-tensor) times ``w [N, K]`` (per-tensor or per-output-channel, symmetric) -> fp32."""
    K = x.data.shape[-1]
    if w.zero_point.numel() == 1 and int(w.zero_point) != 0 or w.zero_point.numel() > 1 and bool(w.zero_point.any()):
        raise ValueError("qlinear expects symmetric weights (zero_point 0)")
    xc = (x.data.reshape(-1, K).to(torch.int32) - x.zero_point).clamp(-128, 127).to(torch.int8)
    # one kernel: int8 GEMM with the activation scale, the per-channel weight scales and the bias in its epilogue
    y = int8_gemm(xc, w.data.to(torch.int8), x.scale.reshape(-1)[:1], w.scale.reshape(-1), bias)
    return y.reshape(*x.data.shape[:-1], w.data.shape[0])


def qconv1d(x: QuantizedTensor, w: QuantizedTensor, bias: Optional[torch.Tensor] = None, stride: int = 1, padding: int = 0) -> torch.Tensor:
    return F.conv1d(x.dequantize(), w.dequantize(), bias, stride, padding)


# ------------------------------------------------------------------------------ QAT
class _FakeQuantFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, zp, qmin, qmax):
        q = torch.round(x / scale) + zp
        ctx.save_for_backward((q >= qmin) & (q <= qmax))
        return (q.clamp(qmin, qmax) - zp) * scale

    @staticmethod
    def backward(ctx, g):
        (mask,) = ctx.saved_tensors            # straight-through estimator inside the representable range
        return g * mask, None, None, None, None


class FakeQuantize(nn.Module):
    """Quantize-dequantize with straight-through gradients; the observer tracks the range while enabled."""

    def __init__(self, qtype: QuantizationType = QuantizationType.INT8, symmetric: bool = True, averaging: float = 0.01):
        super().__init__()
        self.qtype, self.symmetric = qtype, symmetric
        self.observer = MinMaxObserver(averaging)
        self.register_buffer("scale", torch.tensor(1.0))
        self.register_buffer("zero_point", torch.tensor(0, dtype=torch.int32))
        self.observer_enabled, self.fake_quant_enabled = True, True

    def with_observer(self, observer: Observer) -> "FakeQuantize":
        self.observer = observer
        return self

    def calibrate(self, data: torch.Tensor) -> None:
        self.observer.observe(data)
        s, z = self.observer.compute_params(self.qtype, self.symmetric)
        self.scale.copy_(s.to(self.scale.device))
        self.zero_point.copy_(z.to(self.zero_point.device))

    def forward(self, x):
        if self.observer_enabled and self.training:
            self.calibrate(x)
        if not self.fake_quant_enabled:
            return x
        qmin, qmax = self.qtype.range()
        return _FakeQuantFn.apply(x, self.scale.to(x.dtype), self.zero_point.to(x.dtype), qmin, qmax)


@dataclass
class QATConfig:
    weight_qtype: QuantizationType = QuantizationType.INT8
    activation_qtype: QuantizationType = QuantizationType.INT8
    symmetric_weights: bool = True
    symmetric_activations: bool = False
    freeze_observer_after: Optional[int] = None


class QATLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, config: Optional[QATConfig] = None):
        super().__init__()
        c = self.config = config or QATConfig()
        self.linear = nn.Linear(in_features, out_features, bias)
        self.weight_fq = FakeQuantize(c.weight_qtype, c.symmetric_weights, averaging=1.0)
        self.act_fq = FakeQuantize(c.activation_qtype, c.symmetric_activations)

    def forward(self, x):
        return F.linear(self.act_fq(x), self.weight_fq(self.linear.weight), self.linear.bias)

    def to_quantized(self) -> Tuple[QuantizedTensor, Optional[torch.Tensor]]:
        w = self.linear.weight.detach()
        return quantize(w, self.weight_fq.scale.to(w.device), self.weight_fq.zero_point.to(w.device), self.config.weight_qtype), self.linear.bias


class QATConv2d(nn.Module):
    def __init__(self, in_ch: int, out_ch: int, kernel_size, stride=1, padding=0, bias: bool = True, config: Optional[QATConfig] = None):
        super().__init__()
        c = self.config = config or QATConfig()
        self.conv = nn.Conv2d(in_ch, out_ch, kernel_size, stride, padding, bias=bias)
        self.weight_fq = FakeQuantize(c.weight_qtype, c.symmetric_weights, averaging=1.0)
        self.act_fq = FakeQuantize(c.activation_qtype, c.symmetric_activations)

    def forward(self, x):
        return F.conv2d(self.act_fq(x), self.weight_fq(self.conv.weight), self.conv.bias, self.conv.stride, self.conv.padding)


class QATTrainer:
    def __init__(self, config: Optional[QATConfig] = None):
        self.config = config or QATConfig()
        self.steps = 0

    def train_step(self, model: nn.Module, optimizer, loss_fn, x, y) -> float:
        model.train()
        optimizer.zero_grad()
        loss = loss_fn(model(x), y)
        loss.backward()
        optimizer.step()
        self.steps += 1
        if self.config.freeze_observer_after is not None and self.steps >= self.config.freeze_observer_after:
            for m in model.modules():
                if isinstance(m, FakeQuantize):
                    m.observer_enabled = False
        return float(loss)

    def prepare_for_deployment(self, model: nn.Module) -> None:
        model.eval()
        for m in model.modules():
            if isinstance(m, FakeQuantize):
                m.observer_enabled = False


def prepare_qat(model: nn.Module, config: Optional[QATConfig] = None) -> nn.Module:
    """Swap every ``nn.Linear`` / ``nn.Conv2d`` for its QAT twin (weights shared)."""
    for name, child in list(model.named_children()):
        if isinstance(child, nn.Linear):
            q = QATLinear(child.in_features, child.out_features, child.bias is not None, config)
            q.linear = child
            setattr(model, name, q)
        elif isinstance(child, nn.Conv2d) and child.groups == 1 and child.dilation == (1, 1):
            q = QATConv2d(child.in_channels, child.out_channels, child.kernel_size, child.stride, child.padding, child.bias is not None, config)
            q.conv = child
            setattr(model, name, q)
        else:
            prepare_qat(child, config)
    return model


def qmatmul_cuda(a: "QuantizedTensor", b: "QuantizedTensor", out_scale=None, out_zp=None) -> "QuantizedTensor":
    """Quantised matmul on the GPU: the integer product runs on the tcgen05 int8 GEMM (``int8_gemm``), the zero-point
    corrections and the requantisation follow.  (The reference's qmatmul_cuda runs CPU loops behind the name,
    src/quantization/hardware/cuda.rs:12-27.)"""
    if torch.cuda.is_available():
        a, b = a.to("cuda") if hasattr(a, "to") else a, b.to("cuda") if hasattr(b, "to") else b
    return QuantizedOps.qmatmul(a, b, out_scale, out_zp)


def qconv2d_cuda(x: "QuantizedTensor", w: "QuantizedTensor", bias=None, stride=1, padding=0) -> torch.Tensor:
    """Quantised conv2d on the GPU: patches x filters as one tcgen05 int8 GEMM with the scales and bias in its epilogue
    (src/quantization/hardware/cuda.rs:29-48 names it, CPU loops run behind it there)."""
    if torch.cuda.is_available():
        x, w = x.to("cuda") if hasattr(x, "to") else x, w.to("cuda") if hasattr(w, "to") else w
    return QuantizedOps.qconv2d(x, w, bias, stride, padding)
