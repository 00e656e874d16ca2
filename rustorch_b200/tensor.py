"""``Tensor``: the RusTorch tensor surface over ``torch.Tensor``.

Method names, argument order and defaults follow the reference's ``Tensor<T>``
(src/tensor/core.rs:25-35,40-114,240-404; ops under src/tensor/ops/*) so code written against
RusTorch's API reads the same here; the data lives in a ``torch.Tensor`` (``.data``), which on a
CUDA device really is on the GPU (the reference's ``device`` is a tag only and its tensors never
leave host memory, src/tensor/core.rs:136-138,168-179).

Anything not spelled out below falls through to the wrapped ``torch.Tensor`` via
``__getattr__`` with results re-wrapped, so the full PyTorch method set is available too.
"""
from __future__ import annotations

import math
from typing import Iterable, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ._interop import FlagValue, IntValue, ShapeValue
from .dtype import DType, to_torch_dtype

Number = Union[int, float]


class Device:
    """``Cpu / Cuda(idx) / Mps / Wasm`` device tag (src/tensor/device.rs:10-47); only cpu/cuda exist here."""

    def __init__(self, kind: str = "cpu", index: int = 0):
        kind = kind.lower()
        if ":" in kind:
            kind, idx = kind.split(":")
            index = int(idx)
        if kind in ("gpu",):
            kind = "cuda"
        if kind not in ("cpu", "cuda"):
            raise ValueError(f"device '{kind}' does not exist in this build (cpu and cuda only)")
        self.kind, self.index = kind, index

    @staticmethod
    def cpu() -> "Device":
        return Device("cpu")

    @staticmethod
    def cuda(index: int = 0) -> "Device":
        return Device("cuda", index)

    def is_cuda(self) -> bool:
        return self.kind == "cuda"

    def to_torch(self) -> torch.device:
        return torch.device(self.kind, self.index) if self.kind == "cuda" else torch.device("cpu")

    def __str__(self) -> str:
        return f"cuda:{self.index}" if self.kind == "cuda" else "cpu"

    __repr__ = __str__

    def __eq__(self, other) -> bool:
        return isinstance(other, Device) and str(self) == str(other)


def _dev(device) -> torch.device:
    if device is None:
        return torch.device("cpu")
    if isinstance(device, Device):
        return device.to_torch()
    return torch.device(device)


def _unwrap(x):
    if isinstance(x, Tensor):
        return x.data
    if isinstance(x, (list, tuple)):
        return type(x)(_unwrap(v) for v in x)
    return x


def _wrap(x):
    if isinstance(x, torch.Tensor):
        return Tensor(x)
    if isinstance(x, (list, tuple)):
        return type(x)(_wrap(v) for v in x)
    return x


class Tensor:
    __slots__ = ("data",)
    __array_priority__ = 100

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        """``torch.*`` / ``torch.nn.functional.*`` calls and ``torch.nn`` layers accept a ``Tensor``: the call runs on
        the wrapped tensors and tensor results come back wrapped."""
        from ._interop import torch_function
        return torch_function(cls, func, types, args, kwargs)

    # ------------------------------------------------------------ construction
    def __init__(self, data=None, shape: Optional[Sequence[int]] = None, dtype=None, device=None,
                 requires_grad: bool = False):
        if isinstance(data, Tensor):
            t = data.data
        elif isinstance(data, torch.Tensor):
            t = data
        else:
            t = torch.as_tensor(np.asarray(data, dtype=np.float32) if dtype is None and not isinstance(data, np.ndarray) else data)
        if dtype is not None:
            t = t.to(to_torch_dtype(dtype))
        if shape is not None:
            if int(np.prod(shape)) != t.numel():
                raise ValueError(f"shape {tuple(shape)} does not match {t.numel()} elements")
            t = t.reshape(tuple(shape))
        if device is not None:
            t = t.to(_dev(device))
        if requires_grad:
            t = t.detach().requires_grad_(True)
        self.data = t

    new = classmethod(lambda cls, data, shape=None, **kw: cls(data, shape, **kw))

    @classmethod
    def from_vec(cls, data: Sequence[Number], shape: Sequence[int], **kw) -> "Tensor":
        return cls(list(data), shape, **kw)

    try_from_vec = from_vec

    @classmethod
    def from_ndarray(cls, arr: np.ndarray, **kw) -> "Tensor":
        return cls(torch.from_numpy(np.ascontiguousarray(arr)), **kw)

    from_numpy = from_ndarray

    @classmethod
    def from_scalar(cls, v: Number, **kw) -> "Tensor":
        return cls(torch.tensor(float(v)), **kw)

    @classmethod
    def _wrap(cls, t: torch.Tensor) -> "Tensor":
        """Wrap an existing torch tensor without the conversions of ``__init__`` (creation fast path)."""
        obj = cls.__new__(cls)
        obj.data = t
        return obj

    @classmethod
    def zeros(cls, shape, dtype=None, device=None) -> "Tensor":
        if dtype is None and device is None:
            return cls._wrap(torch.zeros(shape, dtype=torch.float32))
        return cls(torch.zeros(tuple(shape), dtype=to_torch_dtype(dtype or "f32"), device=_dev(device)))

    @classmethod
    def ones(cls, shape, dtype=None, device=None) -> "Tensor":
        if dtype is None and device is None:
            return cls._wrap(torch.ones(shape, dtype=torch.float32))
        return cls(torch.ones(tuple(shape), dtype=to_torch_dtype(dtype or "f32"), device=_dev(device)))

    @classmethod
    def full(cls, shape, value: Number, dtype=None, device=None) -> "Tensor":
        return cls(torch.full(tuple(shape), value, dtype=to_torch_dtype(dtype or "f32"), device=_dev(device)))

    zeros_on_device = classmethod(lambda cls, shape, device: cls.zeros(shape, device=device))
    ones_on_device = classmethod(lambda cls, shape, device: cls.ones(shape, device=device))
    zeros_auto = classmethod(lambda cls, shape: cls.zeros(shape, device="cuda" if torch.cuda.is_available() else "cpu"))
    ones_auto = classmethod(lambda cls, shape: cls.ones(shape, device="cuda" if torch.cuda.is_available() else "cpu"))

    # creation ops (src/tensor/ops/creation.rs:14-325)
    @classmethod
    def randn(cls, shape, dtype=None, device=None, generator=None) -> "Tensor":
        return cls(torch.randn(tuple(shape), dtype=to_torch_dtype(dtype or "f32"), device=_dev(device), generator=generator))

    @classmethod
    def rand(cls, shape, dtype=None, device=None, generator=None) -> "Tensor":
        return cls(torch.rand(tuple(shape), dtype=to_torch_dtype(dtype or "f32"), device=_dev(device), generator=generator))

    @classmethod
    def uniform(cls, shape, low: float = 0.0, high: float = 1.0, device=None) -> "Tensor":
        return cls(torch.empty(tuple(shape), device=_dev(device)).uniform_(low, high))

    @classmethod
    def randint(cls, low: int, high: int, shape, device=None) -> "Tensor":
        return cls(torch.randint(low, high, tuple(shape), device=_dev(device)).float())

    @classmethod
    def eye(cls, n: int, device=None) -> "Tensor":
        return cls(torch.eye(n, device=_dev(device)))

    @classmethod
    def arange(cls, start: Number, end: Optional[Number] = None, step: Number = 1, device=None) -> "Tensor":
        if end is None:
            start, end = 0, start
        return cls(torch.arange(start, end, step, dtype=torch.float32, device=_dev(device)))

    @classmethod
    def linspace(cls, start: Number, end: Number, steps: int, device=None) -> "Tensor":
        return cls(torch.linspace(start, end, steps, device=_dev(device)))

    @classmethod
    def logspace(cls, start: Number, end: Number, steps: int, base: float = 10.0, device=None) -> "Tensor":
        return cls(torch.logspace(start, end, steps, base=base, device=_dev(device)))

    @classmethod
    def diag(cls, values) -> "Tensor":
        return cls(torch.diag(_unwrap(values) if isinstance(values, Tensor) else torch.as_tensor(values, dtype=torch.float32)))

    @staticmethod
    def meshgrid(*tensors: "Tensor", indexing: str = "ij") -> Tuple["Tensor", ...]:
        return tuple(Tensor(t) for t in torch.meshgrid(*[_unwrap(t) for t in tensors], indexing=indexing))

    # --------------------------------------------------------------- accessors
    # ``shape`` / ``ndim`` / ``numel`` / ``requires_grad`` read as attributes (the Python wheel) or as calls (Rust)
    @property
    def shape(self) -> Tuple[int, ...]:
        return ShapeValue(self.data.shape)

    @property
    def ndim(self) -> int:
        return IntValue(self.data.dim())

    def __call__(self) -> "Tensor":
        """``v.data()`` and ``v.grad()`` (Rust spelling) on the attribute values ``v.data`` / ``v.grad`` (wheel spelling)."""
        return self

    def size(self) -> Tuple[int, ...]:
        return tuple(self.data.shape)

    @property
    def numel(self) -> int:
        return IntValue(self.data.numel())

    def len(self) -> int:
        return self.data.numel()

    def is_empty(self) -> bool:
        return self.data.numel() == 0

    def device(self) -> Device:
        d = self.data.device
        return Device(d.type, d.index or 0)

    def dtype(self) -> DType:
        return DType.from_torch(self.data.dtype)

    @property
    def requires_grad(self) -> bool:
        return FlagValue(self.data.requires_grad)

    def set_requires_grad(self, flag: bool = True) -> "Tensor":
        self.data.requires_grad_(flag)
        return self

    def get(self, index: Sequence[int]) -> float:
        return float(self.data[tuple(index)])

    def set(self, index: Sequence[int], value: Number) -> None:
        self.data[tuple(index)] = value

    def item(self) -> float:
        return float(self.data.item())

    def as_slice(self) -> List[float]:
        return self.data.detach().reshape(-1).tolist()

    to_vec = as_slice
    tolist = lambda self: self.data.detach().tolist()  # noqa: E731

    def numpy(self) -> np.ndarray:
        return self.data.detach().cpu().numpy()

    as_array = numpy

    def to_device(self, device) -> "Tensor":
        return Tensor(self.data.to(_dev(device)))

    to = to_device

    def try_to_gpu(self, index: int = 0) -> "Tensor":
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device available")
        return Tensor(self.data.to(torch.device("cuda", index)))

    def cpu(self) -> "Tensor":
        return Tensor(self.data.cpu())

    def cuda(self, index: int = 0) -> "Tensor":
        return self.try_to_gpu(index)

    def is_cuda(self) -> bool:
        return self.data.is_cuda

    def clone(self) -> "Tensor":
        return Tensor(self.data.clone())

    def detach(self) -> "Tensor":
        return Tensor(self.data.detach())

    def astype(self, dtype) -> "Tensor":
        return Tensor(self.data.to(to_torch_dtype(dtype)))

    def copy_from(self, other: "Tensor") -> "Tensor":
        with torch.no_grad():
            self.data.copy_(_unwrap(other))
        return self

    # ------------------------------------------------------------------ shape
    def reshape(self, shape: Sequence[int]) -> "Tensor":
        return Tensor(self.data.reshape(tuple(shape)))

    view_shape = reshape

    def try_view(self, shape: Sequence[int]) -> "Tensor":
        return Tensor(self.data.view(tuple(shape)))

    view = try_view

    def squeeze(self, dim: Optional[int] = None) -> "Tensor":
        return Tensor(self.data.squeeze() if dim is None else self.data.squeeze(dim))

    def unsqueeze(self, dim: int) -> "Tensor":
        return Tensor(self.data.unsqueeze(dim))

    def expand(self, shape: Sequence[int]) -> "Tensor":
        return Tensor(self.data.expand(*shape))

    def expand_as(self, other: "Tensor") -> "Tensor":
        return Tensor(self.data.expand_as(_unwrap(other)))

    def broadcast_with(self, other: "Tensor") -> Tuple["Tensor", "Tensor"]:
        a, b = torch.broadcast_tensors(self.data, _unwrap(other))
        return Tensor(a), Tensor(b)

    def flatten(self, start_dim: int = 0, end_dim: int = -1) -> "Tensor":
        return Tensor(self.data.flatten(start_dim, end_dim))

    def unflatten(self, dim: int, sizes: Sequence[int]) -> "Tensor":
        return Tensor(self.data.unflatten(dim, tuple(sizes)))

    def repeat(self, repeats: Sequence[int]) -> "Tensor":
        return Tensor(self.data.repeat(*repeats))

    tile = repeat

    def repeat_interleave(self, repeats: int, dim: Optional[int] = None) -> "Tensor":
        return Tensor(self.data.repeat_interleave(repeats, dim=dim))

    def roll(self, shifts, dims=None) -> "Tensor":
        return Tensor(torch.roll(self.data, shifts, dims))

    def rot90(self, k: int = 1, dims: Sequence[int] = (0, 1)) -> "Tensor":
        return Tensor(torch.rot90(self.data, k, list(dims)))

    def flip(self, dims: Sequence[int]) -> "Tensor":
        return Tensor(torch.flip(self.data, list(dims)))

    def fliplr(self) -> "Tensor":
        return Tensor(torch.fliplr(self.data))

    def flipud(self) -> "Tensor":
        return Tensor(torch.flipud(self.data))

    def permute(self, dims: Sequence[int]) -> "Tensor":
        return Tensor(self.data.permute(*dims))

    def movedim(self, src, dst) -> "Tensor":
        return Tensor(self.data.movedim(src, dst))

    def swapaxes(self, a: int, b: int) -> "Tensor":
        return Tensor(self.data.transpose(a, b))

    def transpose(self, dim0: Optional[int] = None, dim1: Optional[int] = None) -> "Tensor":
        """2-D transpose with no arguments (src/tensor/ops/matrix.rs:199-216), else swap two dims."""
        if dim0 is None:
            if self.data.dim() < 2:
                return Tensor(self.data.clone())
            return Tensor(self.data.transpose(-1, -2))
        return Tensor(self.data.transpose(dim0, dim1))

    def transpose_last_two(self) -> "Tensor":
        return Tensor(self.data.transpose(-1, -2))

    t = transpose
    T = property(lambda self: Tensor(self.data.transpose(-1, -2)))

    def contiguous(self) -> "Tensor":
        return Tensor(self.data.contiguous())

    # -------------------------------------------------------------- arithmetic
    def _bin(self, other, fn) -> "Tensor":
        return Tensor(fn(self.data, _unwrap(other)))

    def add(self, other) -> "Tensor":
        return self._bin(other, torch.add)

    def sub(self, other) -> "Tensor":
        return self._bin(other, torch.sub)

    def mul(self, other) -> "Tensor":
        return self._bin(other, torch.mul)

    def div(self, other) -> "Tensor":
        return self._bin(other, torch.div)

    add_scalar = add
    sub_scalar = sub
    mul_scalar = mul
    div_scalar = div

    def neg(self) -> "Tensor":
        return Tensor(-self.data)

    def maximum(self, other) -> "Tensor":
        return self._bin(other, torch.maximum)

    def minimum(self, other) -> "Tensor":
        return self._bin(other, torch.minimum)

    __add__ = add
    __radd__ = add
    __sub__ = sub
    __mul__ = mul
    __rmul__ = mul
    __truediv__ = div
    __neg__ = neg

    def __rsub__(self, other):
        return Tensor(_unwrap(other) - self.data)

    def __rtruediv__(self, other):
        return Tensor(_unwrap(other) / self.data)

    def __pow__(self, e):
        return Tensor(self.data ** _unwrap(e))

    def __matmul__(self, other):
        return self.matmul(other)

    def __getitem__(self, idx):
        return Tensor(self.data[_unwrap(idx)])

    def __setitem__(self, idx, v):
        self.data[_unwrap(idx)] = _unwrap(v)

    def __len__(self):
        return self.data.shape[0]

    def __eq__(self, other):  # elementwise, like torch
        return Tensor(self.data == _unwrap(other))

    def __ne__(self, other):
        return Tensor(self.data != _unwrap(other))

    def __iter__(self):
        """Slices along the first dimension, as ``torch.Tensor`` iterates."""
        if self.data.dim() == 0:
            raise TypeError("iteration over a 0-d tensor")
        return (Tensor(t) for t in self.data)

    def __array__(self, dtype=None, copy=None):
        """NumPy conversion (``np.asarray(t)``); CUDA data is copied to the host."""
        a = self.data.detach().cpu().numpy()
        return a.astype(dtype) if dtype is not None else a

    def __lt__(self, o):
        return Tensor(self.data < _unwrap(o))

    def __gt__(self, o):
        return Tensor(self.data > _unwrap(o))

    def __le__(self, o):
        return Tensor(self.data <= _unwrap(o))

    def __ge__(self, o):
        return Tensor(self.data >= _unwrap(o))

    __hash__ = object.__hash__

    def __repr__(self) -> str:
        return f"Tensor(shape={list(self.data.shape)}, device={self.device()}, data={self.data})"

    def __float__(self):
        return float(self.data)

    def __int__(self):
        return int(self.data)

    def __bool__(self):
        return bool(self.data)

    def __format__(self, spec: str) -> str:
        """One-element tensors format like the number they hold (``f"{loss:.3f}"``: the binding's sum / mean / losses
        are plain floats, python/src/lib.rs:150-165)."""
        if spec and self.data.numel() == 1:
            return format(self.data.item(), spec)
        return str(self) if not spec else format(str(self), spec)

    # ------------------------------------------------------------------ matrix
    def matmul(self, other) -> "Tensor":
        """2D x 2D, 1D x 2D, 2D x 1D and batched products (src/tensor/ops/matrix.rs:42-157).

        bf16 CUDA operands of rank 2/3 run on the hand-written tcgen05 GEMM; everything else on
        torch.matmul.
        """
        a, b = self.data, _unwrap(other)
        if (a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == b.dim()
                and a.dim() in (2, 3) and a.shape[-1] % 8 == 0 and b.shape[-1] % 8 == 0
                and a.stride(-1) == 1 and b.stride(-1) == 1 and not (a.requires_grad or b.requires_grad)):
            from .ops import kernels as K
            return Tensor(K.gemm(a, b, b_mn=True))
        return Tensor(torch.matmul(a, b))

    mm = matmul
    bmm = matmul

    def dot(self, other) -> "Tensor":
        return Tensor(torch.dot(self.data.reshape(-1), _unwrap(other).reshape(-1)))

    def det(self) -> float:
        return float(torch.linalg.det(self.data))

    def trace(self) -> float:
        return float(torch.trace(self.data))

    # -------------------------------------------------------------------- math
    def pow(self, e: Number) -> "Tensor":
        return Tensor(self.data.pow(e))

    def pow_tensor(self, e: "Tensor") -> "Tensor":
        return Tensor(self.data.pow(_unwrap(e)))

    def log(self, base: Optional[float] = None) -> "Tensor":
        return Tensor(self.data.log() if base is None else self.data.log() / math.log(base))

    ln = lambda self: Tensor(self.data.log())  # noqa: E731

    def square(self) -> "Tensor":
        return Tensor(self.data * self.data)

    def cbrt(self) -> "Tensor":
        return Tensor(torch.sign(self.data) * self.data.abs().pow(1.0 / 3.0))

    def clamp(self, lo: Optional[Number] = None, hi: Optional[Number] = None) -> "Tensor":
        return Tensor(self.data.clamp(lo, hi))

    def min_scalar(self, v: Number) -> "Tensor":
        return Tensor(self.data.clamp(max=v))

    def max_scalar(self, v: Number) -> "Tensor":
        return Tensor(self.data.clamp(min=v))

    def fract(self) -> "Tensor":
        return Tensor(self.data - self.data.trunc())

    def is_finite(self) -> bool:
        return bool(torch.isfinite(self.data).all())

    def has_nan(self) -> bool:
        return bool(torch.isnan(self.data).any())

    def has_inf(self) -> bool:
        return bool(torch.isinf(self.data).any())

    def nan_to_num(self, nan: float = 0.0, posinf: Optional[float] = None, neginf: Optional[float] = None) -> "Tensor":
        return Tensor(torch.nan_to_num(self.data, nan, posinf, neginf))

    def inf_to_num(self, value: float = 0.0) -> "Tensor":
        return Tensor(torch.where(torch.isinf(self.data), torch.full_like(self.data, value), self.data))

    def normalize_0_1(self) -> "Tensor":
        lo, hi = self.data.min(), self.data.max()
        return Tensor((self.data - lo) / (hi - lo).clamp_min(1e-12))

    def standardize(self) -> "Tensor":
        return Tensor((self.data - self.data.mean()) / self.data.std(unbiased=False).clamp_min(1e-12))

    def atan2(self, other) -> "Tensor":
        return self._bin(other, torch.atan2)

    def lerp(self, end, weight: float) -> "Tensor":
        return Tensor(torch.lerp(self.data, _unwrap(end), weight))

    def gamma(self) -> "Tensor":
        return Tensor(torch.exp(torch.lgamma(self.data)) * _gamma_sign(self.data))

    def relu(self) -> "Tensor":
        return Tensor(torch.relu(self.data))

    def gelu(self) -> "Tensor":
        return Tensor(torch.nn.functional.gelu(self.data, approximate="tanh"))

    def softmax(self, dim: int = -1) -> "Tensor":
        return Tensor(torch.softmax(self.data, dim))

    # -------------------------------------------------------------- reductions
    def sum(self, dim=None, keepdim: bool = False):
        return Tensor(self.data.sum() if dim is None else self.data.sum(dim, keepdim))

    def mean(self, dim=None, keepdim: bool = False):
        return Tensor(self.data.mean() if dim is None else self.data.mean(dim, keepdim))

    def sum_axis(self, axis: int) -> "Tensor":
        return Tensor(self.data.sum(axis))

    def mean_axis(self, axis: int) -> "Tensor":
        return Tensor(self.data.mean(axis))

    def max(self, dim=None):
        return Tensor(self.data.max()) if dim is None else Tensor(self.data.max(dim).values)

    def min(self, dim=None):
        return Tensor(self.data.min()) if dim is None else Tensor(self.data.min(dim).values)

    max_axis = lambda self, axis: Tensor(self.data.max(axis).values)  # noqa: E731
    min_axis = lambda self, axis: Tensor(self.data.min(axis).values)  # noqa: E731

    def var(self, unbiased: bool = False) -> "Tensor":
        return Tensor(self.data.var(unbiased=unbiased))

    def std(self, unbiased: bool = False) -> "Tensor":
        return Tensor(self.data.std(unbiased=unbiased))

    var_unbiased = lambda self: Tensor(self.data.var(unbiased=True))  # noqa: E731
    var_axis = lambda self, axis, unbiased=False: Tensor(self.data.var(axis, unbiased=unbiased))  # noqa: E731
    std_axis = lambda self, axis, unbiased=False: Tensor(self.data.std(axis, unbiased=unbiased))  # noqa: E731

    def count_nonzero(self) -> int:
        return int(torch.count_nonzero(self.data))

    def argmax(self, dim=None):
        r = self.data.argmax() if dim is None else self.data.argmax(dim)
        return int(r) if r.dim() == 0 else Tensor(r)

    def argmin(self, dim=None):
        r = self.data.argmin() if dim is None else self.data.argmin(dim)
        return int(r) if r.dim() == 0 else Tensor(r)

    argmax_axis = lambda self, axis: Tensor(self.data.argmax(axis))  # noqa: E731
    argmin_axis = lambda self, axis: Tensor(self.data.argmin(axis))  # noqa: E731

    def median(self) -> float:
        return float(self.data.reshape(-1).median())

    def quantile(self, q: float) -> float:
        return float(torch.quantile(self.data.reshape(-1).float(), q))

    def percentile(self, p: float) -> float:
        return self.quantile(p / 100.0)

    def cumsum(self, dim: int = 0) -> "Tensor":
        return Tensor(self.data.cumsum(dim))

    def cumprod(self, dim: int = 0) -> "Tensor":
        return Tensor(self.data.cumprod(dim))

    def topk(self, k: int, dim: int = -1, largest: bool = True) -> Tuple["Tensor", "Tensor"]:
        v, i = self.data.topk(k, dim, largest)
        return Tensor(v), Tensor(i)

    def bottomk(self, k: int, dim: int = -1) -> Tuple["Tensor", "Tensor"]:
        return self.topk(k, dim, largest=False)

    def kthvalue(self, k: int, dim: int = -1) -> Tuple["Tensor", "Tensor"]:
        v, i = self.data.kthvalue(k, dim)
        return Tensor(v), Tensor(i)

    def cov(self) -> "Tensor":
        return Tensor(torch.cov(self.data))

    def corrcoef(self) -> "Tensor":
        return Tensor(torch.corrcoef(self.data))

    def unique(self) -> "Tensor":
        return Tensor(torch.unique(self.data))

    def histogram(self, bins: int = 10, range: Optional[Tuple[float, float]] = None) -> Tuple["Tensor", "Tensor"]:
        x = self.data.detach().float().cpu().reshape(-1)
        lo, hi = (float(x.min()), float(x.max())) if range is None else range
        h = torch.histc(x, bins, lo, hi)
        return Tensor(h), Tensor(torch.linspace(lo, hi, bins + 1))

    # ------------------------------------------------------------------ linalg
    def svd(self, full_matrices: bool = False):
        u, s, vh = torch.linalg.svd(self.data, full_matrices=full_matrices)
        return Tensor(u), Tensor(s), Tensor(vh.transpose(-1, -2))

    def qr(self):
        q, r = torch.linalg.qr(self.data)
        return Tensor(q), Tensor(r)

    def lu(self):
        p, l, u = torch.linalg.lu(self.data)
        return Tensor(l), Tensor(u), Tensor(p)

    def eig(self):
        w, v = torch.linalg.eig(self.data)
        return Tensor(w), Tensor(v)

    def symeig(self, upper: bool = False):
        w, v = torch.linalg.eigh(self.data, UPLO="U" if upper else "L")
        return Tensor(w), Tensor(v)

    eigh = symeig

    def cholesky(self, upper: bool = False) -> "Tensor":
        return Tensor(torch.linalg.cholesky(self.data, upper=upper))

    def inverse(self) -> "Tensor":
        return Tensor(torch.linalg.inv(self.data))

    def pinv(self) -> "Tensor":
        return Tensor(torch.linalg.pinv(self.data))

    def norm(self, p: Union[int, float, str] = 2) -> float:
        return float(torch.linalg.vector_norm(self.data.reshape(-1).float(), p) if not isinstance(p, str)
                     else torch.linalg.matrix_norm(self.data, p))

    norm_p = norm
    frobenius_norm = lambda self: float(torch.linalg.matrix_norm(self.data, "fro"))  # noqa: E731
    nuclear_norm = lambda self: float(torch.linalg.matrix_norm(self.data, "nuc"))  # noqa: E731

    # ------------------------------------------------------------------ signal
    def fft(self, n: Optional[int] = None, dim: Optional[int] = None, norm: Optional[str] = None) -> "Tensor":
        """``fft(n, dim, norm)`` on real or complex data (src/tensor/complex_impl/matrix.rs:154-191)."""
        return Tensor(torch.fft.fft(self.data, n=n, dim=-1 if dim is None else dim, norm=norm or "backward"))

    def ifft(self, n: Optional[int] = None, dim: Optional[int] = None, norm: Optional[str] = None) -> "Tensor":
        return Tensor(torch.fft.ifft(self.data, n=n, dim=-1 if dim is None else dim, norm=norm or "backward"))

    # complex tensors (src/tensor/complex_impl/tensor_ops.rs:28-64, matrix.rs:61-152)
    def is_complex(self) -> bool:
        return self.data.is_complex()

    def real_part(self) -> "Tensor":
        return Tensor(self.data.real.clone() if self.data.is_complex() else self.data.clone())

    def imag_part(self) -> "Tensor":
        return Tensor(self.data.imag.clone() if self.data.is_complex() else torch.zeros_like(self.data))

    def arg(self) -> "Tensor":
        return Tensor(self.data.angle())

    def conj(self) -> "Tensor":
        return Tensor(self.data.conj().resolve_conj())

    def conj_transpose(self) -> "Tensor":
        return Tensor(self.data.transpose(-1, -2).conj().resolve_conj().contiguous())

    def rfft(self) -> "Tensor":
        return Tensor(torch.fft.rfft(self.data))

    def fftshift(self) -> "Tensor":
        return Tensor(torch.fft.fftshift(self.data))

    def ifftshift(self) -> "Tensor":
        return Tensor(torch.fft.ifftshift(self.data))

    def apply_window(self, window: str = "hann") -> "Tensor":
        n = self.data.shape[-1]
        w = {"hann": torch.hann_window, "hanning": torch.hann_window, "hamming": torch.hamming_window,
             "blackman": torch.blackman_window, "bartlett": torch.bartlett_window,
             "rectangular": lambda n, **k: torch.ones(n)}[window.lower()](n, periodic=False)
        return Tensor(self.data * w.to(self.data.device, self.data.dtype))

    # --------------------------------------------------------------- utilities
    def where_(self, cond, other) -> "Tensor":
        return Tensor(torch.where(_unwrap(cond).bool(), self.data, _unwrap(other) if isinstance(other, Tensor)
                                  else torch.as_tensor(other, dtype=self.data.dtype, device=self.data.device)))

    def masked_select(self, mask) -> "Tensor":
        return Tensor(self.data.masked_select(_unwrap(mask).bool()))

    def masked_fill(self, mask, value: Number) -> "Tensor":
        return Tensor(self.data.masked_fill(_unwrap(mask).bool(), value))

    def gather(self, dim: int, index) -> "Tensor":
        return Tensor(self.data.gather(dim, _unwrap(index).long()))

    def scatter(self, dim: int, index, src) -> "Tensor":
        return Tensor(self.data.scatter(dim, _unwrap(index).long(), _unwrap(src)))

    def index_select(self, dim: int, index) -> "Tensor":
        return Tensor(self.data.index_select(dim, _unwrap(index).long()))

    def select(self, dim: int, index: int) -> "Tensor":
        return Tensor(self.data.select(dim, index))

    def chunk(self, chunks: int, dim: int = 0) -> List["Tensor"]:
        return [Tensor(t) for t in self.data.chunk(chunks, dim)]

    def split(self, size, dim: int = 0) -> List["Tensor"]:
        return [Tensor(t) for t in self.data.split(size, dim)]

    def map(self, fn) -> "Tensor":
        flat = [fn(v) for v in self.as_slice()]
        return Tensor(flat, self.shape(), device=self.data.device)

    def zip_with(self, other: "Tensor", fn) -> "Tensor":
        flat = [fn(a, b) for a, b in zip(self.as_slice(), other.as_slice())]
        return Tensor(flat, self.shape(), device=self.data.device)

    @staticmethod
    def stack(tensors: Sequence["Tensor"], dim: int = 0) -> "Tensor":
        return Tensor(torch.stack([_unwrap(t) for t in tensors], dim))

    @staticmethod
    def concatenate(tensors: Sequence["Tensor"], dim: int = 0) -> "Tensor":
        return Tensor(torch.cat([_unwrap(t) for t in tensors], dim))

    concat = cat = concatenate

    # ----------------------------------------------------------------- autograd
    def backward(self, grad=None) -> None:
        self.data.backward(_unwrap(grad))

    @property
    def grad(self) -> Optional["Tensor"]:
        g = self.data.grad
        return None if g is None else Tensor(g)

    def zero_grad(self) -> None:
        self.data.grad = None

    # -------------------------------------------------------------------- save
    def save(self, path: str) -> None:
        """RUSTORCH container, object type ``tensor`` (src/tensor/core.rs:726-734)."""
        from .formats import rustorch_bin
        rustorch_bin.save_tensor(self.data, path)

    @staticmethod
    def load(path: str) -> "Tensor":
        from .formats import rustorch_bin
        return Tensor(rustorch_bin.load_tensor(path))

    # ------------------------------------------------------ torch fall-through
    # ------------------------------------------------ GpuLinearAlgebra / GpuReduction / GpuParallelOp traits
    # (src/gpu/matrix_ops.rs:274-632, src/tensor/gpu_parallel.rs:139-333): the operands move to the GPU when there is
    # one; bf16 matrices go through the tcgen05 GEMM, everything else through the library kernels.
    def _gpu(self) -> torch.Tensor:
        return self.data.cuda() if torch.cuda.is_available() and not self.data.is_cuda else self.data

    def gpu_matmul(self, other) -> "Tensor":
        from .gpu.devices import MatMulKernel
        return Tensor(MatMulKernel()(self._gpu(), Tensor(_unwrap(other))._gpu()))

    def gpu_batch_matmul(self, other) -> "Tensor":
        return Tensor(torch.matmul(self._gpu(), Tensor(_unwrap(other))._gpu()))

    def gpu_matvec(self, vec) -> "Tensor":
        return Tensor(self._gpu() @ Tensor(_unwrap(vec))._gpu())

    def gpu_conv2d(self, weight, bias=None, stride=1, padding=0) -> "Tensor":
        from .ops import conv
        b = None if bias is None else Tensor(_unwrap(bias))._gpu()
        return Tensor(conv.conv2d(self._gpu(), Tensor(_unwrap(weight))._gpu(), b, stride, padding))

    def gpu_sum(self) -> float:
        return float(self._gpu().sum())

    def gpu_mean(self) -> float:
        return float(self._gpu().mean())

    def gpu_max(self) -> float:
        return float(self._gpu().max())

    def gpu_min(self) -> float:
        return float(self._gpu().min())

    def gpu_std(self, unbiased: bool = False) -> float:
        return float(self._gpu().std(unbiased=unbiased))

    def gpu_var(self, unbiased: bool = False) -> float:
        return float(self._gpu().var(unbiased=unbiased))

    def topk_util(self, k: int, dim: int = -1, largest: bool = True):
        return self.topk(k, dim, largest)

    def quantile_util(self, q: float) -> float:
        return self.quantile(q)

    # ------------------------------------------------ device / metadata helpers (src/tensor/core.rs:436-445,640-790)
    def resolve_dim(self, dim: int) -> int:
        """Non-negative index of ``dim`` (negative values count from the end)."""
        n = self.data.dim()
        if not -n <= dim < n:
            raise IndexError(f"Dimension {dim} out of range for tensor with {n} dimensions")
        return dim % n if n else 0

    def to_cpu(self) -> "Tensor":
        return Tensor(self.data.cpu())

    def is_on_gpu(self) -> bool:
        return self.data.is_cuda

    def device_type(self) -> str:
        return self.data.device.type

    def with_device(self, device) -> "Tensor":
        return self.to_device(device)

    def clone_to_device(self, device) -> "Tensor":
        return Tensor(self.data.detach().clone().to(_dev(device)))

    def clone_with_grad(self) -> "Tensor":
        """A copy that keeps ``requires_grad`` and, when there is one, a copy of the gradient."""
        t = self.data.detach().clone().requires_grad_(self.data.requires_grad)
        if self.data.grad is not None:
            t.grad = self.data.grad.detach().clone()
        return Tensor(t)

    def auto_device(self) -> "Tensor":
        """On the GPU when one is there, else unchanged."""
        return self.to_device("cuda") if torch.cuda.is_available() and not self.data.is_cuda else self

    def as_ptr(self) -> int:
        return self.data.data_ptr()

    def get_metadata(self) -> dict:
        """String-valued description used by the serializers (shape, dtype, device, element count, gradient flag)."""
        return {"shape": str(list(self.data.shape)), "dtype": str(self.data.dtype).replace("torch.", ""),
                "device": str(self.data.device), "numel": str(self.data.numel()), "requires_grad": str(self.data.requires_grad).lower()}

    def batch_size(self) -> int:
        return self.data.shape[0] if self.data.dim() else 1

    # ------------------------------------------------ shape variants (src/tensor/ops/shape_operations.rs, advanced_shape.rs)
    def can_broadcast_with(self, other) -> bool:
        a, b = tuple(self.data.shape), tuple(_unwrap(other).shape)
        return all(x == y or x == 1 or y == 1 for x, y in zip(reversed(a), reversed(b)))

    def squeeze_dim(self, dim: int) -> "Tensor":
        d = self.resolve_dim(dim)
        if self.data.shape[d] != 1:
            raise ValueError(f"Cannot squeeze dimension {dim} with size {self.data.shape[d]}")
        return Tensor(self.data.squeeze(d))

    def squeeze_all(self) -> "Tensor":
        return Tensor(self.data.squeeze())

    squeeze_view = squeeze_all

    def squeeze_inplace(self) -> "Tensor":
        self.data = self.data.squeeze()
        return self

    def unsqueeze_view(self, dim: int) -> "Tensor":
        return Tensor(self.data.unsqueeze(dim))

    expand_dims = unsqueeze_view

    def unsqueeze_inplace(self, dim: int) -> "Tensor":
        self.data = self.data.unsqueeze(dim)
        return self

    def unsqueeze_multiple(self, axes: Sequence[int]) -> "Tensor":
        """Singleton dimensions at the positions ``axes`` of the RESULT (ascending insertion)."""
        t = self.data
        for a in sorted(int(x) for x in axes):
            if not 0 <= a <= t.dim():
                raise IndexError(f"axis {a} outside a result of {t.dim() + 1} dimensions")
            t = t.unsqueeze(a)
        return Tensor(t)

    def flatten_from(self, start_dim: int) -> "Tensor":
        return self.flatten_range(start_dim, None)

    def flatten_range(self, start_dim: int = 0, end_dim: Optional[int] = None) -> "Tensor":
        n = self.data.dim()
        end = n - 1 if end_dim is None else end_dim
        if not (0 <= start_dim <= end < max(n, 1)):
            raise IndexError(f"flatten range [{start_dim}, {end}] outside {n} dimensions")
        return Tensor(self.data.flatten(start_dim, end))

    def flatten_view(self) -> "Tensor":
        """Flattened without a copy; fails if the memory layout needs one."""
        return Tensor(self.data.view(-1))

    def flatten_owned(self) -> "Tensor":
        return Tensor(self.data.reshape(-1).clone())

    def flatten_inplace(self) -> "Tensor":
        self.data = self.data.reshape(-1)
        return self

    def expand_shared(self, shape: Sequence[int]) -> "Tensor":
        """Broadcast view (stride-0 dimensions, no copy)."""
        return Tensor(self.data.expand(*shape))

    expand_lazy = expand_shared

    def expand_owned(self, shape: Sequence[int]) -> "Tensor":
        return Tensor(self.data.expand(*shape).contiguous())

    def materialize(self) -> "Tensor":
        return Tensor(self.data.contiguous())

    def repeat_advanced(self, repeats: Sequence[int]) -> "Tensor":
        """``repeats`` may be longer than the rank (leading dimensions are added) but not shorter."""
        if len(repeats) < self.data.dim():
            raise ValueError(f"{len(repeats)} repeat counts for a tensor of {self.data.dim()} dimensions")
        if any(int(r) <= 0 for r in repeats):
            raise ValueError("repeat counts must be positive")
        return Tensor(self.data.repeat(*[int(r) for r in repeats]))

    def repeat_interleave_scalar(self, repeats: int, dim: Optional[int] = None) -> "Tensor":
        return Tensor(self.data.repeat_interleave(int(repeats), dim=dim))

    def roll_1d(self, shifts: int, dim: Optional[int] = None) -> "Tensor":
        """Without ``dim`` the flattened tensor is rolled and reshaped back."""
        return Tensor(self.data.roll(int(shifts)) if dim is None else self.data.roll(int(shifts), self.resolve_dim(dim)))

    # ------------------------------------------------ statistics / linear algebra variants
    def std_unbiased(self) -> float:
        return float(self.data.float().std(unbiased=True)) if self.data.numel() > 1 else 0.0

    def quantile_advanced(self, q: float) -> float:
        if not 0.0 <= q <= 1.0:
            raise ValueError("Quantile must be between 0 and 1")
        if self.data.numel() == 0:
            raise ValueError("quantile of an empty tensor")
        return float(torch.quantile(self.data.detach().double().flatten(), q))

    def count_nonzero_axis(self, axis: int) -> "Tensor":
        return Tensor(torch.count_nonzero(self.data, dim=self.resolve_dim(axis)).float())

    def qr_basic(self):
        return self.qr()

    def eig_basic(self):
        return self.eig()

    def symeig_basic(self, upper: bool = False):
        return self.symeig(upper)

    def matmul_hybrid(self, other) -> "Tensor":
        """The reference picks a device per call (src/tensor/ops/matrix.rs); here the product runs where the data is."""
        return self.matmul(other)

    # ------------------------------------------------ predicate helpers (src/tensor/ops/utils.rs:28-140)
    def _mask(self, condition) -> torch.Tensor:
        """``condition`` maps the whole tensor to a boolean mask, or one element to a bool."""
        try:
            m = condition(self.data)
            if isinstance(m, torch.Tensor) and m.dtype == torch.bool and m.shape == self.data.shape:
                return m
        except Exception:  # noqa: BLE001  (an element-wise predicate may not accept a tensor)
            pass
        flat = [bool(condition(v)) for v in self.data.detach().flatten().tolist()]
        return torch.tensor(flat, dtype=torch.bool, device=self.data.device).view(self.data.shape)

    def count_where(self, condition) -> int:
        return int(self._mask(condition).sum())

    def find_first(self, condition) -> Optional[int]:
        idx = self._mask(condition).flatten().nonzero()
        return int(idx[0]) if idx.numel() else None

    def find_all(self, condition) -> List[int]:
        return self._mask(condition).flatten().nonzero().flatten().tolist()

    def replace_where(self, condition, replacement: Number) -> "Tensor":
        return Tensor(torch.where(self._mask(condition), torch.as_tensor(replacement, dtype=self.data.dtype, device=self.data.device), self.data))

    def map_with_index(self, fn) -> "Tensor":
        """``fn(flat_index, value) -> value`` over the elements in row-major order."""
        vals = [fn(i, v) for i, v in enumerate(self.data.detach().flatten().tolist())]
        return Tensor(torch.tensor(vals, dtype=self.data.dtype, device=self.data.device).view(self.data.shape))

    def map_inplace(self, fn) -> "Tensor":
        self.data = self.map(fn).data
        return self

    def clone_tensor(self) -> "Tensor":
        return self.clone()

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        attr = getattr(self.data, name)
        if callable(attr):
            def call(*a, **k):
                return _wrap(attr(*_unwrap(a), **{kk: _unwrap(v) for kk, v in k.items()}))
            return call
        return _wrap(attr)


def _gamma_sign(x: torch.Tensor) -> torch.Tensor:
    # sign of Gamma(x) for negative non-integers: (-1)^ceil(-x)
    neg = x < 0
    s = torch.where((torch.ceil(-x) % 2) == 1, -torch.ones_like(x), torch.ones_like(x))
    return torch.where(neg, s, torch.ones_like(x))


def tensor(data, shape: Optional[Sequence[int]] = None, **kw) -> Tensor:
    """``rustorch.tensor(data, shape)`` (python/src/lib.rs) and the ``tensor!`` literal macro."""
    return Tensor(data, shape, **kw)


def zeros(shape, **kw) -> Tensor:
    return Tensor.zeros(shape, **kw)


def ones(shape, **kw) -> Tensor:
    return Tensor.ones(shape, **kw)


def select_optimal_device(numel: int, threshold: int = 1 << 14) -> str:
    """``"cuda"`` for tensors worth a kernel launch when a GPU is present, else ``"cpu"`` (src/tensor/gpu_parallel.rs:473)."""
    return "cuda" if torch.cuda.is_available() and numel >= threshold else "cpu"


def optimized_matmul(a, b) -> Tensor:
    """BLAS-backed matrix product (src/linalg/optimized_blas.rs:11-193): MKL / OpenBLAS on the host, the GEMM kernels on the GPU."""
    return Tensor(_unwrap(a) @ _unwrap(b))


def multithreaded_matmul(a, b, num_threads: Optional[int] = None) -> Tensor:
    if num_threads:
        prev = torch.get_num_threads()
        torch.set_num_threads(num_threads)
        try:
            return optimized_matmul(a, b)
        finally:
            torch.set_num_threads(prev)
    return optimized_matmul(a, b)


def memory_optimized(shape, dtype=torch.float32, device="cpu", pinned: bool = False) -> Tensor:
    """A tensor from the pooled / pinned allocators (src/tensor/memory_optimized.rs:155-402)."""
    from .compat import AllocationStrategy
    strat = AllocationStrategy.PINNED if pinned else AllocationStrategy.POOLED
    return Tensor(strat.allocate(tuple(shape), dtype, device).zero_())


def tensor_nd(nested) -> Tensor:
    """Nested-list literal, the proc-macro ``tensor_nd!`` (rustorch-macros/src/lib.rs:43-68)."""
    return Tensor(nested)


# ``rustorch.tensor`` is both this module and the constructor function of the binding: importing the submodule binds the
# module object to that name on the package, so the module itself is made callable and forwards to ``tensor()``.
import sys as _sys
import types as _types


class _CallableModule(_types.ModuleType):
    def __call__(self, data, shape=None, **kw):
        return tensor(data, shape, **kw)


_sys.modules[__name__].__class__ = _CallableModule
