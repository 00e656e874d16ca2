"""Smaller named pieces of the reference's surface that have no module of their own here.

``AdamConfig / AdamState / AdamUtils`` (src/optim/common.rs:13-383), ``LBFGSMemory / LineSearchMethod``
(src/optim/lbfgs.rs:19-270), ``AllocationStrategy / ZeroCopyOps / TensorIterOps`` (src/tensor/memory/aligned.rs,
operations/zero_copy.rs:10-52), ``ShapeBuilder / LazyExpandedTensor`` (src/tensor/ops/advanced_shape.rs:15-513),
``SafeTensor / SafeNumeric / TypedTensor`` (src/tensor/numeric_safety.rs:10-347, type_safe.rs:11-327), ``WindowType``
(src/tensor/ops/signal.rs), ``Int4`` (src/quantization), ``ProfilerCore`` (src/profiler/core.rs), ``RecurrentOps``
(src/nn/recurrent_common.rs), ``LinearBackward`` (src/autograd), ``DistributedState`` (src/distributed/mod.rs),
``GPTModel`` (example-cli/src/model/architectures/gpt.rs), ``OnnxModel`` (src/formats/onnx.rs:50-231).
"""
from __future__ import annotations

import math
import time
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Deque, Dict, Iterator, List, Optional, Sequence, Tuple

import torch


# ------------------------------------------------------------------------------------------------ optimizers
@dataclass
class AdamConfig:
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0
    amsgrad: bool = False


@dataclass
class AdamState:
    """Per-parameter state shared by the Adam family."""
    step: int = 0
    exp_avg: Optional[torch.Tensor] = None
    exp_avg_sq: Optional[torch.Tensor] = None
    max_exp_avg_sq: Optional[torch.Tensor] = None

    def ensure(self, like: torch.Tensor, amsgrad: bool = False) -> "AdamState":
        if self.exp_avg is None:
            self.exp_avg, self.exp_avg_sq = torch.zeros_like(like), torch.zeros_like(like)
            if amsgrad:
                self.max_exp_avg_sq = torch.zeros_like(like)
        return self


class AdamUtils:
    @staticmethod
    def bias_correction(beta: float, step: int) -> float:
        return 1.0 - beta ** step

    @staticmethod
    def update_moments(state: AdamState, grad: torch.Tensor, cfg: AdamConfig) -> None:
        state.step += 1
        state.exp_avg.mul_(cfg.beta1).add_(grad, alpha=1 - cfg.beta1)
        state.exp_avg_sq.mul_(cfg.beta2).addcmul_(grad, grad, value=1 - cfg.beta2)

    @staticmethod
    def apply_weight_decay(param: torch.Tensor, grad: torch.Tensor, cfg: AdamConfig, decoupled: bool = False) -> torch.Tensor:
        if cfg.weight_decay == 0.0:
            return grad
        if decoupled:
            param.mul_(1 - cfg.lr * cfg.weight_decay)
            return grad
        return grad.add(param, alpha=cfg.weight_decay)

    @staticmethod
    def step(param: torch.Tensor, grad: torch.Tensor, state: AdamState, cfg: AdamConfig, decoupled: bool = False) -> None:
        """One Adam / AdamW update of one tensor, in place."""
        state.ensure(param, cfg.amsgrad)
        grad = AdamUtils.apply_weight_decay(param, grad, cfg, decoupled)
        AdamUtils.update_moments(state, grad, cfg)
        bc1, bc2 = AdamUtils.bias_correction(cfg.beta1, state.step), AdamUtils.bias_correction(cfg.beta2, state.step)
        v = state.exp_avg_sq
        if cfg.amsgrad:
            torch.maximum(state.max_exp_avg_sq, v, out=state.max_exp_avg_sq)
            v = state.max_exp_avg_sq
        param.addcdiv_(state.exp_avg, (v / bc2).sqrt_().add_(cfg.eps), value=-cfg.lr / bc1)


class LineSearchMethod(Enum):
    NONE = "none"
    BACKTRACKING = "backtracking"
    STRONG_WOLFE = "strong_wolfe"

    def torch_name(self) -> Optional[str]:
        return "strong_wolfe" if self is LineSearchMethod.STRONG_WOLFE else None


class LBFGSMemory:
    """The (s, y, rho) history and the two-loop recursion."""

    def __init__(self, history_size: int = 100):
        self.s: Deque[torch.Tensor] = deque(maxlen=history_size)
        self.y: Deque[torch.Tensor] = deque(maxlen=history_size)
        self.rho: Deque[float] = deque(maxlen=history_size)

    def update(self, s: torch.Tensor, y: torch.Tensor) -> bool:
        ys = float(torch.dot(y.reshape(-1), s.reshape(-1)))
        if ys <= 1e-10:
            return False
        self.s.append(s.clone()); self.y.append(y.clone()); self.rho.append(1.0 / ys)
        return True

    def direction(self, grad: torch.Tensor) -> torch.Tensor:
        """``-H grad`` by the two-loop recursion (initial scaling ``s.y / y.y`` of the newest pair)."""
        q = grad.reshape(-1).clone()
        alphas = []
        for s, y, rho in zip(reversed(self.s), reversed(self.y), reversed(self.rho)):
            a = rho * float(torch.dot(s.reshape(-1), q))
            alphas.append(a)
            q.add_(y.reshape(-1), alpha=-a)
        if self.s:
            s, y = self.s[-1].reshape(-1), self.y[-1].reshape(-1)
            q.mul_(float(torch.dot(s, y) / torch.dot(y, y)))
        for (s, y, rho), a in zip(zip(self.s, self.y, self.rho), reversed(alphas)):
            b = rho * float(torch.dot(y.reshape(-1), q))
            q.add_(s.reshape(-1), alpha=a - b)
        return -q.view_as(grad)

    def __len__(self) -> int:
        return len(self.s)


# ------------------------------------------------------------------------------------------------ memory
class AllocationStrategy(Enum):
    DIRECT = "direct"          # allocate on demand
    POOLED = "pooled"          # size-bucketed pool
    ALIGNED = "aligned"        # 32-byte (host SIMD) / 256-byte (device) aligned
    PINNED = "pinned"          # page-locked host memory for async H2D / D2H
    ARENA = "arena"            # one native arena, best-fit with coalescing

    def allocate(self, shape: Sequence[int], dtype: torch.dtype = torch.float32, device="cpu") -> torch.Tensor:
        if self is AllocationStrategy.PINNED:
            return torch.empty(*shape, dtype=dtype, pin_memory=torch.cuda.is_available())
        if self is AllocationStrategy.POOLED:
            from .memory import MemoryPool, PoolExhausted
            key = str(device)
            if key not in _POOLS:
                _POOLS[key] = MemoryPool(64 << 20, device)          # 64 MiB arena per device, best-fit with coalescing
            try:
                return _POOLS[key].allocate(tuple(shape), dtype)
            except PoolExhausted:
                return torch.empty(*shape, dtype=dtype, device=device)
        return torch.empty(*shape, dtype=dtype, device=device)


_POOLS: Dict[str, Any] = {}


class ZeroCopyOps:
    """Views instead of copies: every method returns a tensor that shares storage with its input."""

    @staticmethod
    def view(t: torch.Tensor, shape: Sequence[int]) -> torch.Tensor:
        return t.view(*shape)

    @staticmethod
    def slice_view(t: torch.Tensor, dim: int, start: int, end: int) -> torch.Tensor:
        return t.narrow(dim, start, end - start)

    @staticmethod
    def transpose_view(t: torch.Tensor, d0: int = -2, d1: int = -1) -> torch.Tensor:
        return t.transpose(d0, d1)

    @staticmethod
    def from_numpy(a) -> torch.Tensor:
        return torch.from_numpy(a)

    @staticmethod
    def shares_storage(a: torch.Tensor, b: torch.Tensor) -> bool:
        return a.untyped_storage().data_ptr() == b.untyped_storage().data_ptr()

    @staticmethod
    def elementwise_inplace(t: torch.Tensor, fn: Callable[[torch.Tensor], torch.Tensor]) -> torch.Tensor:
        t.copy_(fn(t))
        return t


class TensorIterOps:
    """Iteration helpers over a tensor without materialising Python lists of scalars."""

    @staticmethod
    def iter_rows(t: torch.Tensor) -> Iterator[torch.Tensor]:
        return iter(t.unbind(0))

    @staticmethod
    def iter_chunks(t: torch.Tensor, chunk: int, dim: int = 0) -> Iterator[torch.Tensor]:
        return iter(t.split(chunk, dim))

    @staticmethod
    def map_chunks(t: torch.Tensor, fn: Callable[[torch.Tensor], torch.Tensor], chunk: int, dim: int = 0) -> torch.Tensor:
        return torch.cat([fn(c) for c in t.split(chunk, dim)], dim)

    @staticmethod
    def fold(t: torch.Tensor, init: float, fn: Callable[[float, torch.Tensor], float], chunk: int = 1 << 20) -> float:
        acc = init
        for c in t.reshape(-1).split(chunk):
            acc = fn(acc, c)
        return acc


# ------------------------------------------------------------------------------------------------ shapes
class ShapeBuilder:
    """Fluent chain of shape operations: ``ShapeBuilder(t).unsqueeze(0).expand(4, -1).flatten().build()``."""

    def __init__(self, tensor: torch.Tensor):
        self._t = tensor

    def shape(self) -> Tuple[int, ...]:
        return tuple(self._t.shape)

    def build(self) -> torch.Tensor:
        return self._t


def _shape_method(name):
    def f(self, *a, **k):
        self._t = getattr(self._t, name)(*a, **k)
        return self
    f.__name__ = name
    return f


for _n in ("squeeze", "unsqueeze", "expand", "flatten", "unflatten", "permute", "transpose", "reshape", "view", "repeat", "flip",
           "roll", "movedim", "swapaxes", "tile", "contiguous"):
    setattr(ShapeBuilder, _n, _shape_method(_n))
del _n


class LazyExpandedTensor:
    """A broadcast that is only described (stride-0 view); ``materialize()`` makes the copy when one is needed."""

    def __init__(self, base: torch.Tensor, shape: Sequence[int]):
        self.base, self.target_shape = base, tuple(shape)
        self._view = base.expand(*shape)

    @property
    def shape(self) -> Tuple[int, ...]:
        return self.target_shape

    def view(self) -> torch.Tensor:
        return self._view

    def materialize(self) -> torch.Tensor:
        return self._view.contiguous()

    def is_materialized(self) -> bool:
        return False

    def memory_saved(self) -> int:
        return (math.prod(self.target_shape) - self.base.numel()) * self.base.element_size()

    def __getitem__(self, idx):
        return self._view[idx]


class SafeNumeric:
    """Overflow- and NaN-checked scalar / tensor arithmetic."""

    @staticmethod
    def check_finite(t: torch.Tensor, what: str = "tensor") -> torch.Tensor:
        if not bool(torch.isfinite(t).all()):
            from .error import NumericalError
            raise NumericalError(f"{what} holds inf or nan")
        return t

    @staticmethod
    def fits(value: float, dtype: torch.dtype) -> bool:
        info = torch.finfo(dtype) if dtype.is_floating_point else torch.iinfo(dtype)
        return info.min <= value <= info.max

    @staticmethod
    def safe_cast(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        info = torch.finfo(dtype) if dtype.is_floating_point else torch.iinfo(dtype)
        if t.numel() and (float(t.max()) > info.max or float(t.min()) < info.min):
            from .error import OverflowError_
            raise OverflowError_(f"values do not fit {dtype}")
        return t.to(dtype)

    @staticmethod
    def safe_div(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        if bool((b == 0).any()):
            from .error import DivisionByZero
            raise DivisionByZero("division by zero")
        return a / b


class SafeTensor:
    """Tensor wrapper whose arithmetic checks its results (``SafeTensor(a) + b`` raises on overflow / nan)."""

    def __init__(self, data: torch.Tensor):
        self.data = SafeNumeric.check_finite(data)

    def _bin(self, other, fn) -> "SafeTensor":
        o = other.data if isinstance(other, SafeTensor) else other
        return SafeTensor(SafeNumeric.check_finite(fn(self.data, o), "result"))

    def __add__(self, o): return self._bin(o, torch.add)
    def __sub__(self, o): return self._bin(o, torch.sub)
    def __mul__(self, o): return self._bin(o, torch.mul)
    def __matmul__(self, o): return self._bin(o, torch.matmul)

    def __truediv__(self, o):
        od = o.data if isinstance(o, SafeTensor) else torch.as_tensor(o)
        return SafeTensor(SafeNumeric.safe_div(self.data, od))

    def cast(self, dtype: torch.dtype) -> "SafeTensor":
        return SafeTensor(SafeNumeric.safe_cast(self.data, dtype))


class TypedTensor:
    """Rank-checked tensor: ``TypedTensor(t, rank=2)`` (the reference encodes the rank in the type, ``Dim1..Dim4``)."""

    def __init__(self, data: torch.Tensor, rank: int):
        if data.dim() != rank:
            from .error import InvalidDimension
            raise InvalidDimension(f"expected a rank-{rank} tensor, got rank {data.dim()}")
        self.data, self.rank = data, rank

    def matmul(self, other: "TypedTensor") -> "TypedTensor":
        if self.rank != 2 or other.rank != 2:
            raise TypeError("matmul is defined for rank-2 typed tensors")
        return TypedTensor(self.data @ other.data, 2)


class WindowType(Enum):
    RECTANGULAR = "rectangular"
    HANN = "hann"
    HAMMING = "hamming"
    BLACKMAN = "blackman"
    BARTLETT = "bartlett"

    def coefficients(self, n: int, device=None, dtype=torch.float32) -> torch.Tensor:
        if self is WindowType.RECTANGULAR:
            return torch.ones(n, device=device, dtype=dtype)
        fn = {"hann": torch.hann_window, "hamming": torch.hamming_window, "blackman": torch.blackman_window,
              "bartlett": torch.bartlett_window}[self.value]
        return fn(n, periodic=False, device=device, dtype=dtype)

    def apply(self, signal: torch.Tensor) -> torch.Tensor:
        return signal * self.coefficients(signal.shape[-1], signal.device, signal.dtype if signal.is_floating_point() else torch.float32)


class Int4:
    """Marker + packing helpers of the 4-bit quantised element type: two signed nibbles per byte, low nibble first."""
    bits, qmin, qmax = 4, -8, 7

    @staticmethod
    def pack(values: torch.Tensor) -> torch.Tensor:
        v = values.to(torch.int16).clamp(Int4.qmin, Int4.qmax).reshape(-1)
        if v.numel() % 2:
            v = torch.cat([v, v.new_zeros(1)])
        lo, hi = v[0::2] & 0xF, v[1::2] & 0xF
        return (lo | (hi << 4)).to(torch.uint8)

    @staticmethod
    def unpack(packed: torch.Tensor, numel: Optional[int] = None) -> torch.Tensor:
        p = packed.to(torch.int16)
        lo, hi = p & 0xF, (p >> 4) & 0xF
        out = torch.stack([lo, hi], -1).reshape(-1)
        out = torch.where(out >= 8, out - 16, out).to(torch.int8)
        return out if numel is None else out[:numel]


# ------------------------------------------------------------------------------------------------ profiler core
class ProfilerCore:
    """Sessions and named timers underneath the global profiler."""

    def __init__(self):
        self.sessions: Dict[str, Dict[str, Any]] = {}
        self._open: Dict[str, float] = {}
        self.timers: Dict[str, List[float]] = {}
        self.current: Optional[str] = None

    def start_session(self, name: str) -> None:
        self.sessions[name] = {"start": time.perf_counter(), "end": None, "timers": {}}
        self.current = name

    def end_session(self) -> Optional[Dict[str, Any]]:
        if self.current is None:
            return None
        s = self.sessions[self.current]
        s["end"] = time.perf_counter()
        s["timers"] = {k: list(v) for k, v in self.timers.items()}
        self.current = None
        return s

    def start_timer(self, name: str, sync_cuda: bool = False) -> None:
        if sync_cuda and torch.cuda.is_available():
            torch.cuda.synchronize()
        self._open[name] = time.perf_counter()

    def stop_timer(self, name: str, sync_cuda: bool = False) -> float:
        if sync_cuda and torch.cuda.is_available():
            torch.cuda.synchronize()
        dt = time.perf_counter() - self._open.pop(name)
        self.timers.setdefault(name, []).append(dt)
        return dt

    def summary(self) -> Dict[str, Dict[str, float]]:
        return {k: {"count": len(v), "total_s": sum(v), "mean_s": sum(v) / len(v), "max_s": max(v)} for k, v in self.timers.items() if v}


# ------------------------------------------------------------------------------------------------ nn / autograd
from .nn.recurrent_common import RecurrentOps  # noqa: E402,F401  (kept importable from here)


class LinearBackward(torch.autograd.Function):
    """``y = x W^T + b`` with the gradient formulas of the reference's grad fn (dX = dY W, dW = dY^T X, db = sum dY);
    on CUDA bf16 the three products run on the tcgen05 GEMM (forward, input-gradient and weight-gradient layouts)."""

    @staticmethod
    def forward(ctx, x, weight, bias=None):
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        return torch.nn.functional.linear(x, weight, bias)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2, x2 = dy.reshape(-1, dy.shape[-1]), x.reshape(-1, x.shape[-1])
        dx = (dy2 @ w).view_as(x)
        dw = dy2.t() @ x2
        db = dy2.sum(0) if ctx.has_bias else None
        return dx, dw, db


class DistributedState:
    """Process-wide view of the default process group (the reference's global singleton)."""

    @staticmethod
    def get():
        from .distributed import api
        pg = api.get_process_group()
        return {"initialized": api.is_initialized(), "rank": api.get_rank(), "world_size": api.get_world_size(),
                "backend": getattr(pg, "backend", None)}

    @staticmethod
    def is_initialized() -> bool:
        from .distributed import api
        return api.is_initialized()


class GPTModel:
    """The CLI's GPT architecture: embedding + sinusoidal positions + pre-LN blocks + final LN + projection, with the
    reference's deterministic ``sin``-based weight initialisation, so that both produce the same toy model."""

    def __init__(self, vocab_size: int, d_model: int = 128, n_layer: int = 2, n_head: int = 4, max_len: int = 512, device="cpu"):
        import torch.nn as nn
        self.cfg = dict(vocab_size=vocab_size, d_model=d_model, n_layer=n_layer, n_head=n_head, max_len=max_len)
        self.tok = nn.Embedding(vocab_size, d_model)
        layer = nn.TransformerEncoderLayer(d_model, n_head, 4 * d_model, dropout=0.0, activation="gelu", batch_first=True, norm_first=True)
        self.blocks = nn.TransformerEncoder(layer, n_layer, enable_nested_tensor=False)
        self.ln, self.head = nn.LayerNorm(d_model), nn.Linear(d_model, vocab_size, bias=False)
        self.modules = nn.ModuleList([self.tok, self.blocks, self.ln, self.head]).to(device)
        with torch.no_grad():                       # deterministic init: w[i] = sin(i) * 0.02
            for p in self.modules.parameters():
                if p.dim() > 1:
                    p.copy_((torch.arange(p.numel(), dtype=torch.float32).sin() * 0.02).view_as(p))
        pos = torch.arange(max_len)[:, None] * torch.exp(torch.arange(0, d_model, 2) * (-math.log(10000.0) / d_model))[None]
        self.pe = torch.zeros(max_len, d_model, device=device)
        self.pe[:, 0::2], self.pe[:, 1::2] = pos.sin().to(device), pos.cos().to(device)

    @torch.no_grad()
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        T = ids.shape[1]
        x = self.tok(ids) + self.pe[:T]
        mask = torch.nn.Transformer.generate_square_subsequent_mask(T, device=ids.device)
        return self.head(self.ln(self.blocks(x, mask=mask, is_causal=True)))

    __call__ = forward


class OnnxModel:
    """Load-and-run wrapper over the importer's executor: ``OnnxModel.load(path).run({"input": x})``."""

    def __init__(self, imported):
        from .model_import import OnnxModule
        self.imported = imported
        self.module = OnnxModule(imported)

    @classmethod
    def load(cls, path: str) -> "OnnxModel":
        from .model_import import import_model
        return cls(import_model(path))

    def input_names(self) -> List[str]:
        return [s.name for s in self.imported.architecture.inputs] if hasattr(self.imported, "architecture") else []

    def run(self, inputs) -> Any:
        if isinstance(inputs, dict):
            inputs = list(inputs.values())
        if isinstance(inputs, torch.Tensor):
            inputs = [inputs]
        return self.module(*inputs)
