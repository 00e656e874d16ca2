"""Automatic mixed precision: ``autocast`` context, ``GradScaler``, ``AMPOptimizer``, ``AMPConfig``
(src/amp/autocast.rs:15-116, grad_scaler.rs:67-372, optimizer_wrapper.rs:9-270, mod.rs:21-167).

The reference emulates reduced precision by rounding f32 values (dtype_utils.rs:9-35); here autocast runs
real bf16 / fp16 kernels (torch.autocast on the named device).  ``GradScaler`` keeps the reference defaults
``(init_scale=65536, growth_factor=2, backoff_factor=0.5, growth_interval=2000, enabled=True)`` and its
method names (``scale / unscale_grads / check_overflow / step / step_with_clipping / update_scale /
state_dict``).
"""
from __future__ import annotations

import contextlib
import enum
from dataclasses import dataclass
from typing import Iterable, List, Optional

import torch

_NATIVE_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def _native_ok() -> bool:
    from .. import _native
    return _native.available()


class AutocastMode(enum.Enum):
    """Which dtype ``autocast`` computes in (src/amp/autocast.rs)."""

    NONE = "none"
    FP16 = "fp16"
    BF16 = "bf16"


_DT = {"fp16": torch.float16, "float16": torch.float16, "half": torch.float16, "bf16": torch.bfloat16,
       "bfloat16": torch.bfloat16}


@contextlib.contextmanager
def autocast(device_type: str = "cuda", enabled: bool = True, dtype=None):
    if dtype is None:
        dtype = torch.bfloat16
    elif isinstance(dtype, (str, AutocastMode)):
        dtype = _DT[dtype.value if isinstance(dtype, AutocastMode) else dtype.lower()]
    with torch.autocast(device_type, dtype=dtype, enabled=enabled):
        yield


def is_autocast_enabled(device_type: str = "cuda") -> bool:
    return torch.is_autocast_enabled(device_type)


def cast_to_fp16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float16)


def cast_to_bf16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16)


def cast_to_fp32(t: torch.Tensor) -> torch.Tensor:
    return t.float()


class GradScaler:
    def __init__(self, init_scale: float = 65536.0, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000, enabled: bool = True):
        self._scale, self.growth_factor, self.backoff_factor = float(init_scale), growth_factor, backoff_factor
        self.growth_interval, self.enabled = growth_interval, enabled
        self._growth_tracker = 0
        self._found_inf = False
        self._unscaled = False
        self.overflow_count = 0
        self.step_count = 0

    def get_scale(self) -> float:
        return self._scale if self.enabled else 1.0

    def scale(self, loss: torch.Tensor) -> torch.Tensor:
        return loss * self._scale if self.enabled else loss

    scale_tensor = scale

    def _params(self, optimizer_or_params) -> List[torch.Tensor]:
        if hasattr(optimizer_or_params, "param_groups"):
            return [p for g in optimizer_or_params.param_groups for p in g["params"] if p.grad is not None]
        return [p for p in optimizer_or_params if p.grad is not None]

    def check_overflow(self, optimizer_or_params) -> bool:
        """True when any gradient holds inf / nan (one fused reduction per call)."""
        gs = [p.grad for p in self._params(optimizer_or_params)]
        if not gs:
            return False
        norms = torch._foreach_norm(gs)
        return not bool(torch.isfinite(torch.stack([n.float() for n in norms])).all())

    def unscale_grads(self, optimizer_or_params) -> bool:
        """Divide gradients by the scale in place; returns whether an overflow was found."""
        if not self.enabled:
            return False
        flat = getattr(optimizer_or_params, "flat", None)
        if flat is not None and getattr(flat, "grad", None) is not None and flat.grad.is_cuda and not self._unscaled:
            flat.collect_autograd_grads()
            self._found_inf = self._native_unscale([flat.grad])      # one pass over the flat fp32 gradient buffer
            self._unscaled = True
            return self._found_inf
        ps = self._params(optimizer_or_params)
        gs = [p.grad for p in ps]
        if gs and not self._unscaled and all(g.is_cuda and g.is_contiguous() and g.dtype in _NATIVE_DTYPES for g in gs) and _native_ok():
            self._found_inf = self._native_unscale(gs)
            self._unscaled = True
            return self._found_inf
        self._found_inf = self.check_overflow(ps)
        if not self._found_inf and not self._unscaled and ps:
            torch._foreach_mul_(gs, 1.0 / self._scale)
        self._unscaled = True
        return self._found_inf

    def _native_unscale(self, grads) -> bool:
        """``g *= 1 / scale`` and the inf / nan check in the same pass (csrc/nn/rnn_amp_sparse.cu); one host read."""
        from .. import _native
        C = _native.load(required=True)
        flag = torch.zeros(1, dtype=torch.float32, device=grads[0].device)
        for g in grads:
            C.amp_unscale(g, 1.0 / self._scale, flag)
        return bool(flag.item() != 0.0)

    unscale_ = unscale_grads

    def step(self, optimizer, *args, **kw) -> bool:
        """Unscale (if not done), skip the step on overflow.  Returns True when the step was taken."""
        if not self.enabled:
            optimizer.step(*args, **kw)
            return True
        if not self._unscaled:
            self.unscale_grads(optimizer)
        self.step_count += 1
        if self._found_inf:
            self.overflow_count += 1
            return False
        optimizer.step(*args, **kw)
        return True

    def step_with_clipping(self, optimizer, max_norm: float) -> bool:
        if self.enabled and not self._unscaled:
            self.unscale_grads(optimizer)
        if not self._found_inf:
            torch.nn.utils.clip_grad_norm_(self._params(optimizer), max_norm)
        return self.step(optimizer)

    def update_scale(self) -> None:
        if not self.enabled:
            return
        if self._found_inf:
            self._scale = max(self._scale * self.backoff_factor, 1.0)
            self._growth_tracker = 0
        else:
            self._growth_tracker += 1
            if self._growth_tracker >= self.growth_interval:
                self._scale *= self.growth_factor
                self._growth_tracker = 0
        self._found_inf, self._unscaled = False, False

    update = update_scale

    def state_dict(self) -> dict:
        return {"scale": self._scale, "growth_factor": self.growth_factor, "backoff_factor": self.backoff_factor,
                "growth_interval": self.growth_interval, "growth_tracker": self._growth_tracker,
                "overflow_count": self.overflow_count, "step_count": self.step_count}

    def load_state_dict(self, sd: dict) -> None:
        self._scale, self.growth_factor, self.backoff_factor = sd["scale"], sd["growth_factor"], sd["backoff_factor"]
        self.growth_interval, self._growth_tracker = sd["growth_interval"], sd["growth_tracker"]
        self.overflow_count, self.step_count = sd.get("overflow_count", 0), sd.get("step_count", 0)


@dataclass
class AMPConfig:
    enabled: bool = True
    dtype: str = "bf16"
    use_grad_scaler: bool = False
    init_scale: float = 65536.0
    growth_interval: int = 2000
    max_grad_norm: Optional[float] = None

    @staticmethod
    def bf16() -> "AMPConfig":
        return AMPConfig(True, "bf16", False)

    @staticmethod
    def fp16() -> "AMPConfig":
        return AMPConfig(True, "fp16", True)

    @staticmethod
    def fp16_static(scale: float = 1024.0) -> "AMPConfig":
        return AMPConfig(True, "fp16", True, scale, 10 ** 9)

    @staticmethod
    def disabled() -> "AMPConfig":
        return AMPConfig(False)


class AMPOptimizer:
    """Optimizer wrapper: ``backward(loss)`` scales, ``step()`` unscales / clips / skips on overflow / updates
    the scale; exposes ``success_rate`` like the reference's wrapper."""

    def __init__(self, optimizer, config: Optional[AMPConfig] = None):
        self.optimizer, self.config = optimizer, config or AMPConfig.bf16()
        self.scaler = GradScaler(self.config.init_scale, growth_interval=self.config.growth_interval,
                                 enabled=self.config.enabled and self.config.use_grad_scaler)
        self.steps = self.skipped = 0

    def autocast(self, device_type: str = "cuda"):
        return autocast(device_type, self.config.enabled, self.config.dtype)

    def backward(self, loss: torch.Tensor) -> None:
        self.scaler.scale(loss).backward()

    def step(self) -> bool:
        self.steps += 1
        if self.config.max_grad_norm is not None:
            ok = self.scaler.step_with_clipping(self.optimizer, self.config.max_grad_norm)
        else:
            ok = self.scaler.step(self.optimizer)
        self.scaler.update_scale()
        if not ok:
            self.skipped += 1
        return ok

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.optimizer.zero_grad(set_to_none=set_to_none)

    def success_rate(self) -> float:
        return 1.0 - self.skipped / self.steps if self.steps else 1.0

    def state_dict(self) -> dict:
        return {"optimizer": self.optimizer.state_dict(), "scaler": self.scaler.state_dict()}

    def load_state_dict(self, sd: dict) -> None:
        self.optimizer.load_state_dict(sd["optimizer"])
        self.scaler.load_state_dict(sd["scaler"])
