"""Optimizers with the reference's constructors, defaults and accessor names (src/optim/*).

All are ``torch.optim.Optimizer`` subclasses (so schedulers, ``state_dict`` with moment buffers and
parameter groups work) plus the reference surface: ``learning_rate() / set_learning_rate(lr) /
set_lr(lr)``, the alternate constructors (``Adam.default_params(lr)``, ``SGD.with_momentum`` ...)
and a per-tensor ``step_tensor(param, grad)`` mirroring the trait's ``step(&param, &grad)``
(src/optim/mod.rs:60-78).  Bias correction counts optimizer steps per parameter, not calls
across parameters (the reference's quirk, src/optim/mod.rs:301).  The fused flat-buffer
variants used by the bf16 training path live in :mod:`rustorch_b200.optim.flat`.
"""
from __future__ import annotations

import math
from typing import Iterable, Optional

import torch
from torch.optim import Optimizer as _TorchOptimizer

from .._interop import FlagValue, FloatValue, IntValue


class _RefAPI:
    """Reference accessor names on top of torch's param_groups, and the native multi-tensor ``step``."""

    _MT_KIND: Optional[int] = None          # update rule of csrc/optim/multi_tensor_optim.cu, None: no native step

    def step(self, closure=None, grad=None):           # noqa: D401
        """One optimizer step.  CUDA parameters are updated by the multi-tensor kernel (one launch per 32 tensors,
        see :mod:`rustorch_b200.optim.multi_tensor`); anything it does not cover takes the per-tensor path.
        ``step(param, grad)`` with two tensors is the reference's per-tensor call (``Optimizer::step(&param, &grad)``,
        src/optim/mod.rs:45-60) and goes to :meth:`step_tensor`."""
        if grad is not None:
            from ..tensor import _unwrap
            raw = lambda t: t.tensor if hasattr(t, "tensor") and isinstance(t.tensor, torch.Tensor) else _unwrap(t)   # noqa: E731
            self.step_tensor(raw(closure), raw(grad))
            return None
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self._MT_KIND is not None:
            from . import multi_tensor
            with torch.no_grad():
                if multi_tensor.try_step(self, self._MT_KIND):
                    return loss
        self._fallback_step()
        return loss

    def _fallback_step(self) -> None:
        for base in type(self).__mro__:
            if base.__module__.startswith("torch.optim") and "step" in base.__dict__:
                base.step(self)
                return
        raise NotImplementedError

    # attributes in the Python wheel (python/src/lib.rs:502-505, 731-770), calls in Rust: the values answer both
    @property
    def learning_rate(self) -> float:
        return FloatValue(self.param_groups[0]["lr"])

    def _hyper(self, key: str):
        try:
            return self.param_groups[0][key]
        except KeyError:
            raise AttributeError(f"{type(self).__name__} has no hyper-parameter {key!r}") from None

    @property
    def beta1(self) -> float:
        return FloatValue(self._hyper("betas")[0])

    @property
    def beta2(self) -> float:
        return FloatValue(self._hyper("betas")[1])

    @property
    def eps(self) -> float:
        return FloatValue(self._hyper("eps"))

    @property
    def weight_decay(self) -> float:
        return FloatValue(self._hyper("weight_decay"))

    @property
    def momentum(self) -> float:
        return FloatValue(self._hyper("momentum"))

    @property
    def nesterov(self) -> bool:
        return FlagValue(bool(self._hyper("nesterov")))

    @property
    def amsgrad(self) -> bool:
        return FlagValue(bool(self._hyper("amsgrad")))

    def param_count(self) -> int:
        """Number of parameter tensors the optimizer steps (src/python/optim.rs param_count)."""
        return sum(len(g["params"]) for g in self.param_groups)

    @property
    def step_count(self) -> int:
        """Steps taken so far (the largest per-parameter step in the optimizer state)."""
        n = 0
        for st in self.state.values():
            v = st.get("step", 0) if isinstance(st, dict) else 0
            n = max(n, int(v.item()) if isinstance(v, torch.Tensor) else int(v))
        return IntValue(n)

    def set_learning_rate(self, lr: float) -> None:
        for g in self.param_groups:
            g["lr"] = float(lr)

    set_lr = set_learning_rate

    _NATIVE_KIND: Optional[int] = None      # Adam 0, AdamW 1, Adamax 2, NAdam 3, RAdam 4 (csrc/runtime/cpu_optim.cpp)

    def _native_step(self, param: torch.Tensor, grad: torch.Tensor) -> bool:
        """Host fast path of ``step_tensor``: fp32 CPU tensors are updated by the native runtime from their addresses.
        On a 1000-element parameter the interpreter, not the arithmetic, bounds the step rate; this path keeps its own
        per-tensor state (moments, step count) and uses the same formulas as the torch path."""
        k = self._NATIVE_KIND
        if (k is None or param.device.type != "cpu" or param.dtype != torch.float32 or grad.dtype != torch.float32
                or not param.is_contiguous() or not grad.is_contiguous() or grad.device.type != "cpu"):
            return False
        g = self.param_groups[0]
        flags = ("amsgrad", "maximize", "capturable", "differentiable") + (() if k == 1 else ("decoupled_weight_decay",))
        if any(g.get(f) for f in flags):
            return False
        fs = self.__dict__.setdefault("_fast_state", {})
        st = fs.get(id(param))
        if st is None:
            if any(param is q for q in self.state):     # already stepped through torch's own state: stay on that path
                return False
            from .. import _native
            st = {"m": torch.zeros_like(param), "v": torch.zeros_like(param), "step": 0, "mu": 1.0, "host": _native.host(), "ref": param}
            st["ptrs"] = (param.data_ptr(), st["m"].data_ptr(), st["v"].data_ptr())
            fs[id(param)] = st
        st["step"] += 1
        b1, b2 = g["betas"]
        pp, pm, pv = st["ptrs"]
        st["mu"] = st["host"].cpu_adam_family_step(k, pp, grad.data_ptr(), pm, pv, param.numel(), g["lr"], b1, b2, g["eps"],
                                                   g["weight_decay"], st["step"], g.get("momentum_decay", 0.0), st["mu"])
        return True

    @torch.no_grad()
    def step_tensor(self, param: torch.Tensor, grad: torch.Tensor) -> None:
        """Update one tensor in place from an explicit gradient (the reference's ``step(&param, &grad)``)."""
        if self._native_step(param, grad):
            return
        known = any(param is p for g in self.param_groups for p in g["params"])
        if not known:
            self.add_param_group({"params": [param]})
        saved = [(p, p.grad) for g in self.param_groups for p in g["params"]]
        for p, _ in saved:
            p.grad = None
        param.grad = grad
        self.step()
        for p, g in saved:
            p.grad = g

    def _publish_fast_state(self) -> None:
        """Copy the host fast path's per-tensor state into ``self.state`` under torch's key names."""
        for st in self.__dict__.get("_fast_state", {}).values():
            if "m" not in st:
                continue
            p = st["ref"]
            if not any(p is q for g in self.param_groups for q in g["params"]):
                self.add_param_group({"params": [p]})
            second = "exp_inf" if self._NATIVE_KIND == 2 else "exp_avg_sq"
            self.state[p] = {"step": torch.tensor(float(st["step"])), "exp_avg": st["m"], second: st["v"]}
            if self._NATIVE_KIND == 3:
                self.state[p]["mu_product"] = torch.tensor(st["mu"])

    def hyper_state(self) -> dict:
        """Hyper-parameters only, like the reference's ``state_dict() -> HashMap<String, f32>``."""
        g = self.param_groups[0]
        return {k: v for k, v in g.items() if isinstance(v, (int, float, bool))}


def _raw_param(p):
    """The leaf ``torch.Tensor`` behind a ``Variable`` / ``Tensor`` wrapper: the binding's optimizers take lists of
    Variables (python/src/lib.rs:454-470), and stepping must update the wrapped tensor in place."""
    if isinstance(p, torch.Tensor):
        return p
    inner = getattr(p, "tensor", None)                   # Variable
    if not isinstance(inner, torch.Tensor):
        inner = getattr(p, "data", None)                 # Tensor
    if not isinstance(inner, torch.Tensor):
        raise TypeError(f"optimizer can only optimize tensors, got {type(p).__name__}")
    return inner


def _params(params) -> Iterable:
    if params is None:
        return [torch.nn.Parameter(torch.zeros(0))]
    out = []
    for p in params:
        if isinstance(p, dict):
            out.append({**p, "params": [_raw_param(q) for q in (p["params"] if isinstance(p["params"], (list, tuple)) else [p["params"]])]})
        else:
            out.append(_raw_param(p))
    return out


class SGD(_RefAPI, torch.optim.SGD):
    """``SGD(params, lr, momentum=0, weight_decay=0, nesterov=False, dampening=0)`` (src/optim/mod.rs:93-137)."""

    def __init__(self, params=None, lr: float = 0.01, momentum: float = 0.0, weight_decay: float = 0.0,
                 nesterov: bool = False, dampening: float = 0.0):
        super().__init__(_params(params), lr=lr, momentum=momentum, dampening=dampening,
                         weight_decay=weight_decay, nesterov=nesterov)

    with_momentum = classmethod(lambda cls, params, lr, momentum: cls(params, lr, momentum))
    with_weight_decay = classmethod(lambda cls, params, lr, momentum, wd: cls(params, lr, momentum, wd))
    with_nesterov = classmethod(lambda cls, params, lr, momentum, nesterov=True: cls(params, lr, momentum, 0.0, nesterov))

    def set_dampening(self, d: float) -> None:
        for g in self.param_groups:
            g["dampening"] = d


class Adam(_RefAPI, torch.optim.Adam):
    """``Adam(params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0, amsgrad=False)``; L2 decay
    folded into the gradient (src/optim/mod.rs:233-296)."""

    def __init__(self, params=None, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, amsgrad: bool = False):
        super().__init__(_params(params), lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay,
                         amsgrad=amsgrad)

    default_params = classmethod(lambda cls, params, lr=1e-3: cls(params, lr))
    with_weight_decay = classmethod(lambda cls, params, lr, wd: cls(params, lr, weight_decay=wd))
    with_amsgrad = classmethod(lambda cls, params, lr: cls(params, lr, amsgrad=True))


class AdamW(_RefAPI, torch.optim.AdamW):
    """``AdamW(params, lr, beta1, beta2, eps, weight_decay, amsgrad)``, defaults (0.9, 0.999, 1e-8, 0.01, False),
    decoupled decay ``p *= 1 - lr*wd`` (src/optim/adamw.rs:39-78,159-163)."""

    def __init__(self, params=None, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, amsgrad: bool = False):
        super().__init__(_params(params), lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay,
                         amsgrad=amsgrad)

    default_params = classmethod(lambda cls, params, lr=1e-3: cls(params, lr))


class RMSprop(_RefAPI, torch.optim.RMSprop):
    """``default_params(lr)``: alpha 0.99, eps 1e-8; momentum / centered variants (src/optim/mod.rs:408-755)."""

    def __init__(self, params=None, lr: float = 0.01, alpha: float = 0.99, eps: float = 1e-8,
                 weight_decay: float = 0.0, momentum: float = 0.0, centered: bool = False):
        super().__init__(_params(params), lr=lr, alpha=alpha, eps=eps, weight_decay=weight_decay,
                         momentum=momentum, centered=centered)

    default_params = classmethod(lambda cls, params, lr=0.01: cls(params, lr))


class AdaGrad(_RefAPI, torch.optim.Adagrad):
    """eps 1e-10, optional initial accumulator value (src/optim/mod.rs:646-648)."""

    def __init__(self, params=None, lr: float = 0.01, lr_decay: float = 0.0, weight_decay: float = 0.0,
                 initial_accumulator_value: float = 0.0, eps: float = 1e-10):
        super().__init__(_params(params), lr=lr, lr_decay=lr_decay, weight_decay=weight_decay,
                         initial_accumulator_value=initial_accumulator_value, eps=eps)

    default_params = classmethod(lambda cls, params, lr=0.01: cls(params, lr))


Adagrad = AdaGrad


class NAdam(_RefAPI, torch.optim.NAdam):
    """``(lr, beta1, beta2, eps, wd, momentum_decay=0.004, schedule_decay=0.004)`` (src/optim/nadam.rs:28-31,135-156)."""

    def __init__(self, params=None, lr: float = 2e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, momentum_decay: float = 0.004, schedule_decay: Optional[float] = None):
        super().__init__(_params(params), lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay,
                         momentum_decay=momentum_decay if schedule_decay is None else schedule_decay)


class RAdam(_RefAPI, torch.optim.RAdam):
    """Variance-rectified Adam; rectification applies once rho_t exceeds the threshold (reference 4.0,
    torch 5.0 — torch's is used) (src/optim/radam.rs:25-31,187-205)."""

    def __init__(self, params=None, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0):
        super().__init__(_params(params), lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)


class Adamax(_RefAPI, torch.optim.Adamax):
    """Infinity-norm Adam, eps default 1e-7 (src/optim/common.rs:107-117)."""

    def __init__(self, params=None, lr: float = 2e-3, betas=(0.9, 0.999), eps: float = 1e-7, weight_decay: float = 0.0):
        super().__init__(_params(params), lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)


class AdaBound(_RefAPI, _TorchOptimizer):
    """Adam whose per-element step size is clipped into bounds that converge to ``final_lr``
    (``new(lr)`` = final_lr 0.1, betas 0.9/0.999, eps 1e-8, wd 0, gamma 1e-3; src/optim/adabound.rs:35-64)."""

    def __init__(self, params=None, lr: float = 1e-3, final_lr: float = 0.1, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, gamma: float = 1e-3):
        super().__init__(_params(params), dict(lr=lr, final_lr=final_lr, betas=tuple(betas), eps=eps,
                                               weight_decay=weight_decay, gamma=gamma, base_lr=lr))

    @torch.no_grad()
    def _fallback_step(self) -> None:
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad.float()
                if g["weight_decay"]:
                    grad = grad.add(p.float(), alpha=g["weight_decay"])
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
                t = st["step"]
                st["exp_avg"].mul_(b1).add_(grad, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(grad, grad, value=1 - b2)
                step_size = g["lr"] * math.sqrt(1 - b2 ** t) / (1 - b1 ** t)
                final_lr = g["final_lr"] * g["lr"] / g["base_lr"]
                lower = final_lr * (1 - 1 / (g["gamma"] * t + 1))
                upper = final_lr * (1 + 1 / (g["gamma"] * t))
                denom = st["exp_avg_sq"].sqrt().add_(g["eps"])
                eta = torch.full_like(denom, step_size).div_(denom).clamp_(lower, upper)
                p.add_((-eta * st["exp_avg"]).to(p.dtype))


class LAMB(_RefAPI, _TorchOptimizer):
    """Layer-wise adaptive moments with trust ratio (``new(lr)`` = betas 0.9/0.999, eps 1e-6, wd 0.01,
    bias correction on; src/optim/lamb.rs:34-62)."""

    def __init__(self, params=None, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-6,
                 weight_decay: float = 0.01, bias_correction: bool = True):
        super().__init__(_params(params), dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay,
                                               bias_correction=bias_correction))

    @torch.no_grad()
    def _fallback_step(self) -> None:
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad.float()
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
                t = st["step"]
                st["exp_avg"].mul_(b1).add_(grad, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(grad, grad, value=1 - b2)
                m, v = st["exp_avg"], st["exp_avg_sq"]
                if g["bias_correction"]:
                    m, v = m / (1 - b1 ** t), v / (1 - b2 ** t)
                upd = m / (v.sqrt() + g["eps"])
                if g["weight_decay"]:
                    upd = upd.add(p.float(), alpha=g["weight_decay"])
                wn, un = float(p.float().norm()), float(upd.norm())
                trust = wn / un if wn > 0 and un > 0 else 1.0
                p.add_((-g["lr"] * trust * upd).to(p.dtype))


class LBFGS(_RefAPI, torch.optim.LBFGS):
    """``new(lr)``: max_iter 20, max_eval 20, tol_grad 1e-5, tol_change 1e-9, history 10, strong-Wolfe line
    search (src/optim/lbfgs.rs:35-52,192-203)."""

    def __init__(self, params=None, lr: float = 1.0, max_iter: int = 20, max_eval: Optional[int] = 20,
                 tolerance_grad: float = 1e-5, tolerance_change: float = 1e-9, history_size: int = 10,
                 line_search_fn: Optional[str] = "strong_wolfe"):
        super().__init__(_params(params), lr=lr, max_iter=max_iter, max_eval=max_eval,
                         tolerance_grad=tolerance_grad, tolerance_change=tolerance_change,
                         history_size=history_size, line_search_fn=line_search_fn)

    step = torch.optim.LBFGS.step          # host loop with closure re-evaluation; no multi-tensor form

    @torch.no_grad()
    def step_tensor(self, param: torch.Tensor, grad: torch.Tensor) -> None:
        """One L-BFGS iteration from an explicit gradient, as the reference's ``step(&param, &grad)`` does: two-loop
        direction over the stored (s, y) pairs, ``param += lr * d``.  fp32 CPU tensors run in the native runtime."""
        if (param.device.type != "cpu" or param.dtype != torch.float32 or not param.is_contiguous() or grad.dtype != torch.float32
                or not grad.is_contiguous()):
            from ..compat import LBFGSMemory
            st = self.__dict__.setdefault("_mem", {}).setdefault(id(param), {"mem": LBFGSMemory(self.param_groups[0]["history_size"])})
            if "p" in st:
                st["mem"].update(param - st["p"], grad - st["g"])
            st["p"], st["g"] = param.clone(), grad.clone()
            param.add_(st["mem"].direction(grad), alpha=self.param_groups[0]["lr"])
            return
        fs = self.__dict__.setdefault("_fast_state", {})
        st = fs.get(id(param))
        n, hist = param.numel(), int(self.param_groups[0]["history_size"])
        if st is None:
            from .. import _native
            z = lambda *shape: torch.zeros(*shape, dtype=torch.float32)  # noqa: E731
            st = {"pp": z(n), "pg": z(n), "S": z(hist, n), "Y": z(hist, n), "rho": z(hist), "scratch": z(n + hist), "count": 0, "head": 0,
                  "has_prev": 0, "host": _native.host(), "ref": param}
            fs[id(param)] = st
        packed = st["host"].cpu_lbfgs_step(param.data_ptr(), grad.data_ptr(), st["pp"].data_ptr(), st["pg"].data_ptr(), st["S"].data_ptr(),
                                           st["Y"].data_ptr(), st["rho"].data_ptr(), st["scratch"].data_ptr(), n, hist, st["count"],
                                           st["head"], st["has_prev"], float(self.param_groups[0]["lr"]))
        st["count"], st["head"], st["has_prev"] = packed >> 16, packed & 0xFFFF, 1


def _state_dict_with_fast(self):
    self._publish_fast_state()
    return torch.optim.Optimizer.state_dict(self)


for _k, _cls in enumerate((Adam, AdamW, Adamax, NAdam, RAdam)):
    _cls._NATIVE_KIND = _k
    _cls.state_dict = _state_dict_with_fast

# update rules of the CUDA multi-tensor kernel (rustorch_b200/optim/multi_tensor.py)
for _cls, _kind in ((Adam, 0), (AdamW, 1), (SGD, 2), (NAdam, 3), (RAdam, 4), (Adamax, 5), (RMSprop, 6), (AdaGrad, 7), (AdaBound, 8),
                    (LAMB, 9)):
    _cls._MT_KIND = _kind


# ---- named constructors of the Rust API (``Type::new / default_params / with_*``); the parameters come first here
def _ctor(cls, name: str, fn) -> None:
    """Registers ``fn(cls, params, ...)`` as a classmethod.  A leading number instead of parameters is the Rust call
    (``SGD::new(0.01)``): an optimizer without registered parameters, stepped with ``step(param, grad)``."""
    def make(c, *a, **k):
        if a and isinstance(a[0], (int, float)) and not isinstance(a[0], bool):
            a = (None,) + a
        return fn(c, *a, **k)
    make.__name__ = name
    setattr(cls, name, classmethod(make))


for _cls in (SGD, Adam, AdamW, RMSprop, AdaGrad, NAdam, RAdam, Adamax, AdaBound, LAMB, LBFGS):
    _ctor(_cls, "new", lambda cls, params=None, *a, **k: cls(params, *a, **k))
    for _name in ("default_params", "with_momentum", "with_weight_decay", "with_nesterov", "with_amsgrad"):
        if _name in _cls.__dict__:                      # the ones written in the class bodies take the same two call forms
            _ctor(_cls, _name, _cls.__dict__[_name].__func__)

# src/optim/adamw.rs:66-80
_ctor(AdamW, "with_weight_decay", lambda cls, params, lr, weight_decay: cls(params, lr, weight_decay=weight_decay))
_ctor(AdamW, "with_amsgrad", lambda cls, params, lr, weight_decay=0.01: cls(params, lr, weight_decay=weight_decay, amsgrad=True))
# src/optim/mod.rs:447-500, 646-660
_ctor(RMSprop, "with_momentum", lambda cls, params, lr, alpha=0.99, eps=1e-8, momentum=0.0: cls(params, lr, alpha, eps, momentum=momentum))
_ctor(RMSprop, "with_weight_decay", lambda cls, params, lr, alpha=0.99, eps=1e-8, weight_decay=0.0: cls(params, lr, alpha, eps, weight_decay))
_ctor(AdaGrad, "with_weight_decay", lambda cls, params, lr, eps=1e-10, weight_decay=0.0: cls(params, lr, weight_decay=weight_decay, eps=eps))
# src/optim/nadam.rs:156-175, radam.rs:206-225, adamax.rs:152-171
_ctor(NAdam, "default_params", lambda cls, params, lr=2e-3: cls(params, lr))
_ctor(NAdam, "with_weight_decay", lambda cls, params, lr, weight_decay: cls(params, lr, weight_decay=weight_decay))
_ctor(NAdam, "with_momentum_decay", lambda cls, params, lr, momentum_decay: cls(params, lr, momentum_decay=momentum_decay))
_ctor(RAdam, "default_params", lambda cls, params, lr=1e-3: cls(params, lr))
_ctor(RAdam, "with_weight_decay", lambda cls, params, lr, weight_decay: cls(params, lr, weight_decay=weight_decay))
_ctor(Adamax, "default_params", lambda cls, params, lr=2e-3: cls(params, lr))
_ctor(Adamax, "with_weight_decay", lambda cls, params, lr, weight_decay: cls(params, lr, weight_decay=weight_decay))
_ctor(Adamax, "with_infinity_eps", lambda cls, params, lr, infinity_eps: cls(params, lr, eps=infinity_eps))
# src/optim/lamb.rs:40-75, adabound.rs:41-64, lbfgs.rs:206-250
_ctor(LAMB, "with_params", lambda cls, params, lr, beta1=0.9, beta2=0.999, eps=1e-6, weight_decay=0.01:
      cls(params, lr, (beta1, beta2), eps, weight_decay))
_ctor(LAMB, "without_bias_correction", lambda cls, params, lr, beta1=0.9, beta2=0.999, eps=1e-6, weight_decay=0.01:
      cls(params, lr, (beta1, beta2), eps, weight_decay, bias_correction=False))
_ctor(AdaBound, "with_params", lambda cls, params, lr, final_lr=0.1, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, gamma=1e-3:
      cls(params, lr, final_lr, (beta1, beta2), eps, weight_decay, gamma))


def _lbfgs_with_params(cls, params, lr, max_iter=20, max_eval=20, tolerance_grad=1e-5, tolerance_change=1e-9, history_size=10,
                       line_search_fn="strong_wolfe"):
    if lr <= 0:
        raise ValueError("Learning rate must be positive")
    if tolerance_grad < 0 or tolerance_change < 0:
        raise ValueError("Tolerances must be non-negative")
    if history_size <= 0:
        raise ValueError("History size must be positive")
    ls = getattr(line_search_fn, "value", line_search_fn)
    ls = None if ls in (None, "none", "None") else "strong_wolfe" if "wolfe" in str(ls).lower() else ls
    return cls(params, lr, max_iter, max_eval, tolerance_grad, tolerance_change, history_size, ls)


_ctor(LBFGS, "with_params", _lbfgs_with_params)


def _set_final_lr(self, final_lr: float) -> None:
    for g in self.param_groups:
        g["final_lr"] = float(final_lr)


AdaBound.set_final_lr = _set_final_lr


def _radam_with_threshold(cls, params, lr, threshold: float):
    """The rectification threshold is part of the fused update rules (``rho_t > 5``, as in PyTorch); the reference's
    default is 4 (src/optim/radam.rs:25-40).  Another value takes a per-tensor update written out here."""
    opt = cls(params, lr)
    if float(threshold) != 5.0:
        opt.threshold = float(threshold)
        opt._MT_KIND = opt._NATIVE_KIND = None
        opt._fallback_step = lambda: _radam_step(opt)
    return opt


@torch.no_grad()
def _radam_step(self) -> None:
    for g in self.param_groups:
        b1, b2 = g["betas"]
        rho_inf = 2.0 / (1.0 - b2) - 1.0
        for p in g["params"]:
            if p.grad is None:
                continue
            grad = p.grad.float()
            if g["weight_decay"]:
                grad = grad.add(p.float(), alpha=g["weight_decay"])
            st = self.state[p]
            if not st:
                st["step"] = 0
                st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
            st["step"] += 1
            t = int(st["step"])
            st["exp_avg"].mul_(b1).add_(grad, alpha=1 - b1)
            st["exp_avg_sq"].mul_(b2).addcmul_(grad, grad, value=1 - b2)
            m_hat = st["exp_avg"] / (1 - b1 ** t)
            rho_t = rho_inf - 2.0 * t * b2 ** t / (1 - b2 ** t)
            if rho_t > self.threshold:
                rect = math.sqrt((rho_t - 4) * (rho_t - 2) * rho_inf / ((rho_inf - 4) * (rho_inf - 2) * rho_t))
                v_hat = (st["exp_avg_sq"] / (1 - b2 ** t)).sqrt().add_(g["eps"])
                p.add_((-g["lr"] * rect * m_hat / v_hat).to(p.dtype))
            else:
                p.add_((-g["lr"] * m_hat).to(p.dtype))


_ctor(RAdam, "with_threshold", _radam_with_threshold)
