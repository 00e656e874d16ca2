"""Tape autograd surface: ``Variable``, gradient modes, functional ``grad``, ``gradcheck``,
numerical higher-order derivatives, the explicit ``ComputationGraph`` and gradient-flow
visualisation.

The reference's ``Variable`` holds data + grad behind locks and walks its closures
recursively, re-visiting shared sub-graphs, with backward functions for only ``+ - * matmul
sum mean`` and ``Linear`` (src/autograd/mod.rs:49-56,156-198,202-505; grad_fn.rs:10-295).
Here the tape is torch.autograd (topologically sorted, every op differentiable); the class keeps
the reference's method names (``data() grad() zero_grad() backward() detach() retain_grad()
register_hook() sum() mean_autograd() matmul() ...``).
"""
from __future__ import annotations

import contextlib
import itertools
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ._interop import FlagValue, IntValue, ShapeValue
from .tensor import Tensor, _unwrap

_ids = itertools.count(1)


class Variable:
    """A tensor that records operations for reverse-mode differentiation."""

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        """Layers and ``torch`` functions accept a ``Variable`` and return ``Variable``s (python/src/lib.rs:377-452:
        the reference's layers map Variable to Variable)."""
        from ._interop import torch_function
        return torch_function(cls, func, types, args, kwargs)

    def __init__(self, data, requires_grad: bool = False):
        t = _unwrap(data) if isinstance(data, (Tensor, torch.Tensor)) else torch.as_tensor(data, dtype=torch.float32)
        if isinstance(data, Variable):
            t = data.tensor
        if requires_grad and not t.requires_grad:
            t = t.detach().requires_grad_(True) if t.is_leaf else t
        self.tensor: torch.Tensor = t
        self.id = next(_ids)

    # reference constructors / accessors
    new = classmethod(lambda cls, data, requires_grad=False: cls(data, requires_grad))

    @classmethod
    def from_tensor(cls, t, requires_grad: bool = False) -> "Variable":
        return cls(t, requires_grad)

    # constructors of the Python binding (src/python/autograd.rs: from_data / zeros / ones / randn)
    @classmethod
    def from_data(cls, data, shape, requires_grad: bool = False) -> "Variable":
        return cls(Tensor(list(data), shape), requires_grad)

    @classmethod
    def zeros(cls, shape, requires_grad: bool = False) -> "Variable":
        return cls(torch.zeros(tuple(shape)), requires_grad)

    @classmethod
    def ones(cls, shape, requires_grad: bool = False) -> "Variable":
        return cls(torch.ones(tuple(shape)), requires_grad)

    @classmethod
    def randn(cls, shape, requires_grad: bool = False) -> "Variable":
        return cls(torch.randn(tuple(shape)), requires_grad)

    def requires_grad_(self, requires_grad: bool = True) -> "Variable":
        if self.tensor.is_leaf:
            self.tensor.requires_grad_(requires_grad)
        elif not requires_grad:
            self.tensor = self.tensor.detach()
        return self

    @property
    def numel(self) -> int:
        return IntValue(self.tensor.numel())

    def transpose(self, dim0: Optional[int] = None, dim1: Optional[int] = None) -> "Variable":
        """Without arguments: the last two dimensions swapped (the binding's matrix transpose)."""
        if dim0 is None and dim1 is None:
            dim0, dim1 = -2, -1
        return self._w(self.tensor.transpose(dim0, dim1))

    def dot(self, other) -> "Variable":
        return self._w((self.tensor.flatten() * _v(other).flatten()).sum())

    def __array__(self, dtype=None, copy=None):
        a = self.tensor.detach().cpu().numpy()
        return a.astype(dtype) if dtype is not None else a

    def __len__(self) -> int:
        return len(self.tensor)

    def __getitem__(self, idx) -> "Variable":
        return self._w(self.tensor[_v(idx)])

    def __copy__(self) -> "Variable":
        return type(self)(self.tensor, self.tensor.requires_grad)            # same storage

    def __deepcopy__(self, memo) -> "Variable":
        return type(self)(self.tensor.detach().clone(), self.tensor.requires_grad)

    # ``data`` / ``grad`` / ``requires_grad`` / ``shape`` are attributes as in the Python wheel
    # (python/src/lib.rs:248-270); their values can also be called, which is the Rust spelling (``v.data()``).
    # ``v.grad`` is None until a backward pass reached ``v``.
    @property
    def data(self) -> Tensor:
        return Tensor(self.tensor.detach())

    @property
    def grad(self) -> Optional[Tensor]:
        g = self.tensor.grad
        return None if g is None else Tensor(g)

    @property
    def requires_grad(self) -> bool:
        return FlagValue(self.tensor.requires_grad)

    def zero_grad(self) -> None:
        self.tensor.grad = None

    def backward(self, grad=None, retain_graph: bool = False) -> None:
        """Seeds with ones (any shape, as the reference does, src/autograd/mod.rs:156-198)."""
        g = _unwrap(grad) if grad is not None else torch.ones_like(self.tensor)
        self.tensor.backward(g, retain_graph=retain_graph)

    backward_with_grad = backward

    def detach(self) -> "Variable":
        return type(self)(self.tensor.detach(), False)

    def retain_grad(self) -> "Variable":
        if not self.tensor.is_leaf:
            self.tensor.retain_grad()
        return self

    def register_hook(self, fn: Callable) -> object:
        return self.tensor.register_hook(lambda g: _unwrap(fn(Tensor(g))) if fn(Tensor(g)) is not None else None)

    def clone(self) -> "Variable":
        return type(self)(self.tensor.clone())

    @property
    def shape(self) -> Tuple[int, ...]:
        return ShapeValue(self.tensor.shape)

    def item(self) -> float:
        return float(self.tensor.item())

    # differentiable ops
    def _w(self, t: torch.Tensor) -> "Variable":
        return type(self)(t)

    def __add__(self, o):
        return self._w(self.tensor + _v(o))

    __radd__ = __add__

    def __sub__(self, o):
        return self._w(self.tensor - _v(o))

    def __rsub__(self, o):
        return self._w(_v(o) - self.tensor)

    def __mul__(self, o):
        return self._w(self.tensor * _v(o))

    __rmul__ = __mul__

    def __truediv__(self, o):
        return self._w(self.tensor / _v(o))

    def __neg__(self):
        return self._w(-self.tensor)

    def __matmul__(self, o):
        return self.matmul(o)

    def matmul(self, o) -> "Variable":
        return self._w(self.tensor @ _v(o))

    attention_matmul = matmul

    def transpose_last_two(self) -> "Variable":
        return self._w(self.tensor.transpose(-1, -2))

    def sum(self, dim=None) -> "Variable":
        return self._w(self.tensor.sum() if dim is None else self.tensor.sum(dim))

    def mean(self, dim=None) -> "Variable":
        return self._w(self.tensor.mean() if dim is None else self.tensor.mean(dim))

    mean_autograd = mean

    def pow(self, e: float) -> "Variable":
        return self._w(self.tensor.pow(e))

    def reshape(self, shape) -> "Variable":
        return self._w(self.tensor.reshape(tuple(shape)))

    def __getattr__(self, name):
        # exp/log/sin/cos/sqrt/tanh/... and every other torch method, result wrapped
        if name.startswith("__"):
            raise AttributeError(name)
        attr = getattr(self.tensor, name)
        if callable(attr):
            def call(*a, **k):
                r = attr(*[_v(x) for x in a], **{kk: _v(x) for kk, x in k.items()})
                return self._w(r) if isinstance(r, torch.Tensor) else r
            return call
        return attr

    def __repr__(self) -> str:
        return f"Variable(id={self.id}, shape={list(self.tensor.shape)}, requires_grad={self.tensor.requires_grad})"


def _v(x):
    if isinstance(x, Variable):
        return x.tensor
    return _unwrap(x)


# ----------------------------------------------------------------- gradient modes
# thread-local in torch as in the reference's GradientContext (src/autograd/context.rs:10-155)
no_grad = torch.no_grad
enable_grad = torch.enable_grad
set_grad_enabled = torch.set_grad_enabled
is_grad_enabled = torch.is_grad_enabled


@contextlib.contextmanager
def detect_anomaly(check_nan: bool = True):
    with torch.autograd.detect_anomaly(check_nan=check_nan):
        yield


class NoGradGuard:
    """RAII-style guard object (``with NoGradGuard(): ...``)."""

    def __enter__(self):
        self._prev = torch.is_grad_enabled()
        torch.set_grad_enabled(False)
        return self

    def __exit__(self, *exc):
        torch.set_grad_enabled(self._prev)
        return False


class EnableGradGuard(NoGradGuard):
    """Context manager that turns gradient recording on inside a ``no_grad`` region (src/autograd/context.rs:10-155)."""

    def __enter__(self):
        self._prev = torch.is_grad_enabled()
        torch.set_grad_enabled(True)
        return self


class AnomalyDetectionGuard:
    """Guard that turns autograd anomaly detection on (NaN checks in backward, forward stack traces in the errors) and
    puts the previous setting back on exit (src/autograd/context.rs:107-127)."""

    def __init__(self, check_nan: bool = True):
        self.check_nan = check_nan

    def __enter__(self):
        self._prev = torch.is_anomaly_enabled()
        self._prev_nan = torch.is_anomaly_check_nan_enabled()
        torch.autograd.set_detect_anomaly(True, check_nan=self.check_nan)
        return self

    def __exit__(self, *exc):
        torch.autograd.set_detect_anomaly(self._prev, check_nan=self._prev_nan)
        return False


def is_anomaly_detection_enabled() -> bool:
    return torch.is_anomaly_enabled()


def set_anomaly_detection(enabled: bool) -> None:
    torch.autograd.set_detect_anomaly(bool(enabled))


class GradientContext:
    """The current thread's gradient mode as one object: ``grad_enabled`` and ``anomaly_detection`` flags that read
    and write torch's thread-local state (src/autograd/context.rs:10-60 keeps the same two flags in a thread-local)."""

    @property
    def grad_enabled(self) -> bool:
        return torch.is_grad_enabled()

    @grad_enabled.setter
    def grad_enabled(self, on: bool) -> None:
        torch.set_grad_enabled(bool(on))

    @property
    def anomaly_detection(self) -> bool:
        return torch.is_anomaly_enabled()

    @anomaly_detection.setter
    def anomaly_detection(self, on: bool) -> None:
        torch.autograd.set_detect_anomaly(bool(on))

    @classmethod
    def current(cls) -> "GradientContext":
        return cls()

    def __repr__(self) -> str:
        return f"GradientContext(grad_enabled={self.grad_enabled}, anomaly_detection={self.anomaly_detection})"


# ------------------------------------------------------------------ functional API
def grad(outputs: Sequence[Variable], inputs: Sequence[Variable], grad_outputs=None, retain_graph: bool = False,
         create_graph: bool = False, allow_unused: bool = False) -> List[Optional[Tensor]]:
    """Gradients of ``outputs`` w.r.t. ``inputs`` (src/autograd/grad_utils.rs:18-209)."""
    outs = [_v(o) for o in (outputs if isinstance(outputs, (list, tuple)) else [outputs])]
    ins = [_v(i) for i in (inputs if isinstance(inputs, (list, tuple)) else [inputs])]
    validate_grad_setup(outs, ins)
    go = None
    if grad_outputs is not None:
        go = [_v(g) for g in grad_outputs]
    elif any(o.numel() != 1 for o in outs):
        go = [torch.ones_like(o) for o in outs]
    gs = torch.autograd.grad(outs, ins, go, retain_graph=retain_graph or create_graph, create_graph=create_graph,
                             allow_unused=allow_unused)
    return [None if g is None else Tensor(g) for g in gs]


gradient = grad


def validate_grad_setup(outputs, inputs) -> None:
    if not outputs or not inputs:
        raise ValueError("grad: outputs and inputs must be non-empty")
    for i in inputs:
        if not _v(i).requires_grad:
            raise ValueError("grad: every input must require grad")


@dataclass
class GradCheckConfig:
    eps: float = 1e-6
    atol: float = 1e-5
    rtol: float = 1e-3


def gradcheck(fn: Callable, inputs: Sequence, config: Optional[GradCheckConfig] = None,
              raise_exception: bool = False) -> bool:
    """Central finite differences vs autograd (src/autograd/gradcheck.rs:16-192), in float64."""
    cfg = config or GradCheckConfig()
    xs = [_v(x).detach().double().requires_grad_(True) for x in inputs]

    def f(*a):
        r = fn(*[Variable(t) for t in a])
        return _v(r)

    return bool(torch.autograd.gradcheck(f, xs, eps=cfg.eps, atol=cfg.atol, rtol=cfg.rtol,
                                         raise_exception=raise_exception))


def _numeric_grad(f: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.detach().double()
    y0 = f(x)
    J = torch.zeros(y0.numel(), x.numel(), dtype=torch.float64)
    flat = x.reshape(-1)
    for i in range(flat.numel()):
        xp, xm = flat.clone(), flat.clone()
        xp[i] += eps
        xm[i] -= eps
        J[:, i] = (f(xp.view_as(x)) - f(xm.view_as(x))).reshape(-1) / (2 * eps)
    return J


def jacobian(fn: Callable, x, eps: float = 1e-5) -> Tensor:
    """Numerical Jacobian ``[out, in]`` (src/autograd/higher_order.rs:14-105)."""
    return Tensor(_numeric_grad(lambda t: _v(fn(Variable(t))).double().reshape(-1), _v(x), eps).float())


def hessian(fn: Callable, x, eps: float = 1e-4) -> Tensor:
    """Numerical Hessian of a scalar function."""
    xt = _v(x).detach().double()

    def g(t: torch.Tensor) -> torch.Tensor:
        return _numeric_grad(lambda u: _v(fn(Variable(u))).double().reshape(1), t, eps).reshape(-1)

    return Tensor(_numeric_grad(g, xt, eps).float())


def hvp(fn: Callable, x, v, eps: float = 1e-4) -> Tensor:
    """Hessian-vector product by differencing gradients."""
    xt, vt = _v(x).detach().double(), _v(v).detach().double()

    def g(t: torch.Tensor) -> torch.Tensor:
        t = t.clone().requires_grad_(True)
        (gr,) = torch.autograd.grad(_v(fn(Variable(t))).sum(), t)
        return gr

    return Tensor(((g(xt + eps * vt) - g(xt - eps * vt)) / (2 * eps)).float())


# ------------------------------------------------------- explicit computation graph
class Function:
    """Forward/backward pair for the explicit graph (src/autograd/function.rs:9-112)."""

    name = "function"

    def forward(self, *inputs: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def backward(self, grad: torch.Tensor, *inputs: torch.Tensor) -> List[torch.Tensor]:
        raise NotImplementedError


class AddFunction(Function):
    name = "add"
    forward = lambda self, a, b: a + b  # noqa: E731
    backward = lambda self, g, a, b: [_reduce_to(g, a), _reduce_to(g, b)]  # noqa: E731


class SubFunction(Function):
    name = "sub"
    forward = lambda self, a, b: a - b  # noqa: E731
    backward = lambda self, g, a, b: [_reduce_to(g, a), _reduce_to(-g, b)]  # noqa: E731


class MulFunction(Function):
    name = "mul"
    forward = lambda self, a, b: a * b  # noqa: E731
    backward = lambda self, g, a, b: [_reduce_to(g * b, a), _reduce_to(g * a, b)]  # noqa: E731


class MatMulFunction(Function):
    name = "matmul"
    forward = lambda self, a, b: a @ b  # noqa: E731
    backward = lambda self, g, a, b: [g @ b.transpose(-1, -2), a.transpose(-1, -2) @ g]  # noqa: E731


class SumFunction(Function):
    name = "sum"
    forward = lambda self, a: a.sum()  # noqa: E731
    backward = lambda self, g, a: [g.expand_as(a)]  # noqa: E731


def _reduce_to(g: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    while g.dim() > like.dim():
        g = g.sum(0)
    for d, (gs, ls) in enumerate(zip(g.shape, like.shape)):
        if ls == 1 and gs != 1:
            g = g.sum(d, keepdim=True)
    return g


class ComputationGraph:
    """Node graph with an explicit topological sort (src/autograd/graph.rs:12-213)."""

    def __init__(self):
        self.nodes: Dict[int, dict] = {}
        self._next = 0

    def add_leaf(self, value: torch.Tensor, requires_grad: bool = True) -> int:
        nid = self._next
        self._next += 1
        self.nodes[nid] = {"fn": None, "inputs": [], "value": _unwrap(value), "grad": None, "requires_grad": requires_grad}
        return nid

    def add_node(self, fn: Function, inputs: Sequence[int]) -> int:
        vals = [self.nodes[i]["value"] for i in inputs]
        nid = self._next
        self._next += 1
        self.nodes[nid] = {"fn": fn, "inputs": list(inputs), "value": fn.forward(*vals), "grad": None,
                           "requires_grad": any(self.nodes[i]["requires_grad"] for i in inputs)}
        return nid

    def topological_sort(self) -> List[int]:
        seen, order = set(), []

        def visit(n):
            if n in seen:
                return
            seen.add(n)
            for i in self.nodes[n]["inputs"]:
                visit(i)
            order.append(n)

        for n in self.nodes:
            visit(n)
        return order

    def backward(self, node: int) -> None:
        for n in self.nodes.values():
            n["grad"] = None
        self.nodes[node]["grad"] = torch.ones_like(self.nodes[node]["value"])
        for nid in reversed(self.topological_sort()):
            n = self.nodes[nid]
            if n["fn"] is None or n["grad"] is None:
                continue
            vals = [self.nodes[i]["value"] for i in n["inputs"]]
            for i, g in zip(n["inputs"], n["fn"].backward(n["grad"], *vals)):
                tgt = self.nodes[i]
                if tgt["requires_grad"]:
                    tgt["grad"] = g if tgt["grad"] is None else tgt["grad"] + g

    def value(self, node: int) -> Tensor:
        return Tensor(self.nodes[node]["value"])

    def grad(self, node: int) -> Optional[Tensor]:
        g = self.nodes[node]["grad"]
        return None if g is None else Tensor(g)


# --------------------------------------------------------------- gradient-flow tools
class GradientFlowVisualizer:
    """DOT export of the autograd graph reachable from a Variable (src/autograd/visualization.rs:14-556)."""

    def to_dot(self, root: Variable, max_nodes: int = 2000) -> str:
        lines = ["digraph autograd {", "  rankdir=BT;"]
        seen, stack = set(), [_v(root).grad_fn]
        while stack and len(seen) < max_nodes:
            fn = stack.pop()
            if fn is None or id(fn) in seen:
                continue
            seen.add(id(fn))
            lines.append(f'  n{id(fn)} [label="{type(fn).__name__}"];')
            for nxt, _ in fn.next_functions:
                if nxt is not None:
                    lines.append(f"  n{id(nxt)} -> n{id(fn)};")
                    stack.append(nxt)
        lines.append("}")
        return "\n".join(lines)

    def save_dot(self, root: Variable, path: str) -> None:
        with open(path, "w") as f:
            f.write(self.to_dot(root))


class GradientFlowAnalyzer:
    """Tracks per-parameter gradient norms over time and flags vanishing / exploding gradients."""

    def __init__(self, vanishing: float = 1e-7, exploding: float = 1e3):
        self.vanishing, self.exploding = vanishing, exploding
        self.history: Dict[str, List[float]] = {}

    def record(self, named_parameters) -> None:
        for name, p in named_parameters:
            g = getattr(p, "grad", None)
            if g is not None:
                self.history.setdefault(name, []).append(float(g.detach().float().norm()))

    def issues(self) -> Dict[str, str]:
        out = {}
        for name, h in self.history.items():
            if h and h[-1] < self.vanishing:
                out[name] = "vanishing"
            elif h and (h[-1] > self.exploding or h[-1] != h[-1]):
                out[name] = "exploding"
        return out

    def trend(self, name: str) -> float:
        h = self.history.get(name, [])
        return 0.0 if len(h) < 2 else (h[-1] - h[0]) / (len(h) - 1)
