"""Keras-style model API: ``Sequential`` builder, ``HighLevelModel`` with ``compile / fit / evaluate / predict``,
``FitConfig``, ``TrainingHistory``; the ``Model`` protocol, ``ModelBuilder``, ``InferenceEngine`` and model
save/load helpers (src/models/mod.rs:48-177, sequential.rs:45-497, sequential_basic.rs:13-261,
high_level.rs:19-421, serialization.rs:18-543, training.rs:157-231).

The reference's models-level trainer reports simulated losses (training.rs:157-231); ``fit`` here trains.
"""
from __future__ import annotations

import enum
import json
import os
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple, Union

import torch
import torch.nn as nn

from .._interop import DictValue, FloatValue, ListValue
from ..data import DataLoader, RandomSampler, SequentialSampler, TensorDataset


class ModelMode(enum.Enum):
    """Training or evaluation mode of a model (src/models/mod.rs:48-60)."""

    TRAIN = "train"
    EVAL = "eval"


class Model(nn.Module):
    """Protocol of the reference's ``Model`` trait: ``train() / eval() / mode() / config() / summary()``."""

    def mode(self) -> ModelMode:
        return ModelMode.TRAIN if self.training else ModelMode.EVAL

    def config(self) -> Dict[str, object]:
        return dict(getattr(self, "_config", {}))

    def summary(self) -> str:
        rows = [f"{type(self).__name__}"]
        total = 0
        for name, p in self.named_parameters():
            rows.append(f"  {name:<40} {str(tuple(p.shape)):<20} {p.numel():>12,}")
            total += p.numel()
        rows.append(f"  total parameters: {total:,}")
        return "\n".join(rows)


@dataclass
class Metrics:
    """Classification summary ``accuracy / precision / recall / f1_score / loss`` (src/models/mod.rs:118-152).
    ``from_predictions`` fills it from logits (or class ids) and targets with macro-averaged precision / recall."""
    accuracy: float = 0.0
    precision: float = 0.0
    recall: float = 0.0
    f1_score: float = 0.0
    loss: float = 0.0

    @classmethod
    def new(cls) -> "Metrics":
        return cls()

    @classmethod
    def with_values(cls, accuracy: float, precision: float, recall: float, f1_score: float, loss: float) -> "Metrics":
        return cls(float(accuracy), float(precision), float(recall), float(f1_score), float(loss))

    @classmethod
    def from_predictions(cls, outputs: torch.Tensor, targets: torch.Tensor, loss: float = 0.0, num_classes: Optional[int] = None) -> "Metrics":
        pred = outputs.argmax(-1) if outputs.is_floating_point() and outputs.dim() > targets.dim() else outputs
        pred, tgt = pred.flatten().long(), targets.flatten().long()
        k = int(num_classes or max(int(pred.max()), int(tgt.max())) + 1)
        cm = torch.bincount(tgt * k + pred, minlength=k * k).view(k, k).double()      # rows: truth, columns: prediction
        tp = cm.diag()
        seen = (cm.sum(1) + cm.sum(0)) > 0
        prec = torch.where(cm.sum(0) > 0, tp / cm.sum(0).clamp_min(1), torch.zeros_like(tp))[seen].mean()
        rec = torch.where(cm.sum(1) > 0, tp / cm.sum(1).clamp_min(1), torch.zeros_like(tp))[seen].mean()
        f1 = 0.0 if float(prec + rec) == 0 else float(2 * prec * rec / (prec + rec))
        return cls(float(tp.sum() / cm.sum().clamp_min(1)), float(prec), float(rec), f1, float(loss))


def count_parameters(module: nn.Module, trainable_only: bool = False) -> int:
    return sum(p.numel() for p in module.parameters() if p.requires_grad or not trainable_only)


@dataclass
class FitConfig:
    epochs: int = 10
    batch_size: int = 32
    validation_split: float = 0.0
    shuffle: bool = True
    verbose: bool = False
    seed: Optional[int] = None


@dataclass
class TrainingHistory:
    """Per-epoch record of a ``fit``.  The binding's accessors (src/python/training.rs:66-117: ``train_loss()``,
    ``val_loss()``, ``metrics()``, ``training_time()``, ``best_val_loss()``, ``best_epoch()``, ``summary()``,
    ``plot_data()``) read the same lists; list / dict / float members can be read as attributes or called."""
    loss: List[float] = field(default_factory=ListValue)
    val_loss: List[float] = field(default_factory=ListValue)
    metrics: Dict[str, List[float]] = field(default_factory=DictValue)
    epoch_time_s: List[float] = field(default_factory=ListValue)
    total_time_s: Optional[float] = None

    def __post_init__(self):
        self.loss, self.val_loss = ListValue(self.loss), ListValue(self.val_loss)
        self.metrics, self.epoch_time_s = DictValue(self.metrics), ListValue(self.epoch_time_s)

    def add_epoch(self, train_loss: float, val_loss: Optional[float] = None, metrics: Optional[Dict[str, float]] = None,
                  seconds: Optional[float] = None) -> None:
        self.loss.append(float(train_loss))
        if val_loss is not None:
            self.val_loss.append(float(val_loss))
        for k, v in (metrics or {}).items():
            self.metrics.setdefault(k, []).append(float(v))
        if seconds is not None:
            self.epoch_time_s.append(float(seconds))

    @property
    def train_loss(self) -> List[float]:
        return self.loss

    @property
    def training_time(self) -> float:
        return FloatValue(self.total_time_s if self.total_time_s is not None else sum(self.epoch_time_s))

    @training_time.setter
    def training_time(self, seconds: float) -> None:
        self.total_time_s = float(seconds)

    def best_val_loss(self) -> Optional[float]:
        return min(self.val_loss) if self.val_loss else None

    def best_epoch(self) -> int:
        """Index of the epoch with the lowest validation loss (training loss without validation); -1 when empty."""
        src = self.val_loss or self.loss
        return min(range(len(src)), key=src.__getitem__) if src else -1

    def summary(self) -> str:
        if not self.loss:
            return "TrainingHistory: no epochs"
        rows = [f"TrainingHistory: {len(self.loss)} epochs in {float(self.training_time):.2f} s",
                f"  final train loss {self.loss[-1]:.6f}"]
        if self.val_loss:
            rows.append(f"  final val loss   {self.val_loss[-1]:.6f}  (best {self.best_val_loss():.6f} at epoch {self.best_epoch() + 1})")
        for k, v in self.metrics.items():
            if v:
                rows.append(f"  {k}: {v[-1]:.4f}")
        return "\n".join(rows)

    def plot_data(self) -> Tuple[List[float], List[float], List[float]]:
        """``(epochs 1.., train losses, validation losses)`` for a loss curve."""
        return [float(i + 1) for i in range(len(self.loss))], list(self.loss), list(self.val_loss)

    def to_json(self) -> str:
        return json.dumps({"loss": list(self.loss), "val_loss": list(self.val_loss), "metrics": dict(self.metrics)})


_LOSSES = {"mse": nn.MSELoss, "cross_entropy": nn.CrossEntropyLoss, "categorical_crossentropy": nn.CrossEntropyLoss,
           "bce": nn.BCEWithLogitsLoss, "binary_crossentropy": nn.BCEWithLogitsLoss, "l1": nn.L1Loss, "huber": nn.HuberLoss}


def _metric(name: str) -> Callable:
    if name in ("accuracy", "acc"):
        return lambda out, y: float((out.argmax(-1) == y).float().mean())
    if name == "mae":
        return lambda out, y: float((out - y).abs().mean())
    raise ValueError(f"unknown metric '{name}'")


def _is_loader(x) -> bool:
    """This package's ``DataLoader`` (stepping API) or a ``torch.utils.data.DataLoader``."""
    return hasattr(x, "next_batch") or isinstance(x, torch.utils.data.DataLoader)


def _rewind(loader) -> None:
    if hasattr(loader, "reset"):
        loader.reset()


def _raw(t):
    """The ``torch.Tensor`` inside a ``Tensor`` / ``Variable`` wrapper (or the argument itself)."""
    if t is None or isinstance(t, torch.Tensor):
        return t
    from ..autograd import Variable
    if isinstance(t, Variable):
        return t.tensor
    return getattr(t, "data", t)


_ACTIVATIONS = {"linear": None, "none": None, "relu": nn.ReLU, "sigmoid": nn.Sigmoid, "tanh": nn.Tanh, "gelu": nn.GELU,
                "softmax": lambda: nn.Softmax(dim=-1), "leaky_relu": nn.LeakyReLU, "elu": nn.ELU, "selu": nn.SELU,
                "swish": nn.SiLU, "silu": nn.SiLU}


def _activation(name: Optional[str]) -> Optional[nn.Module]:
    key = (name or "linear").strip().lower()
    if key not in _ACTIVATIONS:
        raise ValueError(f"unknown activation '{name}'")
    f = _ACTIVATIONS[key]
    return None if f is None else f()


class _Deferred(nn.Module):
    """A layer described without its input width; ``inner`` is built from the first input."""

    def __init__(self, activation: Optional[str]):
        super().__init__()
        self.inner: Optional[nn.Module] = None
        self.act = _activation(activation)
        self.activation = (activation or "linear").lower()
        self.last_output_shape = None

    def _build(self, x: torch.Tensor) -> nn.Module:
        raise NotImplementedError

    def _prepare(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def _build_from_weight(self, weight: torch.Tensor) -> nn.Module:
        raise NotImplementedError

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        """A checkpoint can be loaded into a layer that has not seen data yet: the stored weight tells the input width."""
        w = state_dict.get(prefix + "inner.weight")
        if self.inner is None and w is not None:
            self.inner = self._build_from_weight(w).to(w.dtype)
        return super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def forward(self, x):
        x = self._prepare(x)
        if self.inner is None:
            self.inner = self._build(x).to(device=x.device, dtype=x.dtype if x.is_floating_point() else None)
        y = self.inner(x)
        y = y if self.act is None else self.act(y)
        self.last_output_shape = (None, *y.shape[1:])
        return y


class Dense(_Deferred):
    """``Dense(units, activation)``: this package's ``Linear`` (tcgen05 GEMM on CUDA) + activation; inputs with more
    than two dimensions are flattened per sample first."""

    def __init__(self, units: int, activation: Optional[str] = None):
        super().__init__(activation)
        if int(units) <= 0:
            raise ValueError("units must be positive")
        self.units = int(units)

    def _prepare(self, x):
        return x.flatten(1) if x.dim() > 2 else x

    def _build(self, x):
        from ..nn import Linear
        return Linear(x.shape[-1], self.units)

    def _build_from_weight(self, weight):
        from ..nn import Linear
        if weight.shape[0] != self.units:
            raise ValueError(f"checkpoint has {weight.shape[0]} units, the layer {self.units}")
        return Linear(weight.shape[1], self.units)

    def extra_repr(self) -> str:
        return f"{self.units}, activation={self.activation}"


class Conv2D(_Deferred):
    """``Conv2D(filters, kernel_size, activation)`` over ``[N, C, H, W]`` inputs."""

    def __init__(self, filters: int, kernel_size: int, activation: Optional[str] = "relu"):
        super().__init__(activation)
        if int(filters) <= 0 or int(kernel_size) <= 0:
            raise ValueError("filters and kernel_size must be positive")
        self.filters, self.kernel_size = int(filters), int(kernel_size)

    def _build(self, x):
        from ..nn import Conv2d
        if x.dim() != 4:
            raise ValueError(f"Conv2D needs [N, C, H, W] inputs, got {tuple(x.shape)}")
        return Conv2d(x.shape[1], self.filters, (self.kernel_size, self.kernel_size))

    def _build_from_weight(self, weight):
        from ..nn import Conv2d
        if weight.shape[0] != self.filters or tuple(weight.shape[2:]) != (self.kernel_size, self.kernel_size):
            raise ValueError(f"checkpoint holds a {tuple(weight.shape)} filter bank, the layer wants {self.filters} filters of size {self.kernel_size}")
        return Conv2d(weight.shape[1], self.filters, (self.kernel_size, self.kernel_size))

    def extra_repr(self) -> str:
        return f"{self.filters}, {self.kernel_size}, activation={self.activation}"


def _layer_kind(l: nn.Module) -> str:
    return {"Dense": "Dense", "Conv2D": "Conv2D"}.get(type(l).__name__, type(l).__name__)


def layer_from_spec(spec: str) -> nn.Module:
    """Parses ``Name(arg, ..., key=value)`` as written by :class:`ModelBuilder` of the binding."""
    import re
    m = re.fullmatch(r"\s*([A-Za-z_][A-Za-z0-9_]*)\s*(?:\((.*)\))?\s*", spec)
    if not m:
        raise ValueError(f"cannot parse layer description '{spec}'")
    name, body = m.group(1).lower(), (m.group(2) or "").strip()
    pos, kw = [], {}
    for part in [p.strip() for p in body.split(",") if p.strip()]:
        if "=" in part:
            k, v = part.split("=", 1)
            kw[k.strip().lower()] = v.strip().strip("'\"")
        else:
            pos.append(part.strip("'\""))
    if name == "dense":
        return Dense(int(pos[0]), kw.get("activation", pos[1] if len(pos) > 1 else None))
    if name in ("conv2d",):
        return Conv2D(int(pos[0]), int(pos[1]), kw.get("activation", pos[2] if len(pos) > 2 else "relu"))
    if name == "dropout":
        return nn.Dropout(float(pos[0]) if pos else float(kw.get("rate", kw.get("p", 0.5))))
    if name == "flatten":
        return nn.Flatten()
    if name in _ACTIVATIONS and _ACTIVATIONS[name] is not None:
        return _ACTIVATIONS[name]()
    raise ValueError(f"unknown layer '{spec}'")


class Sequential(Model):
    """``Sequential().add(layer)...compile(optimizer, loss, metrics).fit(x, y, ...)``."""

    def __init__(self, layers: Optional[Sequence[nn.Module]] = None, name: str = "sequential"):
        super().__init__()
        self.layers = nn.ModuleList(layers or [])
        self.name = name
        self._optimizer = self._loss = None
        self._optimizer_spec = ("sgd", 1e-3)
        self.compiled = False
        self._metrics: Dict[str, Callable] = {}

    def to(self, *args, **kwargs):
        """Also remembers the device for layers that do not exist yet and for the batches ``fit`` / ``evaluate`` feed in."""
        dev = torch._C._nn._parse_to(*args, **kwargs)[0]
        if dev is not None:
            self.__dict__["_target_device"] = dev
        return super().to(*args, **kwargs)

    def _dev(self) -> torch.device:
        for p in self.parameters():
            return p.device
        return self.__dict__.get("_target_device", torch.device("cpu"))

    def add(self, layer: Union[nn.Module, str]) -> "Sequential":
        """A module, or a layer description as the binding's builder writes them (src/python/training.rs:326-347):
        ``"Dense(64, activation=relu)"``, ``"Conv2D(32, 3, activation=relu)"``, ``"Dropout(0.5)"``, ``"Flatten"``, or an
        activation name.  Described layers take their input width from the first batch they see."""
        self.layers.append(layer_from_spec(layer) if isinstance(layer, str) else layer)
        return self

    def forward(self, x):
        shapes = self.__dict__.setdefault("_out_shapes", {})
        for i, l in enumerate(self.layers):
            x = l(x)
            if isinstance(x, torch.Tensor):
                shapes[i] = (None, *x.shape[1:])
        return x

    def compile(self, optimizer: Union[str, torch.optim.Optimizer, None] = "adam", loss: Union[str, nn.Module, None] = "mse",
                metrics: Optional[Sequence[str]] = (), lr: float = 1e-3) -> "Sequential":
        self._optimizer_spec = (optimizer or "sgd", lr)      # the binding's defaults: sgd / mse (training.rs:228-238)
        self._optimizer = None
        self._loss = _LOSSES[loss or "mse"]() if isinstance(loss or "mse", str) else loss
        self._metrics = {m: _metric(m) for m in (metrics or ())}
        self.compiled = True
        if not any(isinstance(m, _Deferred) and m.inner is None for m in self.modules()):
            self._make_optimizer()
        return self

    def _make_optimizer(self) -> None:
        from ..optim import OptimizerFactory
        opt, lr = self._optimizer_spec
        self._optimizer = OptimizerFactory.create(opt, self.parameters(), lr=lr) if isinstance(opt, str) else opt

    def _ready(self, sample: torch.Tensor) -> None:
        """Described layers are built by a forward pass of the first batch; the optimizer is made after that."""
        if self._optimizer is None:
            if not getattr(self, "compiled", False):
                raise RuntimeError("Model must be compiled before training")
            with torch.no_grad():
                self(sample)
            self._make_optimizer()

    def _loader(self, x, y, batch_size, shuffle, seed=None):
        ds = TensorDataset(x, y)
        sampler = RandomSampler(len(ds), seed=seed) if shuffle else SequentialSampler(len(ds))
        return DataLoader(ds, sampler, batch_size)

    def fit(self, x, y=None, config: Optional[FitConfig] = None, validation_data=None, epochs: Optional[int] = None,
            verbose: Optional[bool] = None, **kw) -> TrainingHistory:
        """``fit(x, y, config | epochs=, batch_size=, ...)`` on tensors, or the binding's
        ``fit(train_loader, validation_loader=None, epochs=10, verbose=True)`` on data loaders
        (src/python/training.rs:239-275; the reference returns made-up losses there, this trains)."""
        if not getattr(self, "compiled", False):
            raise RuntimeError("Model must be compiled before training")
        if _is_loader(x):
            val = validation_data if validation_data is not None else (y if _is_loader(y) else None)
            return self._fit_loaders(x, val, 10 if epochs is None else epochs, True if verbose is None else verbose)
        x, y = _raw(x), _raw(y)
        self._ready(x[:2])
        if epochs is not None:
            kw["epochs"] = epochs
        if verbose is not None:
            kw["verbose"] = verbose
        cfg = config or FitConfig(**kw)
        n_val = int(len(x) * cfg.validation_split)
        xt, yt = (x[:-n_val], y[:-n_val]) if n_val else (x, y)
        hist = TrainingHistory(metrics={m: [] for m in self._metrics})
        for epoch in range(cfg.epochs):
            t0 = time.time()
            self.train()
            tot, n = 0.0, 0
            for xb, yb in self._loader(xt, yt, cfg.batch_size, cfg.shuffle, None if cfg.seed is None else cfg.seed + epoch):
                xb, yb = xb.to(self._dev(), non_blocking=True), yb.to(self._dev(), non_blocking=True)
                self._optimizer.zero_grad()
                loss = self._loss(self(xb), yb)
                loss.backward()
                self._optimizer.step()
                tot += float(loss) * len(xb)
                n += len(xb)
            hist.loss.append(tot / max(1, n))
            if n_val:
                ev = self.evaluate(x[-n_val:], y[-n_val:], cfg.batch_size)
                hist.val_loss.append(ev["loss"])
                for m in self._metrics:
                    hist.metrics[m].append(ev[m])
            else:
                ev = self.evaluate(xt, yt, cfg.batch_size) if self._metrics else {}
                for m in self._metrics:
                    hist.metrics[m].append(ev[m])
            hist.epoch_time_s.append(time.time() - t0)
            if cfg.verbose:
                print(f"epoch {epoch + 1}/{cfg.epochs} loss {hist.loss[-1]:.4f}")
        return hist

    def _fit_loaders(self, train, val, epochs: int, verbose: bool) -> TrainingHistory:
        hist = TrainingHistory(metrics={m: [] for m in self._metrics})
        t_all = time.time()
        for epoch in range(epochs):
            t0 = time.time()
            self.train()
            tot, n = 0.0, 0
            _rewind(train)
            for batch in train:
                xb, yb = _raw(batch[0]).to(self._dev(), non_blocking=True), _raw(batch[1]).to(self._dev(), non_blocking=True)
                self._ready(xb)
                self._optimizer.zero_grad()
                loss = self._loss(self(xb), yb)
                loss.backward()
                self._optimizer.step()
                tot += float(loss.detach()) * len(xb)
                n += len(xb)
            ev = self.evaluate(val) if val is not None else (self.evaluate(train) if self._metrics else {})
            hist.add_epoch(tot / max(1, n), ev.get("loss") if val is not None else None,
                           {m: ev[m] for m in self._metrics if m in ev}, time.time() - t0)
            if verbose:
                tail = f" val_loss={hist.val_loss[-1]:.4f}" if val is not None else ""
                print(f"Epoch {epoch + 1}/{epochs}: loss={hist.loss[-1]:.4f}{tail}")
        hist.training_time = time.time() - t_all
        return hist

    @torch.no_grad()
    def evaluate(self, x, y=None, batch_size: int = 32) -> Dict[str, float]:
        """``evaluate(x, y)`` on tensors or ``evaluate(loader)``: mean loss and the compiled metrics."""
        if not getattr(self, "compiled", False):
            raise RuntimeError("Model must be compiled before evaluation")
        self.eval()
        tot: Dict[str, float] = {"loss": 0.0, **{m: 0.0 for m in self._metrics}}
        n = 0
        if _is_loader(x):
            _rewind(x)
            batches = ((_raw(b[0]).to(self._dev()), _raw(b[1]).to(self._dev())) for b in x)
        else:
            batches = self._loader(_raw(x), _raw(y), batch_size, False)
        for xb, yb in batches:
            xb, yb = xb.to(self._dev()), yb.to(self._dev())
            out = self(xb)
            tot["loss"] += float(self._loss(out, yb)) * len(xb)
            for m, fn in self._metrics.items():
                tot[m] += fn(out, yb) * len(xb)
            n += len(xb)
        return {k: v / max(1, n) for k, v in tot.items()}

    @torch.no_grad()
    def predict(self, x, batch_size: int = 32):
        """Outputs for ``x`` in evaluation mode; a ``Tensor`` / ``Variable`` argument gives a result of its own kind."""
        self.eval()
        from .._interop import call_unwrapped
        return call_unwrapped(lambda t: torch.cat([self(t[i:i + batch_size].to(self._dev())) for i in range(0, len(t), batch_size)]), (x,), {})

    def summary(self) -> str:
        line = "_" * 65
        rows = [f"Model: {self.name}", line, f"{'Layer (type)':<29}{'Output Shape':<26}Param #", "=" * 65]
        total = 0
        for i, l in enumerate(self.layers):
            n = sum(p.numel() for p in l.parameters())
            total += n
            shape = self.__dict__.get("_out_shapes", {}).get(i, getattr(l, "last_output_shape", None))
            rows.append(f"{f'{type(l).__name__.lower().lstrip(chr(95))}_{i} ({_layer_kind(l)})':<29}"
                        f"{str(shape) if shape is not None else '?':<26}{n:,}")
        rows += ["=" * 65, f"Total params: {total:,}", f"Compiled: {bool(getattr(self, 'compiled', False))}"]
        return "\n".join(rows)


BasicSequential = Sequential
HighLevelModel = Sequential


class BindingModel(Sequential):
    """``Model(name)`` of the Python binding (src/python/training.rs:208-313): ``add`` (layer descriptions or modules),
    ``compile``, ``fit`` / ``evaluate`` on data loaders, ``predict``, ``summary``."""

    def __init__(self, name: Optional[str] = None, layers: Optional[Sequence[nn.Module]] = None):
        super().__init__(layers, name or "Model")

    def __repr__(self) -> str:
        return f"Model(name='{self.name}', layers={len(self.layers)}, compiled={self.compiled})"


class ModelBuilder:
    """Fluent construction of a :class:`Sequential` from layer specs."""

    def __init__(self, name: str = "model"):
        self._layers: List[nn.Module] = []
        self._name = name

    def linear(self, i: int, o: int, bias: bool = True):
        from ..nn import Linear
        self._layers.append(Linear(i, o, bias))
        return self

    def relu(self):
        self._layers.append(nn.ReLU())
        return self

    def gelu(self):
        from ..nn import GELU
        self._layers.append(GELU())
        return self

    def dense(self, units: int, activation: Optional[str] = None):
        """Binding form (src/python/training.rs:326-331): the input width comes from the data."""
        self._layers.append(Dense(units, activation))
        return self

    def dropout(self, p: float):
        if not 0.0 <= float(p) < 1.0:
            raise ValueError("dropout rate must be in [0, 1)")
        self._layers.append(nn.Dropout(p))
        return self

    def conv2d(self, *args, activation: Optional[str] = None, stride=1, padding=0):
        """``conv2d(in_channels, out_channels, kernel, stride, padding)``, or the binding's
        ``conv2d(filters, kernel_size, activation="relu")`` whose input channels come from the data."""
        if len(args) == 2 or (len(args) == 3 and (args[2] is None or isinstance(args[2], str))):
            act = args[2] if len(args) == 3 else activation
            self._layers.append(Conv2D(args[0], args[1], "relu" if act is None else act))
            return self
        i, o, k = args[:3]
        stride = args[3] if len(args) > 3 else stride
        padding = args[4] if len(args) > 4 else padding
        from ..nn import Conv2d
        self._layers.append(Conv2d(i, o, k if isinstance(k, (tuple, list)) else (k, k),
                                   stride if isinstance(stride, (tuple, list)) else (stride, stride),
                                   padding if isinstance(padding, (tuple, list)) else (padding, padding)))
        if activation:
            self._layers.append(_activation(activation))
        return self

    def flatten(self):
        self._layers.append(nn.Flatten())
        return self

    def layer(self, m: nn.Module):
        self._layers.append(m)
        return self

    def build(self, name: Optional[str] = None) -> Sequential:
        """A new model with its own copies of the layers, so one builder can make several independent models."""
        import copy
        return BindingModel(name or self._name, [copy.deepcopy(l) for l in self._layers])

    def __repr__(self) -> str:
        return f"ModelBuilder(layers={len(self._layers)})"


class InferenceEngine:
    """Batched no-grad prediction with optional autocast and latency statistics."""

    def __init__(self, model: nn.Module, device: str = "cpu", dtype: Optional[torch.dtype] = None):
        self.model, self.device, self.dtype = model.to(device).eval(), torch.device(device), dtype
        self.latencies_ms: List[float] = []

    @torch.no_grad()
    def predict(self, x: torch.Tensor) -> torch.Tensor:
        t0 = time.perf_counter()
        x = x.to(self.device)
        if self.dtype is not None:
            with torch.autocast(self.device.type, dtype=self.dtype):
                y = self.model(x)
        else:
            y = self.model(x)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self.latencies_ms.append((time.perf_counter() - t0) * 1e3)
        return y

    def predict_batch(self, xs: Iterable[torch.Tensor]) -> List[torch.Tensor]:
        return [self.predict(x) for x in xs]

    def stats(self) -> Dict[str, float]:
        l = sorted(self.latencies_ms)
        if not l:
            return {}
        return {"n": len(l), "mean_ms": sum(l) / len(l), "p50_ms": l[len(l) // 2], "p99_ms": l[min(len(l) - 1, int(len(l) * 0.99))]}


# ------------------------------------------------------------------ save / load
class SerializationFormat(enum.Enum):
    """File formats ``ModelSaver`` / ``ModelLoader`` handle (src/models/serialization.rs:18-60)."""

    RUSTORCH = "rustorch"
    SAFETENSORS = "safetensors"
    PYTORCH = "pytorch"
    JSON = "json"


class ModelSaver:
    @staticmethod
    def save(model: nn.Module, path: str, fmt: SerializationFormat = SerializationFormat.RUSTORCH, config: Optional[dict] = None) -> None:
        from ..formats import rustorch_bin, safetensors as st
        sd = {k: v.detach().cpu() for k, v in model.state_dict().items()}
        if fmt is SerializationFormat.RUSTORCH:
            rustorch_bin.save_module(model, path, config=config)
        elif fmt is SerializationFormat.SAFETENSORS:
            st.save_safetensors(sd, path, {k: str(v) for k, v in (config or {}).items()})
        elif fmt is SerializationFormat.PYTORCH:
            torch.save(sd, path)
        else:
            st.save_json_state_dict(sd, path, config)

    @staticmethod
    def save_checkpoint(model: nn.Module, optimizer, path: str, epoch: int = 0, step: int = 0, metrics: Optional[dict] = None) -> None:
        from ..formats import rustorch_bin
        opt_blobs = {}
        if optimizer is not None and hasattr(optimizer, "state_dict"):
            import io
            buf = io.BytesIO()
            torch.save(optimizer.state_dict(), buf)
            opt_blobs["torch_state_dict"] = buf.getvalue()
        rustorch_bin.save_checkpoint(path, epoch, step, {k: v.detach() for k, v in model.named_parameters()},
                                     {k: v.detach() for k, v in model.named_buffers()}, opt_blobs, None, metrics,
                                     type(model).__name__)


def load_state_dict_file(path: str) -> Dict[str, torch.Tensor]:
    """Read a state dict from any supported container (RusTorch binary, safetensors, torch / PYTORCH1, JSON, HF dir)."""
    from ..formats import rustorch_bin, safetensors as st
    kind = st.detect_format(path)
    if kind == "rustorch":
        params, buffers, _ = rustorch_bin.load_state_dict(path)
        return {**params, **buffers}
    if kind == "safetensors":
        return st.load_safetensors(path)
    if kind == "mlx":
        from ..formats.mlx import MLXLoader
        return MLXLoader.load(path)[0]
    if kind in ("torch", "pth"):
        return st.load_pth(path)
    if kind == "json":
        return st.load_json_state_dict(path)[0]
    if kind == "huggingface":
        return st.load_huggingface(path)[0]
    raise ValueError(f"unrecognised model file '{path}'")


class ModelLoader:
    @staticmethod
    def load(model: nn.Module, path: str, strict: bool = True) -> nn.Module:
        from ..formats import rustorch_bin, safetensors as st
        kind = st.detect_format(path)
        if kind == "rustorch":
            rustorch_bin.load_module(model, path, strict)
            return model
        if kind == "safetensors":
            sd = st.load_safetensors(path)
        elif kind in ("torch", "pth"):
            sd = st.load_pth(path)
        elif kind == "json":
            sd, _ = st.load_json_state_dict(path)
        else:
            raise ValueError(f"unrecognised model file '{path}'")
        own = model.state_dict()
        # names the model does not have (yet) go through untouched: layers built from their first input create
        # them while loading, and with ``strict`` a genuinely unknown name must fail rather than vanish
        model.load_state_dict({k: (v.to(own[k].dtype) if k in own else v) for k, v in sd.items() if k in own or strict}, strict=strict)
        return model

    @staticmethod
    def load_checkpoint(model: nn.Module, optimizer, path: str, strict: bool = True) -> dict:
        """Restores ``model`` (and ``optimizer``) from a checkpoint file; returns the checkpoint (epoch, step, metrics).
        With ``strict`` a checkpoint that does not cover the model's tensors exactly is an error: resuming from the
        wrong file must not pass for a resume."""
        from ..formats import rustorch_bin
        ck = rustorch_bin.load_checkpoint(path)
        own = model.state_dict()
        tensors = {**ck["parameters"], **ck["buffers"]}
        model.load_state_dict({k: (v.to(own[k].dtype) if k in own else v) for k, v in tensors.items() if k in own or strict}, strict=strict)
        blob = ck["optimizer_state"].get("torch_state_dict")
        if optimizer is not None and blob:
            import io
            optimizer.load_state_dict(torch.load(io.BytesIO(blob), weights_only=False))
        return ck


@dataclass
class ModelInfo:
    name: str
    num_parameters: int
    size_bytes: int
    format: str

    @staticmethod
    def of(model: nn.Module, path: Optional[str] = None) -> "ModelInfo":
        from ..formats.safetensors import detect_format
        return ModelInfo(type(model).__name__, count_parameters(model),
                         os.path.getsize(path) if path and os.path.isfile(path) else sum(p.numel() * p.element_size() for p in model.parameters()),
                         detect_format(path) if path else "memory")


class ModelConverter:
    """Re-save a checkpoint in another format."""

    @staticmethod
    def convert(model: nn.Module, src: str, dst: str, fmt: SerializationFormat) -> None:
        ModelLoader.load(model, src, strict=False)
        ModelSaver.save(model, dst, fmt)
