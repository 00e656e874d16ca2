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

from ..data import DataLoader, RandomSampler, SequentialSampler, TensorDataset


class ModelMode(enum.Enum):
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
    loss: List[float] = field(default_factory=list)
    val_loss: List[float] = field(default_factory=list)
    metrics: Dict[str, List[float]] = field(default_factory=dict)
    epoch_time_s: List[float] = field(default_factory=list)

    def best_epoch(self) -> int:
        src = self.val_loss or self.loss
        return min(range(len(src)), key=src.__getitem__) if src else -1

    def to_json(self) -> str:
        return json.dumps({"loss": self.loss, "val_loss": self.val_loss, "metrics": self.metrics})


_LOSSES = {"mse": nn.MSELoss, "cross_entropy": nn.CrossEntropyLoss, "categorical_crossentropy": nn.CrossEntropyLoss,
           "bce": nn.BCEWithLogitsLoss, "binary_crossentropy": nn.BCEWithLogitsLoss, "l1": nn.L1Loss, "huber": nn.HuberLoss}


def _metric(name: str) -> Callable:
    if name in ("accuracy", "acc"):
        return lambda out, y: float((out.argmax(-1) == y).float().mean())
    if name == "mae":
        return lambda out, y: float((out - y).abs().mean())
    raise ValueError(f"unknown metric '{name}'")


class Sequential(Model):
    """``Sequential().add(layer)...compile(optimizer, loss, metrics).fit(x, y, ...)``."""

    def __init__(self, layers: Optional[Sequence[nn.Module]] = None, name: str = "sequential"):
        super().__init__()
        self.layers = nn.ModuleList(layers or [])
        self.name = name
        self._optimizer = self._loss = None
        self._metrics: Dict[str, Callable] = {}

    def add(self, layer: nn.Module) -> "Sequential":
        self.layers.append(layer)
        return self

    def forward(self, x):
        for l in self.layers:
            x = l(x)
        return x

    def compile(self, optimizer: Union[str, torch.optim.Optimizer] = "adam", loss: Union[str, nn.Module] = "mse",
                metrics: Sequence[str] = (), lr: float = 1e-3) -> "Sequential":
        from ..optim import OptimizerFactory
        self._optimizer = OptimizerFactory.create(optimizer, self.parameters(), lr=lr) if isinstance(optimizer, str) else optimizer
        self._loss = _LOSSES[loss]() if isinstance(loss, str) else loss
        self._metrics = {m: _metric(m) for m in metrics}
        return self

    def _loader(self, x, y, batch_size, shuffle, seed=None):
        ds = TensorDataset(x, y)
        sampler = RandomSampler(len(ds), seed=seed) if shuffle else SequentialSampler(len(ds))
        return DataLoader(ds, sampler, batch_size)

    def fit(self, x: torch.Tensor, y: torch.Tensor, config: Optional[FitConfig] = None, **kw) -> TrainingHistory:
        if self._optimizer is None:
            raise RuntimeError("call compile() before fit()")
        cfg = config or FitConfig(**kw)
        n_val = int(len(x) * cfg.validation_split)
        xt, yt = (x[:-n_val], y[:-n_val]) if n_val else (x, y)
        hist = TrainingHistory(metrics={m: [] for m in self._metrics})
        for epoch in range(cfg.epochs):
            t0 = time.time()
            self.train()
            tot, n = 0.0, 0
            for xb, yb in self._loader(xt, yt, cfg.batch_size, cfg.shuffle, None if cfg.seed is None else cfg.seed + epoch):
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

    @torch.no_grad()
    def evaluate(self, x, y, batch_size: int = 32) -> Dict[str, float]:
        self.eval()
        tot: Dict[str, float] = {"loss": 0.0, **{m: 0.0 for m in self._metrics}}
        n = 0
        for xb, yb in self._loader(x, y, batch_size, False):
            out = self(xb)
            tot["loss"] += float(self._loss(out, yb)) * len(xb)
            for m, fn in self._metrics.items():
                tot[m] += fn(out, yb) * len(xb)
            n += len(xb)
        return {k: v / max(1, n) for k, v in tot.items()}

    @torch.no_grad()
    def predict(self, x, batch_size: int = 32) -> torch.Tensor:
        self.eval()
        return torch.cat([self(x[i:i + batch_size]) for i in range(0, len(x), batch_size)])


BasicSequential = Sequential
HighLevelModel = Sequential


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

    def dropout(self, p: float):
        self._layers.append(nn.Dropout(p))
        return self

    def conv2d(self, i, o, k, stride=1, padding=0):
        self._layers.append(nn.Conv2d(i, o, k, stride, padding))
        return self

    def flatten(self):
        self._layers.append(nn.Flatten())
        return self

    def layer(self, m: nn.Module):
        self._layers.append(m)
        return self

    def build(self) -> Sequential:
        return Sequential(self._layers, self._name)


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
        model.load_state_dict({k: v.to(own[k].dtype) for k, v in sd.items() if k in own}, strict=strict)
        return model

    @staticmethod
    def load_checkpoint(model: nn.Module, optimizer, path: str) -> dict:
        from ..formats import rustorch_bin
        ck = rustorch_bin.load_checkpoint(path)
        own = model.state_dict()
        model.load_state_dict({k: v.to(own[k].dtype) for k, v in {**ck["parameters"], **ck["buffers"]}.items() if k in own}, strict=False)
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
