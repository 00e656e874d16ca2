"""Training loop, callbacks, checkpoint manager, metrics and state
(src/training/trainer.rs:19-683, callbacks.rs:12-562, checkpoint.rs:14-606, metrics.rs:12-414, state.rs:11-288).

The reference's loop never calls ``optimizer.step`` and reports a constant loss of 0.5
(trainer.rs:241-243,325-329); this one steps, clips, accumulates and measures for real while keeping
the reference's protocol: ``TrainerConfig`` fields, callback hook names, ``CallbackSignal.Stop``,
gradient accumulation every ``accumulation_steps`` batches and validation every
``validation_frequency`` epochs.
"""
from __future__ import annotations

import enum
import json
import math
import os
import shutil
import time
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple

import torch

from .._interop import FlagValue, FloatValue, IntValue, StrValue


# ----------------------------------------------------------------------- state
@dataclass
class BatchState:
    batch: int = 0
    loss: float = 0.0
    batch_size: int = 0
    duration_s: float = 0.0


@dataclass
class EpochState:
    epoch: int = 0
    train_loss: float = 0.0
    val_loss: Optional[float] = None
    metrics: Dict[str, float] = field(default_factory=dict)
    duration_s: float = 0.0
    batches: int = 0


@dataclass
class TrainingState:
    epoch: int = 0
    global_step: int = 0
    best_metric: Optional[float] = None
    history: List[EpochState] = field(default_factory=list)
    should_stop: bool = False
    start_time: float = field(default_factory=time.time)

    def elapsed(self) -> float:
        return time.time() - self.start_time


class CallbackSignal(enum.Enum):
    """What a callback asks the trainer to do after an epoch: go on or stop (src/training/callbacks.rs:12-30)."""

    CONTINUE = "continue"
    STOP = "stop"


# --------------------------------------------------------------------- metrics
class ConfusionMatrix:
    def __init__(self, num_classes: int):
        self.n = num_classes
        self.m = torch.zeros(num_classes, num_classes, dtype=torch.long)

    def update(self, pred: torch.Tensor, target: torch.Tensor) -> None:
        idx = target.reshape(-1).long().cpu() * self.n + pred.reshape(-1).long().cpu()
        self.m += torch.bincount(idx, minlength=self.n * self.n).view(self.n, self.n)

    def accuracy(self) -> float:
        t = int(self.m.sum())
        return float(self.m.diag().sum()) / t if t else 0.0

    def precision(self) -> torch.Tensor:
        return self.m.diag().float() / self.m.sum(0).clamp_min(1).float()

    def recall(self) -> torch.Tensor:
        return self.m.diag().float() / self.m.sum(1).clamp_min(1).float()

    def f1(self) -> torch.Tensor:
        p, r = self.precision(), self.recall()
        return 2 * p * r / (p + r).clamp_min(1e-12)


class MetricsCollector:
    """Running averages per epoch plus user metrics ``name -> fn(outputs, targets) -> float``."""

    def __init__(self, metric_fns: Optional[Dict[str, Callable]] = None):
        self.metric_fns = metric_fns or {}
        self.reset()
        self.epochs: List[Dict[str, float]] = []

    def reset(self) -> None:
        self._sum: Dict[str, float] = {}
        self._n = 0

    def update(self, loss: float, outputs=None, targets=None, batch_size: int = 1) -> None:
        self._sum["loss"] = self._sum.get("loss", 0.0) + loss * batch_size
        for name, fn in self.metric_fns.items():
            self._sum[name] = self._sum.get(name, 0.0) + float(fn(outputs, targets)) * batch_size
        self._n += batch_size

    def compute(self) -> Dict[str, float]:
        return {k: v / max(1, self._n) for k, v in self._sum.items()}

    def finalize_epoch(self, prefix: str = "") -> Dict[str, float]:
        out = {prefix + k: v for k, v in self.compute().items()}
        self.epochs.append(out)
        self.reset()
        return out

    def finalize(self, state: TrainingState) -> Dict[str, Any]:
        return {"epochs": len(state.history), "steps": state.global_step, "best_metric": state.best_metric,
                "elapsed_s": state.elapsed(), "history": [asdict(e) for e in state.history]}


def accuracy(outputs: torch.Tensor, targets: torch.Tensor) -> float:
    return float((outputs.argmax(-1) == targets).float().mean())


# ------------------------------------------------------------------- callbacks
class Callback:
    def on_train_begin(self, state: TrainingState) -> None: ...
    def on_train_end(self, state: TrainingState) -> None: ...
    def on_epoch_begin(self, state: TrainingState) -> None: ...
    def on_epoch_end(self, state: TrainingState, epoch: EpochState) -> Optional[CallbackSignal]: ...
    def on_batch_begin(self, state: TrainingState, batch: int) -> None: ...
    def on_batch_end(self, state: TrainingState, batch: BatchState) -> None: ...


class RegistryCallback(Callback):
    """Bridges a ``CallbackRegistry`` of named host functions into the training loop: ``"progress"(epoch, epochs,
    percent)`` after every epoch, ``"log"("info", text)`` with the epoch's losses, ``"completed"(epochs_run)`` at the end.
    A ``"progress"`` function that returns ``False`` stops training.  Entries that are not registered are skipped."""

    def __init__(self, registry, total_epochs: Optional[int] = None):
        self.registry, self.total_epochs = registry, total_epochs

    def on_epoch_end(self, state: TrainingState, epoch: EpochState) -> Optional[CallbackSignal]:
        total = int(self.total_epochs or max(epoch.epoch + 1, 1))
        val = "" if epoch.val_loss is None else f", val_loss {epoch.val_loss:.6f}"
        self.registry.call_if_registered("log", "info", f"epoch {epoch.epoch + 1}/{total}: train_loss {epoch.train_loss:.6f}{val}")
        go_on = self.registry.call_if_registered("progress", epoch.epoch + 1, total, 100.0 * (epoch.epoch + 1) / total)
        return CallbackSignal.STOP if go_on is False else None

    def on_train_end(self, state: TrainingState) -> None:
        self.registry.call_if_registered("completed", len(state.history))


class EarlyStopping(Callback):
    """``(monitor, patience, min_delta, mode_max)`` (callbacks.rs:89-109)."""

    def __init__(self, monitor: str = "val_loss", patience: int = 5, min_delta: float = 0.0, mode_max: bool = False):
        self.monitor, self.patience, self.min_delta, self.mode_max = monitor, patience, min_delta, mode_max
        self.best: Optional[float] = None
        self.wait = 0
        self.stopped_epoch: Optional[int] = None

    def _value(self, e: EpochState) -> Optional[float]:
        if self.monitor == "val_loss":
            return e.val_loss
        if self.monitor in ("loss", "train_loss"):
            return e.train_loss
        return e.metrics.get(self.monitor)

    def on_epoch_end(self, state, epoch):
        v = self._value(epoch)
        if v is None:
            return None
        better = self.best is None or (v > self.best + self.min_delta if self.mode_max else v < self.best - self.min_delta)
        if better:
            self.best, self.wait = v, 0
            return None
        self.wait += 1
        if self.wait >= self.patience:
            self.stopped_epoch = epoch.epoch
            return CallbackSignal.STOP
        return None


class LearningRateScheduler(Callback):
    """Steps an LR scheduler at each epoch end (``step_with_metric`` for plateau schedulers)."""

    def __init__(self, scheduler, monitor: str = "val_loss"):
        self.scheduler, self.monitor = scheduler, monitor

    def on_epoch_end(self, state, epoch):
        if hasattr(self.scheduler, "step_with_metric"):
            v = epoch.val_loss if self.monitor == "val_loss" else epoch.metrics.get(self.monitor, epoch.train_loss)
            self.scheduler.step_with_metric(epoch.train_loss if v is None else v)
        else:
            self.scheduler.step()
        return None


class ProgressBar(Callback):
    def __init__(self, log_frequency: int = 100, stream=None):
        self.log_frequency, self.stream = log_frequency, stream
        self.lines: List[str] = []

    def _emit(self, s: str) -> None:
        self.lines.append(s)
        if self.stream is not None:
            print(s, file=self.stream, flush=True)

    def on_batch_end(self, state, batch):
        if self.log_frequency and (batch.batch + 1) % self.log_frequency == 0:
            self._emit(f"epoch {state.epoch} batch {batch.batch + 1} loss {batch.loss:.4f}")

    def on_epoch_end(self, state, epoch):
        v = "" if epoch.val_loss is None else f" val_loss {epoch.val_loss:.4f}"
        self._emit(f"epoch {epoch.epoch} done: loss {epoch.train_loss:.4f}{v} ({epoch.duration_s:.2f}s)")
        return None


# ---------------------------------------------------------- checkpoint manager
@dataclass
class SaveConfig:
    directory: str = "checkpoints"
    max_to_keep: Optional[int] = 5
    monitor: str = "val_loss"
    mode_max: bool = False
    save_best_only: bool = False
    prefix: str = "checkpoint"


@dataclass
class CheckpointMetadata:
    name: str
    epoch: int
    step: int
    metrics: Dict[str, float]
    timestamp: float
    size_bytes: int = 0
    is_best: bool = False


class CheckpointManager:
    """Writes ``<name>.meta.json`` + ``<name>.bin`` per checkpoint, keeps the newest ``max_to_keep`` (never
    deleting the best one), and finds the latest / best (checkpoint.rs:206-246,291-340)."""

    def __init__(self, config: Optional[SaveConfig] = None):
        self.config = config or SaveConfig()
        os.makedirs(self.config.directory, exist_ok=True)
        self.checkpoints: List[CheckpointMetadata] = []
        self._load_index()

    def _paths(self, name: str) -> Tuple[str, str]:
        d = self.config.directory
        return os.path.join(d, name + ".meta.json"), os.path.join(d, name + ".bin")

    def _load_index(self) -> None:
        for f in sorted(os.listdir(self.config.directory)):
            if f.endswith(".meta.json"):
                with open(os.path.join(self.config.directory, f)) as fh:
                    self.checkpoints.append(CheckpointMetadata(**json.load(fh)))
        self.checkpoints.sort(key=lambda c: (c.step, c.timestamp))

    def _is_better(self, v: float, best: Optional[float]) -> bool:
        return best is None or (v > best if self.config.mode_max else v < best)

    def best_value(self) -> Optional[float]:
        vals = [c.metrics[self.config.monitor] for c in self.checkpoints if self.config.monitor in c.metrics]
        if not vals:
            return None
        return max(vals) if self.config.mode_max else min(vals)

    def save_checkpoint(self, epoch: int, step: int, metrics: Dict[str, float], data: bytes) -> Optional[CheckpointMetadata]:
        v = metrics.get(self.config.monitor)
        best = self.best_value()
        is_best = v is not None and self._is_better(v, best)
        if self.config.save_best_only and not is_best:
            return None
        name = f"{self.config.prefix}_epoch{epoch:04d}_step{step:08d}"
        meta_p, bin_p = self._paths(name)
        tmp = bin_p + ".tmp"
        with open(tmp, "wb") as f:
            f.write(data)
        os.replace(tmp, bin_p)                      # atomic: a crash never leaves a half-written checkpoint
        md = CheckpointMetadata(name, epoch, step, dict(metrics), time.time(), len(data), is_best)
        if is_best:
            for c in self.checkpoints:
                if c.is_best:
                    c.is_best = False
                    with open(self._paths(c.name)[0], "w") as f:
                        json.dump(asdict(c), f)
        with open(meta_p, "w") as f:
            json.dump(asdict(md), f)
        self.checkpoints.append(md)
        self._cleanup()
        return md

    def _cleanup(self) -> None:
        k = self.config.max_to_keep
        if k is None:
            return
        removable = [c for c in self.checkpoints if not c.is_best]
        excess = len(self.checkpoints) - k
        for c in removable[: max(0, excess)]:
            for p in self._paths(c.name):
                if os.path.exists(p):
                    os.remove(p)
            self.checkpoints.remove(c)

    def latest(self) -> Optional[CheckpointMetadata]:
        return self.checkpoints[-1] if self.checkpoints else None

    def best(self) -> Optional[CheckpointMetadata]:
        for c in self.checkpoints:
            if c.is_best:
                return c
        return None

    def load_checkpoint(self, md: Optional[CheckpointMetadata] = None) -> bytes:
        md = md or self.latest()
        if md is None:
            raise FileNotFoundError("no checkpoint available")
        with open(self._paths(md.name)[1], "rb") as f:
            return f.read()

    def list(self) -> List[CheckpointMetadata]:
        return list(self.checkpoints)


def pack_training_state(model: torch.nn.Module, optimizer=None, scheduler=None, extra: Optional[dict] = None) -> bytes:
    """Model + full optimizer state (moment buffers included) + scheduler as one ``torch.save`` blob."""
    import io
    buf = io.BytesIO()
    torch.save({"model": model.state_dict(),
                "optimizer": optimizer.state_dict() if optimizer is not None and hasattr(optimizer, "state_dict") else None,
                "scheduler": scheduler.state_dict() if scheduler is not None and hasattr(scheduler, "state_dict") else None,
                "extra": extra or {}}, buf)
    return buf.getvalue()


def unpack_training_state(data: bytes, model: torch.nn.Module, optimizer=None, scheduler=None) -> dict:
    import io
    sd = torch.load(io.BytesIO(data), map_location="cpu", weights_only=False)
    model.load_state_dict(sd["model"])
    if optimizer is not None and sd.get("optimizer") is not None:
        optimizer.load_state_dict(sd["optimizer"])
    if scheduler is not None and sd.get("scheduler") is not None:
        scheduler.load_state_dict(sd["scheduler"])
    return sd.get("extra", {})


class ModelCheckpoint(Callback):
    """``(filepath, monitor, mode_max, save_all)``: saves through a :class:`CheckpointManager` at epoch end
    (callbacks.rs:421-439)."""

    def __init__(self, filepath: str, monitor: str = "val_loss", mode_max: bool = False, save_all: bool = False,
                 max_to_keep: Optional[int] = 5):
        self.manager = CheckpointManager(SaveConfig(filepath, max_to_keep, monitor, mode_max, save_best_only=not save_all))
        self.model = self.optimizer = self.scheduler = None

    def bind(self, model, optimizer=None, scheduler=None) -> "ModelCheckpoint":
        self.model, self.optimizer, self.scheduler = model, optimizer, scheduler
        return self

    def on_epoch_end(self, state, epoch):
        if self.model is None:
            return None
        metrics = dict(epoch.metrics, train_loss=epoch.train_loss)
        if epoch.val_loss is not None:
            metrics["val_loss"] = epoch.val_loss
        if self.manager.config.monitor not in metrics:
            metrics[self.manager.config.monitor] = epoch.train_loss
        self.manager.save_checkpoint(epoch.epoch, state.global_step, metrics,
                                     pack_training_state(self.model, self.optimizer, self.scheduler,
                                                         {"epoch": epoch.epoch, "global_step": state.global_step}))
        return None


# --------------------------------------------------------------------- trainer
class TrainerConfig:
    """``epochs=10, log_frequency=100, validation_frequency=1, gradient_clip_value=None, device="cpu",
    use_mixed_precision=False, accumulation_steps=1`` (src/training/trainer.rs:19-48).  The Python binding's constructor
    also takes ``learning_rate`` and ``batch_size`` and reads ``epochs() / device() / use_mixed_precision()`` as calls
    with ``set_*`` mutators (src/python/training.rs:11-64); the members answer both spellings."""

    _FIELDS = ("epochs", "learning_rate", "batch_size", "log_frequency", "validation_frequency", "gradient_clip_value", "device",
               "use_mixed_precision", "accumulation_steps")

    def __init__(self, epochs: int = 10, log_frequency: int = 100, validation_frequency: int = 1,
                 gradient_clip_value: Optional[float] = None, device: str = "cpu", use_mixed_precision: bool = False,
                 accumulation_steps: int = 1, learning_rate: Optional[float] = None, batch_size: Optional[int] = None):
        if int(epochs) < 0 or int(accumulation_steps) < 1:
            raise ValueError("epochs must be >= 0 and accumulation_steps >= 1")
        self._v = dict(epochs=int(epochs), log_frequency=int(log_frequency), validation_frequency=int(validation_frequency),
                       gradient_clip_value=gradient_clip_value, device=str(device), use_mixed_precision=bool(use_mixed_precision),
                       accumulation_steps=int(accumulation_steps), learning_rate=learning_rate, batch_size=batch_size)

    def __getattr__(self, name):
        v = self.__dict__.get("_v", {})
        if name in v:
            x = v[name]
            if isinstance(x, bool):
                return FlagValue(x)
            if isinstance(x, int):
                return IntValue(x)
            if isinstance(x, float):
                return FloatValue(x)
            if isinstance(x, str):
                return StrValue(x)
            return x
        raise AttributeError(name)

    def __setattr__(self, name, value):
        if name in self._FIELDS:
            self._v[name] = value
        else:
            object.__setattr__(self, name, value)

    def set_epochs(self, epochs: int) -> None:
        self._v["epochs"] = int(epochs)

    def set_device(self, device: str) -> None:
        self._v["device"] = str(device)

    def set_mixed_precision(self, use_mixed_precision: bool) -> None:
        self._v["use_mixed_precision"] = bool(use_mixed_precision)

    def __eq__(self, other) -> bool:
        return isinstance(other, TrainerConfig) and self._v == other._v

    def __repr__(self) -> str:
        return f"TrainerConfig(epochs={self._v['epochs']}, device='{self._v['device']}', mixed_precision={self._v['use_mixed_precision']})"


class Trainer:
    def __init__(self, config: Optional[TrainerConfig] = None, callbacks: Optional[List[Callback]] = None,
                 metric_fns: Optional[Dict[str, Callable]] = None):
        self.config = config or TrainerConfig()
        if hasattr(callbacks, "call_if_registered"):                  # a CallbackRegistry in place of a list
            callbacks = [RegistryCallback(callbacks)]
        self.callbacks: List[Callback] = list(callbacks or [])
        self.metrics = MetricsCollector(metric_fns)
        self.state = TrainingState()

    def add_callback(self, cb: Callback) -> "Trainer":
        self.callbacks.append(cb)
        return self

    def _to_device(self, x):
        dev = torch.device(self.config.device)
        if isinstance(x, torch.Tensor):
            return x.to(dev, non_blocking=True)
        if isinstance(x, (list, tuple)):
            return type(x)(self._to_device(v) for v in x)
        return x

    def _autocast(self):
        dev = torch.device(self.config.device)
        return torch.autocast(dev.type, dtype=torch.bfloat16, enabled=bool(self.config.use_mixed_precision))

    def clip_gradients(self, model: torch.nn.Module) -> Optional[float]:
        c = self.config.gradient_clip_value
        if c is None:
            return None
        return float(torch.nn.utils.clip_grad_norm_([p for p in model.parameters() if p.grad is not None], c))

    def train_epoch(self, model, loader, loss_fn, optimizer) -> EpochState:
        cfg, st = self.config, self.state
        model.train()
        t0 = time.time()
        acc = max(1, cfg.accumulation_steps)
        n_batches = 0
        optimizer.zero_grad()
        for bi, batch in enumerate(loader):
            tb = time.time()
            for cb in self.callbacks:
                cb.on_batch_begin(st, bi)
            inputs, targets = self._to_device(batch[0]), self._to_device(batch[1])
            with self._autocast():
                outputs = model(inputs)
                loss = loss_fn(outputs, targets)
            (loss / acc).backward()
            if (bi + 1) % acc == 0:
                self.clip_gradients(model)
                optimizer.step()
                optimizer.zero_grad()
                st.global_step += 1
            lv = float(loss.detach())
            bs = inputs.shape[0] if isinstance(inputs, torch.Tensor) else 1
            self.metrics.update(lv, outputs.detach(), targets, bs)
            b_state = BatchState(bi, lv, bs, time.time() - tb)
            for cb in self.callbacks:
                cb.on_batch_end(st, b_state)
            n_batches += 1
        if n_batches % acc != 0:                     # flush a trailing partial accumulation window
            self.clip_gradients(model)
            optimizer.step()
            optimizer.zero_grad()
            st.global_step += 1
        m = self.metrics.finalize_epoch()
        return EpochState(st.epoch, m.pop("loss", float("nan")), None, m, time.time() - t0, n_batches)

    @torch.no_grad()
    def validate_epoch(self, model, loader, loss_fn) -> Dict[str, float]:
        model.eval()
        for batch in loader:
            inputs, targets = self._to_device(batch[0]), self._to_device(batch[1])
            with self._autocast():
                outputs = model(inputs)
                loss = loss_fn(outputs, targets)
            bs = inputs.shape[0] if isinstance(inputs, torch.Tensor) else 1
            self.metrics.update(float(loss), outputs, targets, bs)
        return self.metrics.finalize_epoch("val_")

    def _binding_form(self, model, third) -> bool:
        """``train(model, train_loader, val_loader=None)`` / ``evaluate(model, loader)`` of the Python binding
        (src/python/training.rs:131-200): the model was ``compile``d and carries its own loss and optimizer."""
        return hasattr(model, "_fit_loaders") and (third is None or hasattr(third, "next_batch")
                                                   or isinstance(third, torch.utils.data.DataLoader))

    def train(self, model, train_loader, loss_fn=None, optimizer=None, val_loader=None):
        """``train(model, train_loader, loss_fn, optimizer, val_loader=None)`` -> metrics dictionary
        (src/training/trainer.rs), or the binding's ``train(compiled_model, train_loader, val_loader=None)`` ->
        ``TrainingHistory`` (real training; the reference's binding reports placeholder losses)."""
        if optimizer is None and self._binding_form(model, loss_fn):
            model.to(torch.device(self.config.device))
            return model.fit(train_loader, loss_fn if loss_fn is not None else val_loader, epochs=int(self.config.epochs),
                             verbose=False)
        cfg, st = self.config, self.state
        model.to(torch.device(cfg.device))
        for cb in self.callbacks:
            if isinstance(cb, ModelCheckpoint) and cb.model is None:
                cb.bind(model, optimizer)
            if isinstance(cb, RegistryCallback) and cb.total_epochs is None:
                cb.total_epochs = int(cfg.epochs)
            cb.on_train_begin(st)
        for epoch in range(st.epoch, cfg.epochs):
            st.epoch = epoch
            for cb in self.callbacks:
                cb.on_epoch_begin(st)
            es = self.train_epoch(model, train_loader, loss_fn, optimizer)
            if val_loader is not None and (epoch + 1) % max(1, cfg.validation_frequency) == 0:
                v = self.validate_epoch(model, val_loader, loss_fn)
                es.val_loss = v.pop("val_loss", None)
                es.metrics.update(v)
            st.history.append(es)
            monitored = es.val_loss if es.val_loss is not None else es.train_loss
            if st.best_metric is None or monitored < st.best_metric:
                st.best_metric = monitored
            stop = False
            for cb in self.callbacks:
                if cb.on_epoch_end(st, es) is CallbackSignal.STOP:
                    stop = True
            if stop:
                st.should_stop = True
                break
        st.epoch = len(st.history)
        for cb in self.callbacks:
            cb.on_train_end(st)
        return self.metrics.finalize(st)

    def evaluate(self, model, loader, loss_fn=None) -> Dict[str, float]:
        if loss_fn is None and self._binding_form(model, None):
            return model.evaluate(loader)
        return self.validate_epoch(model, loader, loss_fn)

    def __repr__(self) -> str:
        return f"Trainer(epochs={int(self.config.epochs)}, device='{self.config.device}')"


class TrainerBuilder:
    def __init__(self):
        self._cfg = TrainerConfig()
        self._cbs: List[Callback] = []
        self._metrics: Dict[str, Callable] = {}

    def epochs(self, n: int):
        self._cfg.epochs = n
        return self

    def log_frequency(self, n: int):
        self._cfg.log_frequency = n
        return self

    def validation_frequency(self, n: int):
        self._cfg.validation_frequency = n
        return self

    def gradient_clip_value(self, v: float):
        self._cfg.gradient_clip_value = v
        return self

    def device(self, d: str):
        self._cfg.device = d
        return self

    def use_mixed_precision(self, on: bool = True):
        self._cfg.use_mixed_precision = on
        return self

    def accumulation_steps(self, n: int):
        self._cfg.accumulation_steps = n
        return self

    def callback(self, cb: Callback):
        self._cbs.append(cb)
        return self

    def metric(self, name: str, fn: Callable):
        self._metrics[name] = fn
        return self

    def build(self) -> Trainer:
        return Trainer(self._cfg, self._cbs, self._metrics)


def __getattr__(name: str):
    """``training.sharded`` members (sharded checkpoints, ``AsyncCheckpointer``) load on first use."""
    if name in ("ShardSpec", "save_sharded", "merge_sharded", "load_sharded", "infer_spec", "shard_tensor", "merge_tensors", "AsyncCheckpointer"):
        from . import sharded
        return getattr(sharded, name)
    raise AttributeError(name)
