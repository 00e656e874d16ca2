"""The reference's ``hybrid_f32`` universe (src/hybrid_f32: tensor/core.rs, autograd, nn.rs:16-5060, trainer, memory).

There it is a second, f32-only tensor / autograd / layer stack that routes each op to Metal, CoreML or the CPU.  Here
the routing target is the B200 (large ops) or the host (tiny ones, where a launch costs more than the math), the
tensors are ordinary fp32 torch tensors, and the layers are this framework's layers built in fp32; the trainer keeps
the reference's features (early stopping, checkpoints, mixed precision, LR schedulers, history).
"""
from __future__ import annotations

import copy
import os
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from .nn import layers as L
from .nn import rnn as R


class F32Device:
    """Device names of the fp32 universe; only ``cpu`` / ``cuda`` / ``auto`` route anywhere here (src/hybrid_f32/mod.rs)."""

    CPU, GPU, AUTO = "cpu", "cuda", "auto"


def _route(numel: int, preferred: str = F32Device.AUTO, threshold: int = 1 << 14) -> torch.device:
    """Small tensors stay on the host; everything else goes to the GPU when there is one."""
    if preferred == F32Device.CPU or not torch.cuda.is_available():
        return torch.device("cpu")
    if preferred == F32Device.GPU or numel >= threshold:
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


class F32Tensor:
    """fp32 tensor with the reference's constructors and a device hint."""

    def __init__(self, data, shape: Optional[Sequence[int]] = None, device: str = F32Device.AUTO):
        t = data if isinstance(data, torch.Tensor) else torch.as_tensor(data, dtype=torch.float32)
        t = t.to(torch.float32)
        if shape is not None:
            t = t.reshape(*shape)
        self.data = t.to(_route(t.numel(), device))

    @classmethod
    def zeros(cls, shape: Sequence[int], device: str = F32Device.AUTO) -> "F32Tensor":
        return cls(torch.zeros(*shape), device=device)

    @classmethod
    def ones(cls, shape: Sequence[int], device: str = F32Device.AUTO) -> "F32Tensor":
        return cls(torch.ones(*shape), device=device)

    @classmethod
    def randn(cls, shape: Sequence[int], device: str = F32Device.AUTO) -> "F32Tensor":
        return cls(torch.randn(*shape), device=device)

    @classmethod
    def from_vec(cls, values: Sequence[float], shape: Sequence[int]) -> "F32Tensor":
        return cls(list(values), shape)

    def shape(self) -> Tuple[int, ...]:
        return tuple(self.data.shape)

    def numel(self) -> int:
        return self.data.numel()

    def to_vec(self) -> List[float]:
        return self.data.reshape(-1).cpu().tolist()

    def _other(self, o) -> torch.Tensor:
        return (o.data if isinstance(o, F32Tensor) else torch.as_tensor(o, dtype=torch.float32)).to(self.data.device)

    def __add__(self, o): return F32Tensor(self.data + self._other(o))
    def __sub__(self, o): return F32Tensor(self.data - self._other(o))
    def __mul__(self, o): return F32Tensor(self.data * self._other(o))
    def __truediv__(self, o): return F32Tensor(self.data / self._other(o))
    def __neg__(self): return F32Tensor(-self.data)

    def matmul(self, o) -> "F32Tensor":
        return F32Tensor(self.data @ self._other(o))

    __matmul__ = matmul

    def transpose(self) -> "F32Tensor":
        return F32Tensor(self.data.transpose(-2, -1).contiguous())

    def sum(self) -> float:
        return float(self.data.sum())

    def mean(self) -> float:
        return float(self.data.mean())

    def relu(self) -> "F32Tensor":
        return F32Tensor(L.relu(self.data))

    def sigmoid(self) -> "F32Tensor":
        return F32Tensor(L.sigmoid(self.data))

    def softmax(self, dim: int = -1) -> "F32Tensor":
        return F32Tensor(L.softmax(self.data, dim))

    def reshape(self, shape: Sequence[int]) -> "F32Tensor":
        return F32Tensor(self.data.reshape(*shape))

    def __repr__(self) -> str:
        return f"F32Tensor(shape={self.shape()}, device={self.data.device})"


class F32Variable:
    """Autograd node: ``F32Variable(t, requires_grad=True)``, ``backward()``, ``grad()``, ``zero_grad()``."""

    def __init__(self, data, requires_grad: bool = False):
        t = data.data if isinstance(data, (F32Tensor, F32Variable)) else torch.as_tensor(data, dtype=torch.float32)
        self.data = t.detach().clone().requires_grad_(requires_grad) if not (isinstance(data, F32Variable)) else data.data

    @classmethod
    def _wrap(cls, t: torch.Tensor) -> "F32Variable":
        v = cls.__new__(cls)
        v.data = t
        return v

    def _o(self, o):
        return o.data if isinstance(o, (F32Variable, F32Tensor)) else o

    def __add__(self, o): return F32Variable._wrap(self.data + self._o(o))
    def __sub__(self, o): return F32Variable._wrap(self.data - self._o(o))
    def __mul__(self, o): return F32Variable._wrap(self.data * self._o(o))
    def matmul(self, o): return F32Variable._wrap(self.data @ self._o(o))
    __matmul__ = matmul
    def relu(self): return F32Variable._wrap(L.relu(self.data))
    def sum(self): return F32Variable._wrap(self.data.sum())
    def mean(self): return F32Variable._wrap(self.data.mean())
    def pow(self, p: float): return F32Variable._wrap(self.data.pow(p))

    def backward(self) -> None:
        self.data.backward()

    def grad(self) -> Optional[F32Tensor]:
        return None if self.data.grad is None else F32Tensor(self.data.grad)

    def zero_grad(self) -> None:
        self.data.grad = None

    def requires_grad(self) -> bool:
        return self.data.requires_grad

    def value(self) -> F32Tensor:
        return F32Tensor(self.data.detach())


def _f32(cls):
    """The framework layer of the same name, parameters in fp32."""
    def make(*a, **k):
        return cls(*a, **k).float()
    make.__name__ = "F32" + cls.__name__
    make.__doc__ = f"``{cls.__name__}`` built in fp32 (src/hybrid_f32/nn.rs)."
    return make


F32Linear = _f32(L.Linear)
F32Conv1d = _f32(L.Conv1d)
F32Conv2d = _f32(L.Conv2d)
F32Conv3d = _f32(L.Conv3d)
F32BatchNorm2d = _f32(L.BatchNorm2d)
F32Dropout = _f32(L.Dropout)
F32RNN = _f32(R.RNN)
F32LSTM = _f32(R.LSTM)
F32GRU = _f32(R.GRU)
F32MultiHeadAttention = _f32(nn.MultiheadAttention)
F32Transformer = _f32(nn.Transformer)


@dataclass
class F32TrainerConfig:
    epochs: int = 10
    learning_rate: float = 1e-3
    early_stopping_patience: int = 0          # 0: off
    min_delta: float = 0.0
    checkpoint_dir: Optional[str] = None
    checkpoint_every: int = 0                 # epochs; 0: only the best model
    mixed_precision: bool = False
    grad_clip: float = 0.0
    scheduler: Optional[str] = None           # "step", "cosine", "plateau"
    scheduler_step: int = 10
    scheduler_gamma: float = 0.1


class F32Trainer:
    """Training loop with early stopping, checkpoints, mixed precision and LR schedules."""

    def __init__(self, model: nn.Module, loss_fn: Callable, config: Optional[F32TrainerConfig] = None,
                 optimizer: Optional[torch.optim.Optimizer] = None, device: Optional[str] = None):
        self.cfg = config or F32TrainerConfig()
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.model, self.loss_fn = model.to(self.device), loss_fn
        self.opt = optimizer or torch.optim.Adam(model.parameters(), lr=self.cfg.learning_rate)
        c = self.cfg
        self.sched = None
        if c.scheduler == "step":
            self.sched = torch.optim.lr_scheduler.StepLR(self.opt, c.scheduler_step, c.scheduler_gamma)
        elif c.scheduler == "cosine":
            self.sched = torch.optim.lr_scheduler.CosineAnnealingLR(self.opt, c.epochs)
        elif c.scheduler == "plateau":
            self.sched = torch.optim.lr_scheduler.ReduceLROnPlateau(self.opt, factor=c.scheduler_gamma, patience=max(1, c.scheduler_step))
        self.history: Dict[str, List[float]] = {"train_loss": [], "val_loss": [], "lr": [], "epoch_s": []}
        self.best_loss, self.best_state, self.stopped_epoch = float("inf"), None, None

    def _run(self, batches: Iterable, train: bool) -> float:
        self.model.train(train)
        total, n = 0.0, 0
        amp = self.cfg.mixed_precision and self.device.type == "cuda"
        for x, y in batches:
            x, y = x.to(self.device), y.to(self.device)
            with torch.set_grad_enabled(train), torch.autocast(self.device.type, dtype=torch.bfloat16, enabled=amp):
                loss = self.loss_fn(self.model(x), y)
            if train:
                self.opt.zero_grad(set_to_none=True)
                loss.backward()
                if self.cfg.grad_clip > 0:
                    torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.cfg.grad_clip)
                self.opt.step()
            total += float(loss.detach()) * x.shape[0]
            n += x.shape[0]
        return total / max(1, n)

    def save_checkpoint(self, path: str, epoch: int) -> None:
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        torch.save({"epoch": epoch, "model": self.model.state_dict(), "optimizer": self.opt.state_dict(), "history": self.history,
                    "best_loss": self.best_loss}, path)

    def load_checkpoint(self, path: str) -> int:
        ck = torch.load(path, map_location=self.device, weights_only=False)
        self.model.load_state_dict(ck["model"])
        self.opt.load_state_dict(ck["optimizer"])
        self.history, self.best_loss = ck["history"], ck["best_loss"]
        return int(ck["epoch"])

    def fit(self, train_batches, val_batches=None) -> Dict[str, List[float]]:
        c, bad = self.cfg, 0
        for epoch in range(c.epochs):
            t0 = time.perf_counter()
            tl = self._run(train_batches, True)
            vl = self._run(val_batches, False) if val_batches is not None else tl
            self.history["train_loss"].append(tl); self.history["val_loss"].append(vl)
            self.history["lr"].append(self.opt.param_groups[0]["lr"]); self.history["epoch_s"].append(time.perf_counter() - t0)
            if self.sched is not None:
                self.sched.step(vl) if isinstance(self.sched, torch.optim.lr_scheduler.ReduceLROnPlateau) else self.sched.step()
            if vl < self.best_loss - c.min_delta:
                self.best_loss, bad = vl, 0
                self.best_state = copy.deepcopy(self.model.state_dict())
                if c.checkpoint_dir:
                    self.save_checkpoint(os.path.join(c.checkpoint_dir, "best.pt"), epoch)
            else:
                bad += 1
            if c.checkpoint_dir and c.checkpoint_every and (epoch + 1) % c.checkpoint_every == 0:
                self.save_checkpoint(os.path.join(c.checkpoint_dir, f"epoch_{epoch + 1}.pt"), epoch)
            if c.early_stopping_patience and bad >= c.early_stopping_patience:
                self.stopped_epoch = epoch
                break
        if self.best_state is not None:
            self.model.load_state_dict(self.best_state)
        return self.history
