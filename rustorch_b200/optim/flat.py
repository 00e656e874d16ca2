"""Flat parameter storage + fused optimizers for the bf16 training path.

``FlatParams`` re-homes a module's parameters into one contiguous bf16 buffer (the compute
copy the kernels read) and keeps, in matching layout, fp32 master weights, an fp32 gradient
buffer and the optimizer moments.  Every parameter gains a ``main_grad`` fp32 view that the
wgrad GEMM / norm / embedding backward kernels accumulate into directly.  ``FusedAdamW`` and
``FusedSGD`` then update everything with one kernel launch per decay group (the kernel also
refreshes the bf16 copy and zeroes the gradient).

Reference semantics: AdamW defaults (0.9, 0.999, 1e-8, 0.01) and decoupled decay
(src/optim/adamw.rs:66-68,159-163); SGD momentum/dampening/nesterov (src/optim/mod.rs:82-214).
Unlike the reference (src/optim/mod.rs:301) the bias-correction step counts optimizer steps,
not parameter tensors, and the moments are part of ``state_dict`` (the reference drops them,
src/optim/mod.rs:369-379).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch

from ..ops import kernels as K

_ALIGN = 64  # elements; keeps every parameter view 128-byte aligned in bf16 (TMA needs 16)


def default_decay_filter(name: str, p: torch.Tensor) -> bool:
    """Weight decay on matrices / embeddings, none on biases and norm scales."""
    return p.dim() >= 2


def _is_channels_last(t: torch.Tensor) -> bool:
    return t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last) and not t.is_contiguous()


class FlatParams:
    def __init__(self, module: torch.nn.Module, decay_filter: Callable = default_decay_filter,
                 alloc: Optional[Callable] = None, alloc_f32: Optional[Callable] = None,
                 group_align: int = _ALIGN):
        """``alloc(n)`` / ``alloc_f32(n)`` let a caller place the bf16 parameter buffer and the fp32
        gradient buffer in special memory (e.g. symmetric memory visible to peer GPUs);
        ``group_align`` pads the decay / no-decay groups to a multiple of that many elements."""
        named = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
        seen, uniq = set(), []
        for n, p in named:
            if id(p) not in seen:
                seen.add(id(p))
                uniq.append((n, p))
        decay = [(n, p) for n, p in uniq if decay_filter(n, p)]
        nodecay = [(n, p) for n, p in uniq if not decay_filter(n, p)]
        self.entries: List[Tuple[str, torch.nn.Parameter, int, int]] = []
        off = 0
        for n, p in decay:
            self.entries.append((n, p, off, p.numel()))
            off += -(-p.numel() // _ALIGN) * _ALIGN
        off = -(-off // group_align) * group_align
        self.n_decay = off
        for n, p in nodecay:
            self.entries.append((n, p, off, p.numel()))
            off += -(-p.numel() // _ALIGN) * _ALIGN
        off = -(-off // group_align) * group_align
        self.numel = off
        dev = uniq[0][1].device if uniq else torch.device("cpu")
        self.device = dev
        lp_dtype = uniq[0][1].dtype if uniq else torch.bfloat16
        self.lp_dtype = lp_dtype
        alloc = alloc or (lambda n: torch.zeros(n, dtype=lp_dtype, device=dev))
        alloc_f32 = alloc_f32 or (lambda n: torch.zeros(n, dtype=torch.float32, device=dev))
        self.lp = alloc(off)
        self.master = torch.zeros(off, dtype=torch.float32, device=dev)
        self.grad = alloc_f32(off)
        with torch.no_grad():
            for n, p, o, k in self.entries:
                src = getattr(p, "_fp32_init", None)
                base = src if src is not None else p.data
                # channels-last 4-D parameters (conv filters) keep their physical [Cout, KH, KW, Cin] order in the flat
                # buffers, so the conv kernels read them without a copy and accumulate dW straight into ``main_grad``
                cl = _is_channels_last(p.data)
                self.master[o:o + k].copy_((base.permute(0, 2, 3, 1) if cl else base).reshape(-1).float())
                if src is not None:
                    del p._fp32_init
                self.lp[o:o + k].copy_(self.master[o:o + k])
                if cl:
                    co, ci, kh, kw = p.shape
                    p.data = self.lp[o:o + k].view(co, kh, kw, ci).permute(0, 3, 1, 2)
                else:
                    p.data = self.lp[o:o + k].view(p.shape)
                p._flat_ohwi = cl
                p.main_grad = self.grad[o:o + k]
                p.grad = None

    def collect_autograd_grads(self) -> int:
        """Fold ``p.grad`` tensors written by ordinary autograd (modules that do not accumulate into ``main_grad``
        themselves) into the flat fp32 gradient buffer and drop them.  Returns how many were folded."""
        n = 0
        for _, p, o, k in self.entries:
            if p.grad is not None:
                g = p.grad.permute(0, 2, 3, 1) if getattr(p, "_flat_ohwi", False) else p.grad
                self.grad[o:o + k].add_(g.reshape(-1))
                p.grad = None
                n += 1
        return n

    def groups(self) -> List[Tuple[int, int, bool]]:
        """[(start, stop, decays)] contiguous ranges."""
        out = []
        if self.n_decay:
            out.append((0, self.n_decay, True))
        if self.numel > self.n_decay:
            out.append((self.n_decay, self.numel, False))
        return out

    def zero_grad(self):
        self.grad.zero_()

    def grad_norm(self) -> torch.Tensor:
        if self.grad.is_cuda:
            return K.reduce_all(self.grad, "sumsq").sqrt()
        return self.grad.norm().reshape(1)

    def named_views(self, buf: torch.Tensor) -> Dict[str, torch.Tensor]:
        def view(p, t):
            if getattr(p, "_flat_ohwi", False):
                co, ci, kh, kw = p.shape
                return t.view(co, kh, kw, ci).permute(0, 3, 1, 2)
            return t.view(p.shape)
        return {n: view(p, buf[o:o + k]) for n, p, o, k in self.entries}


class _FusedBase:
    def __init__(self, flat: FlatParams, lr: float):
        self.flat = flat
        self.lr = float(lr)
        self.step_count = 0
        self.grad_scale = 1.0

    # reference API names (src/optim/mod.rs:60-78)
    def learning_rate(self) -> float:
        return self.lr

    def set_learning_rate(self, lr: float) -> None:
        self.lr = float(lr)

    set_lr = set_learning_rate

    def zero_grad(self, set_to_none: bool = False) -> None:
        self.flat.zero_grad()

    @property
    def param_groups(self):
        return [{"lr": self.lr, "params": [p for _, p, _, _ in self.flat.entries]}]


class FusedAdamW(_FusedBase):
    """AdamW (``decoupled=True``) or Adam with L2 decay over a :class:`FlatParams`."""

    def __init__(self, flat: FlatParams, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, decoupled: bool = True):
        super().__init__(flat, lr)
        self.betas = (float(betas[0]), float(betas[1]))
        self.eps = float(eps)
        self.weight_decay = float(weight_decay)
        self.decoupled = decoupled
        self.m = torch.zeros_like(flat.master)
        self.v = torch.zeros_like(flat.master)

    def step(self, clip_grad_norm: Optional[float] = None) -> None:
        f = self.flat
        f.collect_autograd_grads()
        self.step_count += 1
        b1, b2 = self.betas
        bc1 = 1.0 - b1 ** self.step_count
        bc2 = 1.0 - b2 ** self.step_count
        scale = self.grad_scale
        if clip_grad_norm is not None:
            norm = float(f.grad_norm()) * scale
            if norm > clip_grad_norm:
                scale *= clip_grad_norm / (norm + 1e-6)
        for start, stop, decays in f.groups():
            wd = self.weight_decay if decays else 0.0
            if f.master.is_cuda:
                K.fused_optim_step(
                    f.master[start:stop], f.grad[start:stop], self.m[start:stop], self.v[start:stop],
                    f.lp[start:stop] if f.lp_dtype == torch.bfloat16 else None,
                    mode=K.OPT_ADAMW if self.decoupled else K.OPT_ADAM, lr=self.lr, beta1=b1,
                    beta2=b2, eps=self.eps, weight_decay=wd, bias_corr1=bc1, bias_corr2=bc2,
                    grad_scale=scale, zero_grad=True)
                if f.lp_dtype != torch.bfloat16:
                    f.lp[start:stop].copy_(f.master[start:stop])
            else:
                self._step_reference(start, stop, wd, bc1, bc2, scale)

    def _step_reference(self, start, stop, wd, bc1, bc2, scale):
        f = self.flat
        b1, b2 = self.betas
        p, g = f.master[start:stop], f.grad[start:stop] * scale
        m, v = self.m[start:stop], self.v[start:stop]
        if not self.decoupled:
            g = g + wd * p
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        if self.decoupled:
            p.mul_(1 - self.lr * wd)
        p.addcdiv_(m / bc1, (v / bc2).sqrt() + self.eps, value=-self.lr)
        f.lp[start:stop].copy_(p)
        f.grad[start:stop].zero_()

    def state_dict(self) -> dict:
        return {"lr": self.lr, "betas": self.betas, "eps": self.eps, "weight_decay": self.weight_decay,
                "step": self.step_count, "master": self.flat.master.clone(), "exp_avg": self.m.clone(),
                "exp_avg_sq": self.v.clone()}

    def load_state_dict(self, sd: dict) -> None:
        self.lr, self.betas, self.eps = sd["lr"], tuple(sd["betas"]), sd["eps"]
        self.weight_decay, self.step_count = sd["weight_decay"], sd["step"]
        self.flat.master.copy_(sd["master"])
        self.flat.lp.copy_(self.flat.master)
        self.m.copy_(sd["exp_avg"])
        self.v.copy_(sd["exp_avg_sq"])


class FusedSGD(_FusedBase):
    """SGD with momentum / dampening / nesterov / L2 weight decay over a :class:`FlatParams`."""

    def __init__(self, flat: FlatParams, lr: float, momentum: float = 0.0, dampening: float = 0.0,
                 weight_decay: float = 0.0, nesterov: bool = False, decay_all: bool = True):
        super().__init__(flat, lr)
        self.momentum, self.dampening = float(momentum), float(dampening)
        self.weight_decay, self.nesterov = float(weight_decay), nesterov
        self.decay_all = decay_all
        self.buf = torch.zeros_like(flat.master) if momentum != 0.0 else None

    def step(self) -> None:
        f = self.flat
        f.collect_autograd_grads()
        self.step_count += 1
        first = self.step_count == 1
        for start, stop, decays in f.groups():
            wd = self.weight_decay if (decays or self.decay_all) else 0.0
            if f.master.is_cuda:
                K.fused_optim_step(
                    f.master[start:stop], f.grad[start:stop],
                    self.buf[start:stop] if self.buf is not None else None, None,
                    f.lp[start:stop] if f.lp_dtype == torch.bfloat16 else None, mode=K.OPT_SGD,
                    lr=self.lr, beta1=self.momentum, beta2=self.dampening, weight_decay=wd,
                    grad_scale=self.grad_scale, zero_grad=True, nesterov=self.nesterov,
                    first_step=first)
                if f.lp_dtype != torch.bfloat16:
                    f.lp[start:stop].copy_(f.master[start:stop])
            else:
                p = f.master[start:stop]
                g = f.grad[start:stop] * self.grad_scale + wd * p
                d = g
                if self.buf is not None:
                    b = self.buf[start:stop]
                    if first:
                        b.copy_(g)
                    else:
                        b.mul_(self.momentum).add_(g, alpha=1 - self.dampening)
                    d = g + self.momentum * b if self.nesterov else b
                p.add_(d, alpha=-self.lr)
                f.lp[start:stop].copy_(p)
                f.grad[start:stop].zero_()

    def state_dict(self) -> dict:
        return {"lr": self.lr, "momentum": self.momentum, "step": self.step_count,
                "master": self.flat.master.clone(),
                "momentum_buffer": None if self.buf is None else self.buf.clone()}

    def load_state_dict(self, sd: dict) -> None:
        self.lr, self.momentum, self.step_count = sd["lr"], sd["momentum"], sd["step"]
        self.flat.master.copy_(sd["master"])
        self.flat.lp.copy_(self.flat.master)
        if self.buf is not None and sd.get("momentum_buffer") is not None:
            self.buf.copy_(sd["momentum_buffer"])
