"""Data-parallel training step fused into one peer-memory kernel per gradient bucket.

``FusedDDP`` (``optimizer="adamw" | "adam" | "sgd"``; ``FusedDDPAdamW`` / ``FusedDDPSGD`` are the named
variants) wraps a model whose parameters live in a :class:`FlatParams`:

* the bf16 parameter buffer, the fp32 gradient buffer and a small flag array are *symmetric*
  allocations (``torch.distributed._symmetric_memory``), so every rank holds device pointers
  to every peer's copy over NVLink;
* the gradient buffer is cut into buckets of ``bucket_cap_mb`` (25 MB, the reference's default,
  src/distributed/ddp.rs:86-131); inside a bucket rank ``r`` owns the ``r``-th 1/N slice;
* when the backward pass has finished the last gradient of a bucket (the fused autograd
  Functions report it through ``fused.grad_ready_hook``) the bucket's kernel is queued on a side
  stream: it reduces the owned slice across all ranks, zeroes the gradients, applies scale + the
  optimizer rule to the fp32 master weights / moments and stores the new bf16 parameters into every
  rank's parameter buffer (csrc/collective/ddp_fused.cu).  Where the symmetric allocation also has a
  multicast (NVLS) mapping the reduction is one ``multimem.ld_reduce`` per 16 bytes (the NVSwitch adds
  the ranks' values) and the zero / parameter stores are one ``multimem.st`` each (default from four ranks
  up); otherwise plain peer loads and stores (``RUSTORCH_DDP_NVLS=0`` / ``1`` forces either).  Backward keeps
  running underneath;
* ``step()`` queues whatever is left, waits for the peers' end signals and joins the streams.

With one rank the same kernel runs without flags (a fused AdamW over the buckets).

Parameters used more than once per backward (tied weights) must say so through a
``_grad_contribs`` attribute (number of backward Functions that accumulate into them); the GPT
model does this itself.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native
from ..nn import fused
from ..optim.flat import FlatParams, default_decay_filter


def _symm_empty(numel: int, dtype: torch.dtype, device: torch.device, group) -> Tuple[torch.Tensor, List[int], object]:
    """Allocate a zeroed symmetric tensor and return (tensor, peer pointers, handle)."""
    import torch.distributed._symmetric_memory as symm

    t = symm.empty(numel, dtype=dtype, device=device)
    t.zero_()
    name = group.group_name if hasattr(group, "group_name") else group
    try:
        hdl = symm.rendezvous(t, name)
    except Exception:  # older signature wants the group registered first
        symm.enable_symm_mem_for_group(name)
        hdl = symm.rendezvous(t, name)
    ptrs = [int(p) for p in hdl.buffer_ptrs]
    return t, ptrs, hdl


def _multicast_ptr(hdl) -> int:
    """Device address of the multicast (NVLS) mapping of a symmetric allocation, 0 when there is none."""
    try:
        return int(getattr(hdl, "multicast_ptr", 0) or 0)
    except Exception:
        return 0


_OPT_MODES = {"adamw": 0, "adam": 1, "sgd": 2}


class FusedDDP:
    """Data-parallel wrapper + optimizer in one object; see the module docstring.

    ``optimizer``: ``"adamw"`` (decoupled decay), ``"adam"`` (L2 decay in the gradient) or ``"sgd"``
    (``momentum`` / ``dampening`` / ``nesterov`` / L2 decay, src/optim/mod.rs:82-214).  ``decay_all`` applies the
    weight decay to biases and norm scales too (the usual SGD recipe for ResNets).  ``n_ctas = 0`` launches two
    CTAs per SM of the device.  ``timeout_s`` bounds every cross-rank flag wait inside the kernels.
    """

    def __init__(self, module: torch.nn.Module, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, bucket_cap_mb: float = 25.0, process_group=None,
                 decay_filter=default_decay_filter, n_ctas: int = 0, timeout_s: float = 10.0,
                 overlap: bool = True, optimizer: str = "adamw", momentum: float = 0.0, dampening: float = 0.0,
                 nesterov: bool = False, decay_all: bool = False, use_nvls: Optional[bool] = None):
        assert optimizer in _OPT_MODES, f"optimizer must be one of {sorted(_OPT_MODES)}"
        self.module = module
        self.optimizer = optimizer
        self.opt_mode = _OPT_MODES[optimizer]
        self.momentum, self.dampening, self.nesterov, self.decay_all = float(momentum), float(dampening), bool(nesterov), bool(decay_all)
        self.lr, self.betas, self.eps, self.weight_decay = float(lr), (float(betas[0]), float(betas[1])), float(eps), float(weight_decay)
        self.n_ctas, self.timeout_s, self.overlap = int(n_ctas), float(timeout_s), overlap
        self.step_count = 0
        self.grad_scale = 1.0
        if dist.is_initialized():
            self.group = process_group or dist.group.WORLD
            self.world = dist.get_world_size(self.group)
            self.rank = dist.get_rank(self.group)
        else:
            self.group, self.world, self.rank = None, 1, 0
        dev = next(module.parameters()).device
        self.device = dev
        self._handles = []
        W = self.world
        ptrs: Dict[str, List[int]] = {}
        mc: Dict[str, int] = {}
        # Host emulation (CPU tensors, gloo): same ownership and state layout, the bucket step is an all-reduce, the
        # update of the owned slice and an all-gather of the new parameters.  Used to test checkpoint logic.
        self.host = dev.type != "cuda"

        def alloc(kind, dtype):
            def _a(n):
                if W == 1 or self.host:
                    t = torch.zeros(n, dtype=dtype, device=dev)
                    ptrs[kind] = [t.data_ptr()]
                    return t
                t, pp, h = _symm_empty(n, dtype, dev, self.group)
                self._handles.append(h)
                ptrs[kind] = pp
                mc[kind] = _multicast_ptr(h)
                return t
            return _a

        lp_dtype = next(module.parameters()).dtype
        assert lp_dtype == torch.bfloat16, "FusedDDP needs bf16 parameters"
        self.flat = FlatParams(module, decay_filter=decay_filter, alloc=alloc("lp", torch.bfloat16),
                               alloc_f32=alloc("grad", torch.float32), group_align=64 * W)
        f = self.flat
        if W > 1:
            # identical starting point on every rank
            dist.broadcast(f.master, 0, group=self.group)
            f.lp.copy_(f.master)
        if self.opt_mode == 2:
            self.m = torch.zeros_like(f.master) if self.momentum != 0.0 else None
            self.v = None
        else:
            self.m = torch.zeros_like(f.master)
            self.v = torch.zeros_like(f.master)
        self.lp_ptrs, self.grad_ptrs = ptrs["lp"], ptrs["grad"]
        if use_nvls is None:
            # auto: through the switch from four ranks up (one multimem load replaces N - 1 peer loads); with two
            # ranks the single peer load is faster (22.0 vs 21.2 ms per GPT-2 step).  RUSTORCH_DDP_NVLS=0 / 1 forces it.
            env = os.environ.get("RUSTORCH_DDP_NVLS", "auto")
            use_nvls = W >= 4 if env == "auto" else env != "0"
        self.mc_grad, self.mc_lp = (mc.get("grad", 0), mc.get("lp", 0)) if (use_nvls and W > 1) else (0, 0)
        if W > 1 and not self.host:  # every rank must take the same path: the multicast stores also zero / refresh the peers' buffers
            have = torch.tensor([1 if (self.mc_grad and self.mc_lp) else 0], device=dev, dtype=torch.int32)
            dist.all_reduce(have, op=dist.ReduceOp.MIN, group=self.group)
            if int(have.item()) == 0:
                self.mc_grad = self.mc_lp = 0
        self.nvls = bool(self.mc_grad and self.mc_lp)

        # ---- buckets: never straddle the decay / no-decay boundary; length divisible by 4*W
        per = max(64 * W, int(bucket_cap_mb * 1024 * 1024 / 4) // (64 * W) * (64 * W))
        self.buckets: List[Tuple[int, int, bool]] = []
        for start, stop, decays in f.groups():
            s = start
            while s < stop:
                e = min(stop, s + per)
                self.buckets.append((s, e, decays))
                s = e
        nb = len(self.buckets)
        self.n_buckets = nb
        n_flags = max(64, 2 * nb * W)
        if W == 1 or self.host:
            self.flags = torch.zeros(n_flags, dtype=torch.int32, device=dev)
            self.flag_ptrs = [self.flags.data_ptr()]
        else:
            self.flags, self.flag_ptrs, h = _symm_empty(n_flags, torch.int32, dev, self.group)
            self._handles.append(h)
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=dev)

        # ---- readiness bookkeeping
        self._param_buckets: Dict[int, List[int]] = {}
        self._bucket_need = [0] * nb
        for name, p, off, n in f.entries:
            contribs = int(getattr(p, "_grad_contribs", 1))
            hit = [i for i, (s, e, _) in enumerate(self.buckets) if off < e and off + n > s]
            self._param_buckets[id(p)] = hit
            p._ddp_contribs = contribs
            for i in hit:
                self._bucket_need[i] += contribs
        self._pending = list(self._bucket_need)
        self._launched = [False] * nb
        self._comm = None if self.host else torch.cuda.Stream(device=dev, priority=-1)
        self._in_step = False
        fused.grad_ready_hook = self._on_grads_ready
        # Parameters of ordinary autograd modules (convolutions, BatchNorm, ...) get their gradient in ``.grad``: a
        # post-accumulate hook folds it into the flat fp32 buffer at once and reports the parameter as ready, so their
        # buckets overlap with the rest of backward too.  Parameters of the fused Functions never see the hook fire.
        self._ag_hooks = [p.register_post_accumulate_grad_hook(self._on_autograd_grad) for _, p, _, _ in f.entries]
        self._entry_of = {id(p): (o, n) for _, p, o, n in f.entries}
        if W > 1:
            dist.barrier(group=self.group)
        if not self.host:
            torch.cuda.synchronize(dev)

    # ------------------------------------------------------------------ hooks
    def _hyper(self):
        if self.opt_mode == 2:      # SGD: beta1 carries the momentum, beta2 the dampening
            return self.momentum, self.dampening, 1.0, 1.0
        b1, b2 = self.betas
        t = self.step_count + 1
        return b1, b2, 1.0 - b1 ** t, 1.0 - b2 ** t

    def _launch_bucket(self, i: int) -> None:
        s, e, decays = self.buckets[i]
        W = self.world
        chunk = (e - s) // W
        b1, b2, bc1, bc2 = self._hyper()
        if self.host:
            self._host_bucket_step(s, e, chunk, self.weight_decay if (decays or self.decay_all) else 0.0, b1, b2, bc1, bc2)
            self._launched[i] = True
            return
        C = _native.load(required=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self._comm.wait_event(ev)
        with torch.cuda.stream(self._comm):
            C.ddp_bucket_step(self.grad_ptrs, self.lp_ptrs, self.flag_ptrs, self.flat.master, self.m, self.v,
                              self.done_counter, s, chunk, self.rank, self.step_count + 1, i * W,
                              (self.n_buckets + i) * W, self.timeout_s, self.lr, b1, b2, self.eps,
                              self.weight_decay if (decays or self.decay_all) else 0.0, bc1, bc2,
                              self.grad_scale / W, self.n_ctas, self.opt_mode, self.nesterov,
                              self.step_count == 0, self.mc_grad, self.mc_lp)
        self._launched[i] = True

    @torch.no_grad()
    def _host_bucket_step(self, s: int, e: int, chunk: int, wd: float, b1: float, b2: float, bc1: float, bc2: float) -> None:
        f, W, R = self.flat, self.world, self.rank
        g_all = f.grad[s:e]
        if W > 1:
            dist.all_reduce(g_all, group=self.group)
        lo, hi = s + R * chunk, s + (R + 1) * chunk
        p, g = f.master[lo:hi], f.grad[lo:hi] * (self.grad_scale / W)
        if self.opt_mode == 2:
            g = g + wd * p
            d = g
            if self.m is not None:
                m = self.m[lo:hi]
                if self.step_count == 0:
                    m.copy_(g)
                else:
                    m.mul_(b1).add_(g, alpha=1.0 - b2)
                d = g + b1 * m if self.nesterov else m
            p.add_(d, alpha=-self.lr)
        else:
            m, v = self.m[lo:hi], self.v[lo:hi]
            if self.opt_mode == 1:
                g = g + wd * p
            m.mul_(b1).add_(g, alpha=1.0 - b1)
            v.mul_(b2).addcmul_(g, g, value=1.0 - b2)
            if self.opt_mode == 0:
                p.mul_(1.0 - self.lr * wd)
            p.addcdiv_(m / bc1, (v / bc2).sqrt() + self.eps, value=-self.lr)
        g_all.zero_()
        mine = p.to(f.lp.dtype)
        if W > 1:
            parts = [torch.empty_like(mine) for _ in range(W)]
            dist.all_gather(parts, mine, group=self.group)
            f.lp[s:e].copy_(torch.cat(parts))
        else:
            f.lp[s:e].copy_(mine)

    def _on_autograd_grad(self, p) -> None:
        if p.grad is None:
            return
        o, n = self._entry_of[id(p)]
        g = p.grad.permute(0, 2, 3, 1) if getattr(p, "_flat_ohwi", False) else p.grad
        self.flat.grad[o:o + n].add_(g.reshape(-1))
        p.grad = None
        self._on_grads_ready([p])

    def _on_grads_ready(self, params) -> None:
        if not self.overlap:
            return
        for p in params:
            for i in self._param_buckets.get(id(p), ()):
                self._pending[i] -= 1
                if self._pending[i] == 0 and not self._launched[i]:
                    self._launch_bucket(i)

    # ------------------------------------------------------------------- step
    def step(self) -> None:
        """Finish the data-parallel optimizer step for the gradients of the last backward."""
        self.flat.collect_autograd_grads()      # gradients left in ``.grad`` by ordinary autograd modules
        for i in range(self.n_buckets):
            if not self._launched[i]:
                self._launch_bucket(i)
        W = self.world
        if self.host:
            self.step_count += 1
            self._pending = list(self._bucket_need)
            self._launched = [False] * self.n_buckets
            return
        if W > 1:
            C = _native.load(required=True)
            with torch.cuda.stream(self._comm):
                C.ddp_wait_end(self.flags.data_ptr() + 4 * self.n_buckets * W, self.n_buckets, W, self.rank,
                               self.step_count + 1, self.timeout_s, self.device.index or 0)
                # every peer has read its slices of this rank's gradients: clear them for the next backward pass
                # (the kernels only zero the slice their own rank owns)
                self.flat.grad.zero_()
        torch.cuda.current_stream(self.device).wait_stream(self._comm)
        self.step_count += 1
        self._pending = list(self._bucket_need)
        self._launched = [False] * self.n_buckets

    def _rearm(self) -> None:
        """Clears the cross-rank flag words, the CTA counter and the bucket bookkeeping (all ranks together, between
        two host barriers, so that nobody clears while a peer's kernel still signals and nobody launches against
        flags that a slower rank has yet to clear).  The flag words hold step numbers and the kernels wait for
        ``flag >= step``; they must therefore go back to zero whenever the step count can move backwards."""
        if self.host:
            self._pending = list(self._bucket_need)
            self._launched = [False] * self.n_buckets
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)
        self.flags.zero_()
        self.done_counter.zero_()
        self._pending = list(self._bucket_need)
        self._launched = [False] * self.n_buckets
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)

    def reset_after_timeout(self) -> None:
        """Re-arms the object after a step reported a peer timeout.  CTAs that gave up leave the kernel before they
        count themselves in ``done_counter``, so the next launch would see its "last CTA" early; the gradient
        buffer may also hold slices that nobody cleared.  All ranks call this together, then restore a checkpoint
        with ``load_state_dict`` (the step that timed out is lost) before they train on."""
        self._rearm()
        if not self.host:
            self.flat.grad.zero_()
            torch.cuda.synchronize(self.device)
            if self.world > 1:
                dist.barrier(group=self.group)

    def zero_grad(self, set_to_none: bool = False) -> None:
        """Gradients are zeroed by the bucket kernel itself; kept for API parity."""

    def set_learning_rate(self, lr: float) -> None:
        self.lr = float(lr)

    def learning_rate(self) -> float:
        return self.lr

    def _gather_owned(self, buf: torch.Tensor) -> torch.Tensor:
        """Full-length copy of a flat fp32 buffer of which each rank only keeps its own bucket slices current."""
        if self.world == 1:
            return buf.clone()
        out = buf.clone()
        for s, e, _ in self.buckets:
            chunk = (e - s) // self.world
            parts = [torch.empty(chunk, dtype=torch.float32, device=self.device) for _ in range(self.world)]
            mine = buf[s + self.rank * chunk: s + (self.rank + 1) * chunk].contiguous()
            dist.all_gather(parts, mine, group=self.group)
            out[s:e] = torch.cat(parts)
        return out

    def gather_master(self) -> torch.Tensor:
        """Full fp32 master weights (each rank only keeps its own slices current)."""
        return self._gather_owned(self.flat.master)

    def state_dict(self) -> dict:
        """World-size independent optimizer state: master weights and moments are gathered from their owners, so
        any rank's dictionary is a complete checkpoint that :meth:`load_state_dict` accepts at any world size.
        Collective: every rank must call it."""
        return {"optimizer": self.optimizer, "lr": self.lr, "betas": self.betas, "eps": self.eps,
                "weight_decay": self.weight_decay, "momentum": self.momentum, "dampening": self.dampening,
                "nesterov": self.nesterov, "step": self.step_count, "master": self.gather_master(),
                "exp_avg": None if self.m is None else self._gather_owned(self.m),
                "exp_avg_sq": None if self.v is None else self._gather_owned(self.v),
                "rank": self.rank, "world": self.world}

    def load_state_dict(self, sd: dict) -> None:
        """Restore master weights, the bf16 parameter copy, the moments and the step count from ``state_dict()``
        output (written at any world size: the buffers are full length)."""
        assert sd.get("optimizer", self.optimizer) == self.optimizer, "state dict belongs to another optimizer rule"
        n = self.flat.master.numel()
        assert sd["master"].numel() == n, f"state dict holds {sd['master'].numel()} parameters, this model {n}"
        self.lr, self.betas, self.eps = float(sd["lr"]), tuple(sd["betas"]), float(sd["eps"])
        self.weight_decay, self.step_count = float(sd["weight_decay"]), int(sd["step"])
        self.momentum = float(sd.get("momentum", self.momentum))
        self.dampening = float(sd.get("dampening", self.dampening))
        self.nesterov = bool(sd.get("nesterov", self.nesterov))
        with torch.no_grad():
            self.flat.master.copy_(sd["master"].to(self.device))
            self.flat.lp.copy_(self.flat.master)
            if self.m is not None and sd.get("exp_avg") is not None:
                self.m.copy_(sd["exp_avg"].to(self.device))
            if self.v is not None and sd.get("exp_avg_sq") is not None:
                self.v.copy_(sd["exp_avg_sq"].to(self.device))
        self._rearm()                           # the step count may have moved backwards: flags back to zero
        if self.world > 1:
            dist.barrier(group=self.group)      # nobody launches a bucket into a peer that is still loading

    def close(self) -> None:
        if fused.grad_ready_hook == self._on_grads_ready:
            fused.grad_ready_hook = None
        for h in getattr(self, "_ag_hooks", []):
            h.remove()
        self._ag_hooks = []


class FusedDDPAdamW(FusedDDP):
    """:class:`FusedDDP` with the AdamW rule (the GPT-2 / Llama recipes)."""

    def __init__(self, module, *args, **kw):
        kw.setdefault("optimizer", "adamw")
        super().__init__(module, *args, **kw)


class FusedDDPSGD(FusedDDP):
    """:class:`FusedDDP` with SGD + momentum and L2 decay on every parameter (the ResNet recipe)."""

    def __init__(self, module, lr: float = 0.1, momentum: float = 0.9, weight_decay: float = 1e-4, nesterov: bool = False,
                 dampening: float = 0.0, **kw):
        kw.setdefault("decay_all", True)
        super().__init__(module, lr=lr, weight_decay=weight_decay, optimizer="sgd", momentum=momentum, dampening=dampening,
                         nesterov=nesterov, **kw)
