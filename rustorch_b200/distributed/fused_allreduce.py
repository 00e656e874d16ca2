"""Data-parallel training step fused into one peer-memory kernel per gradient bucket.

``FusedDDPAdamW`` wraps a model whose parameters live in a :class:`FlatParams`:

* the bf16 parameter buffer, the fp32 gradient buffer and a small flag array are *symmetric*
  allocations (``torch.distributed._symmetric_memory``), so every rank holds device pointers
  to every peer's copy over NVLink;
* the gradient buffer is cut into buckets of ``bucket_cap_mb`` (25 MB, the reference's default,
  src/distributed/ddp.rs:86-131); inside a bucket rank ``r`` owns the ``r``-th 1/N slice;
* when the backward pass has finished the last gradient of a bucket (the fused autograd
  Functions report it through ``fused.grad_ready_hook``) the bucket's kernel is queued on a side
  stream: it reduces the owned slice across all ranks with P2P loads, zeroes the gradients,
  applies scale + AdamW to the fp32 master weights / moments and stores the new bf16
  parameters into every rank's parameter buffer (csrc/collective/ddp_fused.cu).  Backward
  keeps running underneath;
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


class FusedDDPAdamW:
    def __init__(self, module: torch.nn.Module, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, bucket_cap_mb: float = 25.0, process_group=None,
                 decay_filter=default_decay_filter, n_ctas: int = 296, timeout_s: float = 60.0,
                 overlap: bool = True):
        self.module = module
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

        def alloc(kind, dtype):
            def _a(n):
                if W == 1:
                    t = torch.zeros(n, dtype=dtype, device=dev)
                    ptrs[kind] = [t.data_ptr()]
                    return t
                t, pp, h = _symm_empty(n, dtype, dev, self.group)
                self._handles.append(h)
                ptrs[kind] = pp
                return t
            return _a

        lp_dtype = next(module.parameters()).dtype
        assert lp_dtype == torch.bfloat16, "FusedDDPAdamW needs bf16 parameters"
        self.flat = FlatParams(module, decay_filter=decay_filter, alloc=alloc("lp", torch.bfloat16),
                               alloc_f32=alloc("grad", torch.float32), group_align=64 * W)
        f = self.flat
        if W > 1:
            # identical starting point on every rank
            dist.broadcast(f.master, 0, group=self.group)
            f.lp.copy_(f.master)
        self.m = torch.zeros_like(f.master)
        self.v = torch.zeros_like(f.master)
        self.lp_ptrs, self.grad_ptrs = ptrs["lp"], ptrs["grad"]

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
        if W == 1:
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
        self._comm = torch.cuda.Stream(device=dev, priority=-1)
        self._in_step = False
        fused.grad_ready_hook = self._on_grads_ready
        if W > 1:
            dist.barrier(group=self.group)
        torch.cuda.synchronize(dev)

    # ------------------------------------------------------------------ hooks
    def _hyper(self):
        b1, b2 = self.betas
        t = self.step_count + 1
        return b1, b2, 1.0 - b1 ** t, 1.0 - b2 ** t

    def _launch_bucket(self, i: int) -> None:
        s, e, decays = self.buckets[i]
        W = self.world
        chunk = (e - s) // W
        b1, b2, bc1, bc2 = self._hyper()
        C = _native.load(required=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self._comm.wait_event(ev)
        with torch.cuda.stream(self._comm):
            C.ddp_bucket_adamw(self.grad_ptrs, self.lp_ptrs, self.flag_ptrs, self.flat.master, self.m, self.v,
                               self.done_counter, s, chunk, self.rank, self.step_count + 1, i * W,
                               (self.n_buckets + i) * W, self.timeout_s, self.lr, b1, b2, self.eps,
                               self.weight_decay if decays else 0.0, bc1, bc2, self.grad_scale / W,
                               self.n_ctas)
        self._launched[i] = True

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
        if W > 1:
            C = _native.load(required=True)
            with torch.cuda.stream(self._comm):
                C.ddp_wait_end(self.flags.data_ptr() + 4 * self.n_buckets * W, self.n_buckets, W, self.rank,
                               self.step_count + 1, self.timeout_s, self.device.index or 0)
        torch.cuda.current_stream(self.device).wait_stream(self._comm)
        self.step_count += 1
        self._pending = list(self._bucket_need)
        self._launched = [False] * self.n_buckets

    def zero_grad(self, set_to_none: bool = False) -> None:
        """Gradients are zeroed by the bucket kernel itself; kept for API parity."""

    def set_learning_rate(self, lr: float) -> None:
        self.lr = float(lr)

    def learning_rate(self) -> float:
        return self.lr

    def gather_master(self) -> torch.Tensor:
        """Full fp32 master weights (each rank only keeps its own slices current)."""
        f = self.flat
        if self.world == 1:
            return f.master.clone()
        out = f.master.clone()
        for s, e, _ in self.buckets:
            chunk = (e - s) // self.world
            parts = [torch.empty(chunk, dtype=torch.float32, device=self.device) for _ in range(self.world)]
            mine = f.master[s + self.rank * chunk: s + (self.rank + 1) * chunk].contiguous()
            dist.all_gather(parts, mine, group=self.group)
            out[s:e] = torch.cat(parts)
        return out

    def state_dict(self) -> dict:
        return {"lr": self.lr, "betas": self.betas, "eps": self.eps, "weight_decay": self.weight_decay,
                "step": self.step_count, "master": self.gather_master(), "exp_avg": self.m.clone(),
                "exp_avg_sq": self.v.clone(), "rank": self.rank, "world": self.world}

    def close(self) -> None:
        if fused.grad_ready_hook == self._on_grads_ready:
            fused.grad_ready_hook = None
