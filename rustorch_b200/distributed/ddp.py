"""``DistributedDataParallel``, ``DataParallel``, ``DistributedSampler`` and gradient bucketing for
ordinary modules (src/distributed/ddp.rs:23-291, simple_ddp.rs:14-136, data_parallel.rs:22-489).

The reference's wrapper loops over parameters calling a no-op all-reduce and never registers its
hooks (ddp.rs:139-172).  This one is real:

* parameters are broadcast from rank 0 at construction (``broadcast_buffers`` also at every forward);
* gradients are grouped into buckets of ``bucket_cap_mb`` (default 25 MB) in reverse parameter order
  by the same greedy rule as the reference's ``create_buckets`` (ddp.rs:235-271);
* a post-accumulate-grad hook per parameter fires the bucket's asynchronous averaged all-reduce as
  soon as its last gradient arrives, overlapping communication with the rest of backward;
* ``sync_gradients()`` waits for the outstanding reductions (and reduces anything whose hook did not
  fire, e.g. unused parameters when ``find_unused_parameters``).

``DistributedDataParallel(module, fused_optimizer={...})`` takes the flat-buffer bf16 path instead: gradient
reduction, scaling, the optimizer rule (AdamW / Adam / SGD with momentum) and the parameter broadcast run as one
peer-memory kernel per bucket, overlapped with backward
(:class:`rustorch_b200.distributed.fused_allreduce.FusedDDP`); ``step()`` then replaces the separate
``sync_gradients()`` + ``optimizer.step()``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, Iterator, List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from . import api


@dataclass
class GradientBucket:
    index: int
    params: List[nn.Parameter] = field(default_factory=list)
    size_bytes: int = 0
    pending: int = 0
    buffer: Optional[torch.Tensor] = None
    work: object = None

    @staticmethod
    def create_buckets(params: Sequence[nn.Parameter], bucket_cap_mb: float = 25.0) -> List["GradientBucket"]:
        """Greedy: append parameters until the cap would be exceeded, then start a new bucket."""
        cap = int(bucket_cap_mb * 1024 * 1024)
        buckets: List[GradientBucket] = []
        cur = GradientBucket(0)
        for p in params:
            nbytes = p.numel() * p.element_size()
            if cur.params and cur.size_bytes + nbytes > cap:
                buckets.append(cur)
                cur = GradientBucket(len(buckets))
            cur.params.append(p)
            cur.size_bytes += nbytes
        if cur.params:
            buckets.append(cur)
        return buckets


class DistributedDataParallel(nn.Module):
    def __init__(self, module: nn.Module, device_ids: Optional[Sequence[int]] = None, output_device: Optional[int] = None,
                 dim: int = 0, broadcast_buffers: bool = True, process_group: Optional[api.ProcessGroup] = None,
                 bucket_cap_mb: float = 25.0, find_unused_parameters: bool = False, check_reduction: bool = False,
                 gradient_as_bucket_view: bool = False, static_graph: bool = False, fused_optimizer: Optional[dict] = None):
        super().__init__()
        if not dist.is_initialized():
            raise RuntimeError("DistributedDataParallel needs init_process_group() first")
        self.module = module
        self.fused = None
        if fused_optimizer is not None:
            # bf16 parameters on a GPU (or, for tests of the bookkeeping, on the CPU over gloo): one fused kernel per
            # gradient bucket does the all-reduce, the optimizer step and the parameter broadcast
            from .fused_allreduce import FusedDDP
            self.device_ids, self.output_device, self.dim = device_ids, output_device, dim
            self.broadcast_buffers, self.bucket_cap_mb = broadcast_buffers, bucket_cap_mb
            self._group = None if process_group is None else process_group.handle
            self.world_size = dist.get_world_size(self._group)
            for b in module.buffers():
                dist.broadcast(b.data, 0, group=self._group)
            self.fused = FusedDDP(module, bucket_cap_mb=bucket_cap_mb, process_group=self._group, **fused_optimizer)
            self.buckets, self._hooks = [], []
            self.require_backward_grad_sync = True
            return
        self.device_ids, self.output_device, self.dim = device_ids, output_device, dim
        self.broadcast_buffers, self.bucket_cap_mb = broadcast_buffers, bucket_cap_mb
        self.find_unused_parameters, self.static_graph = find_unused_parameters, static_graph
        self.gradient_as_bucket_view = gradient_as_bucket_view
        self._group = None if process_group is None else process_group.handle
        self.world_size = dist.get_world_size(self._group)
        params = [p for p in module.parameters() if p.requires_grad]
        # identical replicas
        for p in module.parameters():
            dist.broadcast(p.data, 0, group=self._group)
        for b in module.buffers():
            dist.broadcast(b.data, 0, group=self._group)
        # reverse order ~ order in which backward produces gradients
        self.buckets = GradientBucket.create_buckets(list(reversed(params)), bucket_cap_mb)
        self._bucket_of: Dict[int, GradientBucket] = {}
        for b in self.buckets:
            for p in b.params:
                self._bucket_of[id(p)] = b
        self._hooks = [p.register_post_accumulate_grad_hook(self._on_grad) for p in params]
        self._reset()
        self.require_backward_grad_sync = True

    # ------------------------------------------------------------- reduction
    def _reset(self) -> None:
        for b in self.buckets:
            b.pending, b.work, b.buffer = len(b.params), None, None

    def _launch(self, b: GradientBucket) -> None:
        grads = [p.grad if p.grad is not None else torch.zeros_like(p) for p in b.params]
        flat = torch.cat([g.reshape(-1) for g in grads])
        b.buffer = flat
        b.work = dist.all_reduce(flat, dist.ReduceOp.SUM, group=self._group, async_op=True)

    def _on_grad(self, p: nn.Parameter) -> None:
        if not self.require_backward_grad_sync:
            return
        b = self._bucket_of[id(p)]
        b.pending -= 1
        if b.pending == 0 and b.work is None:
            self._launch(b)

    def step(self) -> None:
        """Fused mode only: finish the data-parallel optimizer step for the gradients of the last backward."""
        if self.fused is None:
            raise RuntimeError("step() belongs to the fused mode; pass fused_optimizer={...} or use an optimizer with sync_gradients()")
        self.fused.step()

    def sync_gradients(self) -> None:
        """Block until every bucket is averaged and written back into ``.grad`` (a no-op in fused mode, where the
        reduction is part of ``step()``)."""
        if self.fused is not None:
            return
        for b in self.buckets:
            if b.work is None:
                if not self.find_unused_parameters and any(p.grad is None for p in b.params) \
                        and any(p.grad is not None for p in b.params):
                    raise RuntimeError("a parameter produced no gradient; pass find_unused_parameters=True")
                self._launch(b)
        for b in self.buckets:
            b.work.wait()
            flat = b.buffer.div_(self.world_size)
            off = 0
            for p in b.params:
                n = p.numel()
                g = flat[off:off + n].view_as(p)
                if p.grad is None:
                    p.grad = g.clone()
                else:
                    p.grad.copy_(g)
                off += n
        self._reset()

    class _NoSync:
        def __init__(self, ddp):
            self.ddp = ddp

        def __enter__(self):
            self.ddp.require_backward_grad_sync = False

        def __exit__(self, *exc):
            self.ddp.require_backward_grad_sync = True
            return False

    def no_sync(self):
        """Skip reduction inside the block (gradient accumulation across micro-batches)."""
        return DistributedDataParallel._NoSync(self)

    # --------------------------------------------------------------- forward
    def forward(self, *args, **kw):
        if self.broadcast_buffers and self.training:
            for b in self.module.buffers():
                dist.broadcast(b.data, 0, group=self._group)
        return self.module(*args, **kw)

    def get_module(self) -> nn.Module:
        return self.module


def wrap_module(module: nn.Module, device_ids: Optional[Sequence[int]] = None, **kw) -> DistributedDataParallel:
    return DistributedDataParallel(module, device_ids, **kw)


class SimpleDistributedDataParallel(nn.Module):
    """No buckets, no hooks: ``sync_gradients`` averages every gradient in one flat all-reduce."""

    def __init__(self, module: nn.Module, process_group: Optional[api.ProcessGroup] = None):
        super().__init__()
        self.module = module
        self._group = None if process_group is None else process_group.handle
        if dist.is_initialized():
            for p in module.parameters():
                dist.broadcast(p.data, 0, group=self._group)

    def forward(self, *a, **k):
        return self.module(*a, **k)

    def sync_gradients(self) -> None:
        if not dist.is_initialized() or dist.get_world_size(self._group) == 1:
            return
        ps = [p for p in self.module.parameters() if p.grad is not None]
        if not ps:
            return
        flat = torch.cat([p.grad.reshape(-1) for p in ps])
        dist.all_reduce(flat, group=self._group)
        flat.div_(dist.get_world_size(self._group))
        off = 0
        for p in ps:
            p.grad.copy_(flat[off:off + p.numel()].view_as(p))
            off += p.numel()


wrap_simple = SimpleDistributedDataParallel


class GradientSyncStrategy:
    SYNCHRONOUS = "synchronous"
    ASYNCHRONOUS = "asynchronous"

    @staticmethod
    def local_sgd(sync_frequency: int) -> dict:
        return {"kind": "local_sgd", "sync_frequency": sync_frequency}


class DataParallel(nn.Module):
    """Single-process data parallelism over ``device_ids``: the batch is split along ``dim``, each chunk
    runs on a replica on its own device and stream, outputs are gathered on ``output_device``."""

    def __init__(self, module: nn.Module, device_ids: Optional[Sequence[int]] = None, output_device: Optional[int] = None,
                 dim: int = 0):
        super().__init__()
        self.module = module
        n = torch.cuda.device_count() if torch.cuda.is_available() else 0
        self.device_ids = list(device_ids) if device_ids is not None else list(range(n))
        self.output_device = output_device if output_device is not None else (self.device_ids[0] if self.device_ids else None)
        self.dim = dim

    def replicate_input(self, x: torch.Tensor) -> List[torch.Tensor]:
        n = max(1, len(self.device_ids))
        chunks = list(x.chunk(n, self.dim))
        if self.device_ids and torch.cuda.is_available():
            chunks = [c.to(torch.device("cuda", d), non_blocking=True) for c, d in zip(chunks, self.device_ids)]
        return chunks

    def gather_outputs(self, outs: List[torch.Tensor]) -> torch.Tensor:
        if self.output_device is not None and torch.cuda.is_available():
            outs = [o.to(torch.device("cuda", self.output_device)) for o in outs]
        return torch.cat(outs, self.dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if len(self.device_ids) <= 1 or not torch.cuda.is_available():
            return self.module(x)
        replicas = nn.parallel.replicate(self.module, self.device_ids[: len(x.chunk(len(self.device_ids), self.dim))])
        outs = nn.parallel.parallel_apply(replicas, [(c,) for c in self.replicate_input(x)][: len(replicas)])
        return self.gather_outputs(outs)


class DistributedSampler:
    """``(num_samples, num_replicas, rank, drop_last, seed)``: seed+epoch shuffle, pad to a multiple of the
    world size, then a **contiguous block per rank** (``indices[rank*n : (rank+1)*n]``) as in the
    reference (src/distributed/data_parallel.rs:396-489) — not PyTorch's strided split."""

    def __init__(self, num_samples: int, num_replicas: Optional[int] = None, rank: Optional[int] = None,
                 shuffle: bool = True, seed: int = 0, drop_last: bool = False):
        if hasattr(num_samples, "__len__"):
            num_samples = len(num_samples)
        self.num_total = int(num_samples)
        self.num_replicas = api.get_world_size() if num_replicas is None else num_replicas
        self.rank = api.get_rank() if rank is None else rank
        if not 0 <= self.rank < self.num_replicas:
            raise ValueError("rank out of range")
        self.shuffle, self.seed, self.drop_last, self.epoch = shuffle, seed, drop_last, 0
        if drop_last:
            self.num_samples = self.num_total // self.num_replicas
        else:
            self.num_samples = -(-self.num_total // self.num_replicas)
        self.total_size = self.num_samples * self.num_replicas

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def sample_indices(self) -> List[int]:
        if self.shuffle:
            g = torch.Generator().manual_seed(self.seed + self.epoch)
            idx = torch.randperm(self.num_total, generator=g).tolist()
        else:
            idx = list(range(self.num_total))
        if self.drop_last:
            idx = idx[: self.total_size]
        else:
            pad = self.total_size - len(idx)
            if pad > 0:
                idx += (idx * (pad // max(1, len(idx)) + 1))[:pad]
        s = self.rank * self.num_samples
        return idx[s:s + self.num_samples]

    get_indices = sample_indices            # name in the Python binding (src/python/distributed.rs)

    def __iter__(self) -> Iterator[int]:
        return iter(self.sample_indices())

    def __len__(self) -> int:
        return self.num_samples

    len = __len__

    # Sampler protocol of rustorch_b200.data
    def reset(self) -> None:
        self._it = iter(self.sample_indices())

    def sample(self) -> Optional[int]:
        if not hasattr(self, "_it"):
            self.reset()
        return next(self._it, None)


class DistributedDataLoader:
    """A :class:`rustorch_b200.data.DataLoader` over this rank's shard; ``set_epoch`` reshuffles."""

    def __init__(self, dataset, batch_size: int, num_replicas: Optional[int] = None, rank: Optional[int] = None,
                 shuffle: bool = True, seed: int = 0, drop_last: bool = False, **loader_kw):
        from ..data import DataLoader
        self.sampler = DistributedSampler(len(dataset), num_replicas, rank, shuffle, seed, drop_last)
        self.loader = DataLoader(dataset, self.sampler, batch_size, drop_last=drop_last, **loader_kw)

    def set_epoch(self, epoch: int) -> None:
        self.sampler.set_epoch(epoch)

    def __iter__(self):
        return iter(self.loader)

    def __len__(self):
        return len(self.loader)
