"""Data-parallel gradient synchronisation for the flat-buffer training path.

``FlatDDP`` owns the gradient all-reduce of a :class:`~rustorch_b200.optim.flat.FlatParams`:
the gradient buffer is cut into buckets of ``bucket_cap_mb`` (25 MB like the reference's
``BackendOptimizations`` / ``DistributedDataParallel`` defaults, src/distributed/common.rs:131-190,
src/distributed/ddp.rs:86-131) and averaged across ranks; the reference's own all-reduce is a
no-op stub (src/distributed/common.rs:49-56).  Two mechanisms:

* ``mode="nccl"``: one NCCL all-reduce per bucket on a side stream (the library baseline);
* ``mode="fused"``: the hand-written peer-memory kernel that reduces a rank's shard over
  NVLink, applies the 1/N scale and the AdamW update, and writes the new bf16 parameters
  back to every peer (see :mod:`rustorch_b200.distributed.fused_allreduce`).
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


def bucket_ranges(numel: int, bucket_cap_mb: float, elem_bytes: int = 4, align: int = 1024) -> List[Tuple[int, int]]:
    """Greedy fixed-size cut of ``[0, numel)``; boundaries are multiples of ``align`` elements."""
    per = max(align, int(bucket_cap_mb * 1024 * 1024 / elem_bytes) // align * align)
    out, s = [], 0
    while s < numel:
        e = min(numel, s + per)
        out.append((s, e))
        s = e
    return out


class FlatDDP:
    def __init__(self, flat, process_group=None, bucket_cap_mb: float = 25.0, mode: str = "nccl"):
        self.flat = flat
        self.group = process_group
        self.world_size = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        self.mode = mode
        self.buckets = bucket_ranges(flat.numel, bucket_cap_mb)
        self._stream = torch.cuda.Stream() if flat.grad.is_cuda else None

    def broadcast_parameters(self, src: int = 0) -> None:
        """Make every rank start from rank ``src``'s weights (master and compute copies)."""
        if self.world_size == 1:
            return
        dist.broadcast(self.flat.master, src, group=self.group)
        self.flat.lp.copy_(self.flat.master)

    def sync_gradients(self) -> None:
        """Sum gradients across ranks (the optimizer applies the 1/N through ``grad_scale``)."""
        if self.world_size == 1:
            return
        g = self.flat.grad
        if self._stream is not None:
            self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream):
                for s, e in self.buckets:
                    dist.all_reduce(g[s:e], group=self.group)
            torch.cuda.current_stream().wait_stream(self._stream)
        else:
            for s, e in self.buckets:
                dist.all_reduce(g[s:e], group=self.group)
