"""``DistributedOptimizer``: a base optimizer plus a gradient synchronisation strategy
(src/distributed/optimizer.rs:35-608).

Strategies: ``Synchronous`` (bucketed averaged all-reduce before every step), ``Asynchronous`` (hand the
buckets to the :class:`AsyncGradientSynchronizer` worker), ``LocalSGD{sync_frequency}`` (step locally,
average the parameters every k steps), ``Compressed{ratio}`` (top-k with error feedback before the
all-reduce) and ``Hierarchical`` (reduce inside a sub-group, then across group leaders, then broadcast).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from . import api
from .async_gradient import AsyncGradientSynchronizer, GradientCompressor
from .ddp import GradientBucket


@dataclass
class SyncStrategy:
    kind: str = "synchronous"
    sync_frequency: int = 1
    ratio: float = 0.01
    group_size: int = 8

    Synchronous = staticmethod(lambda: SyncStrategy("synchronous"))
    Asynchronous = staticmethod(lambda: SyncStrategy("asynchronous"))
    LocalSGD = staticmethod(lambda sync_frequency: SyncStrategy("local_sgd", sync_frequency=sync_frequency))
    Compressed = staticmethod(lambda ratio: SyncStrategy("compressed", ratio=ratio))
    Hierarchical = staticmethod(lambda group_size=8: SyncStrategy("hierarchical", group_size=group_size))


class DistributedOptimizer:
    def __init__(self, base: torch.optim.Optimizer, strategy: Optional[SyncStrategy] = None,
                 group: Optional[api.ProcessGroup] = None, bucket_size_mb: float = 25.0):
        self.base, self.strategy, self.group = base, strategy or SyncStrategy(), group
        self.params = [p for g in base.param_groups for p in g["params"] if p.requires_grad]
        self.buckets = GradientBucket.create_buckets(list(reversed(self.params)), bucket_size_mb)
        self.step_count = 0
        self._async = AsyncGradientSynchronizer(group=group) if self.strategy.kind == "asynchronous" else None
        self._compressor = GradientCompressor("topk", self.strategy.ratio) if self.strategy.kind == "compressed" else None
        self._intra = self._leaders = None
        if self.strategy.kind == "hierarchical" and api.is_initialized():
            W, G, r = api.get_world_size(), self.strategy.group_size, api.get_rank()
            for s in range(0, W, G):
                ranks = list(range(s, min(W, s + G)))
                pg = api.new_group(ranks)
                if r in ranks:
                    self._intra = pg
            self._leaders = api.new_group(list(range(0, W, G)))

    @classmethod
    def builder(cls):
        return _Builder(cls)

    def _flat(self, b: GradientBucket) -> torch.Tensor:
        return torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in b.params])

    def _unflat(self, b: GradientBucket, flat: torch.Tensor) -> None:
        off = 0
        for p in b.params:
            n = p.numel()
            if p.grad is None:
                p.grad = flat[off:off + n].view_as(p).clone()
            else:
                p.grad.copy_(flat[off:off + n].view_as(p))
            off += n

    def sync_bucket_with_backend(self, b: GradientBucket) -> None:
        flat = self._flat(b)
        k = self.strategy.kind
        if k == "compressed":
            flat = self._compressor.compress_decompress(flat, key=b.index)
        if k == "hierarchical" and self._intra is not None:
            api.all_reduce(flat, api.ReduceOp.SUM, self._intra)
            if api.get_rank() % self.strategy.group_size == 0:
                api.all_reduce(flat, api.ReduceOp.SUM, self._leaders)
            api.broadcast(flat, self._intra.ranks()[0], self._intra)
            flat.div_(api.get_world_size())
        elif k == "asynchronous":
            rid = self._async.submit_gradient(flat)
            self._async.wait_for_completion(rid)
        else:
            api.all_reduce(flat, api.ReduceOp.AVERAGE, self.group)
        self._unflat(b, flat)

    def sync_gradients(self) -> None:
        for b in self.buckets:
            self.sync_bucket_with_backend(b)

    def step(self) -> None:
        self.step_count += 1
        if self.strategy.kind == "local_sgd":
            self.base.step()
            if self.step_count % self.strategy.sync_frequency == 0:
                for p in self.params:
                    api.all_reduce(p.data, api.ReduceOp.AVERAGE, self.group)
            return
        self.sync_gradients()
        self.base.step()

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.base.zero_grad(set_to_none=set_to_none)

    def state_dict(self) -> dict:
        return {"base": self.base.state_dict(), "step": self.step_count, "strategy": self.strategy.__dict__}

    def load_state_dict(self, sd: dict) -> None:
        self.base.load_state_dict(sd["base"])
        self.step_count = sd["step"]


class _Builder:
    def __init__(self, cls):
        self.cls, self.kw = cls, {}
        self._base = None

    def optimizer(self, base):
        self._base = base
        return self

    def strategy(self, s: SyncStrategy):
        self.kw["strategy"] = s
        return self

    def bucket_size_mb(self, mb: float):
        self.kw["bucket_size_mb"] = mb
        return self

    def group(self, g):
        self.kw["group"] = g
        return self

    def build(self):
        if self._base is None:
            raise ValueError("DistributedOptimizer builder needs a base optimizer")
        return self.cls(self._base, **self.kw)
