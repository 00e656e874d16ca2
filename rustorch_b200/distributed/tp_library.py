"""Tensor + sequence parallel linears on library kernels only (NCCL collectives + cuBLAS matmuls).

Same interface and sharding as the fused layers in ``tp_fused.py`` (input / output rows are sequence-sharded, weights
are split over the feature dimension), so a model can be built on either and timed against the other:
``benchmarks/llama_tp_bench.py --impl library``.  Column parallel: all-gather of the input rows, then ``X W^T``;
row parallel: ``X W^T`` of this rank's feature slice, then reduce-scatter of the partial sums.  The reference's
tensor-parallel layer returns zeros (src/distributed/model_parallel.rs:429-503); this is the baseline arm, not the
product.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

__all__ = ["LibraryColumnParallelLinear", "LibraryRowParallelLinear"]


def _all_gather_rows(x: torch.Tensor, group, world: int) -> torch.Tensor:
    out = torch.empty((world * x.shape[0], x.shape[1]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def _reduce_scatter_rows(x: torch.Tensor, group, world: int) -> torch.Tensor:
    out = torch.empty((x.shape[0] // world, x.shape[1]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
    return out


class _ColumnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, w, group, world):
        xg = _all_gather_rows(x_shard, group, world)
        ctx.save_for_backward(xg, w)
        ctx.group, ctx.world = group, world
        return xg @ w.t()

    @staticmethod
    def backward(ctx, dy):
        xg, w = ctx.saved_tensors
        dx = _reduce_scatter_rows(dy @ w, ctx.group, ctx.world)
        return dx, dy.t() @ xg, None, None


class _RowFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, group, world):
        ctx.save_for_backward(x, w)
        ctx.group, ctx.world = group, world
        return _reduce_scatter_rows(x @ w.t(), group, world)

    @staticmethod
    def backward(ctx, dy_shard):
        x, w = ctx.saved_tensors
        dy = _all_gather_rows(dy_shard, ctx.group, ctx.world)
        return dy @ w, dy.t() @ x, None, None


class LibraryColumnParallelLinear(nn.Module):
    """Input: this rank's rows ``[rows, in]``.  Output: all rows, this rank's output features ``[W rows, out / W]``."""

    def __init__(self, in_features: int, out_features: int, rows_per_rank: int = 0, bias: bool = False, group=None, device="cuda",
                 init_std: float = 0.02, dtype=torch.bfloat16):
        super().__init__()
        if bias:
            raise ValueError("the library arm has no bias")
        self.group = group
        self.world = dist.get_world_size(group)
        self.weight = nn.Parameter(torch.randn(out_features // self.world, in_features, device=device, dtype=dtype) * init_std)

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        return _ColumnFn.apply(x_shard, self.weight, self.group, self.world)


class LibraryRowParallelLinear(nn.Module):
    """Input: all rows, this rank's input features ``[W rows, in / W]``.  Output: this rank's rows ``[rows, out]``."""

    def __init__(self, in_features: int, out_features: int, rows_per_rank: int = 0, bias: bool = False, group=None, device="cuda",
                 init_std: float = 0.02, dtype=torch.bfloat16):
        super().__init__()
        if bias:
            raise ValueError("the library arm has no bias")
        self.group = group
        self.world = dist.get_world_size(group)
        self.weight = nn.Parameter(torch.randn(out_features, in_features // self.world, device=device, dtype=dtype) * init_std)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _RowFn.apply(x, self.weight, self.group, self.world)
