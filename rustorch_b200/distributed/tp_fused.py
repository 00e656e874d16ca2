"""Tensor-parallel linear layers whose collective runs inside the GEMM kernel (csrc/collective/tp_gemm.cu).

Megatron-style sequence-parallel sharding: activations between the two linears of a block are sharded over
rows (tokens), the weights over output features (column-parallel) or input features (row-parallel):

* ``FusedColumnParallelLinear``:  ``y[M, N/W] = all_gather(x)[M, K] @ W_r[N/W, K]^T``  — one all-gather -> GEMM kernel;
  backward: ``dW_r = dy^T @ x_gathered`` (tcgen05 wgrad on the gather buffer the forward filled) and
  ``dx_r = reduce_scatter(dy @ W_r)`` — one GEMM -> reduce-scatter kernel.
* ``FusedRowParallelLinear``:  ``y_r[M/W, N] = reduce_scatter(x[M, K/W] @ W_r[N, K/W]^T)`` — one GEMM -> reduce-scatter
  kernel; backward: ``dx = all_gather(dy) @ W_r`` (all-gather -> GEMM) and ``dW_r = dy_gathered^T @ x``.

Every op instance owns its symmetric buffers (``torch.distributed._symmetric_memory``), flag words and epoch
counter; shapes are fixed per instance (rows per rank a multiple of 128).  The reference's
ColumnParallel / RowParallel layers slice weights on the host and call a blocking all-reduce stub
(src/distributed/model_parallel.rs:429-503); the NCCL equivalent of these layers is
``rustorch_b200.distributed.model_parallel`` and serves as the baseline in the tests and benchmarks.
"""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import _native
from ..ops import kernels as K


def _group_info(group) -> Tuple[object, int, int]:
    if dist.is_available() and dist.is_initialized():
        g = group or dist.group.WORLD
        return g, dist.get_world_size(g), dist.get_rank(g)
    return None, 1, 0


def _symm(numel: int, dtype: torch.dtype, device, group, world: int):
    """Zeroed buffer + the pointers of every rank's copy (symmetric memory for world > 1)."""
    if world == 1:
        t = torch.zeros(numel, dtype=dtype, device=device)
        return t, [t.data_ptr()], None
    from .fused_allreduce import _symm_empty
    return _symm_empty(numel, dtype, device, group)


class AllGatherGemm:
    """``out[W*rows, N] = all_gather(shards)[W*rows, K] @ weight^T (+ bias)`` as one kernel.  Write this rank's rows into
    ``self.x_shard`` (or pass ``x``), then call."""

    def __init__(self, rows_per_rank: int, K_: int, device, group=None, timeout_s: float = 20.0, n_comm: Optional[int] = None):
        if rows_per_rank % 128:
            raise ValueError("rows per rank must be a multiple of 128")
        self.group, self.world, self.rank = _group_info(group)
        self.rows, self.K, self.device = rows_per_rank, K_, torch.device(device)
        W = self.world
        flat, self.x_ptrs, self._h1 = _symm(rows_per_rank * K_, torch.bfloat16, self.device, self.group, W)
        self.x_shard = flat.view(rows_per_rank, K_)
        self.flags, self.flag_ptrs, self._h2 = _symm(2 * W + (rows_per_rank // 128) * W, torch.int32, self.device, self.group, W)
        self.gather = torch.empty(W * rows_per_rank, K_, dtype=torch.bfloat16, device=self.device)
        self.mb_ready = torch.zeros(W * rows_per_rank // 128, dtype=torch.int32, device=self.device)
        self.comm_done = torch.zeros(1, dtype=torch.int32, device=self.device)
        if n_comm is None:
            # copy CTAs: the bytes they keep in flight (a few hundred KB each) over the NVLink latency set the pull rate.
            # Eight of them moved 235 MB at ~250 GB/s on 8 ranks (transfer-bound), while 2 ranks need no more than 8.
            n_comm = int(os.environ.get("RUSTORCH_TP_NCOMM", "0")) or (8 if W <= 2 else 16 if W <= 4 else 24)
        self.epoch, self.timeout_s, self.n_comm = 0, timeout_s, n_comm

    def __call__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, x: Optional[torch.Tensor] = None,
                 b_mn: bool = False, out: Optional[torch.Tensor] = None, gather: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``gather``: where the kernel leaves the gathered input (default: this op's own buffer).  Layers that need
        it again in backward pass their own, so that one op (symmetric shard + flags) can serve many layers."""
        if x is not None:
            self.x_shard.copy_(x.reshape(self.rows, self.K))
        N = weight.shape[1] if b_mn else weight.shape[0]
        if out is None:
            out = torch.empty(self.world * self.rows, N, dtype=torch.bfloat16, device=self.device)
        self.epoch += 1
        _native.load(required=True).tp_ag_gemm(self.x_ptrs, self.flag_ptrs, self.gather if gather is None else gather, self.mb_ready,
                                               self.comm_done, weight, b_mn, out, bias, self.rank, self.epoch, self.rows,
                                               self.timeout_s, self.n_comm)
        return out


class GemmReduceScatter:
    """``out[rows, N] = reduce_scatter(x[W*rows, K] @ weight^T) (+ bias) (+ residual)`` as one kernel."""

    def __init__(self, rows_per_rank: int, N: int, device, group=None, timeout_s: float = 20.0):
        if rows_per_rank % 128:
            raise ValueError("rows per rank must be a multiple of 128")
        self.group, self.world, self.rank = _group_info(group)
        self.rows, self.N, self.device = rows_per_rank, N, torch.device(device)
        W = self.world
        self.stage, self.stage_ptrs, self._h1 = _symm(2 * W * rows_per_rank * N, torch.bfloat16, self.device, self.group, W)
        self.flags, self.flag_ptrs, self._h2 = _symm(2 * W + (rows_per_rank // 128) * W, torch.int32, self.device, self.group, W)
        self.epoch, self.timeout_s = 0, timeout_s

    def __call__(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 residual: Optional[torch.Tensor] = None, b_mn: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty(self.rows, self.N, dtype=torch.bfloat16, device=self.device)
        self.epoch += 1
        _native.load(required=True).tp_gemm_rs(x, weight, b_mn, self.stage_ptrs, self.flag_ptrs, out, bias, residual, self.rank,
                                               self.epoch, self.timeout_s)
        return out


_OPS = {}


def _wgrad_splits(n_out: int, n_in: int, rows: int) -> int:
    """Split count of a weight-gradient GEMM [n_out, n_in] over ``rows`` contraction rows: one wave of work units."""
    from ..nn.fused import _split_k_for
    return _split_k_for(-(-n_out // 128) * -(-n_in // 256), -(-rows // 64))


def shared_op(kind: str, rows: int, dim: int, device, group):
    """One op object (symmetric buffers, flags, epoch counter) per (kind, rows, dim, group): layers of equal shape use
    it one after the other, which the kernels' double buffering and end-of-kernel flags make safe.  A 32-layer model then
    holds 4 sets of communication buffers instead of 128."""
    key = (kind, rows, dim, str(torch.device(device)), id(group) if group is not None else None)
    if key not in _OPS:
        _OPS[key] = AllGatherGemm(rows, dim, device, group) if kind == "ag" else GemmReduceScatter(rows, dim, device, group)
    return _OPS[key]


class _ColumnParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, weight, bias, layer):
        y = layer.ag(weight, bias, x=x_shard, gather=layer.gather)
        ctx.layer = layer
        ctx.save_for_backward(weight)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        (weight,) = ctx.saved_tensors
        L = ctx.layer
        dy = dy.contiguous()
        # dW[N_local, K] = dy^T @ x_gathered : both operands read "MN-major", fp32 accumulate
        dw = K.gemm(dy, L.gather, a_mn=True, b_mn=True, out_dtype=torch.float32, split_k=_wgrad_splits(dy.shape[1], L.gather.shape[1], dy.shape[0]), accumulate=True)
        db = dy.float().sum(0).to(weight.dtype) if ctx.has_bias else None
        # dx_shard[rows, K] = reduce_scatter(dy[M, N_local] @ W[N_local, K]) : W read as [K_red = N_local][N_out = K]
        dx = L.rs_bwd(dy, weight, b_mn=True)
        return dx, dw.to(weight.dtype), db, None


class _RowParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, layer):
        y = layer.rs(x, weight, bias)          # each output row is reduced once, by its owner: the bias is added there
        ctx.layer = layer
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        x, weight = ctx.saved_tensors
        L = ctx.layer
        # dx[M, K_local] = all_gather(dy)[M, N] @ W[N, K_local]  (W read as [K_red = N][N_out = K_local])
        dx = L.ag_bwd(weight, None, x=dy_shard.contiguous(), b_mn=True)
        dw = K.gemm(L.ag_bwd.gather, x, a_mn=True, b_mn=True, out_dtype=torch.float32, split_k=_wgrad_splits(L.ag_bwd.gather.shape[1], x.shape[1], x.shape[0]), accumulate=True)
        db = None
        if ctx.has_bias:
            db = L.ag_bwd.gather.float().sum(0).to(weight.dtype)
        return dx, dw.to(weight.dtype), db, None


class FusedColumnParallelLinear(nn.Module):
    """Input: this rank's rows ``[rows, in_features]`` (sequence-parallel).  Output: all rows, this rank's output features
    ``[W*rows, out_features / W]``."""

    def __init__(self, in_features: int, out_features: int, rows_per_rank: int, bias: bool = True, group=None, device="cuda",
                 init_std: float = 0.02):
        super().__init__()
        g, W, r = _group_info(group)
        if out_features % W:
            raise ValueError("out_features must divide by the tensor-parallel world size")
        self.world, self.rank = W, r
        self.in_features, self.out_features, self.out_local = in_features, out_features, out_features // W
        self.weight = nn.Parameter(torch.randn(self.out_local, in_features, device=device, dtype=torch.bfloat16) * init_std)
        self.bias = nn.Parameter(torch.zeros(self.out_local, device=device, dtype=torch.bfloat16)) if bias else None
        self.ag = shared_op("ag", rows_per_rank, in_features, device, g)
        self.rs_bwd = shared_op("rs", rows_per_rank, in_features, device, g)
        # this layer's gathered input, kept for its weight gradient
        self.gather = torch.empty(W * rows_per_rank, in_features, dtype=torch.bfloat16, device=device)

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        return _ColumnParallelFn.apply(x_shard, self.weight, self.bias, self)


class FusedRowParallelLinear(nn.Module):
    """Input: all rows, this rank's input features ``[W*rows, in_features / W]``.  Output: this rank's rows
    ``[rows, out_features]`` (sequence-parallel), summed over ranks; the bias is added once."""

    def __init__(self, in_features: int, out_features: int, rows_per_rank: int, bias: bool = True, group=None, device="cuda",
                 init_std: float = 0.02):
        super().__init__()
        g, W, r = _group_info(group)
        if in_features % W:
            raise ValueError("in_features must divide by the tensor-parallel world size")
        self.world, self.rank = W, r
        self.in_features, self.out_features, self.in_local = in_features, out_features, in_features // W
        self.weight = nn.Parameter(torch.randn(out_features, self.in_local, device=device, dtype=torch.bfloat16) * init_std)
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=torch.bfloat16)) if bias else None
        self.rs = shared_op("rs", rows_per_rank, out_features, device, g)
        self.ag_bwd = shared_op("ag", rows_per_rank, out_features, device, g)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _RowParallelFn.apply(x, self.weight, self.bias, self)
