"""Tensor-, pipeline- and expert-parallel building blocks with real data paths
(src/distributed/model_parallel.rs:22-573, src/gpu/multi_gpu.rs:1123-1179).

The reference's classes are API shells that return zeros (model_parallel.rs:231-252,462-502,549-563);
only its 1F1B schedule list is real (multi_gpu.rs:1123-1170).  Here:

* ``TensorParallel.split_tensor / gather_tensors / all_reduce_tensor`` move real data (collectives from
  :mod:`rustorch_b200.distributed.api`); ``ColumnParallelLinear`` / ``RowParallelLinear`` are the
  Megatron-style layers built on them;
* ``PipelineScheduler.generate_schedule`` emits GPipe or 1F1B op lists and ``PipelineStage.run`` executes them
  with point-to-point sends/receives (NCCL p2p on GPUs, Gloo on CPU ranks);
* ``ExpertParallel.route_tokens`` does top-k gating, all-to-all dispatch, local expert compute and all-to-all
  combine.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from . import api


class PartitionStrategy(enum.Enum):
    """How a model is cut for model parallelism: by layer, by tensor, by expert."""

    LAYER_WISE = "layer_wise"
    TENSOR_WISE = "tensor_wise"
    COLUMN_WISE = "column_wise"
    ROW_WISE = "row_wise"
    HYBRID = "hybrid"


# ------------------------------------------------------------------ tensor parallel
class TensorParallel:
    """``(num_partitions, partition_rank, parallel_dim)`` (model_parallel.rs:429-503)."""

    def __init__(self, num_partitions: int, partition_rank: int, parallel_dim: int = -1,
                 group: Optional[api.ProcessGroup] = None):
        if not 0 <= partition_rank < num_partitions:
            raise ValueError("partition_rank out of range")
        self.num_partitions, self.partition_rank, self.parallel_dim, self.group = num_partitions, partition_rank, parallel_dim, group

    def split_tensor(self, t: torch.Tensor) -> torch.Tensor:
        """This rank's slice along ``parallel_dim`` (must divide evenly)."""
        d = self.parallel_dim % t.dim()
        if t.shape[d] % self.num_partitions:
            raise ValueError(f"dim {d} of size {t.shape[d]} is not divisible by {self.num_partitions}")
        return t.chunk(self.num_partitions, d)[self.partition_rank].contiguous()

    def gather_tensors(self, local: torch.Tensor) -> torch.Tensor:
        """All-gather the slices back along ``parallel_dim``."""
        parts = api.all_gather(local, self.group)
        if len(parts) == 1 and self.num_partitions > 1:   # not running distributed: caller passes all parts
            return local
        return torch.cat(parts, self.parallel_dim % local.dim())

    def all_reduce_tensor(self, t: torch.Tensor) -> torch.Tensor:
        api.all_reduce(t, api.ReduceOp.SUM, self.group)
        return t


class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        api.all_reduce(g, api.ReduceOp.SUM, ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        api.all_reduce(x, api.ReduceOp.SUM, group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class ColumnParallelLinear(nn.Module):
    """``y_local = x W_r^T`` where ``W`` is split by output rows; ``gather_output`` concatenates."""

    def __init__(self, in_features: int, out_features: int, tp: TensorParallel, bias: bool = True,
                 gather_output: bool = False, device=None, dtype=None, init_std: float = 0.02):
        super().__init__()
        if out_features % tp.num_partitions:
            raise ValueError("out_features must be divisible by the tensor-parallel size")
        self.tp, self.gather_output = tp, gather_output
        self.out_local = out_features // tp.num_partitions
        self.weight = nn.Parameter(torch.empty(self.out_local, in_features, device=device, dtype=dtype).normal_(0, init_std))
        self.bias = nn.Parameter(torch.zeros(self.out_local, device=device, dtype=dtype)) if bias else None

    def forward(self, x):
        x = _CopyToTP.apply(x, self.tp.group)
        y = F.linear(x, self.weight, self.bias)
        return self.tp.gather_tensors(y) if self.gather_output else y


class RowParallelLinear(nn.Module):
    """``y = sum_r x_r W_r^T`` where ``W`` is split by input columns; the sum is an all-reduce."""

    def __init__(self, in_features: int, out_features: int, tp: TensorParallel, bias: bool = True,
                 input_is_parallel: bool = True, device=None, dtype=None, init_std: float = 0.02):
        super().__init__()
        if in_features % tp.num_partitions:
            raise ValueError("in_features must be divisible by the tensor-parallel size")
        self.tp, self.input_is_parallel = tp, input_is_parallel
        self.in_local = in_features // tp.num_partitions
        self.weight = nn.Parameter(torch.empty(out_features, self.in_local, device=device, dtype=dtype).normal_(0, init_std))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None

    def forward(self, x):
        if not self.input_is_parallel:
            x = TensorParallel(self.tp.num_partitions, self.tp.partition_rank, -1, self.tp.group).split_tensor(x)
        y = _ReduceFromTP.apply(F.linear(x, self.weight), self.tp.group)
        return y if self.bias is None else y + self.bias


# ---------------------------------------------------------------- pipeline parallel
class PipelineSchedule(enum.Enum):
    """Order of micro-batch forward / backward passes in a pipeline (fill-drain or one-forward-one-backward)."""

    GPIPE = "gpipe"
    PIPEDREAM = "pipedream"
    ONE_F_ONE_B = "1f1b"
    INTERLEAVED_1F1B = "interleaved_1f1b"


class CommunicationType(enum.Enum):
    """Collective that connects two partitions of a model-parallel layer (src/distributed/model_parallel.rs)."""

    P2P = "p2p"
    ALL_TO_ALL = "all_to_all"
    ALL_REDUCE = "all_reduce"
    BROADCAST = "broadcast"


@dataclass
class PipelineConfig:
    num_micro_batches: int = 4
    num_stages: int = 2
    gradient_accumulation_steps: int = 1
    use_1f1b: bool = True


@dataclass
class PipelineOp:
    kind: str          # "forward" | "backward"
    micro_batch: int
    stage: int


class PipelineScheduler:
    """Per-stage op lists.  1F1B: ``min(S - stage - 1, M)`` warm-up forwards, then alternate one forward /
    one backward, then drain the remaining backwards; GPipe: all forwards then all backwards."""

    def __init__(self, config: PipelineConfig, schedule: Optional[PipelineSchedule] = None):
        self.config = config
        self.schedule = schedule or (PipelineSchedule.ONE_F_ONE_B if config.use_1f1b else PipelineSchedule.GPIPE)

    def generate_schedule(self, stage: int) -> List[PipelineOp]:
        M, S = self.config.num_micro_batches, self.config.num_stages
        if not 0 <= stage < S:
            raise ValueError("stage out of range")
        if self.schedule is PipelineSchedule.GPIPE:
            return [PipelineOp("forward", m, stage) for m in range(M)] + \
                   [PipelineOp("backward", m, stage) for m in reversed(range(M))]
        warm = min(S - stage - 1, M)
        ops = [PipelineOp("forward", m, stage) for m in range(warm)]
        f, b = warm, 0
        while f < M:
            ops.append(PipelineOp("forward", f, stage))
            f += 1
            ops.append(PipelineOp("backward", b, stage))
            b += 1
        while b < M:
            ops.append(PipelineOp("backward", b, stage))
            b += 1
        return ops

    def max_in_flight(self, stage: int) -> int:
        live = peak = 0
        for op in self.generate_schedule(stage):
            live += 1 if op.kind == "forward" else -1
            peak = max(peak, live)
        return peak


class PipelineStage:
    """Runs one stage's module under a schedule with p2p activation / gradient exchange."""

    def __init__(self, module: nn.Module, stage: int, config: PipelineConfig, group: Optional[api.ProcessGroup] = None,
                 schedule: Optional[PipelineSchedule] = None, prev_rank: Optional[int] = None, next_rank: Optional[int] = None):
        self.module, self.stage, self.config, self.group = module, stage, config, group
        self.scheduler = PipelineScheduler(config, schedule)
        self.prev_rank = stage - 1 if prev_rank is None else prev_rank
        self.next_rank = stage + 1 if next_rank is None else next_rank
        self.is_first, self.is_last = stage == 0, stage == config.num_stages - 1

    def run(self, micro_inputs: Optional[Sequence[torch.Tensor]], loss_fn: Optional[Callable] = None,
            micro_targets: Optional[Sequence[torch.Tensor]] = None, act_shape: Optional[Sequence[int]] = None,
            act_dtype=torch.float32, device=None) -> List[float]:
        """One training pass over all micro-batches.  The first stage gets ``micro_inputs``, the last stage
        ``loss_fn`` and ``micro_targets``; the others receive activations of ``act_shape``."""
        saved: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        losses: List[float] = []
        # Sends are non-blocking (two neighbouring stages may both want to send at the same point of a
        # 1F1B schedule); the requests and their buffers are kept until the end of the pass.
        pending: List[Tuple[object, torch.Tensor]] = []
        M = self.config.num_micro_batches
        for op in self.scheduler.generate_schedule(self.stage):
            m = op.micro_batch
            if op.kind == "forward":
                if self.is_first:
                    x = micro_inputs[m]
                else:
                    x = torch.empty(tuple(act_shape), dtype=act_dtype, device=device)
                    api.recv(x, self.prev_rank, self.group, tag=m)
                    x.requires_grad_(True)
                y = self.module(x)
                if self.is_last:
                    y = loss_fn(y, micro_targets[m]) / M
                    losses.append(float(y.detach()) * M)
                else:
                    buf = y.detach().contiguous()
                    pending.append((api.isend(buf, self.next_rank, self.group, tag=m), buf))
                saved[m] = (x, y)
            else:
                x, y = saved.pop(m)
                if self.is_last:
                    y.backward()
                else:
                    g = torch.empty_like(y)
                    api.recv(g, self.next_rank, self.group, tag=1000 + m)
                    y.backward(g)
                if not self.is_first:
                    buf = x.grad.contiguous()
                    pending.append((api.isend(buf, self.prev_rank, self.group, tag=1000 + m), buf))
        for req, _ in pending:
            req.wait()
        return losses


class ModelParallel(nn.Module):
    """``(partitions, device_map)``: consecutive sub-modules placed on different devices of one process,
    activations hop between devices in ``forward`` (model_parallel.rs:22-227)."""

    def __init__(self, partitions: Sequence[nn.Module], device_map: Optional[Sequence] = None,
                 config: Optional[PipelineConfig] = None):
        super().__init__()
        self.partitions = nn.ModuleList(partitions)
        self.device_map = [torch.device(d) for d in device_map] if device_map else [None] * len(partitions)
        self.config = config or PipelineConfig(num_stages=len(partitions))
        for p, d in zip(self.partitions, self.device_map):
            if d is not None:
                p.to(d)

    def forward(self, x):
        for p, d in zip(self.partitions, self.device_map):
            if d is not None:
                x = x.to(d, non_blocking=True)
            x = p(x)
        return x

    def forward_micro_batches(self, x: torch.Tensor) -> torch.Tensor:
        return torch.cat([self.forward(c) for c in x.chunk(self.config.num_micro_batches, 0)], 0)


# ------------------------------------------------------------------ expert parallel
class ExpertParallel(nn.Module):
    """``(num_experts, experts_per_device, device_rank, experts)``: top-k softmax gating; tokens travel to the
    rank that owns their expert by all-to-all and come back the same way (model_parallel.rs:507-573)."""

    def __init__(self, num_experts: int, experts_per_device: int, device_rank: int, experts: Sequence[nn.Module],
                 d_model: int, top_k: int = 1, group: Optional[api.ProcessGroup] = None):
        super().__init__()
        if len(experts) != experts_per_device:
            raise ValueError("this rank must be given exactly experts_per_device experts")
        self.num_experts, self.experts_per_device, self.device_rank, self.top_k = num_experts, experts_per_device, device_rank, top_k
        self.experts = nn.ModuleList(experts)
        self.gate = nn.Linear(d_model, num_experts, bias=False)
        self.group = group
        self.n_ranks = num_experts // experts_per_device

    def get_local_experts(self) -> List[int]:
        s = self.device_rank * self.experts_per_device
        return list(range(s, s + self.experts_per_device))

    def gate_tokens(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        probs = torch.softmax(self.gate(x).float(), -1)
        w, idx = probs.topk(self.top_k, -1)
        return (w / w.sum(-1, keepdim=True)).to(x.dtype), idx

    def route_tokens(self, x: torch.Tensor) -> torch.Tensor:
        """``x [N, d]`` -> mixture of expert outputs ``[N, d]``."""
        N, d = x.shape
        w, idx = self.gate_tokens(x)
        flat_tok = torch.arange(N, device=x.device).repeat_interleave(self.top_k)
        flat_exp = idx.reshape(-1)
        flat_w = w.reshape(-1)
        distributed = dist.is_initialized() and api.get_world_size() > 1 and self.n_ranks > 1
        out = torch.zeros(N, d, dtype=x.dtype, device=x.device)
        if not distributed:
            for e_local, e in enumerate(self.get_local_experts() if self.n_ranks == 1 else range(self.num_experts)):
                sel = flat_exp == e
                if sel.any():
                    y = self.experts[e_local % len(self.experts)](x[flat_tok[sel]])
                    out.index_add_(0, flat_tok[sel], y * flat_w[sel].unsqueeze(-1))
            return out
        # ---- dispatch: sort assignments by owning rank, exchange counts, then tokens
        owner = flat_exp // self.experts_per_device
        order = torch.argsort(owner, stable=True)
        send_counts = torch.bincount(owner, minlength=self.n_ranks)
        recv_counts = torch.empty_like(send_counts)
        api.all_to_all(list(recv_counts.split(1)), list(send_counts.split(1)), self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        send_x = x[flat_tok[order]]
        send_e = flat_exp[order]
        recv_x = [torch.empty(n, d, dtype=x.dtype, device=x.device) for n in rc]
        recv_e = [torch.empty(n, dtype=send_e.dtype, device=x.device) for n in rc]
        api.all_to_all(recv_x, list(send_x.split(sc)), self.group)
        api.all_to_all(recv_e, list(send_e.split(sc)), self.group)
        rx, re = torch.cat(recv_x), torch.cat(recv_e)
        ry = torch.zeros_like(rx)
        for e_local, e in enumerate(self.get_local_experts()):
            sel = re == e
            if sel.any():
                ry[sel] = self.experts[e_local](rx[sel]).to(ry.dtype)
        # ---- combine: send results back along the same routes
        back = [torch.empty(n, d, dtype=x.dtype, device=x.device) for n in sc]
        api.all_to_all(back, list(ry.split(rc)), self.group)
        y = torch.cat(back)
        out.index_add_(0, flat_tok[order], y * flat_w[order].unsqueeze(-1))
        return out

    forward = route_tokens
