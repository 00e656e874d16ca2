"""Batch-parallel tensor operations (src/tensor/parallel_ops.rs:14-424, parallel_traits.rs:103-291, parallel_impl.rs,
src/parallel.rs:7-28, src/utils/mod.rs:7-45).

The reference spreads a batch over rayon worker threads.  On a B200 a batch is one kernel (``bmm``, a fused
normalisation, a channels-last convolution): the "parallel strategy" decides only between a single launch, chunked
launches on several CUDA streams (for batches whose chunks differ in shape or that do not fit one workspace) and,
on the CPU, torch's intra-op thread pool.  The trait names are kept as mix-in classes over ``torch.Tensor`` lists.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from enum import Enum
from typing import Callable, List, Optional, Sequence

import torch
import torch.nn.functional as F


class ParallelStrategy(Enum):
    """How a batch operation is split across workers (src/tensor/parallel_traits.rs)."""

    AUTO = "auto"
    SEQUENTIAL = "sequential"
    FORCE_PARALLEL = "force_parallel"


@dataclass
class ParallelConfig:
    """``strategy``, the element count from which work is split (reference default 1000), chunk size and workers."""
    strategy: ParallelStrategy = ParallelStrategy.AUTO
    threshold: int = 1000
    chunk_size: int = 0
    num_threads: int = 0

    def should_parallelize(self, numel: int) -> bool:
        if self.strategy is ParallelStrategy.SEQUENTIAL:
            return False
        return self.strategy is ParallelStrategy.FORCE_PARALLEL or numel >= self.threshold


class ParallelContext:
    """Scoped configuration: sets torch's CPU thread count and hands out CUDA side streams for chunked launches."""

    _current: Optional["ParallelContext"] = None

    def __init__(self, config: Optional[ParallelConfig] = None, streams: int = 4):
        self.config = config or ParallelConfig()
        self._n_streams, self._streams, self._saved_threads = streams, None, None

    def __enter__(self) -> "ParallelContext":
        self._prev, ParallelContext._current = ParallelContext._current, self
        if self.config.num_threads > 0:
            self._saved_threads = torch.get_num_threads()
            torch.set_num_threads(self.config.num_threads)
        return self

    def __exit__(self, *exc) -> None:
        ParallelContext._current = self._prev
        if self._saved_threads is not None:
            torch.set_num_threads(self._saved_threads)

    @classmethod
    def current(cls) -> "ParallelContext":
        return cls._current or cls()

    def streams(self, device) -> List["torch.cuda.Stream"]:
        if self._streams is None:
            self._streams = [torch.cuda.Stream(device) for _ in range(self._n_streams)]
        return self._streams

    def map_chunks(self, fn: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor) -> torch.Tensor:
        """``fn`` over chunks of dim 0: on CUDA each chunk runs on its own stream, on the CPU they run in turn."""
        cfg = self.config
        n = x.shape[0]
        chunk = cfg.chunk_size or max(1, math.ceil(n / self._n_streams))
        if not cfg.should_parallelize(x.numel()) or n <= chunk:
            return fn(x)
        parts = list(x.split(chunk, 0))
        if not x.is_cuda:
            return torch.cat([fn(p) for p in parts], 0)
        cur = torch.cuda.current_stream(x.device)
        outs = []
        for i, p in enumerate(parts):
            s = self.streams(x.device)[i % self._n_streams]
            s.wait_stream(cur)
            with torch.cuda.stream(s):
                outs.append(fn(p))
        for s in self.streams(x.device):
            cur.wait_stream(s)
        return torch.cat(outs, 0)


# ------------------------------------------------------------------------------------ free functions of the reference
def batch_matmul_parallel(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``[B, M, K] @ [B, K, N]`` (or a shared ``[K, N]``): one batched GEMM."""
    return torch.matmul(a, b)


def batch_add_parallel(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return a + b


def batch_mul_parallel(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return a * b


def batch_scalar_mul_parallel(a: torch.Tensor, s: float) -> torch.Tensor:
    return a * s


def batch_normalize_parallel(x: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """Every batch item to zero mean / unit variance over its own elements."""
    flat = x.reshape(x.shape[0], -1).float()
    mean, var = flat.mean(1, keepdim=True), flat.var(1, unbiased=False, keepdim=True)
    return ((flat - mean) * torch.rsqrt(var + eps)).reshape(x.shape).to(x.dtype)


def batch_conv2d_parallel(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, stride=1, padding=0) -> torch.Tensor:
    from ..ops import conv as _conv
    return _conv.conv2d(x, weight, bias, stride, padding)


def batch_sum_parallel(x: torch.Tensor, dim: int = 0) -> torch.Tensor:
    return x.sum(dim)


def batch_mean_parallel(x: torch.Tensor, dim: int = 0) -> torch.Tensor:
    return x.mean(dim)


def parallel_map(fn: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, config: Optional[ParallelConfig] = None) -> torch.Tensor:
    return ParallelContext(config).map_chunks(fn, x)


# ------------------------------------------------------------------------------------ trait mix-ins
class ParallelOp:
    """Base trait: the configuration and the decision whether an op is worth splitting."""
    parallel_config = ParallelConfig()

    def should_parallelize(self, numel: int) -> bool:
        return self.parallel_config.should_parallelize(numel)


class BatchParallelOp(ParallelOp):
    def batch_elementwise_op(self, a: torch.Tensor, b: torch.Tensor, op: Callable) -> torch.Tensor:
        return op(a, b)

    def batch_scalar_op(self, a: torch.Tensor, s: float, op: Callable) -> torch.Tensor:
        return op(a, s)

    def batch_normalize(self, a: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
        return batch_normalize_parallel(a, eps)


class MatrixParallelOp(ParallelOp):
    def batch_matmul(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        return batch_matmul_parallel(a, b)

    def batch_conv2d(self, x, weight, bias=None, stride=1, padding=0) -> torch.Tensor:
        return batch_conv2d_parallel(x, weight, bias, stride, padding)


class ReductionParallelOp(ParallelOp):
    def parallel_sum(self, x: torch.Tensor, dim: Optional[int] = None) -> torch.Tensor:
        return x.sum() if dim is None else x.sum(dim)

    def parallel_mean(self, x: torch.Tensor, dim: Optional[int] = None) -> torch.Tensor:
        return x.mean() if dim is None else x.mean(dim)

    def parallel_max(self, x: torch.Tensor) -> torch.Tensor:
        return x.max()

    def parallel_min(self, x: torch.Tensor) -> torch.Tensor:
        return x.min()

    def parallel_variance(self, x: torch.Tensor, unbiased: bool = False) -> torch.Tensor:
        return x.var(unbiased=unbiased)


class SimdParallelOp(ParallelOp):
    """The reference pairs rayon with AVX2 lanes; the device analogue is 16-byte vector access in the native kernels."""

    def simd_parallel_add(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        from ..ops import elementwise as E
        return E.add(a, b)

    def simd_parallel_mul(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        from ..ops import elementwise as E
        return E.mul(a, b)

    def simd_parallel_dot(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        return (a.reshape(-1).float() * b.reshape(-1).float()).sum()


class GpuParallelOp(ParallelOp):
    """Reductions and batched products that pick the device by size (src/tensor/gpu_parallel.rs:139-333)."""

    @staticmethod
    def _place(x: torch.Tensor) -> torch.Tensor:
        from ..tensor import select_optimal_device
        return x.to(select_optimal_device(x.numel())) if not x.is_cuda else x

    def gpu_sum(self, x): return self._place(x).sum()
    def gpu_mean(self, x): return self._place(x).mean()
    def gpu_max(self, x): return self._place(x).max()
    def gpu_min(self, x): return self._place(x).min()
    def gpu_std(self, x, unbiased: bool = False): return self._place(x).std(unbiased=unbiased)
    def gpu_var(self, x, unbiased: bool = False): return self._place(x).var(unbiased=unbiased)
    def gpu_batch_matmul(self, a, b): return torch.matmul(self._place(a), self._place(b).to(self._place(a).device))


class ParallelTensor(BatchParallelOp, MatrixParallelOp, ReductionParallelOp, SimdParallelOp, GpuParallelOp):
    """A tensor with the parallel traits attached (src/parallel.rs:7-28)."""

    def __init__(self, data: torch.Tensor, config: Optional[ParallelConfig] = None):
        self.data = data
        if config is not None:
            self.parallel_config = config

    def map(self, fn: Callable[[torch.Tensor], torch.Tensor]) -> "ParallelTensor":
        return ParallelTensor(ParallelContext(self.parallel_config).map_chunks(fn, self.data), self.parallel_config)

    def matmul(self, other) -> "ParallelTensor":
        o = other.data if isinstance(other, ParallelTensor) else other
        return ParallelTensor(self.batch_matmul(self.data, o), self.parallel_config)

    def sum(self) -> torch.Tensor:
        return self.parallel_sum(self.data)


# ------------------------------------------------------------------------------------ src/utils/mod.rs helpers
def kaiming_init(shape: Sequence[int], fan_in: Optional[int] = None, device=None, dtype=torch.float32) -> torch.Tensor:
    """``N(0, sqrt(2 / fan_in))`` with ``fan_in`` defaulting to the first dimension (src/utils/mod.rs:7-19)."""
    fan = fan_in if fan_in is not None else int(shape[0])
    return torch.randn(*shape, device=device, dtype=dtype) * math.sqrt(2.0 / max(1, fan))


def softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    from ..ops import elementwise as E
    return E.softmax(x, dim)


def mse_loss(pred: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    return F.mse_loss(pred, target)


def num_cpu_threads() -> int:
    return int(os.environ.get("RAYON_NUM_THREADS", torch.get_num_threads()))
