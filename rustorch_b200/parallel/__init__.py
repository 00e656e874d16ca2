"""Parallel execution: batch-parallel tensor operations and traits (``batch_ops``), and the multi-GPU strategies,
which live in :mod:`rustorch_b200.distributed` (data / tensor / pipeline / expert parallelism) and are re-exported
here under the names a user of the reference's ``parallel`` / ``distributed`` modules looks for."""
from .batch_ops import (BatchParallelOp, GpuParallelOp, MatrixParallelOp, ParallelConfig, ParallelContext, ParallelOp, ParallelStrategy,
                        ParallelTensor, ReductionParallelOp, SimdParallelOp, batch_add_parallel, batch_conv2d_parallel,
                        batch_matmul_parallel, batch_mean_parallel, batch_mul_parallel, batch_normalize_parallel,
                        batch_scalar_mul_parallel, batch_sum_parallel, kaiming_init, mse_loss, num_cpu_threads, parallel_map,
                        softmax)


def __getattr__(name):
    # DistributedDataParallel, ColumnParallelLinear, PipelineStage ... without importing torch.distributed eagerly
    from .. import distributed
    if hasattr(distributed, name):
        return getattr(distributed, name)
    raise AttributeError(f"module 'rustorch_b200.parallel' has no attribute '{name}'")
