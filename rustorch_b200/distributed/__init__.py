"""``rustorch.distributed``: process groups, collectives, DDP / TP / PP / EP, cluster management
(src/distributed/mod.rs)."""
from .api import (CommunicationStats, DistributedBackend, DistributedRequest, ProcessGroup, ReduceOp, all_gather,
                  all_reduce, all_to_all, barrier, broadcast, cleanup_distributed, destroy_process_group, finalize,
                  gather, get_process_group, get_rank, get_world_size, init_distributed, init_process_group,
                  irecv, is_available, is_initialized, is_master, isend, monitoring, new_group, recv, reduce, reduce_scatter,
                  scatter, send)
from .async_gradient import (AsyncConfig, AsyncGradientSynchronizer, CommunicationScheduler, GradientBucketManager,
                             GradientCompressor, Priority, QuantizationCompressor, TensorMemoryPool, TopKCompressor)
from .backends import (BackendFactory, BackendOptimizations, DataParallelTrainer, DeviceInfo, DistributedOps, GlooBackend,
                       GlooTransport, GpuMetrics, MultiGpuProfiler, MultiGpuValidator, NCCLBackend, NCCLBackendOptimized,
                       NCCLCommunicator, NCCLUniqueId, P2PBackend, ScalingBenchmark, TCPBackend, ValidationReport)
from .cluster import (ClusterConfig, ClusterManager, ClusterTopology, FaultToleranceConfig, HeartbeatMonitor,
                      NodeCapabilities, NodeInfo, NodeStatus, ResourceScheduler, SchedulingPolicy, StoreHeartbeat, retry)
from .ddp import (DataParallel, DistributedDataLoader, DistributedDataParallel, DistributedSampler, GradientBucket,
                  GradientSyncStrategy, SimpleDistributedDataParallel, wrap_module, wrap_simple)
from .ddp_flat import FlatDDP, bucket_ranges
from .model_parallel import (ColumnParallelLinear, CommunicationType, ExpertParallel, ModelParallel, PartitionStrategy,
                             PipelineConfig, PipelineOp, PipelineSchedule, PipelineScheduler, PipelineStage,
                             RowParallelLinear, TensorParallel)
from .multi_gpu import (AllReduceAlgorithm, CommBackend, DistributedTrainer, GpuTopology, LearningRateSchedule,
                        LoadBalancer, MultiGpuBarrier, MultiGpuContext, NCCLOps, NCCLOptimizations, NCCLProfiler,
                        ParallelismStrategy, ParameterServer, StreamManager, StreamPriority, TransferStatistics)
from .optimizer import DistributedOptimizer, SyncStrategy
from .context_parallel import RingAttention, gather_sequence, ring_attention, shard_sequence
