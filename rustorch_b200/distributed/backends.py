"""Communication back-end objects, NCCL integration helpers, multi-GPU validator and profiler
(src/distributed/backends.rs:13-239, common.rs:131-190, nccl_integration.rs:23-397, multi_gpu_validation.rs:29-616,
src/gpu/multi_gpu_profiler.rs:20-873, src/gpu/multi_gpu.rs DataParallelTrainer).

The reference's back-ends are shells whose collectives return immediately.  Here every back-end object performs
the collective through ``torch.distributed`` (NCCL on GPUs, gloo on CPU) or, for ``P2PBackend``, through the
peer-memory kernels of this framework.  The validator and profiler measure (CUDA events, max over ranks) instead
of sleeping and cloning.
"""
from __future__ import annotations

import os
import time
import uuid
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from . import api
from .api import DistributedBackend, ReduceOp


@dataclass
class BackendOptimizations:
    """Defaults of the reference (common.rs:131-190): 25 MB buckets, 512 MB pool, 4 streams, zero-copy on."""
    bucket_size_mb: int = 25
    memory_pool_mb: int = 512
    num_streams: int = 4
    zero_copy: bool = True
    compression: bool = False


class GlooTransport(Enum):
    """Transports gloo can run over; TCP is the one available here."""

    TCP = "tcp"
    INFINIBAND = "ib"
    SHARED_MEMORY = "shm"


class DistributedOps:
    """The ``DistributedOps<T>`` trait: six collectives on one process group."""

    name = "base"

    def __init__(self, group=None, optimizations: Optional[BackendOptimizations] = None):
        self.group, self.opt = group, optimizations or BackendOptimizations()

    def all_reduce(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
        api.all_reduce(t, op, self.group)
        return t

    def all_gather(self, t: torch.Tensor) -> List[torch.Tensor]:
        return api.all_gather(t, self.group)

    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        api.broadcast(t, src, self.group)
        return t

    def reduce(self, t: torch.Tensor, dst: int = 0, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
        api.reduce(t, dst, op, self.group)
        return t

    def scatter(self, t: torch.Tensor, scatter_list=None, src: int = 0) -> torch.Tensor:
        api.scatter(t, scatter_list, src, self.group)
        return t

    def gather(self, t: torch.Tensor, dst: int = 0):
        return api.gather(t, dst, self.group)

    def all_reduce_bucketed(self, tensors: Sequence[torch.Tensor], op: ReduceOp = ReduceOp.SUM) -> None:
        """Flatten into buckets of ``bucket_size_mb`` and reduce each bucket with one collective."""
        cap = self.opt.bucket_size_mb * 1024 * 1024
        bucket, size = [], 0

        def flush():
            nonlocal bucket, size
            if not bucket:
                return
            flat = torch.cat([b.reshape(-1).float() for b in bucket])
            self.all_reduce(flat, op)
            o = 0
            for b in bucket:
                b.copy_(flat[o:o + b.numel()].view_as(b))
                o += b.numel()
            bucket, size = [], 0
        for t in tensors:
            nbytes = t.numel() * t.element_size()
            if bucket and (size + nbytes > cap or t.device != bucket[0].device):
                flush()
            bucket.append(t)
            size += nbytes
        flush()


class NCCLBackend(DistributedOps):
    """Back-end object for NCCL over NVLink / NVSwitch (src/distributed/nccl_integration.rs)."""

    name = "nccl"


class GlooBackend(DistributedOps):
    """Back-end object for the gloo transport (CPU tensors) (src/distributed/backends.rs)."""

    name = "gloo"

    def __init__(self, group=None, optimizations=None, transport: GlooTransport = GlooTransport.TCP):
        super().__init__(group, optimizations)
        self.transport = transport


class TCPBackend(GlooBackend):
    """Plain TCP back-end, served by gloo's TCP transport (src/distributed/backends.rs)."""

    name = "tcp"


class P2PBackend(DistributedOps):
    """All-reduce through the peer-memory kernels (one kernel per call); other collectives as the base class."""
    name = "p2p"

    def __init__(self, group=None, optimizations=None, max_numel: int = 1 << 24, dtype: torch.dtype = torch.float32):
        super().__init__(group, optimizations)
        from .p2p_collectives import P2PCollectives
        self.pc = P2PCollectives(max_numel, dtype, group=group.handle if hasattr(group, "handle") else group)

    def all_reduce(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
        if op not in (ReduceOp.SUM, ReduceOp.AVERAGE) or t.dtype != self.pc.dtype or t.numel() > self.pc.max_numel or not t.is_cuda:
            return super().all_reduce(t, op)
        self.pc.all_reduce_(t)
        if op is ReduceOp.AVERAGE:
            t.div_(self.pc.world)
        return t


class BackendFactory:
    @staticmethod
    def create_backend(backend: DistributedBackend, group=None, optimizations: Optional[BackendOptimizations] = None) -> DistributedOps:
        name = backend.value if isinstance(backend, DistributedBackend) else str(backend).lower()
        if name == "nccl":
            return NCCLBackend(group, optimizations)
        if name == "gloo":
            return GlooBackend(group, optimizations)
        if name == "tcp":
            return TCPBackend(group, optimizations)
        if name == "p2p":
            return P2PBackend(group, optimizations)
        raise ValueError(f"backend '{name}' is not available (MPI is not supported)")


# ------------------------------------------------------------------------------ NCCL integration
class NCCLUniqueId:
    """128 opaque bytes identifying a communicator bootstrap; produced on rank 0 and shared through the store."""

    def __init__(self, data: Optional[bytes] = None):
        self.data = data if data is not None else (uuid.uuid4().bytes * 8)
        if len(self.data) != 128:
            raise ValueError("an NCCL unique id is 128 bytes")

    def hex(self) -> str:
        return self.data.hex()


class NCCLCommunicator:
    """A communicator bound to one device: wraps a ``torch.distributed`` NCCL process group (the reference stores a
    null ``comm`` pointer) and a set of side streams."""

    def __init__(self, device_id: int, rank: int, nranks: int, unique_id: Optional[NCCLUniqueId] = None, group=None, num_streams: int = 4):
        self.device_id, self.rank, self.nranks, self.unique_id = device_id, rank, nranks, unique_id or NCCLUniqueId()
        self.group = group
        self.streams = [torch.cuda.Stream(device_id) for _ in range(num_streams)] if torch.cuda.is_available() else []
        self.ops = DistributedOps(group)

    def all_reduce(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
        return self.ops.all_reduce(t, op)

    def all_gather(self, t: torch.Tensor) -> List[torch.Tensor]:
        return self.ops.all_gather(t)

    def broadcast(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        return self.ops.broadcast(t, root)

    def synchronize(self) -> None:
        for s in self.streams:
            s.synchronize()


class NCCLBackendOptimized(NCCLBackend):
    """Bucketed all-reduce with overlap: buckets go out on a side stream while the caller keeps computing."""

    def __init__(self, group=None, optimizations: Optional[BackendOptimizations] = None):
        super().__init__(group, optimizations)
        self._stream = torch.cuda.Stream() if torch.cuda.is_available() else None

    def all_reduce_bucketed_async(self, tensors: Sequence[torch.Tensor], op: ReduceOp = ReduceOp.SUM) -> Callable[[], None]:
        if self._stream is None:
            self.all_reduce_bucketed(tensors, op)
            return lambda: None
        self._stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._stream):
            self.all_reduce_bucketed(tensors, op)
        return lambda: torch.cuda.current_stream().wait_stream(self._stream)


# ------------------------------------------------------------------------------ validator
@dataclass
class DeviceInfo:
    index: int
    name: str
    total_memory: int
    sms: int


@dataclass
class ValidationReport:
    devices: List[DeviceInfo]
    world_size: int
    collectives_ok: bool
    max_error: float
    p2p_matrix: List[List[bool]] = field(default_factory=list)
    messages: List[str] = field(default_factory=list)


@dataclass
class ScalingBenchmark:
    world_size: int
    step_ms: float
    comm_ms: float
    throughput: float
    comm_overhead: float


class MultiGpuValidator:
    """Checks that the devices and the process group really work, and measures collective cost."""

    def __init__(self, tolerance: float = 1e-5):
        self.tol = tolerance

    def discover_devices(self) -> List[DeviceInfo]:
        out = []
        for i in range(torch.cuda.device_count() if torch.cuda.is_available() else 0):
            p = torch.cuda.get_device_properties(i)
            out.append(DeviceInfo(i, p.name, p.total_memory, p.multi_processor_count))
        return out

    def p2p_matrix(self) -> List[List[bool]]:
        n = torch.cuda.device_count() if torch.cuda.is_available() else 0
        return [[i == j or torch.cuda.can_device_access_peer(i, j) for j in range(n)] for i in range(n)]

    def validate_distributed(self, device: Optional[torch.device] = None) -> ValidationReport:
        """Every rank contributes ``rank + 1``; the sums, gathers and broadcasts must come back exact."""
        msgs, ok, err = [], True, 0.0
        world, rank = api.get_world_size(), api.get_rank()
        dev = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and dist.is_initialized()
                         and dist.get_backend() == "nccl" else torch.device("cpu"))
        if dist.is_initialized():
            t = torch.full((1024,), float(rank + 1), device=dev)
            dist.all_reduce(t)
            want = world * (world + 1) / 2
            err = max(err, float((t - want).abs().max()))
            lst = [torch.empty(4, device=dev) for _ in range(world)]
            dist.all_gather(lst, torch.full((4,), float(rank), device=dev))
            err = max(err, max(float((lst[r] - r).abs().max()) for r in range(world)))
            b = torch.full((8,), float(rank), device=dev)
            dist.broadcast(b, world - 1)
            err = max(err, float((b - (world - 1)).abs().max()))
            ok = err <= self.tol
            msgs.append(f"all_reduce / all_gather / broadcast on {world} ranks: max error {err:.2e}")
        else:
            msgs.append("no process group: single-process validation only")
        return ValidationReport(self.discover_devices(), world, ok, err, self.p2p_matrix(), msgs)

    def benchmark(self, step_fn: Callable[[], None], sync_fn: Callable[[], None], items_per_step: int, iters: int = 5) -> ScalingBenchmark:
        """Time ``step_fn`` (compute) and ``sync_fn`` (communication) separately; report overhead and throughput."""
        cuda = torch.cuda.is_available()

        def timed(fn):
            for _ in range(2):
                fn()
            if cuda:
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(iters):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / iters
            else:
                t0 = time.perf_counter()
                for _ in range(iters):
                    fn()
                ms = (time.perf_counter() - t0) / iters * 1e3
            if dist.is_initialized():
                t = torch.tensor([ms], device="cuda" if cuda and dist.get_backend() == "nccl" else "cpu")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t)
            return ms
        step_ms, comm_ms = timed(step_fn), timed(sync_fn)
        world = api.get_world_size()
        total = step_ms + comm_ms
        return ScalingBenchmark(world, step_ms, comm_ms, items_per_step * world / (total / 1e3), comm_ms / total if total else 0.0)

    @staticmethod
    def scaling_efficiency(throughput_1: float, throughput_n: float, n: int) -> float:
        return throughput_n / (n * throughput_1) if throughput_1 > 0 else 0.0


# ------------------------------------------------------------------------------ profiler
@dataclass
class GpuMetrics:
    index: int
    compute_ms: float = 0.0
    comm_ms: float = 0.0
    idle_ms: float = 0.0
    memory_used: int = 0
    samples: int = 0


class MultiGpuProfiler:
    """Per-GPU compute / communication time from CUDA events around user-marked regions."""

    def __init__(self):
        self.gpus: Dict[int, GpuMetrics] = {}
        self.comm_events: List[Dict[str, float]] = []
        self._open: Dict[str, tuple] = {}

    def _gpu(self, i: int) -> GpuMetrics:
        return self.gpus.setdefault(i, GpuMetrics(i))

    def start(self, kind: str, device: int = 0, nbytes: int = 0) -> str:
        key = f"{kind}:{device}:{len(self._open)}:{time.perf_counter_ns()}"
        if torch.cuda.is_available():
            e = torch.cuda.Event(enable_timing=True)
            with torch.cuda.device(device):
                e.record()
            self._open[key] = (kind, device, nbytes, e, None)
        else:
            self._open[key] = (kind, device, nbytes, None, time.perf_counter())
        return key

    def stop(self, key: str) -> float:
        kind, device, nbytes, ev, t0 = self._open.pop(key)
        if ev is not None:
            e1 = torch.cuda.Event(enable_timing=True)
            with torch.cuda.device(device):
                e1.record()
            e1.synchronize()
            ms = ev.elapsed_time(e1)
        else:
            ms = (time.perf_counter() - t0) * 1e3
        return self.record(kind, device, ms, nbytes)

    def record(self, kind: str, device: int, ms: float, nbytes: int = 0) -> float:
        g = self._gpu(device)
        g.samples += 1
        if kind == "compute":
            g.compute_ms += ms
        elif kind == "comm":
            g.comm_ms += ms
            self.comm_events.append({"device": device, "ms": ms, "bytes": nbytes, "gbps": nbytes / ms / 1e6 if ms > 0 else 0.0})
        else:
            g.idle_ms += ms
        if torch.cuda.is_available() and device < torch.cuda.device_count():
            g.memory_used = max(g.memory_used, torch.cuda.memory_allocated(device))
        return ms

    def bottlenecks(self) -> List[str]:
        out = []
        for g in self.gpus.values():
            tot = g.compute_ms + g.comm_ms + g.idle_ms
            if tot and g.comm_ms / tot > 0.3:
                out.append(f"GPU {g.index}: {g.comm_ms / tot:.0%} of the time in communication: overlap it with backward or fuse it into the kernels")
            if tot and g.idle_ms / tot > 0.2:
                out.append(f"GPU {g.index}: idle {g.idle_ms / tot:.0%}: load imbalance or host-bound launches")
        comp = [g.compute_ms for g in self.gpus.values() if g.compute_ms]
        if len(comp) > 1 and max(comp) > 1.2 * min(comp):
            out.append("compute time differs by more than 20% between GPUs: rebalance the shards")
        return out

    def report(self) -> str:
        rows = [f"{'gpu':<5}{'compute ms':>12}{'comm ms':>10}{'idle ms':>10}{'mem MB':>10}"]
        for g in sorted(self.gpus.values(), key=lambda x: x.index):
            rows.append(f"{g.index:<5}{g.compute_ms:>12.2f}{g.comm_ms:>10.2f}{g.idle_ms:>10.2f}{g.memory_used / 2 ** 20:>10.1f}")
        if self.comm_events:
            bw = sum(e["gbps"] for e in self.comm_events) / len(self.comm_events)
            rows.append(f"mean collective bandwidth {bw:.1f} GB/s over {len(self.comm_events)} calls")
        return "\n".join(rows + self.bottlenecks())


class DataParallelTrainer:
    """Single-process multi-GPU data parallel (the ``multi_gpu.rs`` trainer): replicas on each device, batch split,
    gradients averaged on device 0 and parameters re-broadcast."""

    def __init__(self, module: torch.nn.Module, device_ids: Optional[Sequence[int]] = None):
        self.device_ids = list(device_ids) if device_ids is not None else list(range(max(1, torch.cuda.device_count())))
        self.cuda = torch.cuda.is_available()
        import copy
        devs = [torch.device("cuda", i) for i in self.device_ids] if self.cuda else [torch.device("cpu")] * len(self.device_ids)
        self.replicas = [module.to(devs[0])] + [copy.deepcopy(module).to(d) for d in devs[1:]]
        self.devices = devs

    def train_step(self, x: torch.Tensor, y: torch.Tensor, loss_fn: Callable, optimizer: torch.optim.Optimizer) -> float:
        xs, ys = x.chunk(len(self.replicas)), y.chunk(len(self.replicas))
        losses = []
        for m, d, xi, yi in zip(self.replicas, self.devices, xs, ys):
            m.zero_grad(set_to_none=True)
            loss = loss_fn(m(xi.to(d)), yi.to(d))
            loss.backward()
            losses.append(float(loss.detach()) * xi.shape[0])
        main = self.replicas[0]
        with torch.no_grad():
            for ps in zip(*[list(m.parameters()) for m in self.replicas]):
                g = sum(p.grad.to(self.devices[0]) * xi.shape[0] for p, xi in zip(ps, xs)) / x.shape[0]
                ps[0].grad = g
        optimizer.step()
        with torch.no_grad():
            for ps in zip(*[list(m.parameters()) for m in self.replicas]):
                for p in ps[1:]:
                    p.copy_(ps[0].to(p.device))
        return sum(losses) / x.shape[0]
