"""Single-process multi-GPU context, collectives over device lists, sync primitives, the
distributed trainer / parameter server and NCCL tuning helpers
(src/gpu/multi_gpu.rs:16-1121, src/gpu/sync_primitives.rs:14-313, src/gpu/distributed_training.rs:17-636,
src/distributed/nccl_integration.rs:234-585).

The reference runs these over host vectors; here the lists hold real tensors that may sit on different
CUDA devices (peer copies over NVLink) or all on the CPU (then everything is host arithmetic, which is
also what the tests use).  The math oracle is the reference's: ``all_reduce`` leaves the element-wise
mean (``[1,2,3,4]`` & ``[5,6,7,8]`` -> ``[3,4,5,6]``, tests/multi_gpu_operations_test.rs:93-120).
"""
from __future__ import annotations

import enum
import math
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch


class ParallelismStrategy(enum.Enum):
    """Data, model, pipeline or hybrid parallelism of a multi-GPU context."""

    DATA_PARALLEL = "data_parallel"
    MODEL_PARALLEL = "model_parallel"
    PIPELINE_PARALLEL = "pipeline_parallel"
    HYBRID = "hybrid"
    EXPERT_PARALLEL = "expert_parallel"


class CommBackend(enum.Enum):
    """Communication library a multi-GPU context uses."""

    NCCL = "nccl"
    P2P = "p2p"
    HOST_STAGED = "host_staged"


class AllReduceAlgorithm(enum.Enum):
    """Algorithm choices of the multi-GPU all-reduce (src/gpu/multi_gpu.rs:583-701)."""

    RING = "ring"
    TREE = "tree"
    BUTTERFLY = "butterfly"
    DOUBLE_BINARY_TREE = "double_binary_tree"


@dataclass
class GpuTopology:
    num_gpus: int
    p2p_matrix: List[List[bool]]
    bandwidth_matrix: List[List[float]]     # GB/s per direction
    nvlink: bool = True

    @staticmethod
    def probe(device_ids: Sequence[int]) -> "GpuTopology":
        n = len(device_ids)
        p2p = [[True] * n for _ in range(n)]
        if torch.cuda.is_available():
            for i, a in enumerate(device_ids):
                for j, b in enumerate(device_ids):
                    if i != j and a < torch.cuda.device_count() and b < torch.cuda.device_count():
                        p2p[i][j] = bool(torch.cuda.can_device_access_peer(a, b))
        # NVLink 5 through NVSwitch: uniform 900 GB/s per direction nominal; local = HBM
        bw = [[7700.0 if i == j else (900.0 if p2p[i][j] else 64.0) for j in range(n)] for i in range(n)]
        return GpuTopology(n, p2p, bw, all(all(r) for r in p2p))


@dataclass
class TransferStatistics:
    bytes_moved: int = 0
    transfers: int = 0
    seconds: float = 0.0

    def bandwidth_gbs(self) -> float:
        return self.bytes_moved / self.seconds / 1e9 if self.seconds > 0 else 0.0


class MultiGpuBarrier:
    """Host barrier for ``len(gpu_ids)`` participants; ``wait`` raises ``TimeoutError`` after ``timeout`` s."""

    def __init__(self, gpu_ids: Sequence[int], timeout: float = 30.0):
        self.n, self.timeout = len(gpu_ids), timeout
        self._cv = threading.Condition()
        self._count, self._gen = 0, 0

    def wait(self, gpu_id: int = 0, timeout: Optional[float] = None) -> None:
        t = self.timeout if timeout is None else timeout
        with self._cv:
            gen = self._gen
            self._count += 1
            if self._count == self.n:
                self._count = 0
                self._gen += 1
                self._cv.notify_all()
                return
            if not self._cv.wait_for(lambda: self._gen != gen, t):
                self._count -= 1
                raise TimeoutError(f"barrier timed out after {t} s (gpu {gpu_id})")


class StreamPriority(enum.IntEnum):
    """Priority class of a CUDA stream."""

    LOW = 0
    NORMAL = 1
    HIGH = 2


class StreamManager:
    """CUDA streams and events by id (``create_stream / create_event / record_event / wait_event /
    query_event / synchronize_device``); on a machine without CUDA the same calls keep host bookkeeping."""

    def __init__(self):
        self.streams: Dict[int, object] = {}
        self.events: Dict[int, object] = {}
        self._host_events: Dict[int, threading.Event] = {}
        self._next = 0

    def create_stream(self, device: int = 0, priority: StreamPriority = StreamPriority.NORMAL) -> int:
        sid = self._next
        self._next += 1
        if torch.cuda.is_available():
            self.streams[sid] = torch.cuda.Stream(device=device, priority=-1 if priority is StreamPriority.HIGH else 0)
        else:
            self.streams[sid] = None
        return sid

    def create_event(self) -> int:
        eid = self._next
        self._next += 1
        if torch.cuda.is_available():
            self.events[eid] = torch.cuda.Event()
        else:
            self._host_events[eid] = threading.Event()
        return eid

    def record_event(self, event_id: int, stream_id: Optional[int] = None) -> None:
        if torch.cuda.is_available():
            self.events[event_id].record(self.streams[stream_id] if stream_id is not None else None)
        else:
            self._host_events[event_id].set()

    def query_event(self, event_id: int) -> bool:
        if torch.cuda.is_available():
            return bool(self.events[event_id].query())
        return self._host_events[event_id].is_set()

    def wait_event(self, event_id: int, timeout: float = 30.0) -> None:
        deadline = time.monotonic() + timeout
        while not self.query_event(event_id):
            if time.monotonic() > deadline:
                raise TimeoutError(f"event {event_id} not reached within {timeout} s")
            time.sleep(0.0005)

    def synchronize_device(self, device: int = 0) -> None:
        if torch.cuda.is_available():
            torch.cuda.synchronize(device)


class MultiGpuContext:
    def __init__(self, device_ids: Sequence[int], strategy: ParallelismStrategy = ParallelismStrategy.DATA_PARALLEL,
                 backend: CommBackend = CommBackend.P2P):
        if not device_ids:
            raise ValueError("device_ids must not be empty")
        self.device_ids = list(device_ids)
        self.strategy, self.backend = strategy, backend
        self.topology = GpuTopology.probe(self.device_ids)
        self.stats = TransferStatistics()
        self.barrier = MultiGpuBarrier(self.device_ids)
        self.comm_groups: Dict[str, List[int]] = {"world": list(self.device_ids)}

    def num_gpus(self) -> int:
        return len(self.device_ids)

    def execute(self, fn: Callable[[int], object]) -> List[object]:
        """Run ``fn(gpu_id)`` for every device in its own thread (its own CUDA current device)."""
        out: List[object] = [None] * len(self.device_ids)
        errs: List[BaseException] = []

        def run(i, d):
            try:
                if torch.cuda.is_available() and d < torch.cuda.device_count():
                    with torch.cuda.device(d):
                        out[i] = fn(d)
                else:
                    out[i] = fn(d)
            except BaseException as e:  # noqa: BLE001
                errs.append(e)

        ts = [threading.Thread(target=run, args=(i, d)) for i, d in enumerate(self.device_ids)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        if errs:
            raise errs[0]
        return out

    def _account(self, nbytes: int, t0: float) -> None:
        self.stats.bytes_moved += nbytes
        self.stats.transfers += 1
        self.stats.seconds += time.perf_counter() - t0

    # collectives over a list of per-device tensors (in place)
    def all_reduce(self, tensors: List[torch.Tensor], average: bool = True,
                   algorithm: AllReduceAlgorithm = AllReduceAlgorithm.RING) -> List[torch.Tensor]:
        n = len(tensors)
        t0 = time.perf_counter()
        if algorithm is AllReduceAlgorithm.RING and n > 1 and tensors[0].numel() >= n:
            self._ring_all_reduce(tensors)
        else:
            total = tensors[0].clone()
            for t in tensors[1:]:
                total += t.to(total.device)
            for t in tensors:
                t.copy_(total.to(t.device))
        if average:
            for t in tensors:
                t.div_(n)
        self._account(2 * (n - 1) * tensors[0].numel() * tensors[0].element_size(), t0)
        return tensors

    @staticmethod
    def _ring_all_reduce(tensors: List[torch.Tensor]) -> None:
        """Reduce-scatter then all-gather over ``n`` chunks (``n - 1`` steps each)."""
        n = len(tensors)
        flats = [t.view(-1) for t in tensors]
        bounds = [(i * flats[0].numel()) // n for i in range(n + 1)]
        ch = lambda r, c: flats[r][bounds[c]:bounds[c + 1]]  # noqa: E731
        for step in range(n - 1):
            sends = [(r, (r - step) % n, ch(r, (r - step) % n).clone()) for r in range(n)]
            for r, c, data in sends:
                dst = (r + 1) % n
                ch(dst, c).add_(data.to(flats[dst].device))
        for step in range(n - 1):
            sends = [(r, (r + 1 - step) % n, ch(r, (r + 1 - step) % n).clone()) for r in range(n)]
            for r, c, data in sends:
                dst = (r + 1) % n
                ch(dst, c).copy_(data.to(flats[dst].device))

    def broadcast(self, tensors: List[torch.Tensor], root: int = 0) -> List[torch.Tensor]:
        """Binary-tree order: rank ``r`` receives from ``(r - 1) // 2`` relative to the root."""
        n = len(tensors)
        t0 = time.perf_counter()
        order = [(root + i) % n for i in range(n)]
        for i in range(1, n):
            src, dst = order[(i - 1) // 2], order[i]
            tensors[dst].copy_(tensors[src].to(tensors[dst].device))
        self._account((n - 1) * tensors[0].numel() * tensors[0].element_size(), t0)
        return tensors

    def scatter(self, tensor: torch.Tensor, dim: int = 0) -> List[torch.Tensor]:
        chunks = tensor.chunk(len(self.device_ids), dim)
        if torch.cuda.is_available():
            return [c.to(torch.device("cuda", d)) if d < torch.cuda.device_count() else c for c, d in zip(chunks, self.device_ids)]
        return [c.clone() for c in chunks]

    def gather(self, tensors: List[torch.Tensor], dim: int = 0, root: int = 0) -> torch.Tensor:
        dev = tensors[root].device
        return torch.cat([t.to(dev) for t in tensors], dim)


class LoadBalancer:
    """Splits a batch proportionally to per-device throughput estimates."""

    def __init__(self, n: int):
        self.speed = [1.0] * n

    def update(self, device: int, samples_per_s: float, momentum: float = 0.5) -> None:
        self.speed[device] = momentum * self.speed[device] + (1 - momentum) * samples_per_s

    def split(self, batch: int) -> List[int]:
        tot = sum(self.speed)
        parts = [int(batch * s / tot) for s in self.speed]
        for i in range(batch - sum(parts)):
            parts[i % len(parts)] += 1
        return parts


# ------------------------------------------------------- distributed trainer (host)
class LearningRateSchedule(enum.Enum):
    """Learning-rate policy of the distributed trainer (src/gpu/distributed_training.rs)."""

    CONSTANT = "constant"
    LINEAR_DECAY = "linear_decay"
    EXPONENTIAL_DECAY = "exponential_decay"
    COSINE_ANNEALING = "cosine_annealing"
    WARMUP_DECAY = "warmup_decay"


@dataclass
class TrainingFaultConfig:
    max_retries: int = 3
    retry_delay: float = 0.1
    checkpoint_frequency: int = 1000
    accumulate_on_failure: bool = True


class ParameterServer:
    """Keeps the canonical parameters; ``push`` averages worker gradients and applies SGD."""

    def __init__(self, params: List[torch.Tensor], lr: float = 0.01):
        self.params = [p.clone() for p in params]
        self.lr, self.version = lr, 0

    def push(self, worker_grads: List[List[torch.Tensor]]) -> None:
        n = len(worker_grads)
        for i, p in enumerate(self.params):
            g = sum(w[i].to(p.device) for w in worker_grads) / n
            p.sub_(self.lr * g)
        self.version += 1

    def pull(self) -> List[torch.Tensor]:
        return [p.clone() for p in self.params]


class DistributedTrainer:
    """``training_step(params, grads)``: all-reduce -> optional top-k compression -> parameter-server or local
    SGD update, with LR schedule, periodic checkpoints and ``handle_failure`` (reload + redistribute)."""

    def __init__(self, ctx: MultiGpuContext, lr: float = 0.01, schedule: LearningRateSchedule = LearningRateSchedule.CONSTANT,
                 total_steps: int = 1000, warmup_steps: int = 0, compression_ratio: Optional[float] = None,
                 use_parameter_server: bool = False, fault: Optional[TrainingFaultConfig] = None):
        self.ctx, self.base_lr, self.schedule = ctx, lr, schedule
        self.total_steps, self.warmup_steps = total_steps, warmup_steps
        self.compression_ratio, self.use_ps = compression_ratio, use_parameter_server
        self.fault = fault or TrainingFaultConfig()
        self.step_count = 0
        self.checkpoint: Optional[dict] = None
        self.active = list(range(ctx.num_gpus()))
        self.server: Optional[ParameterServer] = None
        self.profiling = False
        self.timings: List[Dict[str, float]] = []

    def enable_profiling(self, on: bool = True) -> None:
        self.profiling = on

    def current_lr(self) -> float:
        t, T, lr = self.step_count, max(1, self.total_steps), self.base_lr
        s = self.schedule
        if s is LearningRateSchedule.CONSTANT:
            return lr
        if s is LearningRateSchedule.LINEAR_DECAY:
            return lr * max(0.0, 1 - t / T)
        if s is LearningRateSchedule.EXPONENTIAL_DECAY:
            return lr * 0.96 ** (t / max(1, T / 100))
        if s is LearningRateSchedule.COSINE_ANNEALING:
            return lr * 0.5 * (1 + math.cos(math.pi * min(t, T) / T))
        if t < self.warmup_steps:
            return lr * (t + 1) / self.warmup_steps
        return lr * max(0.0, 1 - (t - self.warmup_steps) / max(1, T - self.warmup_steps))

    @staticmethod
    def compress_topk(g: torch.Tensor, ratio: float) -> torch.Tensor:
        k = max(1, int(g.numel() * ratio))
        flat = g.reshape(-1)
        thr = flat.abs().topk(k).values[-1]
        return torch.where(g.abs() >= thr, g, torch.zeros_like(g))

    def training_step(self, params: List[List[torch.Tensor]], grads: List[List[torch.Tensor]]) -> float:
        """``params[w][i]`` / ``grads[w][i]``: tensor ``i`` of worker ``w``.  Returns the lr used."""
        t0 = time.perf_counter()
        workers = [w for w in range(len(grads)) if w in self.active]
        n_t = len(grads[workers[0]])
        for i in range(n_t):
            gs = [grads[w][i] for w in workers]
            if self.compression_ratio:
                for g in gs:
                    g.copy_(self.compress_topk(g, self.compression_ratio))
            self.ctx.all_reduce(gs, average=True)
        t1 = time.perf_counter()
        lr = self.current_lr()
        if self.use_ps:
            if self.server is None:
                self.server = ParameterServer(params[workers[0]], lr)
            self.server.lr = lr
            self.server.push([grads[workers[0]]])
            new = self.server.pull()
            for w in workers:
                for p, q in zip(params[w], new):
                    p.copy_(q.to(p.device))
        else:
            for w in workers:
                for p, g in zip(params[w], grads[w]):
                    p.sub_(lr * g)
        self.step_count += 1
        if self.step_count % self.fault.checkpoint_frequency == 0:
            self.save_checkpoint(params[workers[0]])
        if self.profiling:
            self.timings.append({"comm_s": t1 - t0, "update_s": time.perf_counter() - t1})
        return lr

    def save_checkpoint(self, params: List[torch.Tensor]) -> None:
        self.checkpoint = {"step": self.step_count, "params": [p.detach().cpu().clone() for p in params]}

    def load_checkpoint(self, params: List[List[torch.Tensor]]) -> int:
        if self.checkpoint is None:
            return self.step_count
        for w in self.active:
            for p, q in zip(params[w], self.checkpoint["params"]):
                p.copy_(q.to(p.device))
        self.step_count = self.checkpoint["step"]
        return self.step_count

    def handle_failure(self, failed_gpu: int, params: Optional[List[List[torch.Tensor]]] = None) -> List[int]:
        """Drop the failed worker, restore the survivors from the last checkpoint, return the new worker set."""
        if failed_gpu in self.active:
            self.active.remove(failed_gpu)
        if not self.active:
            raise RuntimeError("no workers left")
        if params is not None:
            self.load_checkpoint(params)
        return list(self.active)

    def redistribute_workload(self, global_batch: int) -> List[int]:
        n = len(self.active)
        parts = [global_batch // n] * n
        for i in range(global_batch % n):
            parts[i] += 1
        return parts


# ---------------------------------------------------------------- NCCL helpers
@dataclass
class NCCLOptimizations:
    compression: bool = False
    bucket_size_mb: int = 25
    num_streams: int = 4
    async_ops: bool = True
    timeout_s: float = 300.0


class NCCLOps:
    @staticmethod
    def get_optimal_config(num_gpus: int, memory_per_gpu_gb: float) -> NCCLOptimizations:
        """50 MB buckets above 16 GB per GPU, 8 streams above 4 GPUs (nccl_integration.rs:402-485)."""
        return NCCLOptimizations(bucket_size_mb=50 if memory_per_gpu_gb > 16 else 25,
                                 num_streams=8 if num_gpus > 4 else 4)


    @staticmethod
    def init_multi_gpu(device_ids: Optional[List[int]] = None) -> "MultiGpuContext":
        """A context over the given (default: all visible) devices (nccl_integration.rs:402-440)."""
        ids = list(device_ids) if device_ids is not None else list(range(max(1, torch.cuda.device_count())))
        return MultiGpuContext(ids)

    @staticmethod
    def all_reduce_multi_gpu(tensors: List[torch.Tensor], average: bool = True) -> List[torch.Tensor]:
        """In-place all-reduce over one tensor per device (nccl_integration.rs:441-470)."""
        return p2p_all_reduce(tensors, average)


def p2p_all_reduce(tensors: List[torch.Tensor], average: bool = False) -> List[torch.Tensor]:
    """Ring all-reduce (reduce-scatter + all-gather, chunk = numel / devices) over one tensor per device, in place
    (src/gpu/multi_gpu.rs:583-700)."""
    if len(tensors) > 1 and tensors[0].numel() >= len(tensors):
        MultiGpuContext._ring_all_reduce(tensors)
    elif len(tensors) > 1:
        host_staged_all_reduce(tensors, average=False)
    if average:
        for t in tensors:
            t.div_(len(tensors))
    return tensors


def host_staged_all_reduce(tensors: List[torch.Tensor], average: bool = True) -> List[torch.Tensor]:
    """Sum on the host, copy the result back to every device (src/gpu/multi_gpu.rs:704-751)."""
    total = torch.zeros_like(tensors[0], device="cpu", dtype=torch.float32)
    for t in tensors:
        total += t.detach().to("cpu", torch.float32)
    if average:
        total /= len(tensors)
    for t in tensors:
        t.copy_(total.to(t.device, t.dtype))
    return tensors


def nccl_all_reduce(tensor: torch.Tensor, average: bool = False, group=None) -> torch.Tensor:
    """All-reduce across the process group when one is initialised (NCCL on GPUs, gloo on CPU), else identity
    (``CommunicationManager::nccl_all_reduce``, src/gpu/multi_gpu.rs:560-582)."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(tensor, group=group)
        if average:
            tensor.div_(dist.get_world_size(group))
    return tensor


class NCCLProfiler:
    """Times collectives and reports bandwidth (``TimingGuard`` is the context manager)."""

    def __init__(self):
        self.records: List[Dict[str, float]] = []

    class TimingGuard:
        def __init__(self, prof, op, nbytes):
            self.prof, self.op, self.nbytes = prof, op, nbytes

        def __enter__(self):
            if torch.cuda.is_available():
                self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                self.e0.record()
            self.t0 = time.perf_counter()
            return self

        def __exit__(self, *exc):
            if torch.cuda.is_available():
                self.e1.record()
                self.e1.synchronize()
                dt = self.e0.elapsed_time(self.e1) * 1e-3
            else:
                dt = time.perf_counter() - self.t0
            self.prof.records.append({"op": self.op, "bytes": self.nbytes, "seconds": dt,
                                      "gbps": self.nbytes * 8 / dt / 1e9 if dt > 0 else 0.0})
            return False

    def time(self, op: str, nbytes: int) -> "NCCLProfiler.TimingGuard":
        return NCCLProfiler.TimingGuard(self, op, nbytes)

    def summary(self) -> Dict[str, Dict[str, float]]:
        out: Dict[str, Dict[str, float]] = {}
        for r in self.records:
            s = out.setdefault(r["op"], {"calls": 0, "bytes": 0, "seconds": 0.0})
            s["calls"] += 1
            s["bytes"] += r["bytes"]
            s["seconds"] += r["seconds"]
        for s in out.values():
            s["gbps"] = s["bytes"] * 8 / s["seconds"] / 1e9 if s["seconds"] > 0 else 0.0
        return out
