"""GPU runtime layer: device types and manager, contexts with streams and a memory pool, transfers, availability
cache, size-based device selection, performance advice, validation, the kernel executor façade and a
runtime-compiled custom-kernel manager
(src/gpu/mod.rs:227-835, memory.rs:11-513, device.rs:9-374, device_cache.rs:15-263,
smart_device_selector.rs:13-280, performance_optimizer.rs:19-518, validation.rs:11-478, kernels.rs:10-674,
unified_kernel_simple.rs:14-435, custom_kernels.rs:14-680, matrix_ops.rs / conv_ops.rs / activation_ops.rs /
reduction_ops.rs).

The reference enumerates CUDA / Metal / OpenCL / CoreML back-ends and dispatches per call.  This framework
has one GPU target (CUDA on B200) plus the CPU for tests, so ``DeviceType`` keeps the reference's names for API
compatibility but only ``Cpu`` and ``Cuda(i)`` can ever be available; selecting another raises
``DeviceNotAvailable``.  Nothing here changes a GPU setting (clocks, power, modes): telemetry is read-only.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import tempfile
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .. import _native
from ..memory import MemoryPool


class DeviceNotAvailable(RuntimeError):
    pass


@dataclass(frozen=True)
class DeviceType:
    kind: str = "cpu"           # cpu | cuda | metal | opencl | coreml | coreml_hybrid | mac_hybrid | auto
    index: int = 0

    @staticmethod
    def Cpu() -> "DeviceType":
        return DeviceType("cpu", 0)

    @staticmethod
    def Cuda(index: int = 0) -> "DeviceType":
        return DeviceType("cuda", index)

    @staticmethod
    def Metal(index: int = 0) -> "DeviceType":
        return DeviceType("metal", index)

    @staticmethod
    def OpenCL(index: int = 0) -> "DeviceType":
        return DeviceType("opencl", index)

    @staticmethod
    def CoreML(index: int = 0) -> "DeviceType":
        return DeviceType("coreml", index)

    @staticmethod
    def Auto() -> "DeviceType":
        return DeviceType("auto", 0)

    def is_available(self) -> bool:
        if self.kind == "cpu":
            return True
        if self.kind == "cuda":
            return torch.cuda.is_available() and self.index < torch.cuda.device_count()
        if self.kind == "auto":
            return True
        return False

    def torch_device(self) -> torch.device:
        if self.kind == "auto":
            return torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
        if self.kind in ("cpu", "cuda"):
            return torch.device(self.kind, self.index) if self.kind == "cuda" else torch.device("cpu")
        raise DeviceNotAvailable(f"{self.kind} back-end does not exist on this platform (CUDA / CPU only)")

    def __str__(self) -> str:
        return "cpu" if self.kind == "cpu" else f"{self.kind}:{self.index}"


class GpuContext:
    """A device with its stream set and (optionally) an arena memory pool."""

    def __init__(self, device: DeviceType, pool_bytes: int = 0, n_streams: int = 4):
        if not device.is_available():
            raise DeviceNotAvailable(f"device {device} is not available")
        self._device = device
        self.tdev = device.torch_device()
        self.streams = [torch.cuda.Stream(self.tdev) for _ in range(n_streams)] if self.tdev.type == "cuda" else []
        self.pool = MemoryPool(pool_bytes, self.tdev) if pool_bytes else None

    def device(self) -> DeviceType:
        return self._device

    def is_gpu_available(self) -> bool:
        return self.tdev.type == "cuda"

    def memory_pool_size(self) -> int:
        return self.pool.stats()["capacity"] if self.pool else 0

    def stream_count(self) -> int:
        return len(self.streams)

    def stream(self, i: int = 0):
        return self.streams[i % len(self.streams)] if self.streams else None

    def synchronize(self) -> None:
        if self.tdev.type == "cuda":
            torch.cuda.synchronize(self.tdev)

    def properties(self) -> dict:
        if self.tdev.type != "cuda":
            return {"name": "cpu", "cores": os.cpu_count()}
        p = torch.cuda.get_device_properties(self.tdev)
        return {"name": p.name, "compute_capability": (p.major, p.minor), "sms": p.multi_processor_count,
                "total_memory": p.total_memory, "l2_bytes": getattr(p, "L2_cache_size", 0)}


class DeviceManager:
    def __init__(self):
        self._contexts: Dict[DeviceType, GpuContext] = {}
        self._current = DeviceType.Cuda(0) if torch.cuda.is_available() else DeviceType.Cpu()

    def available_devices(self) -> List[DeviceType]:
        return [DeviceType.Cpu()] + [DeviceType.Cuda(i) for i in range(torch.cuda.device_count() if torch.cuda.is_available() else 0)]

    def set_device(self, device: DeviceType) -> None:
        if device.kind == "auto":
            device = DeviceType.Cuda(0) if torch.cuda.is_available() else DeviceType.Cpu()
        if not device.is_available():
            raise DeviceNotAvailable(f"device {device} is not available")
        if device.kind == "cuda":
            torch.cuda.set_device(device.index)
        self._current = device

    def current_device(self) -> DeviceType:
        return self._current

    def current_context(self) -> GpuContext:
        if self._current not in self._contexts:
            self._contexts[self._current] = GpuContext(self._current)
        return self._contexts[self._current]

    @staticmethod
    def is_cuda_available() -> bool:
        return torch.cuda.is_available()

    @staticmethod
    def is_metal_available() -> bool:
        return False

    @staticmethod
    def is_opencl_available() -> bool:
        return False


_MANAGER: Optional[DeviceManager] = None


def get_device_manager() -> DeviceManager:
    global _MANAGER
    if _MANAGER is None:
        _MANAGER = DeviceManager()
    return _MANAGER


def set_device(device: DeviceType) -> None:
    get_device_manager().set_device(device)


def current_device() -> DeviceType:
    return get_device_manager().current_device()


def is_gpu_available() -> bool:
    return torch.cuda.is_available()


# ------------------------------------------------------------------------------ memory / transfer
class GpuMemoryPool(MemoryPool):
    """Arena pool on a CUDA device (or the CPU for tests)."""

    def __init__(self, device: DeviceType, capacity_bytes: int):
        super().__init__(capacity_bytes, device.torch_device())


class GpuMemoryManager:
    def __init__(self):
        self.pools: Dict[DeviceType, GpuMemoryPool] = {}

    def pool(self, device: DeviceType, capacity_bytes: int = 1 << 30) -> GpuMemoryPool:
        if device not in self.pools:
            self.pools[device] = GpuMemoryPool(device, capacity_bytes)
        return self.pools[device]

    def usage(self) -> Dict[str, dict]:
        return {str(d): p.stats() for d, p in self.pools.items()}


class DataTransfer:
    """Host<->device copies through pinned staging buffers on a side stream (asynchronous with compute)."""

    def __init__(self, device: DeviceType):
        self.tdev = device.torch_device()
        self.stream = torch.cuda.Stream(self.tdev) if self.tdev.type == "cuda" else None
        self._pinned: Dict[Tuple[torch.dtype, int], torch.Tensor] = {}
        self.bytes_h2d = self.bytes_d2h = 0

    def _staging(self, t: torch.Tensor) -> torch.Tensor:
        key = (t.dtype, t.numel())
        if key not in self._pinned:
            self._pinned[key] = torch.empty(t.numel(), dtype=t.dtype, pin_memory=self.tdev.type == "cuda")
        return self._pinned[key]

    def to_device(self, host: torch.Tensor, non_blocking: bool = True) -> torch.Tensor:
        self.bytes_h2d += host.numel() * host.element_size()
        if self.tdev.type != "cuda":
            return host.clone()
        src = host if host.is_pinned() else self._staging(host).copy_(host.reshape(-1)).view(host.shape)
        with torch.cuda.stream(self.stream):
            out = src.to(self.tdev, non_blocking=non_blocking)
        torch.cuda.current_stream(self.tdev).wait_stream(self.stream)
        return out

    def to_host(self, dev: torch.Tensor) -> torch.Tensor:
        self.bytes_d2h += dev.numel() * dev.element_size()
        return dev.detach().cpu()


# ------------------------------------------------------------------------------ availability cache
class DeviceStatus(Enum):
    """Availability state of a device in the device manager (src/gpu/device.rs)."""

    AVAILABLE = "available"
    UNAVAILABLE = "unavailable"
    ERROR = "error"


@dataclass
class CachedDevice:
    status: DeviceStatus
    checked_at: float = field(default_factory=time.time)
    init_time_s: float = 0.0
    ttl_s: float = 30.0

    def is_valid(self, now: Optional[float] = None) -> bool:
        return ((now if now is not None else time.time()) - self.checked_at) < self.ttl_s


class DeviceCache:
    _global: Optional["DeviceCache"] = None

    def __init__(self, ttl_s: float = 30.0):
        self.ttl_s = ttl_s
        self._cache: Dict[DeviceType, CachedDevice] = {}
        self.hits = self.misses = 0

    @classmethod
    def global_(cls) -> "DeviceCache":
        if cls._global is None:
            cls._global = DeviceCache()
        return cls._global

    def is_device_available(self, device: DeviceType) -> bool:
        c = self._cache.get(device)
        if c is not None and c.is_valid():
            self.hits += 1
            return c.status is DeviceStatus.AVAILABLE
        self.misses += 1
        t0 = time.perf_counter()
        try:
            st = DeviceStatus.AVAILABLE if device.is_available() else DeviceStatus.UNAVAILABLE
        except Exception:  # noqa: BLE001
            st = DeviceStatus.ERROR
        self._cache[device] = CachedDevice(st, init_time_s=time.perf_counter() - t0, ttl_s=self.ttl_s)
        return st is DeviceStatus.AVAILABLE

    def get_cached_status(self, device: DeviceType) -> Optional[CachedDevice]:
        return self._cache.get(device)

    def update_cache(self, device: DeviceType, cached: CachedDevice) -> None:
        self._cache[device] = cached

    def cleanup_expired(self) -> None:
        self._cache = {d: c for d, c in self._cache.items() if c.is_valid()}

    def get_stats(self) -> dict:
        return {"entries": len(self._cache), "hits": self.hits, "misses": self.misses}

    def warmup(self) -> None:
        for d in get_device_manager().available_devices():
            self.is_device_available(d)


# ------------------------------------------------------------------------------ selection / optimisation
class OperationType(Enum):
    """Operation classes the device selectors and the performance optimizer distinguish (src/gpu/smart_device_selector.rs)."""

    MATMUL = "matmul"
    CONV = "conv"
    ELEMENTWISE = "elementwise"
    REDUCTION = "reduction"
    ACTIVATION = "activation"


@dataclass
class OperationProfile:
    op_type: OperationType
    dimensions: Sequence[int]
    data_type_size: int = 4

    def memory_footprint(self) -> int:
        n = 1
        for d in self.dimensions:
            n *= d
        return n * self.data_type_size


@dataclass
class DeviceThresholds:
    """Below these element counts the launch + transfer overhead exceeds the GPU gain."""
    matmul: int = 64 * 64
    conv: int = 16 * 16 * 8
    elementwise: int = 1 << 16
    reduction: int = 1 << 16
    activation: int = 1 << 16


class SmartDeviceSelector:
    def __init__(self, available: Optional[List[DeviceType]] = None):
        self.available = available if available is not None else get_device_manager().available_devices()
        self.thresholds = DeviceThresholds()

    def with_thresholds(self, t: DeviceThresholds) -> "SmartDeviceSelector":
        self.thresholds = t
        return self

    def select_device(self, profile: OperationProfile) -> DeviceType:
        gpus = [d for d in self.available if d.kind == "cuda"]
        n = profile.memory_footprint() // max(1, profile.data_type_size)
        if gpus and n >= getattr(self.thresholds, profile.op_type.value):
            return gpus[0]
        return DeviceType.Cpu()

    def get_fallback_chain(self, profile: OperationProfile) -> List[DeviceType]:
        first = self.select_device(profile)
        return [first] + [d for d in self.available if d != first]


class PerformanceOptimizer:
    """Read-only telemetry (NVML) -> execution advice.  Never changes a device setting."""

    def __init__(self, device_index: int = 0):
        self.device_index = device_index
        self.history: List[dict] = []

    def sample(self) -> dict:
        s = {"t": time.time()}
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.device_index)
            s["temperature_c"] = pynvml.nvmlDeviceGetTemperature(h, pynvml.NVML_TEMPERATURE_GPU)
            s["sm_mhz"] = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
            s["power_w"] = pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
            u = pynvml.nvmlDeviceGetUtilizationRates(h)
            s["gpu_util"], s["mem_util"] = u.gpu, u.memory
        except Exception:  # noqa: BLE001  (no GPU / no NVML)
            pass
        self.history.append(s)
        return s

    def feed(self, sample: dict) -> None:
        self.history.append(sample)

    def strategy(self) -> str:
        if not self.history:
            return "normal"
        s = self.history[-1]
        if s.get("temperature_c", 0) >= 85:
            return "throttle"            # reduce batch / insert gaps; clocks are not touched
        if s.get("gpu_util", 100) < 30 and len(self.history) > 3:
            return "increase_batch"
        return "normal"

    def recommendations(self) -> List[str]:
        st = self.strategy()
        return {"throttle": ["GPU is hot: lower the per-step work or overlap less until it cools"],
                "increase_batch": ["GPU utilisation is low: raise the batch size or capture the step in a CUDA graph"],
                "normal": []}[st]


class HybridExecutor:
    """Runs ``fn(device)`` on the first device of the fallback chain that succeeds."""

    def __init__(self, selector: Optional[SmartDeviceSelector] = None):
        self.selector = selector or SmartDeviceSelector()
        self.fallbacks = 0

    def execute(self, profile: OperationProfile, fn: Callable[[torch.device], object]):
        last: Optional[Exception] = None
        for i, d in enumerate(self.selector.get_fallback_chain(profile)):
            try:
                out = fn(d.torch_device())
                self.fallbacks += i
                return out
            except (RuntimeError, DeviceNotAvailable) as e:
                last = e
        raise RuntimeError(f"operation failed on every device: {last}")


# ------------------------------------------------------------------------------ validation
@dataclass
class ValidationResult:
    name: str
    device: str
    passed: bool
    max_error: float
    time_ms: float
    message: str = ""


class GpuValidator:
    """CPU-vs-device checks of the native kernels and of memory round trips."""

    def __init__(self, tolerance: float = 1e-5):
        self.tol = tolerance

    def _run(self, name: str, device: DeviceType, fn: Callable[[torch.device], float]) -> ValidationResult:
        t0 = time.perf_counter()
        try:
            err = fn(device.torch_device())
            return ValidationResult(name, str(device), err <= self.tol, err, (time.perf_counter() - t0) * 1e3)
        except Exception as e:  # noqa: BLE001
            return ValidationResult(name, str(device), False, float("inf"), (time.perf_counter() - t0) * 1e3, str(e))

    def validate_elementwise_add(self, device: DeviceType) -> ValidationResult:
        def f(dev):
            from ..ops import elementwise as ew
            a, b = torch.randn(4097), torch.randn(4097)
            return float((ew.add(a.to(dev), b.to(dev)).cpu() - (a + b)).abs().max())
        return self._run("elementwise_add", device, f)

    def validate_matrix_multiplication(self, device: DeviceType) -> ValidationResult:
        def f(dev):
            a, b = torch.randn(128, 256), torch.randn(256, 64)
            ref = a.double() @ b.double()
            if dev.type == "cuda":
                from ..ops import kernels as K
                out = K.gemm(a.to(dev).bfloat16(), b.t().contiguous().to(dev).bfloat16(), out_dtype=torch.float32).cpu()
                return float((out - ref).abs().max() / ref.abs().max()) * 1e-3      # bf16 inputs: scaled to the tolerance
            return float((a @ b - ref).abs().max() / ref.abs().max())
        return self._run("matrix_multiplication", device, f)

    def validate_memory_operations(self, device: DeviceType) -> List[ValidationResult]:
        def roundtrip(dev):
            x = torch.randn(1 << 16)
            return float((DataTransfer(device).to_host(DataTransfer(device).to_device(x)) - x).abs().max())

        def pool(dev):
            p = GpuMemoryPool(device, 1 << 20)
            t = p.zeros((1000,))
            t += 1
            err = float((t.cpu() - 1).abs().max())
            p.deallocate(t)
            return err + (0.0 if p.stats()["in_use"] == 0 else 1.0)
        return [self._run("transfer_roundtrip", device, roundtrip), self._run("memory_pool", device, pool)]

    def validate_all_devices(self) -> List[ValidationResult]:
        out = []
        for d in get_device_manager().available_devices():
            out += [self.validate_elementwise_add(d), self.validate_matrix_multiplication(d)] + self.validate_memory_operations(d)
        return out

    def generate_report(self, results: List[ValidationResult]) -> str:
        lines = [f"{'check':<26}{'device':<10}{'ok':<6}{'max err':>12}{'ms':>10}"]
        for r in results:
            lines.append(f"{r.name:<26}{r.device:<10}{'yes' if r.passed else 'NO':<6}{r.max_error:>12.3e}{r.time_ms:>10.2f} {r.message}")
        lines.append(f"{sum(r.passed for r in results)}/{len(results)} passed")
        return "\n".join(lines)


# ------------------------------------------------------------------------------ kernel executor façade
class KernelOp(Enum):
    """Operation a kernel executor is asked to run (src/gpu/kernels.rs)."""

    ADD = "add"
    SUB = "sub"
    MUL = "mul"
    DIV = "div"
    MATMUL = "matmul"
    RELU = "relu"
    SIGMOID = "sigmoid"
    TANH = "tanh"
    GELU = "gelu"
    SOFTMAX = "softmax"
    SUM = "sum"
    MEAN = "mean"
    MAX = "max"
    MIN = "min"
    CONV2D = "conv2d"
    BATCH_NORM = "batch_norm"


@dataclass
class KernelMetrics:
    launches: int = 0
    total_ms: float = 0.0
    per_op: Dict[str, List[float]] = field(default_factory=dict)

    def record(self, op: str, ms: float) -> None:
        self.launches += 1
        self.total_ms += ms
        self.per_op.setdefault(op, []).append(ms)


class UnifiedKernelExecutor:
    """``execute(op, *tensors)`` on one device: native kernels on CUDA, PyTorch on CPU."""

    def __init__(self, device: DeviceType):
        if not device.is_available():
            raise DeviceNotAvailable(f"device {device} is not available")
        self._device, self.tdev = device, device.torch_device()
        self.metrics = KernelMetrics()

    def supports_operation(self, op: KernelOp) -> bool:
        return True

    def device_type(self) -> DeviceType:
        return self._device

    def get_metrics(self) -> KernelMetrics:
        return self.metrics

    def execute(self, op: KernelOp, *inputs: torch.Tensor, **kw) -> torch.Tensor:
        from ..ops import elementwise as ew
        from ..ops.batchnorm import batch_norm
        xs = [t.to(self.tdev) for t in inputs]
        t0 = time.perf_counter()
        v = op.value
        if v in ("add", "sub", "mul", "div"):
            out = ew.binary(v, xs[0], xs[1])
        elif v in ("relu", "sigmoid", "tanh", "gelu"):
            out = ew.unary(v, xs[0])
        elif v == "softmax":
            out = ew.softmax(xs[0], kw.get("dim", -1))
        elif v in ("sum", "mean", "max", "min"):
            out = ew.reduce_last(xs[0].reshape(1, -1), v)[0]
        elif v == "matmul":
            if self.tdev.type == "cuda" and xs[0].dtype == torch.bfloat16 and _native.available():
                from ..ops import kernels as K
                out = K.gemm(xs[0].contiguous(), xs[1], b_mn=True)
            else:
                out = xs[0] @ xs[1]
        elif v == "conv2d":
            out = torch.nn.functional.conv2d(xs[0], xs[1], xs[2] if len(xs) > 2 else None, kw.get("stride", 1), kw.get("padding", 0))
        else:
            out = batch_norm(xs[0], None, None, xs[1] if len(xs) > 1 else None, xs[2] if len(xs) > 2 else None, True)
        if self.tdev.type == "cuda":
            torch.cuda.synchronize(self.tdev)
        self.metrics.record(v, (time.perf_counter() - t0) * 1e3)
        return out

    execute_f32 = execute
    execute_f64 = execute


class KernelSelector:
    def __init__(self):
        self.executors: List[UnifiedKernelExecutor] = []

    def add_executor(self, ex: UnifiedKernelExecutor) -> None:
        self.executors.append(ex)

    def select_best(self, op: KernelOp) -> Optional[UnifiedKernelExecutor]:
        gpu = [e for e in self.executors if e.tdev.type == "cuda" and e.supports_operation(op)]
        return (gpu or self.executors or [None])[0]

    def execute(self, op: KernelOp, *inputs, **kw) -> torch.Tensor:
        ex = self.select_best(op)
        if ex is None:
            raise RuntimeError("no executor registered")
        return ex.execute(op, *inputs, **kw)

    def available_devices(self) -> List[DeviceType]:
        return [e.device_type() for e in self.executors]


KernelExecutor = UnifiedKernelExecutor


# ------------------------------------------------------------------------------ runtime-compiled kernels
@dataclass
class KernelConfig:
    name: str                       # __global__ function name (compiled with extern "C")
    source: str                     # CUDA C++ source
    block: Tuple[int, int, int] = (256, 1, 1)
    shared_bytes: int = 0


@dataclass
class KernelStats:
    compile_ms: float = 0.0
    launches: int = 0
    cache_hit: bool = False


class CustomKernelManager:
    """Compiles user CUDA source to a cubin for sm_100a with nvcc (cached by content hash), loads it through the
    driver API and launches it on the current stream.  The reference only stores the source strings
    (src/gpu/custom_kernels.rs:124-146 never compiles them)."""

    def __init__(self, device: Optional[DeviceType] = None, cache_dir: Optional[str] = None):
        self.device = device or (DeviceType.Cuda(0) if torch.cuda.is_available() else DeviceType.Cpu())
        self.cache_dir = cache_dir or os.path.join(tempfile.gettempdir(), "rustorch_b200_kernels")
        os.makedirs(self.cache_dir, exist_ok=True)
        self.compiled: Dict[str, str] = {}            # name -> cubin path
        self.stats: Dict[str, KernelStats] = {}
        self._functions: Dict[str, object] = {}

    def compile_kernel(self, cfg: KernelConfig, arch: str = "sm_100a") -> str:
        digest = hashlib.sha256((cfg.source + arch).encode()).hexdigest()[:16]
        cubin = os.path.join(self.cache_dir, f"{cfg.name}.{digest}.cubin")
        st = self.stats.setdefault(cfg.name, KernelStats())
        if os.path.exists(cubin):
            st.cache_hit = True
        else:
            src = os.path.join(self.cache_dir, f"{cfg.name}.{digest}.cu")
            with open(src, "w") as f:
                f.write(cfg.source)
            t0 = time.perf_counter()
            nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
            r = subprocess.run([nvcc, "-cubin", f"-arch={arch}", "-O3", "-lineinfo", "-o", cubin, src], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"compilation of '{cfg.name}' failed:\n{r.stderr}")
            st.compile_ms = (time.perf_counter() - t0) * 1e3
        self.compiled[cfg.name] = cubin
        return cubin

    def execute_kernel(self, cfg: KernelConfig, grid: Tuple[int, int, int], args: Sequence[object]) -> None:
        """``args``: tensors (passed as device pointers), ints (int64) and floats (fp32)."""
        if self.device.kind != "cuda":
            raise DeviceNotAvailable("custom kernels run on CUDA devices only")
        import ctypes

        import numpy as np
        from cuda import cuda as drv
        if cfg.name not in self.compiled:
            self.compile_kernel(cfg)
        if cfg.name not in self._functions:
            torch.cuda.init()
            torch.zeros(1, device=self.device.torch_device())          # make the primary context current
            with open(self.compiled[cfg.name], "rb") as f:
                img = f.read()
            err, mod = drv.cuModuleLoadData(img)
            if int(err) != 0:
                raise RuntimeError(f"cuModuleLoadData failed: {err}")
            err, fn = drv.cuModuleGetFunction(mod, cfg.name.encode())
            if int(err) != 0:
                raise RuntimeError(f"kernel '{cfg.name}' not found in the module (declare it extern \"C\"): {err}")
            self._functions[cfg.name] = (mod, fn)
        _, fn = self._functions[cfg.name]
        vals, types = [], []
        for a in args:
            if isinstance(a, torch.Tensor):
                vals.append(a.data_ptr()); types.append(ctypes.c_void_p)
            elif isinstance(a, float):
                vals.append(a); types.append(ctypes.c_float)
            else:
                vals.append(int(a)); types.append(ctypes.c_longlong)
        stream = torch.cuda.current_stream(self.device.torch_device()).cuda_stream
        (err,) = drv.cuLaunchKernel(fn, *grid, *cfg.block, cfg.shared_bytes, stream, (tuple(vals), tuple(types)), 0)
        if int(err) != 0:
            raise RuntimeError(f"launch of '{cfg.name}' failed: {err}")
        self.stats[cfg.name].launches += 1

    def get_kernel_stats(self, name: str) -> KernelStats:
        return self.stats[name]
