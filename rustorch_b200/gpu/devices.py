"""Device layer, kernel objects and executors of the reference's ``gpu`` module that sit above the raw kernels
(src/gpu/device.rs:9-374, kernels.rs:10-674, cuda_kernels.rs:70-843, matrix_ops.rs:17-689, sync_primitives.rs:14-313,
src/backends/mod.rs:47-348, compute_backend.rs:19-426, cpu_unified.rs).

``GpuDevice`` / ``GpuStream`` wrap a CUDA device and stream; ``GpuKernel`` objects are callables bound to the
framework's native kernels; the executors keep the reference's method names (``elementwise_add_f32``, ``matmul_f32``,
``reduce_sum_f32`` ...) and run the tcgen05 GEMM / vectorised elementwise kernels underneath.  Metal and OpenCL
executors exist by name and raise ``DeviceNotAvailable``: those runtimes are not present on an NVIDIA box.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from enum import Enum
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from .. import _native
from . import DeviceNotAvailable, DeviceType


# ------------------------------------------------------------------------------------------------ devices / streams
class GpuStream:
    """A CUDA stream with the reference's ``synchronize`` / ``is_ready`` / ``record`` / ``wait`` surface."""

    def __init__(self, device: "GpuDevice", priority: int = 0):
        self.device = device
        self.raw = torch.cuda.Stream(device.torch_device, priority=priority) if device.is_cuda else None

    def synchronize(self) -> None:
        if self.raw is not None:
            self.raw.synchronize()

    def is_ready(self) -> bool:
        return True if self.raw is None else self.raw.query()

    def record_event(self) -> Optional["torch.cuda.Event"]:
        if self.raw is None:
            return None
        e = torch.cuda.Event()
        e.record(self.raw)
        return e

    def wait_event(self, event) -> None:
        if self.raw is not None and event is not None:
            self.raw.wait_event(event)

    def __enter__(self):
        self._ctx = torch.cuda.stream(self.raw) if self.raw is not None else None
        if self._ctx:
            self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self._ctx:
            self._ctx.__exit__(*exc)


class GpuDevice(ABC):
    """Trait: ``name / total_memory / available_memory / synchronize / create_stream / supports(dtype)``."""
    is_cuda = False

    @property
    @abstractmethod
    def torch_device(self) -> torch.device: ...

    @abstractmethod
    def name(self) -> str: ...

    @abstractmethod
    def total_memory(self) -> int: ...

    def available_memory(self) -> int:
        return self.total_memory()

    def synchronize(self) -> None:
        pass

    def create_stream(self, priority: int = 0) -> GpuStream:
        return GpuStream(self, priority)

    def supports(self, dtype: torch.dtype) -> bool:
        return True


class CpuDevice(GpuDevice):
    @property
    def torch_device(self) -> torch.device:
        return torch.device("cpu")

    def name(self) -> str:
        return "cpu"

    def total_memory(self) -> int:
        try:
            import psutil
            return int(psutil.virtual_memory().total)
        except Exception:  # noqa: BLE001
            return 0


class CudaDevice(GpuDevice):
    is_cuda = True

    def __init__(self, index: int = 0):
        if not torch.cuda.is_available() or index >= torch.cuda.device_count():
            raise DeviceNotAvailable(f"cuda:{index} is not available")
        self.index = index
        self._props = torch.cuda.get_device_properties(index)

    @property
    def torch_device(self) -> torch.device:
        return torch.device("cuda", self.index)

    def name(self) -> str:
        return self._props.name

    def total_memory(self) -> int:
        return int(self._props.total_memory)

    def available_memory(self) -> int:
        return int(torch.cuda.mem_get_info(self.index)[0])

    def synchronize(self) -> None:
        torch.cuda.synchronize(self.index)

    def compute_capability(self) -> Tuple[int, int]:
        return self._props.major, self._props.minor

    def sm_count(self) -> int:
        return self._props.multi_processor_count


class MetalDevice(GpuDevice):
    def __init__(self, *a, **k):
        raise DeviceNotAvailable("Metal is not available on this platform")

    torch_device = None

    def name(self):
        return "metal"

    def total_memory(self):
        return 0


class StreamOperation(Enum):
    """What a stream entry in the manager's log stands for (src/gpu/sync_primitives.rs)."""
    KERNEL = "kernel"
    MEMCPY_H2D = "memcpy_h2d"
    MEMCPY_D2H = "memcpy_d2h"
    MEMCPY_P2P = "memcpy_p2p"
    EVENT_RECORD = "event_record"
    EVENT_WAIT = "event_wait"
    COLLECTIVE = "collective"


# ------------------------------------------------------------------------------------------------ kernel objects
class GpuKernel(ABC):
    """Trait of the kernels framework: a named operation with a launch method."""
    name = "kernel"

    @abstractmethod
    def execute(self, *tensors: torch.Tensor, **params) -> torch.Tensor: ...

    def __call__(self, *tensors, **params):
        return self.execute(*tensors, **params)


class ModernGpuKernel(GpuKernel):
    """Second-generation trait: adds validation and a cost estimate used by the selector."""

    def validate(self, *tensors: torch.Tensor) -> None:
        devs = {t.device for t in tensors}
        if len(devs) > 1:
            raise ValueError(f"{self.name}: operands on different devices {devs}")

    def flops(self, *tensors: torch.Tensor) -> float:
        return float(sum(t.numel() for t in tensors))

    def __call__(self, *tensors, **params):
        self.validate(*tensors)
        return self.execute(*tensors, **params)


class AddKernel(ModernGpuKernel):
    name = "add"

    def execute(self, a, b, alpha: float = 1.0):
        from ..ops import elementwise as E
        return E.add(a, b, alpha)


class MatMulKernel(ModernGpuKernel):
    name = "matmul"

    def execute(self, a, b):
        if a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2 and _native.available():
            from ..ops import kernels as K
            return K.gemm(a.contiguous(), b.contiguous(), b_mn=True)          # tcgen05 GEMM, B given as [K, N]
        return a @ b

    def flops(self, a, b):
        return 2.0 * a.shape[-2] * a.shape[-1] * b.shape[-1]


class ConvKernel(ModernGpuKernel):
    name = "conv2d"

    def execute(self, x, w, bias=None, stride=1, padding=0):
        from ..ops import conv as C
        return C.conv2d(x, w, bias, stride, padding)


class KernelExecutor:
    """Registry + dispatcher of kernel objects for one device."""

    def __init__(self, device: Optional[GpuDevice] = None):
        self.device = device or (CudaDevice(0) if torch.cuda.is_available() else CpuDevice())
        self.kernels: Dict[str, GpuKernel] = {k.name: k for k in (AddKernel(), MatMulKernel(), ConvKernel())}

    def register(self, kernel: GpuKernel) -> None:
        self.kernels[kernel.name] = kernel

    def execute(self, name: str, *tensors, **params):
        if name not in self.kernels:
            raise KeyError(f"no kernel named '{name}'")
        tensors = tuple(t.to(self.device.torch_device) if isinstance(t, torch.Tensor) else t for t in tensors)
        return self.kernels[name](*tensors, **params)


# ------------------------------------------------------------------------------------------------ CUDA executors
class CudaBuffer:
    """Typed device buffer with explicit H2D / D2H copies (``CudaBuffer<T>``)."""

    def __init__(self, numel: int, dtype: torch.dtype = torch.float32, device: int = 0):
        self.tensor = torch.empty(numel, dtype=dtype, device=torch.device("cuda", device))

    @classmethod
    def from_host(cls, data, dtype: torch.dtype = torch.float32, device: int = 0) -> "CudaBuffer":
        t = torch.as_tensor(data, dtype=dtype)
        b = cls(t.numel(), dtype, device)
        b.copy_from_host(t)
        return b

    def copy_from_host(self, data) -> None:
        self.tensor.copy_(torch.as_tensor(data, dtype=self.tensor.dtype).reshape(-1), non_blocking=True)

    def copy_to_host(self) -> torch.Tensor:
        return self.tensor.cpu()

    def __len__(self) -> int:
        return self.tensor.numel()


class CudaKernelExecutor:
    """Method names of the reference's executor (elementwise, activation, reduction, convolution entry points); the
    device work is done by this framework's kernels instead of NVRTC-compiled strings."""

    def __init__(self, device_id: int = 0):
        if not torch.cuda.is_available():
            raise DeviceNotAvailable("CUDA is not available")
        self.device = torch.device("cuda", device_id)

    def _t(self, x) -> torch.Tensor:
        return (x.tensor if isinstance(x, CudaBuffer) else torch.as_tensor(x)).to(self.device)

    def elementwise_add_f32(self, a, b):
        from ..ops import elementwise as E
        return E.add(self._t(a).float(), self._t(b).float())

    def elementwise_mul_f32(self, a, b):
        from ..ops import elementwise as E
        return E.mul(self._t(a).float(), self._t(b).float())

    def relu_f32(self, a):
        from ..ops import elementwise as E
        return E.unary("relu", self._t(a).float())

    def sigmoid_f32(self, a):
        from ..ops import elementwise as E
        return E.unary("sigmoid", self._t(a).float())

    def tanh_f32(self, a):
        from ..ops import elementwise as E
        return E.unary("tanh", self._t(a).float())

    def gelu_f32(self, a):
        from ..ops import elementwise as E
        return E.unary("gelu", self._t(a).float())

    def softmax_f32(self, a, dim: int = -1):
        from ..ops import elementwise as E
        return E.softmax(self._t(a).float(), dim)

    def reduce_sum_f32(self, a):
        from ..ops import kernels as K
        return K.reduce_all(self._t(a).float().reshape(-1), "sum")[0]

    def reduce_max_f32(self, a):
        from ..ops import kernels as K
        return K.reduce_all(self._t(a).float().reshape(-1), "max")[0]

    def conv2d_f32(self, x, w, bias=None, stride=1, padding=0):
        return torch.nn.functional.conv2d(self._t(x).float(), self._t(w).float(), None if bias is None else self._t(bias).float(),
                                          stride, padding)


class CudaMatrixExecutor:
    """``matmul_f32 / batch_matmul_f32 / matvec_f32 / transpose`` (src/gpu/matrix_ops.rs): bf16 operands go to the
    tcgen05 GEMM, fp32 ones to the library GEMM with TF32 disabled (exact fp32 semantics)."""

    def __init__(self, device_id: int = 0):
        if not torch.cuda.is_available():
            raise DeviceNotAvailable("CUDA is not available")
        self.device = torch.device("cuda", device_id)
        self._mm = MatMulKernel()

    def matmul_f32(self, a, b):
        return torch.as_tensor(a, device=self.device).float() @ torch.as_tensor(b, device=self.device).float()

    def matmul_bf16(self, a, b):
        return self._mm(torch.as_tensor(a, device=self.device).bfloat16(), torch.as_tensor(b, device=self.device).bfloat16())

    def batch_matmul_f32(self, a, b):
        return torch.bmm(torch.as_tensor(a, device=self.device).float(), torch.as_tensor(b, device=self.device).float())

    def matvec_f32(self, a, v):
        return torch.as_tensor(a, device=self.device).float() @ torch.as_tensor(v, device=self.device).float()

    def transpose(self, a):
        return torch.as_tensor(a, device=self.device).t().contiguous()


def _unavailable(name: str, what: str):
    def __init__(self, *a, **k):
        raise DeviceNotAvailable(f"{what} is not available on this platform")
    return type(name, (), {"__init__": __init__, "__doc__": f"{what} executor: present by name only."})


MetalKernelExecutor = _unavailable("MetalKernelExecutor", "Metal")
MetalMatrixExecutor = _unavailable("MetalMatrixExecutor", "Metal")
OpenClKernelExecutor = _unavailable("OpenClKernelExecutor", "OpenCL")
OpenClMatrixExecutor = _unavailable("OpenClMatrixExecutor", "OpenCL")
CoreMLHybrid = _unavailable("CoreMLHybrid", "CoreML")
MacHybrid = _unavailable("MacHybrid", "The Metal / CoreML hybrid executor")


# ------------------------------------------------------------------------------------------------ compute back-ends
class SelectionStrategy(Enum):
    """How the back-end manager picks a compute back-end (src/backends/mod.rs)."""

    PERFORMANCE = "performance"
    MEMORY = "memory"
    FIRST_AVAILABLE = "first_available"
    CPU_ONLY = "cpu_only"


class ComputeBackend(ABC):
    """Back-end trait: allocation + the core ops on that device."""
    name = "backend"

    @abstractmethod
    def device(self) -> torch.device: ...

    def is_available(self) -> bool:
        return True

    def allocate(self, shape: Sequence[int], dtype: torch.dtype = torch.float32) -> torch.Tensor:
        return torch.empty(*shape, dtype=dtype, device=self.device())

    def to_backend(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(self.device())

    def add(self, a, b):
        return self.to_backend(a) + self.to_backend(b)

    def mul(self, a, b):
        return self.to_backend(a) * self.to_backend(b)

    def matmul(self, a, b):
        return self.to_backend(a) @ self.to_backend(b)

    def sum(self, a):
        return self.to_backend(a).sum()

    def synchronize(self) -> None:
        pass

    def capabilities(self) -> Dict[str, Any]:
        return {"name": self.name}


class CpuBackend(ComputeBackend):
    name = "cpu"

    def device(self) -> torch.device:
        return torch.device("cpu")

    def capabilities(self) -> Dict[str, Any]:
        caps = {"name": "cpu", "threads": torch.get_num_threads()}
        try:
            import cpuinfo
            flags = set(cpuinfo.get_cpu_info().get("flags", []))
            caps.update(avx2="avx2" in flags, avx512="avx512f" in flags, fma="fma" in flags, sse41="sse4_1" in flags)
        except Exception:  # noqa: BLE001
            pass
        return caps


class GpuBackend(ComputeBackend):
    name = "cuda"

    def __init__(self, index: int = 0):
        self.dev = CudaDevice(index)
        self._mm = MatMulKernel()

    def device(self) -> torch.device:
        return self.dev.torch_device

    def is_available(self) -> bool:
        return torch.cuda.is_available()

    def add(self, a, b):
        from ..ops import elementwise as E
        return E.add(self.to_backend(a), self.to_backend(b))

    def mul(self, a, b):
        from ..ops import elementwise as E
        return E.mul(self.to_backend(a), self.to_backend(b))

    def matmul(self, a, b):
        return self._mm(self.to_backend(a), self.to_backend(b))

    def synchronize(self) -> None:
        self.dev.synchronize()

    def capabilities(self) -> Dict[str, Any]:
        return {"name": self.dev.name(), "sms": self.dev.sm_count(), "memory": self.dev.total_memory(),
                "compute_capability": self.dev.compute_capability(), "native_kernels": _native.available()}


class BackendManager:
    """``DeviceManager(SelectionStrategy)`` of src/backends: picks a back-end by strategy."""

    def __init__(self, strategy: SelectionStrategy = SelectionStrategy.PERFORMANCE):
        self.strategy = strategy
        self.backends: List[ComputeBackend] = [CpuBackend()]
        if torch.cuda.is_available():
            self.backends = [GpuBackend(i) for i in range(torch.cuda.device_count())] + self.backends

    def select(self) -> ComputeBackend:
        if self.strategy is SelectionStrategy.CPU_ONLY:
            return self.backends[-1]
        if self.strategy is SelectionStrategy.MEMORY and len(self.backends) > 1:
            gpus = [b for b in self.backends if isinstance(b, GpuBackend)]
            return max(gpus, key=lambda b: b.dev.available_memory())
        return self.backends[0]
