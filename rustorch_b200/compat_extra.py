"""More named pieces of the reference's public surface, each a small working object on top of the package:

* explicit backward nodes (``GradFn`` and ``AddBackward`` ... ``MeanBackward``; src/autograd/grad_fn.rs, mod.rs:38)
* state-dict containers (``StateDict``, ``ModelStateDict``, ``TensorMetadata``; src/serialization/model_io.rs:118-392,
  src/models/serialization.rs:18-120)
* the generic Adam family (``GenericAdamOptimizer``, ``AdamVariant``, ``CommonOps``; src/optim/common.rs:20-160)
* gradient compression selector (``GradientCompression``; src/gpu/multi_gpu.rs:83-96)
* device helpers (``GpuBuffer``, ``CudaBlas``, ``CudaSparseOps``, ``GpuActivation``, ``GpuConvolution``,
  ``GpuBatchMatrixExecutor``; src/gpu/memory_ops/buffer.rs, cuda_enhanced.rs, activation_ops.rs, conv_ops.rs, matrix_ops.rs)
* model-parallel communication bookkeeping (``CommunicationOp``, ``CommunicationManager``;
  src/distributed/model_parallel.rs:229-330)
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch


# ------------------------------------------------------------------------------------------------ backward nodes
class GradFn:
    """A node of the backward graph: ``apply(grad_output)`` returns one gradient per input (``None`` where not needed)."""

    name = "GradFn"

    def __init__(self, *inputs: torch.Tensor):
        self.inputs = inputs

    def apply(self, grad_output: torch.Tensor) -> Tuple[Optional[torch.Tensor], ...]:
        raise NotImplementedError

    @staticmethod
    def _unbroadcast(g: torch.Tensor, shape: Sequence[int]) -> torch.Tensor:
        while g.dim() > len(shape):
            g = g.sum(0)
        for i, n in enumerate(shape):
            if n == 1 and g.shape[i] != 1:
                g = g.sum(i, keepdim=True)
        return g


class AddBackward(GradFn):
    name = "AddBackward"

    def apply(self, g):
        a, b = self.inputs
        return self._unbroadcast(g, a.shape), self._unbroadcast(g, b.shape)


class SubBackward(GradFn):
    name = "SubBackward"

    def apply(self, g):
        a, b = self.inputs
        return self._unbroadcast(g, a.shape), self._unbroadcast(-g, b.shape)


class MulBackward(GradFn):
    name = "MulBackward"

    def apply(self, g):
        a, b = self.inputs
        return self._unbroadcast(g * b, a.shape), self._unbroadcast(g * a, b.shape)


class MatMulBackward(GradFn):
    name = "MatMulBackward"

    def apply(self, g):
        a, b = self.inputs
        return g @ b.transpose(-1, -2), a.transpose(-1, -2) @ g


class SumBackward(GradFn):
    name = "SumBackward"

    def apply(self, g):
        (a,) = self.inputs
        return (g.expand_as(a).clone(),)


class MeanBackward(GradFn):
    name = "MeanBackward"

    def apply(self, g):
        (a,) = self.inputs
        return (g.expand_as(a) / a.numel(),)


# ------------------------------------------------------------------------------------------------ state dicts
@dataclass
class TensorMetadata:
    shape: List[int]
    dtype: str
    device: str = "cpu"
    requires_grad: bool = False
    data_offset: int = 0
    data_size: int = 0


@dataclass
class StateDict:
    """Named parameters and buffers plus free-form metadata; saved in the RusTorch binary container."""
    parameters: Dict[str, torch.Tensor] = field(default_factory=dict)
    buffers: Dict[str, torch.Tensor] = field(default_factory=dict)
    metadata: Dict[str, str] = field(default_factory=dict)

    @classmethod
    def from_module(cls, module: torch.nn.Module) -> "StateDict":
        return cls({k: v.detach().clone() for k, v in module.named_parameters()},
                   {k: v.detach().clone() for k, v in module.named_buffers()})

    def add_parameter(self, name: str, t: torch.Tensor) -> None:
        self.parameters[name] = t

    def add_buffer(self, name: str, t: torch.Tensor) -> None:
        self.buffers[name] = t

    def tensor_metadata(self) -> Dict[str, TensorMetadata]:
        out, off = {}, 0
        for k, v in {**self.parameters, **self.buffers}.items():
            n = v.numel() * v.element_size()
            out[k] = TensorMetadata(list(v.shape), str(v.dtype).replace("torch.", ""), str(v.device), bool(v.requires_grad), off, n)
            off += n
        return out

    def load_into(self, module: torch.nn.Module, strict: bool = True):
        return module.load_state_dict({**self.parameters, **self.buffers}, strict=strict)

    def save(self, path: str) -> None:
        from .formats import rustorch_bin
        rustorch_bin.save_state_dict(self.parameters, path, self.buffers)

    @classmethod
    def load(cls, path: str) -> "StateDict":
        from .formats import rustorch_bin
        params, buffers, meta = rustorch_bin.load_state_dict(path)
        return cls(params, buffers, {k: str(v) for k, v in meta.items() if isinstance(v, (str, int, float))})


@dataclass
class ModelStateDict:
    """``parameters: name -> flat list of f64`` with the shapes beside it, the models-level interchange form."""
    parameters: Dict[str, List[float]] = field(default_factory=dict)
    shapes: Dict[str, List[int]] = field(default_factory=dict)

    @classmethod
    def from_module(cls, module: torch.nn.Module) -> "ModelStateDict":
        sd = module.state_dict()
        return cls({k: v.detach().double().flatten().tolist() for k, v in sd.items()}, {k: list(v.shape) for k, v in sd.items()})

    def to_tensors(self, dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
        return {k: torch.tensor(v, dtype=torch.float64).reshape(self.shapes[k]).to(dtype) for k, v in self.parameters.items()}


# ------------------------------------------------------------------------------------------------ generic Adam family
class AdamVariant(enum.Enum):
    """Which member of the Adam family a generic Adam optimizer runs (src/optim/common.rs)."""

    ADAM = "adam"
    ADAMW = "adamw"
    ADAMAX = "adamax"
    NADAM = "nadam"
    RADAM = "radam"


class CommonOps:
    """Moment updates shared by the Adam family (src/optim/common.rs:120-160)."""

    @staticmethod
    def update_momentum(m: torch.Tensor, grad: torch.Tensor, beta1: float) -> torch.Tensor:
        return m.mul_(beta1).add_(grad, alpha=1 - beta1)

    @staticmethod
    def update_velocity(v: torch.Tensor, grad: torch.Tensor, beta2: float) -> torch.Tensor:
        return v.mul_(beta2).addcmul_(grad, grad, value=1 - beta2)

    @staticmethod
    def bias_correction(beta: float, step: int) -> float:
        return 1.0 - beta ** step

    @staticmethod
    def apply_weight_decay(grad: torch.Tensor, param: torch.Tensor, weight_decay: float) -> torch.Tensor:
        return grad.add(param, alpha=weight_decay) if weight_decay else grad


def GenericAdamOptimizer(params, variant: AdamVariant = AdamVariant.ADAM, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                         weight_decay: float = 0.0):
    """The optimizer of the chosen variant (``step`` / ``step_tensor`` / ``state_dict`` as every optimizer of the package)."""
    from . import optim
    cls = {AdamVariant.ADAM: optim.Adam, AdamVariant.ADAMW: optim.AdamW, AdamVariant.ADAMAX: optim.Adamax,
           AdamVariant.NADAM: optim.NAdam, AdamVariant.RADAM: optim.RAdam}[AdamVariant(variant)]
    return cls(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)


# ------------------------------------------------------------------------------------------------ gradient compression
class GradientCompression(enum.Enum):
    NONE = "none"
    TOP_K = "top_k"
    RANDOM = "random"
    QUANTIZATION = "quantization"
    ERROR_FEEDBACK = "error_feedback"

    def compressor(self, ratio: float = 0.01, bits: int = 8):
        """An object whose ``compress_decompress(grad, key=0)`` returns what the receiver would see."""
        from .distributed.async_gradient import GradientCompressor
        if self is GradientCompression.TOP_K:
            return GradientCompressor("topk", ratio, bits, error_feedback=False)
        if self is GradientCompression.ERROR_FEEDBACK:
            return GradientCompressor("topk", ratio, bits, error_feedback=True)
        if self is GradientCompression.QUANTIZATION:
            return GradientCompressor("quantization", ratio, bits)
        if self is GradientCompression.RANDOM:
            return _RandomKCompressor(ratio)
        return GradientCompressor(None)


class _RandomKCompressor:
    """Keeps a random ``ratio`` of the entries, scaled by ``1 / ratio`` so that the expectation is unchanged."""

    def __init__(self, ratio: float, seed: int = 0):
        self.ratio, self.gen = float(ratio), torch.Generator().manual_seed(seed)

    def compress(self, t: torch.Tensor):
        flat = t.flatten()
        k = max(1, int(flat.numel() * self.ratio))
        idx = torch.randperm(flat.numel(), generator=self.gen)[:k].to(flat.device)
        return idx, flat[idx] * (flat.numel() / k), tuple(t.shape)

    def decompress(self, payload):
        idx, vals, shape = payload
        out = torch.zeros(int(torch.tensor(shape).prod()), dtype=vals.dtype, device=vals.device)
        out[idx] = vals
        return out.reshape(shape)

    def compress_decompress(self, g: torch.Tensor, key: int = 0) -> torch.Tensor:
        return self.decompress(self.compress(g))


# ------------------------------------------------------------------------------------------------ device helpers
class GpuBuffer:
    """A typed device allocation (the reference's ``GpuBuffer<T>`` enum over back ends; here CUDA or host memory)."""

    def __init__(self, data: torch.Tensor):
        self.data = data

    @classmethod
    def from_host(cls, values, device: Optional[str] = None, dtype: torch.dtype = torch.float32) -> "GpuBuffer":
        dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
        return cls(torch.as_tensor(values, dtype=dtype).to(dev))

    @classmethod
    def zeros(cls, n: int, device: Optional[str] = None, dtype: torch.dtype = torch.float32) -> "GpuBuffer":
        return cls(torch.zeros(n, dtype=dtype, device=device or ("cuda" if torch.cuda.is_available() else "cpu")))

    def to_host(self) -> torch.Tensor:
        return self.data.detach().cpu()

    def len(self) -> int:
        return self.data.numel()

    __len__ = len

    def is_cuda(self) -> bool:
        return self.data.is_cuda


def _native_bf16(*ts: torch.Tensor) -> bool:
    from . import _native
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts) and _native.available()


class CudaBlas:
    """BLAS-shaped entry points: bf16 CUDA operands run on the tcgen05 GEMM, everything else on the library."""

    @staticmethod
    def gemm(a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0, trans_b: bool = False) -> torch.Tensor:
        if _native_bf16(a, b) and a.dim() == 2 and b.dim() == 2 and a.shape[1] % 8 == 0:
            from .ops import kernels as K
            bt = b if trans_b else b.t().contiguous()              # K.gemm computes a @ bt^T
            if bt.shape[0] % 8 == 0:
                return K.gemm(a.contiguous(), bt.contiguous(), alpha=alpha)
        return alpha * (a @ (b.t() if trans_b else b))

    @staticmethod
    def gemv(a: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        return a @ x

    @staticmethod
    def dot(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        return torch.dot(x.flatten(), y.flatten())

    @staticmethod
    def axpy(alpha: float, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        return y.add_(x, alpha=alpha)


class CudaSparseOps:
    @staticmethod
    def spmv(crow: torch.Tensor, col: torch.Tensor, values: torch.Tensor, x: torch.Tensor, rows: int) -> torch.Tensor:
        return CudaSparseOps.spmm(crow, col, values, x.unsqueeze(1), rows).squeeze(1)

    @staticmethod
    def spmm(crow: torch.Tensor, col: torch.Tensor, values: torch.Tensor, dense: torch.Tensor, rows: int) -> torch.Tensor:
        a = torch.sparse_csr_tensor(crow, col, values, size=(rows, dense.shape[0]))
        return a @ dense


class GpuActivation:
    """Activations on device tensors through the package's elementwise kernels."""

    @staticmethod
    def apply(name: str, x: torch.Tensor) -> torch.Tensor:
        from .nn import layers
        return getattr(layers, name)(x)

    relu = staticmethod(lambda x: GpuActivation.apply("relu", x))
    sigmoid = staticmethod(lambda x: GpuActivation.apply("sigmoid", x))
    tanh = staticmethod(lambda x: GpuActivation.apply("tanh", x))
    gelu = staticmethod(lambda x: GpuActivation.apply("gelu", x))
    swish = staticmethod(lambda x: GpuActivation.apply("swish", x))


class GpuConvolution:
    @staticmethod
    def conv2d(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, stride=1, padding=0) -> torch.Tensor:
        from .ops.conv import conv2d
        return conv2d(x, weight, bias, stride, padding)

    @staticmethod
    def conv_transpose2d(x, weight, bias=None, stride=1, padding=0, output_padding=0) -> torch.Tensor:
        from .ops.conv import conv_transpose2d
        return conv_transpose2d(x, weight, bias, stride, padding, output_padding)


class GpuBatchMatrixExecutor:
    """Batched matrix products ``[B, M, K] x [B, K, N]``."""

    def __init__(self, device: Optional[str] = None):
        self.device = device or ("cuda" if torch.cuda.is_available() else "cpu")

    def batch_matmul(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        return torch.bmm(a.to(self.device), b.to(self.device))

    cuda_batch_matmul = batch_matmul


def get_compute_capability(device: int = 0) -> Tuple[int, int]:
    """``(major, minor)`` of a CUDA device, ``(0, 0)`` without one (src/gpu/cuda_enhanced.rs:160-190)."""
    return tuple(torch.cuda.get_device_capability(device)) if torch.cuda.is_available() else (0, 0)


def execute_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False) -> torch.Tensor:
    """``softmax(q k^T / sqrt(d)) v`` over ``[B, H, T, D]`` (the reference's custom-kernel entry, src/gpu/custom_kernels.rs:
    439-536, computes it on the host): bf16 CUDA inputs with D = 64 / 128 run on the tcgen05 flash-attention kernel."""
    from . import _native
    if q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) and _native.available():
        from .nn.fused import FlashAttentionFn                     # expects [B, T, H, D]
        o = FlashAttentionFn.apply(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal, None)
        return o.transpose(1, 2)
    return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal)


# ------------------------------------------------------------------------------------------------ model-parallel communication
class CommunicationOp(enum.Enum):
    """Kinds of collective operations a communication manager schedules (src/gpu/multi_gpu.rs)."""

    SEND = "send"
    RECV = "recv"
    ALL_REDUCE = "all_reduce"
    ALL_GATHER = "all_gather"
    REDUCE_SCATTER = "reduce_scatter"
    BROADCAST = "broadcast"
    ALL_TO_ALL = "all_to_all"


class CommunicationManager:
    """Queues communication operations of a model-parallel step and runs them in order over ``torch.distributed``
    (a world of one executes them locally)."""

    def __init__(self, group=None):
        self.group = group
        self.pending: List[Tuple[CommunicationOp, torch.Tensor, dict]] = []
        self.completed = 0

    def schedule(self, op: CommunicationOp, tensor: torch.Tensor, **kw) -> int:
        self.pending.append((CommunicationOp(op), tensor, kw))
        return len(self.pending) - 1

    def execute_all(self) -> List[torch.Tensor]:
        import torch.distributed as dist
        live = dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1
        out = []
        for op, t, kw in self.pending:
            if live:
                if op is CommunicationOp.ALL_REDUCE:
                    dist.all_reduce(t, group=self.group)
                elif op is CommunicationOp.BROADCAST:
                    dist.broadcast(t, kw.get("src", 0), group=self.group)
                elif op is CommunicationOp.ALL_GATHER:
                    parts = [torch.empty_like(t) for _ in range(dist.get_world_size(self.group))]
                    dist.all_gather(parts, t, group=self.group)
                    t = torch.cat(parts, kw.get("dim", 0))
                elif op is CommunicationOp.REDUCE_SCATTER:
                    w = dist.get_world_size(self.group)
                    res = torch.empty_like(t.chunk(w, 0)[0])
                    dist.reduce_scatter_tensor(res, t.contiguous(), group=self.group)
                    t = res
                elif op is CommunicationOp.SEND:
                    dist.send(t, kw["dst"], group=self.group)
                elif op is CommunicationOp.RECV:
                    dist.recv(t, kw["src"], group=self.group)
                elif op is CommunicationOp.ALL_TO_ALL:
                    res = torch.empty_like(t)
                    dist.all_to_all_single(res, t.contiguous(), group=self.group)
                    t = res
            out.append(t)
            self.completed += 1
        self.pending.clear()
        return out
