"""Unified error type (src/error.rs:11-535, src/common/error_handling.rs).

The reference has one enum with ~60 variants and helper constructors; here every variant is a subclass of
``RusTorchError`` (so ``except RusTorchError`` catches all of them and ``except ShapeMismatch`` one of them), and the
helper constructors keep their names as class methods.  ``RusTorchResult`` is only an annotation alias: Python
functions raise instead of returning ``Err``.
"""
from __future__ import annotations

from typing import Any, Optional, Sequence, TypeVar, Union

T = TypeVar("T")


class RusTorchError(Exception):
    """Base of all framework errors; ``kind`` names the reference's enum variant."""

    kind = "RusTorchError"

    def __init__(self, message: str = "", error_code: Optional[int] = None, **context: Any):
        super().__init__(message)
        self.message, self.error_code, self.context = message, error_code, context

    def __str__(self) -> str:
        ctx = ", ".join(f"{k}={v}" for k, v in self.context.items())
        return f"{self.kind}: {self.message}" + (f" ({ctx})" if ctx else "")

    # ---- helper constructors of the reference
    @classmethod
    def shape_mismatch(cls, expected: Sequence[int], actual: Sequence[int]) -> "ShapeMismatch":
        return ShapeMismatch(f"expected {list(expected)}, got {list(actual)}", expected=list(expected), actual=list(actual))

    @classmethod
    def tensor_op(cls, message: str) -> "TensorOp":
        return TensorOp(message)

    @classmethod
    def invalid_dimension(cls, dim: int, rank: int) -> "InvalidDimension":
        return InvalidDimension(f"dimension {dim} out of range for a rank-{rank} tensor", dim=dim, rank=rank)

    @classmethod
    def device_not_available(cls, device: str) -> "DeviceNotAvailable":
        return DeviceNotAvailable(f"device '{device}' is not available", device=device)

    @classmethod
    def gpu(cls, message: str) -> "GpuError":
        return GpuError(message)

    @classmethod
    def invalid_params(cls, operation: str, message: str) -> "InvalidParameters":
        return InvalidParameters(message, operation=operation)

    @classmethod
    def io(cls, message: str) -> "IoError":
        return IoError(message)

    @classmethod
    def serialization(cls, message: str) -> "SerializationError":
        return SerializationError(message)

    @classmethod
    def distributed(cls, message: str) -> "DistributedError":
        return DistributedError(message)

    @classmethod
    def not_implemented(cls, feature: str) -> "NotImplementedFeature":
        return NotImplementedFeature(f"{feature} is not implemented", feature=feature)


def _variant(name: str, base=RusTorchError):
    parent = "" if base is RusTorchError else f"; also caught as ``{base.__name__}``"
    return type(name, (base,), {"kind": name, "__doc__": f"Error kind ``{name}``{parent} (kinds are named after the variants of the reference's ``RusTorchError``, src/error.rs:11-535)."})


TensorOp = _variant("TensorOp")
ShapeMismatch = _variant("ShapeMismatch", TensorOp)
InvalidDimension = _variant("InvalidDimension", TensorOp)
IndexOutOfBounds = _variant("IndexOutOfBounds", TensorOp)
BroadcastError = _variant("BroadcastError", TensorOp)
EmptyTensor = _variant("EmptyTensor", TensorOp)
TypeError_ = _variant("TypeError")
DTypeMismatch = _variant("DTypeMismatch", TypeError_)
InvalidParameters = _variant("InvalidParameters")
InvalidOperation = _variant("InvalidOperation")
NumericalError = _variant("NumericalError")
OverflowError_ = _variant("OverflowError", NumericalError)
DivisionByZero = _variant("DivisionByZero", NumericalError)
AutogradError = _variant("AutogradError")
NeuralNetworkError = _variant("NeuralNetworkError")
OptimizerError = _variant("OptimizerError")
DataError = _variant("DataError")
DataLoaderError = _variant("DataLoaderError", DataError)
DeviceError = _variant("DeviceError")
DeviceNotAvailable = _variant("DeviceNotAvailable", DeviceError)
GpuError = _variant("GpuError", DeviceError)
CudaError = _variant("CudaError", GpuError)
KernelError = type("KernelError", (GpuError, RuntimeError), {
    "kind": "KernelError", "__doc__": "A native kernel reported a non-zero status word; also a ``RuntimeError`` and a ``GpuError``."})
KernelTimeout = _variant("KernelTimeout", KernelError)
OutOfMemory = _variant("OutOfMemory", DeviceError)
MemoryError_ = _variant("MemoryError")
AllocationError = _variant("AllocationError", MemoryError_)
IoError = _variant("IoError")
SerializationError = _variant("SerializationError", IoError)
DeserializationError = _variant("DeserializationError", IoError)
ModelFormatError = _variant("ModelFormatError", IoError)
ChecksumMismatch = _variant("ChecksumMismatch", IoError)
ImportError_ = _variant("ImportError")
UnsupportedOperator = _variant("UnsupportedOperator", ImportError_)
DistributedError = _variant("DistributedError")
CommunicationError = _variant("CommunicationError", DistributedError)
ProcessGroupError = _variant("ProcessGroupError", DistributedError)
ClusterError = _variant("ClusterError", DistributedError)
TimeoutError_ = _variant("TimeoutError", DistributedError)
BackendNotAvailable = _variant("BackendNotAvailable", DistributedError)
ProfilerError = _variant("ProfilerError")
ValidationError = _variant("ValidationError")
DebugError = _variant("DebugError")
VisualizationError = _variant("VisualizationError")
QuantizationError = _variant("QuantizationError")
SparseError = _variant("SparseError")
ConfigError = _variant("ConfigError")
NotImplementedFeature = _variant("NotImplementedFeature")
Unsupported = _variant("Unsupported")

RusTorchResult = Union[T, RusTorchError]          # annotation only


def check_status_to_error(code: int, message: Optional[str] = None) -> Optional[RusTorchError]:
    """Device status words of the native kernels (0 = fine) as framework errors."""
    if code == 0:
        return None
    if 101 <= code <= 105:
        return KernelTimeout(message or "a bounded device-side wait ran out", code, code=code)
    if code == 201:
        return IndexOutOfBounds(message or "index or alignment check failed in a kernel", code, code=code)
    return KernelError(message or "kernel reported an error", code, code=code)


__all__ = [n for n, v in list(globals().items()) if isinstance(v, type) and issubclass(v, RusTorchError)] + ["RusTorchResult", "check_status_to_error"]
