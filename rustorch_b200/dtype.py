"""``DType`` enum with sizes, promotion and parsing (src/dtype.rs:7-225).

Unlike the reference, where the enum is metadata only (tensors are f32/f64), every entry here
maps to a real torch dtype.
"""
from __future__ import annotations

import enum

import torch


class DType(enum.Enum):
    F16 = "f16"
    BF16 = "bf16"
    F32 = "f32"
    F64 = "f64"
    I8 = "i8"
    I16 = "i16"
    I32 = "i32"
    I64 = "i64"
    U8 = "u8"
    BOOL = "bool"
    C64 = "c64"
    C128 = "c128"

    def to_torch(self) -> torch.dtype:
        return _TO_TORCH[self]

    @staticmethod
    def from_torch(dt: torch.dtype) -> "DType":
        return _FROM_TORCH[dt]

    def size(self) -> int:
        """Size in bytes of one element."""
        return torch.empty((), dtype=self.to_torch()).element_size()

    size_in_bytes = size

    def is_float(self) -> bool:
        return self in (DType.F16, DType.BF16, DType.F32, DType.F64)

    def is_int(self) -> bool:
        return self in (DType.I8, DType.I16, DType.I32, DType.I64, DType.U8)

    def is_complex(self) -> bool:
        return self in (DType.C64, DType.C128)

    def is_signed(self) -> bool:
        return self not in (DType.U8, DType.BOOL)

    def promote(self, other: "DType") -> "DType":
        return DType.from_torch(torch.promote_types(self.to_torch(), other.to_torch()))

    def __str__(self) -> str:
        return self.value


_TO_TORCH = {
    DType.F16: torch.float16, DType.BF16: torch.bfloat16, DType.F32: torch.float32, DType.F64: torch.float64,
    DType.I8: torch.int8, DType.I16: torch.int16, DType.I32: torch.int32, DType.I64: torch.int64,
    DType.U8: torch.uint8, DType.BOOL: torch.bool, DType.C64: torch.complex64, DType.C128: torch.complex128,
}
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}
_ALIASES = {"float16": "f16", "half": "f16", "bfloat16": "bf16", "float32": "f32", "float": "f32",
            "float64": "f64", "double": "f64", "int8": "i8", "int16": "i16", "int32": "i32", "int": "i32",
            "int64": "i64", "long": "i64", "uint8": "u8", "complex64": "c64", "complex128": "c128"}


def parse_dtype(name: str) -> DType:
    key = name.strip().lower()
    key = _ALIASES.get(key, key)
    try:
        return DType(key)
    except ValueError as e:
        raise ValueError(f"unknown dtype '{name}'") from e


def to_torch_dtype(d) -> torch.dtype:
    if isinstance(d, torch.dtype):
        return d
    if isinstance(d, DType):
        return d.to_torch()
    return parse_dtype(str(d)).to_torch()
