"""Element types, numbered like the reference's on-disk dtype codes
(ghostflow-core/src/dtype.rs:7-29; codes used by ghostflow-core/src/serialize.rs:171-200)."""
from __future__ import annotations

import enum

import torch


class DType(enum.IntEnum):
    F16 = 0
    BF16 = 1
    F32 = 2
    F64 = 3
    I8 = 4
    I16 = 5
    I32 = 6
    I64 = 7
    U8 = 8
    Bool = 9

    def size_bytes(self) -> int:
        return _SIZES[self]

    def is_float(self) -> bool:
        return self in (DType.F16, DType.BF16, DType.F32, DType.F64)

    def to_torch(self) -> torch.dtype:
        return _TO_TORCH[self]

    @staticmethod
    def from_torch(dt: torch.dtype) -> "DType":
        return _FROM_TORCH[dt]


_TO_TORCH = {
    DType.F16: torch.float16, DType.BF16: torch.bfloat16, DType.F32: torch.float32, DType.F64: torch.float64,
    DType.I8: torch.int8, DType.I16: torch.int16, DType.I32: torch.int32, DType.I64: torch.int64,
    DType.U8: torch.uint8, DType.Bool: torch.bool,
}
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}
_SIZES = {DType.F16: 2, DType.BF16: 2, DType.F32: 4, DType.F64: 8, DType.I8: 1, DType.I16: 2, DType.I32: 4,
          DType.I64: 8, DType.U8: 1, DType.Bool: 1}
_NAMES = {"f16": DType.F16, "float16": DType.F16, "half": DType.F16, "bf16": DType.BF16, "bfloat16": DType.BF16,
          "f32": DType.F32, "float32": DType.F32, "float": DType.F32, "f64": DType.F64, "float64": DType.F64,
          "i8": DType.I8, "i16": DType.I16, "i32": DType.I32, "i64": DType.I64, "int64": DType.I64,
          "u8": DType.U8, "bool": DType.Bool}


def to_torch_dtype(d) -> torch.dtype:
    if isinstance(d, torch.dtype):
        return d
    if isinstance(d, DType):
        return _TO_TORCH[d]
    if isinstance(d, str):
        return _TO_TORCH[_NAMES[d.lower()]]
    raise TypeError(f"not a dtype: {d!r}")
