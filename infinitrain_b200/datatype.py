"""Data types, promotion rules and the tagged ``Scalar``.

Reference: infini_train/include/datatype.h:86-132, infini_train/src/datatype.cc:174-198,
infini_train/include/scalar.h:12-82.  Storage and arithmetic are PyTorch's; this module keeps the
reference's 13-entry enum, its names ("bf16", "fp32", ...), its byte sizes and its promotion rules
(fp16 with bf16 promotes to fp32; any float beats any integer; otherwise the wider type wins and the
first operand wins ties).
"""
from __future__ import annotations

import enum

import torch


class DataType(enum.IntEnum):
    kBOOL = 0
    kUINT8 = 1
    kINT8 = 2
    kUINT16 = 3
    kINT16 = 4
    kUINT32 = 5
    kINT32 = 6
    kUINT64 = 7
    kINT64 = 8
    kBFLOAT16 = 9
    kFLOAT16 = 10
    kFLOAT32 = 11
    kFLOAT64 = 12


kDataTypeToSize = {
    DataType.kBOOL: 1, DataType.kUINT8: 1, DataType.kINT8: 1, DataType.kUINT16: 2, DataType.kINT16: 2,
    DataType.kUINT32: 4, DataType.kINT32: 4, DataType.kUINT64: 8, DataType.kINT64: 8, DataType.kBFLOAT16: 2,
    DataType.kFLOAT16: 2, DataType.kFLOAT32: 4, DataType.kFLOAT64: 8,
}
kDataTypeToDesc = {
    DataType.kBOOL: "bool", DataType.kUINT8: "uint8", DataType.kINT8: "int8", DataType.kUINT16: "uint16",
    DataType.kINT16: "int16", DataType.kUINT32: "uint32", DataType.kINT32: "int32", DataType.kUINT64: "uint64",
    DataType.kINT64: "int64", DataType.kBFLOAT16: "bf16", DataType.kFLOAT16: "fp16", DataType.kFLOAT32: "fp32",
    DataType.kFLOAT64: "fp64",
}
_TO_TORCH = {
    DataType.kBOOL: torch.bool, DataType.kUINT8: torch.uint8, DataType.kINT8: torch.int8,
    DataType.kUINT16: torch.uint16, DataType.kINT16: torch.int16, DataType.kUINT32: torch.uint32,
    DataType.kINT32: torch.int32, DataType.kUINT64: torch.uint64, DataType.kINT64: torch.int64,
    DataType.kBFLOAT16: torch.bfloat16, DataType.kFLOAT16: torch.float16, DataType.kFLOAT32: torch.float32,
    DataType.kFLOAT64: torch.float64,
}
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}


def to_torch_dtype(dt) -> torch.dtype:
    if isinstance(dt, torch.dtype):
        return dt
    return _TO_TORCH[DataType(dt)]


def from_torch_dtype(dt: torch.dtype) -> DataType:
    return _FROM_TORCH[dt]


def parse_dtype(name: str) -> DataType:
    """'float32' / 'fp32' / 'bfloat16' / 'bf16' ... as accepted by the trainers' ``--dtype`` flag."""
    alias = {"float32": "fp32", "float": "fp32", "bfloat16": "bf16", "float16": "fp16", "half": "fp16",
             "float64": "fp64", "double": "fp64"}
    name = alias.get(name.lower(), name.lower())
    for k, v in kDataTypeToDesc.items():
        if v == name:
            return k
    raise ValueError(f"unknown dtype '{name}'")


def IsFloatingPointDType(dt: DataType) -> bool:
    return dt in (DataType.kFLOAT16, DataType.kBFLOAT16, DataType.kFLOAT32, DataType.kFLOAT64)


def PromoteDataTypes(a: DataType, b: DataType) -> DataType:
    if a == b:
        return a
    if {a, b} == {DataType.kFLOAT16, DataType.kBFLOAT16}:
        return DataType.kFLOAT32
    a_fp, b_fp = IsFloatingPointDType(a), IsFloatingPointDType(b)
    if a_fp and not b_fp:
        return a
    if b_fp and not a_fp:
        return b
    return a if kDataTypeToSize[a] >= kDataTypeToSize[b] else b


class Scalar:
    """A host scalar tagged bool / double / int64 / uint64 (reference: scalar.h:12-82)."""

    class Kind(enum.IntEnum):
        kBool = 0
        kDouble = 1
        kInt64 = 2
        kUInt64 = 3

    def __init__(self, value=0, unsigned: bool = False):
        if isinstance(value, Scalar):
            self.kind, self.value = value.kind, value.value
        elif isinstance(value, bool):
            self.kind, self.value = Scalar.Kind.kBool, bool(value)
        elif isinstance(value, float):
            self.kind, self.value = Scalar.Kind.kDouble, float(value)
        elif isinstance(value, int):
            self.kind = Scalar.Kind.kUInt64 if unsigned else Scalar.Kind.kInt64
            self.value = int(value)
        elif isinstance(value, torch.Tensor):
            v = value.item()
            self.__init__(v)
        else:
            raise TypeError(f"cannot build a Scalar from {type(value)}")

    def to(self, dtype):
        """Convert with the target type's rounding; half types round through fp32 (double ->
        float -> bf16), the two-step path the reference documents."""
        td = to_torch_dtype(dtype)
        if td in (torch.bfloat16, torch.float16):
            return torch.tensor(float(self.value), dtype=torch.float32).to(td).item()
        if td.is_floating_point:
            return torch.tensor(float(self.value), dtype=td).item()
        if td == torch.bool:
            return bool(self.value)
        return int(self.value)

    def __repr__(self):
        return f"Scalar({self.kind.name}, {self.value})"
