"""Device and dtype vocabulary of the loader API.

Same names and values as upstream ``fastsafetensors/st_types.py`` (``Device``, ``DeviceType``,
``DType``), so that code written against upstream runs unchanged.  ``DType`` additionally knows
how many bits one element of each safetensors dtype occupies in the file, which the shard
geometry needs and which does not depend on any framework.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Optional


class DeviceType(enum.Enum):
    CPU = "cpu"
    CUDA = "cuda"
    GPU = "gpu"


@dataclass(frozen=True)
class Device:
    type: DeviceType = DeviceType.CPU
    index: Optional[int] = None

    def as_str(self) -> str:
        return self.type.value if self.index is None else f"{self.type.value}:{self.index}"

    @classmethod
    def from_str(cls, s: str) -> "Device":
        kind, sep, idx = s.partition(":")
        try:
            dev_type = DeviceType(kind.lower())
        except ValueError:
            raise ValueError(f"Unknown device type: {kind}") from None
        if not sep:
            return cls(type=dev_type, index=None)
        try:
            return cls(type=dev_type, index=int(idx))
        except ValueError:
            raise ValueError(f"Invalid index: {idx}") from None

    @property
    def is_cpu(self) -> bool:
        return self.type == DeviceType.CPU


class DType(enum.Enum):
    BOOL = "BOOL"
    I8 = "I8"
    I16 = "I16"
    I32 = "I32"
    I64 = "I64"
    U8 = "U8"
    U16 = "U16"
    U32 = "U32"
    U64 = "U64"
    F16 = "F16"
    F32 = "F32"
    F64 = "F64"
    BF16 = "BF16"
    F8_E5M2 = "F8_E5M2"
    F8_E4M3 = "F8_E4M3"
    F8_E8M0 = "F8_E8M0"
    F4 = "F4"
    AUTO = "AUTO"

    @property
    def bits(self) -> int:
        """Bits per logical element in a safetensors file (F4 packs two values per byte)."""
        return _BITS[self]


_BITS = {
    DType.BOOL: 8, DType.I8: 8, DType.U8: 8, DType.F8_E5M2: 8, DType.F8_E4M3: 8,
    DType.F8_E8M0: 8, DType.I16: 16, DType.U16: 16, DType.F16: 16, DType.BF16: 16,
    DType.I32: 32, DType.U32: 32, DType.F32: 32, DType.I64: 64, DType.U64: 64,
    DType.F64: 64, DType.F4: 4,
}
