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


class _DTypeBase(enum.Enum):
    @property
    def bits(self) -> int:
        """Bits per logical element in a safetensors file (F4 packs two values per byte)."""
        return _BITS[self.value]


# dtype strings of the safetensors format (member name == value), plus AUTO = "as stored"
_BITS = {
    "BOOL": 8, "I8": 8, "U8": 8, "F8_E5M2": 8, "F8_E4M3": 8, "F8_E8M0": 8,
    "I16": 16, "U16": 16, "F16": 16, "BF16": 16,
    "I32": 32, "U32": 32, "F32": 32,
    "I64": 64, "U64": 64, "F64": 64,
    "F4": 4,
}
DType = _DTypeBase("DType", {name: name for name in list(_BITS) + ["AUTO"]})
DType.__doc__ = "Element type of a tensor in a safetensors file; ``AUTO`` means: keep what the file has."
