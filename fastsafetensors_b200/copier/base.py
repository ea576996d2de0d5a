"""Copier contract: one object per file that moves the file's data section to a buffer.

Same two-phase contract as upstream ``fastsafetensors/copier/base.py``: ``submit_io`` starts
the transfer and returns the destination buffer at once, ``wait_io`` blocks until the bytes are
there and returns the tensors instantiated over it.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Dict

from ..cpp import gds_device_buffer
from ..st_types import DType


class CopierInterface(ABC):
    @abstractmethod
    def submit_io(self, use_buf_register: bool, max_copy_block_size: int) -> gds_device_buffer:
        ...

    @abstractmethod
    def wait_io(self, gbuf: gds_device_buffer, dtype: DType = DType.AUTO,
                noalign: bool = False) -> Dict[str, Any]:
        ...


class DummyDeviceBuffer(gds_device_buffer):
    """Placeholder buffer that owns nothing (never freed)."""

    def __init__(self) -> None:
        super().__init__(0, 0, False)
