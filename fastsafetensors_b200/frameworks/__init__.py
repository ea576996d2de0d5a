"""Framework shim: the small surface through which the loader touches a tensor framework.

Mirrors the contract of upstream ``fastsafetensors/frameworks/__init__.py`` (``TensorBase``,
``ProcessGroupBase``, ``FrameworkOpBase``, ``get_framework_op``).  Only PyTorch is implemented:
the loader targets B200 through torch's allocator, streams and ``torch.distributed``.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, List, Optional, Tuple

from ..st_types import Device, DType


@dataclass
class TensorBase:
    """A framework tensor tagged with the loader's device and dtype vocabulary."""

    device: Device
    dtype: DType

    def get_raw(self) -> Any:
        raise NotImplementedError

    def contiguous(self) -> "TensorBase":
        raise NotImplementedError

    def to(self, device: Optional[Device] = None, dtype: DType = DType.AUTO) -> "TensorBase":
        raise NotImplementedError

    def clone(self) -> "TensorBase":
        raise NotImplementedError

    def detach(self) -> "TensorBase":
        raise NotImplementedError

    def view(self, dtype: DType) -> "TensorBase":
        raise NotImplementedError

    def reshape(self, shape: List[int]) -> "TensorBase":
        raise NotImplementedError(f"{type(self).__name__} does not implement reshape()")

    def data_ptr(self) -> int:
        raise NotImplementedError(f"{type(self).__name__} does not implement data_ptr()")

    def __getitem__(self, _val) -> "TensorBase":
        raise NotImplementedError


class ProcessGroupBase(ABC):
    @abstractmethod
    def size(self) -> int: ...

    @abstractmethod
    def rank(self) -> int: ...

    @abstractmethod
    def broadcast(self, dst: Any, rank: int) -> None: ...

    @abstractmethod
    def scatter(self, dst: Any, scatter_list: List[Any], src: int) -> None: ...

    @abstractmethod
    def send(self, t: Any, dst_rank: int, tag: int) -> None: ...

    @abstractmethod
    def recv(self, t: Any, src_rank: int, tag: int) -> None: ...


class FrameworkOpBase(ABC):
    """Operations the loader needs from a framework (see ``_torch.TorchOp``)."""

    @abstractmethod
    def get_name(self) -> str: ...

    @abstractmethod
    def get_device(self, device: Any, pg: ProcessGroupBase) -> Device: ...

    @abstractmethod
    def set_device(self, device: Device) -> None: ...

    @abstractmethod
    def alloc_tensor_memory(self, length: int, dev: Device) -> Any: ...

    @abstractmethod
    def free_tensor_memory(self, gbuf: Any, dev: Device) -> None: ...

    @abstractmethod
    def get_empty_tensor(self, shape: List[int], dtype: DType, device: Device) -> TensorBase: ...

    @abstractmethod
    def concat_tensors(self, tensors: List[Any], dim: int) -> TensorBase: ...

    @abstractmethod
    def copy_tensor(self, dst: Any, src: Any) -> None: ...

    @abstractmethod
    def get_dtype_size(self, dtype: DType) -> float: ...

    @abstractmethod
    def get_cuda_ver(self) -> str: ...

    @abstractmethod
    def get_device_ptr_align(self) -> int: ...

    @abstractmethod
    def as_workaround_dtype(self, dtype: DType) -> DType: ...

    @abstractmethod
    def get_process_group(self, pg: Optional[Any]) -> ProcessGroupBase: ...

    @abstractmethod
    def is_equal(self, wrapped: Any, real: Any) -> bool: ...

    @abstractmethod
    def randn(self, s: tuple, device: Device, dtype: DType) -> TensorBase: ...

    @abstractmethod
    def support_fp8(self) -> bool: ...

    @abstractmethod
    def get_mem_used(self) -> int: ...

    def get_storage_shape(self, dtype: DType, shape: List[int], strides: List[int]) -> Tuple[List[int], List[int]]:
        return shape, strides

    def get_native_shape(self, dtype: DType, st_shape: List[int]) -> List[int]:
        return st_shape

    def get_native_slices(self, dtype: DType, st_shape: List[int], slices: Tuple) -> Tuple:
        return slices

    def synchronize(self, device: Device) -> None:
        return None

    def get_global_rank(self) -> int:
        return 0

    def get_device_name(self, index: int) -> str:
        return ""


def get_framework_op(name: str) -> FrameworkOpBase:
    if name in ("pt", "pytorch", "torch"):
        from ._torch import get_framework_op as op

        return op()
    if name == "paddle":
        raise Exception("framework paddle is not supported by this build (PyTorch only)")
    raise Exception(f"Unknown framework name: {name}")
