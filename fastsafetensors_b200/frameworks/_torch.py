"""PyTorch side of the framework shim.

Counterpart of upstream ``fastsafetensors/frameworks/_torch.py``.  Differences that matter:

* file images are ordinary ``torch.uint8`` tensors (device or host) wrapped in a
  ``gds_device_buffer``; tensors handed to the caller are views of them, so no DLPack capsule
  is involved and the allocation is returned to torch's caching allocator by reference count;
* collectives do not end in a device-wide ``torch.cuda.synchronize()`` (upstream
  ``_torch.py:148-149`` and siblings): ``torch.distributed`` already orders the result on the
  caller's current stream, which is all a consumer on that stream needs;
* every dtype travels through collectives as raw bytes, so FP8/FP4 need no cast workaround.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..st_types import Device, DeviceType, DType
from . import FrameworkOpBase, ProcessGroupBase, TensorBase

dtype_convert: Dict[DType, Any] = {
    DType.BOOL: torch.bool,
    DType.U8: torch.uint8,
    DType.I8: torch.int8,
    DType.I16: torch.int16,
    DType.I32: torch.int32,
    DType.I64: torch.int64,
    DType.F16: torch.float16,
    DType.BF16: torch.bfloat16,
    DType.F32: torch.float32,
    DType.F64: torch.float64,
}
for _name, _attr in (
    (DType.F8_E5M2, "float8_e5m2"), (DType.F8_E4M3, "float8_e4m3fn"),
    (DType.F8_E8M0, "float8_e8m0fnu"), (DType.F4, "float4_e2m1fn_x2"),
    (DType.U16, "uint16"), (DType.U32, "uint32"), (DType.U64, "uint64"),
):
    if hasattr(torch, _attr):
        dtype_convert[_name] = getattr(torch, _attr)

# dtypes that upstream instantiates through an integer stand-in (its DLPack table lacks them)
need_workaround_dtypes: Dict[DType, DType] = {
    DType.F8_E5M2: DType.I8,
    DType.F8_E4M3: DType.I8,
    DType.F8_E8M0: DType.U8,
    DType.F4: DType.U8,
}


@dataclass
class TorchTensor(TensorBase):
    real_tensor: torch.Tensor

    def get_raw(self) -> torch.Tensor:
        return self.real_tensor

    def contiguous(self) -> "TorchTensor":
        return TorchTensor(self.device, self.dtype, self.real_tensor.contiguous())

    def to(self, device: Optional[Device] = None, dtype: DType = DType.AUTO) -> "TorchTensor":
        target_dev = device if device is not None and device != self.device else None
        target_dt = dtype if dtype not in (DType.AUTO, self.dtype) else None
        if target_dev is None and target_dt is None:
            return self
        moved = self.real_tensor.to(
            device=target_dev.as_str() if target_dev else None,
            dtype=dtype_convert[target_dt] if target_dt else None,
        )
        return TorchTensor(target_dev or self.device, target_dt or self.dtype, moved)

    def clone(self) -> "TorchTensor":
        return TorchTensor(self.device, self.dtype, self.real_tensor.clone())

    def detach(self) -> "TorchTensor":
        return TorchTensor(self.device, self.dtype, self.real_tensor.detach())

    def view(self, dtype: DType) -> "TorchTensor":
        return TorchTensor(self.device, dtype, self.real_tensor.view(dtype_convert[dtype]))

    def reshape(self, shape: List[int]) -> "TorchTensor":
        return TorchTensor(self.device, self.dtype, self.real_tensor.reshape(shape))

    def data_ptr(self) -> int:
        return self.real_tensor.data_ptr()

    def __getitem__(self, _val) -> "TorchTensor":
        return TorchTensor(self.device, self.dtype, self.real_tensor[_val])


def _bytes_view(t: torch.Tensor) -> torch.Tensor:
    """The tensor's bytes as a flat uint8 view (collectives move bytes, whatever the dtype)."""
    if not t.is_contiguous():
        raise ValueError("collectives need contiguous tensors")
    flat = t.reshape(-1)
    return flat if flat.dtype == torch.uint8 else flat.view(torch.uint8)


@dataclass
class TorchProcessGroup(ProcessGroupBase):
    real_pg: Optional[dist.ProcessGroup]

    def size(self) -> int:
        return self.real_pg.size() if self.real_pg else 1

    def rank(self) -> int:
        return self.real_pg.rank() if self.real_pg else 0

    def _global(self, group_rank: int) -> int:
        return dist.get_global_rank(self.real_pg, group_rank)

    def broadcast(self, dst: TorchTensor, rank: int) -> None:
        if self.real_pg:
            dist.broadcast(_bytes_view(dst.real_tensor), self._global(rank), group=self.real_pg)

    def scatter(self, dst: TorchTensor, scatter_list: List[TorchTensor], src: int) -> None:
        if self.real_pg:
            chunks = [_bytes_view(t.real_tensor) for t in scatter_list]
            dist.scatter(
                _bytes_view(dst.real_tensor),
                scatter_list=chunks if chunks else None,
                src=self._global(src),
                group=self.real_pg,
            )

    def send(self, t: TorchTensor, dst_rank: int, tag: int) -> None:
        if self.real_pg:
            dist.send(_bytes_view(t.real_tensor), self._global(dst_rank), group=self.real_pg, tag=tag)

    def recv(self, t: TorchTensor, src_rank: int, tag: int) -> None:
        if self.real_pg:
            dist.recv(_bytes_view(t.real_tensor), self._global(src_rank), group=self.real_pg, tag=tag)


class TorchOp(FrameworkOpBase):
    def __init__(self) -> None:
        self.mem_used = 0

    def get_name(self) -> str:
        return "pytorch"

    def get_device(self, device: Any, pg: ProcessGroupBase) -> Device:
        dev = torch.device(device)
        return Device(DeviceType(dev.type), dev.index)

    def set_device(self, device: Device) -> None:
        if device.type != DeviceType.CPU:
            torch.cuda.set_device(device.as_str())

    def alloc_tensor_memory(self, length: int, dev: Device):
        from ..cpp import gds_device_buffer

        on_gpu = dev.type != DeviceType.CPU
        backing = torch.empty(
            max(int(length), 1), dtype=torch.uint8, device=dev.as_str() if on_gpu else "cpu"
        )
        self.mem_used += length
        return gds_device_buffer(backing.data_ptr(), length, on_gpu, owner=backing)

    def free_tensor_memory(self, gbuf, dev: Device) -> None:
        self.mem_used -= gbuf.get_length()
        gbuf.release()

    def get_empty_tensor(self, shape: List[int], dtype: DType, device: Device) -> TorchTensor:
        native = self.get_native_shape(dtype, shape)
        return TorchTensor(
            device, dtype, torch.empty(size=native, dtype=dtype_convert[dtype], device=device.as_str())
        )

    def concat_tensors(self, tensors: List[TorchTensor], dim: int) -> TorchTensor:
        dtype = tensors[0].dtype
        if dtype in (DType.F8_E8M0, DType.F4):
            parts = [t.real_tensor.view(torch.uint8) for t in tensors]
            return TorchTensor(tensors[0].device, dtype, torch.cat(parts, dim=dim).view(dtype_convert[dtype]))
        return TorchTensor(tensors[0].device, dtype, torch.cat([t.real_tensor for t in tensors], dim=dim))

    def copy_tensor(self, dst: TorchTensor, src: TorchTensor) -> None:
        dst.real_tensor.copy_(src.real_tensor)

    def get_dtype_size(self, dtype: DType) -> float:
        return dtype.bits / 8.0

    def get_cuda_ver(self) -> str:
        if torch.cuda.is_available():
            return f"cuda-{torch.version.cuda}"
        return "0.0"

    def get_device_ptr_align(self) -> int:
        return 16

    def as_workaround_dtype(self, dtype: DType) -> DType:
        return need_workaround_dtypes.get(dtype, dtype)

    def get_storage_shape(self, dtype: DType, shape: List[int], strides: List[int]) -> Tuple[List[int], List[int]]:
        if dtype.bits >= 8:
            return shape, strides
        ratio = 8 // dtype.bits
        if not shape or shape[-1] % ratio:
            raise ValueError(
                f"Malformed input: {shape=}, {ratio=}, last dimension must be divisible by the packing ratio."
            )
        return [math.prod(shape) // ratio], [1]

    def get_native_shape(self, dtype: DType, st_shape: List[int]) -> List[int]:
        if dtype.bits >= 8:
            return st_shape
        ratio = 8 // dtype.bits
        if not st_shape or st_shape[-1] % ratio:
            raise ValueError(
                f"Malformed input: {st_shape=}, {ratio=}, last dimension must be divisible by the packing ratio."
            )
        return list(st_shape[:-1]) + [st_shape[-1] // ratio]

    def get_native_slices(self, dtype: DType, st_shape: List[int], slices: Tuple) -> Tuple:
        if dtype.bits >= 8 or not st_shape or len(slices) < len(st_shape):
            return slices
        ratio = 8 // dtype.bits
        out = list(slices)
        last = out[-1]
        extent = st_shape[-1]
        if isinstance(last, slice):
            if last.step not in (None, 1):
                raise ValueError(
                    f"Malformed input: {slices=}, {ratio=}, packed sub-byte slices only support step=1."
                )
            lo = min(max(0 if last.start is None else last.start, 0), extent)
            hi = min(max(extent if last.stop is None else last.stop, 0), extent)
            if lo % ratio or hi % ratio:
                raise ValueError(
                    f"Malformed input: {slices=}, {ratio=}, packed sub-byte slice bounds must align to storage units."
                )
            out[-1] = slice(lo // ratio, hi // ratio, 1)
        elif isinstance(last, int):
            if last % ratio:
                raise ValueError(
                    f"Malformed input: {slices=}, {ratio=}, packed sub-byte indices must align to storage units."
                )
            out[-1] = last // ratio
        return tuple(out)

    def synchronize(self, device: Device) -> None:
        if device.type != DeviceType.CPU and torch.cuda.is_available():
            torch.cuda.synchronize()

    def current_stream(self, device: Device) -> int:
        """Handle of torch's current stream on ``device`` (0 for the host)."""
        if device.type == DeviceType.CPU:
            return 0
        return int(torch.cuda.current_stream(device.index).cuda_stream)

    def get_global_rank(self) -> int:
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank()
        return 0

    def get_device_name(self, index: int) -> str:
        if not torch.cuda.is_available():
            return ""
        try:
            return torch.cuda.get_device_name(index)
        except Exception:
            return ""

    def get_process_group(self, pg: Optional[Any]) -> TorchProcessGroup:
        from ..common import SingleGroup

        if pg is None or isinstance(pg, SingleGroup):
            return TorchProcessGroup(None)
        if not isinstance(pg, dist.ProcessGroup):
            raise Exception("pg must be an instance of torch.disributed.ProcessGroup")
        return TorchProcessGroup(pg)

    def is_equal(self, wrapped: TorchTensor, real: Any) -> bool:
        if not isinstance(real, torch.Tensor):
            raise Exception("real is not torch.Tensor")
        return bool(torch.all(wrapped.real_tensor.eq(real)))

    def randn(self, s: tuple, device: Device, dtype: DType) -> TorchTensor:
        return TorchTensor(device, dtype, torch.randn(s, device=device.as_str(), dtype=dtype_convert[dtype]))

    def support_fp8(self) -> bool:
        return DType.F8_E5M2 in dtype_convert

    def get_mem_used(self) -> int:
        return self.mem_used


_op: Optional[TorchOp] = None


def get_framework_op() -> TorchOp:
    global _op
    if _op is None:
        _op = TorchOp()
    return _op
