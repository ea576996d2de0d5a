"""The B200 copier: O_DIRECT / page-cache aware multi-threaded reads through a pinned ring,
overlapped with ``cudaMemcpyAsync`` on the reader's copy streams, realigned on the GPU when the
file's header length makes host and device addresses incongruent modulo 16.

It takes the place of both upstream copiers on this path: ``NoGdsFileCopier``
(``copier/nogds.py:15-78``: buffered pread + synchronous ``cudaMemcpy`` per chunk) and
``GdsFileCopier`` (``copier/gds.py:18-162``: cuFile into a 4 KiB-aligned window, then a
``memmove`` through a 1 GiB temporary when ``header_length % 16 != 0``).  It is registered under
both of their names, ``"nogds"`` and ``"gds"``, so that a loader built with either flag gets it.
The whole data section is one request; the native reader cuts it into ring-slot windows itself,
so ``max_copy_block_size`` has nothing left to decide here.
"""

from __future__ import annotations

import os
from typing import Any, Dict, Optional

from .. import _native as nat
from ..common import SafeTensorsMetadata
from ..cpp import Reader, gds_device_buffer, gds_file_reader
from ..st_types import Device, DeviceType, DType
from .base import CopierInterface
from .registry import CopierConstructFunc, register_copier_constructor

DEFAULT_SLOT_KB = 4096
_IO_MODES = {"auto": nat.IO_AUTO, "direct": nat.IO_DIRECT, "buffered": nat.IO_BUFFERED,
             "cufile": nat.IO_CUFILE}


class B200FileCopier(CopierInterface):
    def __init__(self, metadata: SafeTensorsMetadata, device: Device, reader: Reader, framework):
        self.metadata = metadata
        self.device = device
        # upstream's reader objects (cpp.nogds_file_reader / cpp.gds_file_reader) are accepted
        # too: they wrap a native reader
        if isinstance(reader, gds_file_reader):
            reader = reader._reader(False)
        self.reader = getattr(reader, "_reader", reader)
        self.framework = framework
        self.request: Optional[int] = None
        if not os.path.isfile(metadata.src):
            raise Exception(f"B200FileCopier.__init__: failed to open, file={metadata.src}")

    def submit_io(self, use_buf_register: bool, max_copy_block_size: int) -> gds_device_buffer:
        meta = self.metadata
        total = meta.size_bytes - meta.header_length
        gbuf = self.framework.alloc_tensor_memory(total, self.device)
        try:
            if self.device.type != DeviceType.CPU:
                # the image comes from torch's stream-ordered allocator: its memory may have
                # belonged to an image that a gather or a collective queued on the current stream
                # still reads, so the reader's own copy streams must queue behind that stream
                self.reader.order_after(self.framework.current_stream(self.device))
            self.request = self.reader.submit(meta.src, meta.header_length, total, gbuf, 0)
        except Exception:
            self.framework.free_tensor_memory(gbuf, self.device)
            raise
        return gbuf

    def drain(self) -> None:
        """Wait for the read without instantiating anything (the image is about to be dropped)."""
        if self.request is not None:
            request, self.request = self.request, None
            self.reader.wait(request)

    def wait_io(self, gbuf: gds_device_buffer, dtype: DType = DType.AUTO,
                noalign: bool = False) -> Dict[str, Any]:
        if self.request is not None:
            request, self.request = self.request, None
            try:
                self.reader.wait(request)
            except nat.NativeError as e:
                if e.code == nat.EGDS:
                    raise          # a RuntimeError naming "gds": callers retry without it
                raise Exception(f"wait_io: read of {self.metadata.src} failed: {e}") from e
        if dtype != DType.AUTO and self.device.type != DeviceType.CPU:
            tensors = self.metadata.get_tensors(gbuf, self.device, self.metadata.header_length)
            return self._convert_on_device(gbuf, tensors, dtype)
        return self.metadata.get_tensors(gbuf, self.device, self.metadata.header_length, dtype=dtype)

    def _convert_on_device(self, gbuf: gds_device_buffer, tensors: Dict[str, Any], dtype: DType) -> Dict[str, Any]:
        """Load-time narrowing (upstream common.py:355-375) on a CUDA image: every tensor is
        converted out of place into a new, compact image by ONE launch of the convert kernel
        (plus one gather launch for tensors that already have the target type); pairs the kernel
        does not know go through ``torch.Tensor.to`` as upstream's all do.  The old image is
        released and ``gbuf`` takes over the new one."""
        import torch

        from ..frameworks._torch import TorchTensor, dtype_convert

        meta = self.metadata
        for name, frame in meta.tensors.items():
            if dtype.bits > frame.dtype.bits:
                raise Exception(
                    f"Online type conversion to larger sizes is not supported ({frame.dtype} -> {dtype})")
        offsets: Dict[str, int] = {}
        total = 0
        for name, frame in meta.tensors.items():
            offsets[name] = total
            count = 1
            for extent in frame.shape:
                count *= extent
            total += (count * dtype.bits // 8 + 15) // 16 * 16
        new = self.framework.alloc_tensor_memory(total, self.device)
        image = new.owner
        stream = self.framework.current_stream(self.device)
        convert_ops, copy_ops = [], []
        out: Dict[str, Any] = {}
        for name, frame in meta.tensors.items():
            src = tensors[name].get_raw()
            count = src.numel()
            nbytes = count * dtype.bits // 8
            view = image[offsets[name]: offsets[name] + nbytes].view(dtype_convert[dtype]).reshape(frame.shape)
            s_code, d_code = nat.DT_CODES.get(frame.dtype.value), nat.DT_CODES.get(dtype.value)
            if frame.dtype == dtype:
                copy_ops.append((src.data_ptr(), view.data_ptr(), 1, nbytes, 0, 0))
            elif s_code is not None and d_code is not None and d_code != 0:
                convert_ops.append((src.data_ptr(), view.data_ptr(), count, s_code, d_code))
            elif count:
                view.copy_(src.to(dtype=dtype_convert[dtype]))
            frame.dtype = dtype
            out[name] = TorchTensor(self.device, dtype, view)
        nat.convert(convert_ops, stream)
        nat.gather(copy_ops, stream)
        tensors.clear()
        # The launches above still read the old image.  Releasing it now is safe: torch hands
        # the memory only to later allocations of the same stream, and whoever writes it from
        # another stream orders itself behind this one first (submit_io does, for the reader).
        self.framework.free_tensor_memory(gbuf, self.device)
        gbuf.adopt(new)
        return out


def new_b200_file_copier(device: Device, bbuf_size_kb: int = 16 * 1024, max_threads: int = 16,
                         io_mode: Optional[str] = None, slot_kb: Optional[int] = None,
                         copy_streams: int = 4, numa_node: Optional[int] = None,
                         plain_dma_only: bool = False, **kwargs) -> CopierConstructFunc:
    """One native reader per loader, shared by the copiers of all its files.

    ``bbuf_size_kb`` keeps upstream's meaning of a total ring size but only as a lower bound:
    each worker gets two slots of at least ``slot_kb`` KiB (default 4 MiB, or the
    ``FST_B200_SLOT_KB`` environment variable), large enough for direct I/O and DMA to run at
    full rate.  ``io_mode`` is ``"auto"`` (default, or ``FST_B200_IO_MODE``), ``"direct"``,
    ``"buffered"`` or ``"cufile"`` (``cuFileRead`` into a registered device staging ring; a
    ``RuntimeError`` whose text contains "gds" is raised where cuFile cannot be used, which is
    what callers such as vLLM catch to retry with ``nogds=True``).
    """
    on_gpu = device.type != DeviceType.CPU
    if on_gpu and nat.cuda_device_count() == 0:
        raise Exception("[FAIL] no CUDA device is visible but a GPU device was requested")
    mode = (io_mode or os.environ.get("FST_B200_IO_MODE", "auto")).lower()
    if mode not in _IO_MODES:
        raise ValueError(f"io_mode must be one of {sorted(_IO_MODES)}, got {mode!r}")
    slot_kb = int(slot_kb or os.environ.get("FST_B200_SLOT_KB", DEFAULT_SLOT_KB))
    threads = max(1, int(max_threads))
    slot_bytes = max(slot_kb * 1024, bbuf_size_kb * 1024 // (threads * 2))
    index = (device.index if device.index is not None else 0) if on_gpu else -1
    if numa_node is None:
        numa_node = -1
    reader = Reader(index, threads, slot_bytes, 2, io_mode=_IO_MODES[mode],
                    copy_streams=copy_streams, numa_node=numa_node,
                    plain_dma_only=plain_dma_only)

    def construct(metadata: SafeTensorsMetadata, device: Device, framework) -> CopierInterface:
        return B200FileCopier(metadata, device, reader, framework)

    construct.reader = reader  # type: ignore[attr-defined]
    return construct


register_copier_constructor("nogds")(new_b200_file_copier)
register_copier_constructor("gds")(new_b200_file_copier)
register_copier_constructor("b200")(new_b200_file_copier)
