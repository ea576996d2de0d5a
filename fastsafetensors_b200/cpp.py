"""Python face of the native layer, under the names upstream's pybind11 module exports.

Upstream code and tests reach native code through ``fastsafetensors.cpp`` (stub:
``fastsafetensors/cpp.pyi``).  This module offers the same names on top of the C ABI in
``include/fst_b200.h`` so that such code keeps working: ``gds_device_buffer``,
``nogds_file_reader``, ``gds_file_handle``, ``gds_file_reader``, ``get_cpp_metrics`` and the
small query functions.  The loader itself uses ``Reader`` (below) directly.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import byref, c_int64, c_uint64
from typing import Any, Dict, Optional, Tuple

from . import _native as nat
from ._native import NativeError


# ------------------------------------------------------------------------------------------
# buffers
# ------------------------------------------------------------------------------------------
class gds_device_buffer:
    """A (base address, length) pair naming device or host memory; optionally keeps the object
    that owns the memory alive.  Same methods as upstream's class (ext.hpp:128-153)."""

    def __init__(self, devPtr_base: int, length: int, use_cuda: bool, owner: Any = None) -> None:
        self._base = int(devPtr_base)
        self._length = int(length)
        self._use_cuda = bool(use_cuda)
        self._owner = owner

    def get_base_address(self) -> int:
        return self._base

    def get_length(self) -> int:
        return self._length

    @property
    def use_cuda(self) -> bool:
        return self._use_cuda

    @property
    def owner(self) -> Any:
        return self._owner

    def release(self) -> None:
        """Drop the reference to the owning allocation (views of it keep it alive)."""
        self._owner = None

    def adopt(self, other: "gds_device_buffer") -> None:
        """Become ``other`` (address, length, owner); ``other`` is emptied."""
        self._base, self._length, self._use_cuda, self._owner = (
            other._base, other._length, other._use_cuda, other._owner)
        other._owner = None

    def check_range(self, offset: int, length: int) -> int:
        if offset < 0 or length < 0 or offset + length > self._length:
            raise IndexError(
                f"out of bound access: 0x{self._base:x}, length={self._length}, "
                f"request offset={offset}, request length={length}"
            )
        return self._base + offset

    # cuFile registration is a property of the reader's own staging ring here, not of the
    # destination buffer; these stay for callers that follow upstream's call sequence.
    def cufile_register(self, offset: int, length: int) -> int:
        self.check_range(offset, length)
        return 0

    def cufile_deregister(self, offset: int) -> int:
        return 0

    def memmove(self, dst_off: int, src_off: int, tmp: "gds_device_buffer", length: int) -> int:
        """Move ``length`` bytes inside this buffer through ``tmp`` (ext.cpp:606-645).  On a
        device buffer this is two launches of the realign kernel on the current stream followed
        by a stream synchronisation, as upstream's two ``cudaMemcpy`` are synchronous."""
        if self._length < dst_off or self._length < src_off or tmp.get_length() < length:
            return -1
        if length == 0:
            return 0
        src, dst, t = self._base + src_off, self._base + dst_off, tmp.get_base_address()
        if self._use_cuda:
            import torch

            stream = int(torch.cuda.current_stream().cuda_stream)
            try:
                nat.realign(t, src, length, stream)
                nat.realign(dst, t, length, stream)
            except NativeError:
                return -1
            torch.cuda.current_stream().synchronize()
        else:
            ctypes.memmove(t, src, length)
            ctypes.memmove(dst, t, length)
        return 0


# ------------------------------------------------------------------------------------------
# reader
# ------------------------------------------------------------------------------------------
class Reader:
    """Owner of one native reader (``fst_reader_*``)."""

    def __init__(self, device_index: int, threads: int, slot_bytes: int, slots_per_thread: int = 2,
                 io_mode: int = nat.IO_AUTO, copy_streams: int = 4, numa_node: int = -1,
                 plain_dma_only: bool = False) -> None:
        cfg = nat.ReaderConfig()
        cfg.device = device_index
        cfg.threads = threads
        cfg.slots_per_thread = slots_per_thread
        cfg.io_mode = io_mode
        cfg.slot_bytes = slot_bytes
        cfg.copy_streams = copy_streams
        cfg.numa_node = numa_node
        cfg.plain_dma_only = 1 if plain_dma_only else 0
        handle = c_uint64(0)
        nat.check(nat.lib.fst_reader_create(byref(cfg), byref(handle)), "fst_reader_create")
        self._handle: Optional[int] = handle.value

    def submit(self, path: str, file_offset: int, nbytes: int, dst: gds_device_buffer,
               dst_offset: int) -> int:
        req = c_int64(0)
        nat.check(
            nat.lib.fst_reader_submit(self._handle, os.fsencode(path), file_offset, nbytes,
                                      dst.get_base_address(), dst.get_length(), dst_offset,
                                      byref(req)),
            "fst_reader_submit",
        )
        return req.value

    def order_after(self, stream: int) -> None:
        """Order the reader's copies behind the work queued so far on ``stream`` (a
        ``cudaStream_t`` as an integer); see ``fst_reader_order_after``."""
        nat.check(nat.lib.fst_reader_order_after(self._handle, stream), "fst_reader_order_after")

    def wait(self, request: int, timeout_ms: int = -1) -> int:
        done = c_uint64(0)
        nat.check(nat.lib.fst_reader_wait(self._handle, request, timeout_ms, byref(done)),
                  "fst_reader_wait")
        return done.value

    def inject_fault(self, nth: int, err: int = 5, short_bytes: int = -1) -> None:
        nat.check(nat.lib.fst_reader_inject_fault(self._handle, nth, err, short_bytes),
                  "fst_reader_inject_fault")

    def close(self) -> None:
        if self._handle is not None:
            nat.lib.fst_reader_destroy(self._handle)
            self._handle = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass


class nogds_file_reader:
    """Upstream's bounce-buffer reader interface (ext.hpp:155-185) over the native reader.
    ``bbuf_size_kb`` is the total ring size; each of ``max_threads`` workers gets two slots."""

    def __init__(self, use_mmap: bool, bbuf_size_kb: int, max_threads: int, use_cuda: bool,
                 device_id: int) -> None:
        per_thread = (bbuf_size_kb + max_threads - 1) // max_threads * 1024
        slot = max(4096, per_thread // 2)
        self._reader = Reader(device_id if use_cuda else -1, max_threads, slot, 2,
                              io_mode=nat.IO_BUFFERED)
        self._results: Dict[int, int] = {}

    def submit_read(self, fd: int, dst: gds_device_buffer, offset: int, length: int, ptr_off: int) -> int:
        try:
            rid = self._reader.submit(f"/proc/self/fd/{fd}", offset, length, dst, ptr_off)
        except NativeError as e:
            if e.code == nat.ERANGE:
                raise IndexError(str(e)) from None
            return -1
        self._results[rid] = dst.get_base_address() + ptr_off
        return rid

    def wait_read(self, thread_id: int) -> int:
        addr = self._results.pop(thread_id, 0)
        try:
            self._reader.wait(thread_id)
        except NativeError:
            return 0
        return addr


class gds_file_handle:
    """A file named for later reads (ext.hpp:187-208).  No cuFile registration happens here."""

    def __init__(self, filename: str, o_direct: bool, use_cuda: bool) -> None:
        if not os.path.exists(filename):
            raise RuntimeError(f"raw_gds_file_handle: open returned an error = 2 (gds file {filename})")
        self.filename = filename
        self.o_direct = bool(o_direct)
        self.use_cuda = bool(use_cuda)


class gds_file_reader:
    """Upstream's cuFile reader interface (ext.hpp:210-227) over the native reader."""

    def __init__(self, max_threads: int, use_cuda: bool, device_id: int) -> None:
        self._args = (device_id if use_cuda else -1, max_threads)
        self._readers: Dict[bool, Reader] = {}
        self._pending: Dict[int, Tuple[Reader, int]] = {}
        self._next = 1

    def _reader(self, o_direct: bool) -> Reader:
        if o_direct not in self._readers:
            self._readers[o_direct] = Reader(
                self._args[0], self._args[1], 4 << 20, 2,
                io_mode=nat.IO_DIRECT if o_direct else nat.IO_BUFFERED,
            )
        return self._readers[o_direct]

    def submit_read(self, fh: gds_file_handle, dst: gds_device_buffer, offset: int, length: int,
                    ptr_off: int, file_length: int) -> int:
        n = max(0, min(length, file_length - offset))
        dst.check_range(ptr_off, length)
        reader = self._reader(fh.o_direct)
        try:
            rid = reader.submit(fh.filename, offset, n, dst, ptr_off)
        except NativeError:
            return -1
        my_id = self._next
        self._next += 1
        self._pending[my_id] = (reader, rid)
        return my_id

    def wait_read(self, id: int) -> int:
        reader, rid = self._pending.pop(id)
        try:
            return reader.wait(rid)
        except NativeError:
            return -1


# ------------------------------------------------------------------------------------------
# queries and small helpers (names of cpp.pyi)
# ------------------------------------------------------------------------------------------
class cpp_metrics:
    def __init__(self) -> None:
        m = nat.get_metrics()
        for name, _ in m._fields_:
            if name != "reserved":
                setattr(self, name, int(getattr(m, name)))


def get_cpp_metrics() -> cpp_metrics:
    return cpp_metrics()


def is_cuda_found() -> bool:
    return nat.cuda_device_count() > 0


def is_hip_found() -> bool:
    return False


def is_cufile_found() -> bool:
    return bool(nat.lib.fst_cufile_available())


def cufile_version() -> int:
    return 0


def is_gds_supported(deviceId: int) -> int:
    return int(nat.lib.fst_gds_supported(deviceId))


def init_gds() -> int:
    return 0


def close_gds() -> int:
    return 0


def get_alignment_size() -> int:
    return int(nat.lib.fst_io_alignment())


def set_debug_log(debug_log: bool) -> None:
    nat.lib.fst_set_debug(1 if debug_log else 0)


def get_device_pci_bus(deviceId: int) -> str:
    buf = ctypes.create_string_buffer(64)
    if nat.lib.fst_device_pci_bus(deviceId, buf, 64) != 0:
        return ""
    return buf.value.decode()


def set_numa_node(numa_node: int) -> int:
    return int(nat.lib.fst_pin_numa(numa_node))


def read_buffer(dst: int, length: int) -> bytes:
    out = ctypes.create_string_buffer(length)
    nat.check(nat.lib.fst_read_host(dst, length, out), "fst_read_host")
    return out.raw


def cpu_malloc(length: int) -> int:
    return int(nat.lib.fst_host_alloc(length))


def cpu_free(addr: int) -> None:
    nat.lib.fst_host_free(addr)


def gpu_malloc(length: int) -> int:
    """``cudaMalloc`` on the current device; 0 on failure (ext.cpp:559-565)."""
    return int(nat.lib.fst_device_alloc(length))


def gpu_free(addr: int) -> None:
    nat.lib.fst_device_free(addr)


def memcpy_h2d_async(dst: int, src: int, size: int) -> int:
    """``cudaMemcpyAsync`` host -> device on the default stream; returns the CUDA error code,
    -1 without a CUDA device (ext.cpp:959-971)."""
    rc = int(nat.lib.fst_memcpy_h2d_async(dst, src, size))
    return -1 if rc == nat.ENOCUDA else rc


def load_library_functions(cudart_lib_name: str = "") -> None:
    """Nothing to load: the CUDA runtime is linked into the native library."""


_gil_release = True


def set_gil_release(gil_release: bool) -> None:
    """ctypes always drops the GIL around native calls; the flag is kept for callers."""
    global _gil_release
    _gil_release = bool(gil_release)


def get_gil_release() -> bool:
    return _gil_release
