"""ctypes binding of ``libfst_b200.so`` (declared in ``include/fst_b200.h``).

The library is loaded from the package directory only.  If it is missing the import of this
module raises: there is no pure-Python or torch substitute for the native layer.  Build it with
``python fastsafetensors_b200/_build.py``.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import (
    POINTER,
    Structure,
    byref,
    c_char_p,
    c_int,
    c_int32,
    c_int64,
    c_uint64,
    c_void_p,
)
from typing import Sequence, Tuple

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libfst_b200.so")

ABI_VERSION = 2

# status codes of include/fst_b200.h
OK, EINVAL, ERANGE, ENOCUDA, ECUDA, EIO, ETIMEOUT, ENOMEM, ELIMIT, EGDS = (
    0, -1, -2, -3, -4, -5, -6, -7, -8, -9,
)
IO_AUTO, IO_DIRECT, IO_BUFFERED, IO_CUFILE = 0, 1, 2, 3
GATHER_INLINE_OPS = 48
GATHER_STATIC_MAX_OPS = 4096
ARENA_HANDLE_BYTES = 64

# every symbol the header declares; tests check that the library exports each one
EXPORTS = (
    "fst_abi_version", "fst_last_error", "fst_cuda_device_count", "fst_set_debug",
    "fst_device_pci_bus", "fst_device_numa_node", "fst_pin_numa", "fst_host_alloc",
    "fst_host_free", "fst_read_host", "fst_io_alignment", "fst_get_metrics",
    "fst_reader_create", "fst_reader_submit", "fst_reader_wait", "fst_reader_destroy",
    "fst_reader_inject_fault", "fst_gather", "fst_gather_static", "fst_gather_host",
    "fst_realign", "fst_release_workspaces", "fst_arena_create", "fst_arena_export",
    "fst_arena_open_peer", "fst_arena_close_peer", "fst_arena_destroy", "fst_convert",
    "fst_cufile_available", "fst_gds_supported", "fst_reader_order_after", "fst_device_alloc",
    "fst_device_free", "fst_memcpy_h2d_async", "fst_gather_limited",
)


class Metrics(Structure):
    _fields_ = [
        ("bounce_buffer_bytes", c_uint64),
        ("staging_device_bytes", c_uint64),
        ("bytes_read", c_uint64),
        ("bytes_h2d", c_uint64),
        ("bytes_realigned", c_uint64),
        ("bytes_gathered", c_uint64),
        ("kernel_launches", c_uint64),
        ("direct_io_requests", c_uint64),
        ("buffered_io_requests", c_uint64),
        ("read_ns", c_uint64),
        ("reserved", c_uint64 * 6),
    ]


class ReaderConfig(Structure):
    _fields_ = [
        ("device", c_int32),
        ("threads", c_int32),
        ("slots_per_thread", c_int32),
        ("io_mode", c_int32),
        ("slot_bytes", c_uint64),
        ("copy_streams", c_int32),
        ("numa_node", c_int32),
        ("plain_dma_only", c_int32),
        ("reserved", c_int32 * 7),
    ]


class Copy2D(Structure):
    _fields_ = [
        ("src", c_uint64),
        ("dst", c_uint64),
        ("rows", c_uint64),
        ("row_bytes", c_uint64),
        ("src_pitch", c_uint64),
        ("dst_pitch", c_uint64),
    ]


class ConvertOp(Structure):
    _fields_ = [
        ("src", c_uint64),
        ("dst", c_uint64),
        ("n_elements", c_uint64),
        ("src_dtype", c_int32),
        ("dst_dtype", c_int32),
    ]


DT_CODES = {"F64": 0, "F32": 1, "F16": 2, "BF16": 3}


class NativeError(RuntimeError):
    """A native entry point returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the native CUDA layer has not been built "
            "(run `python fastsafetensors_b200/_build.py`); there is no fallback"
        )
    lib = ctypes.CDLL(LIB_PATH)
    lib.fst_abi_version.restype = c_int
    lib.fst_last_error.restype = c_char_p
    lib.fst_cuda_device_count.restype = c_int
    lib.fst_set_debug.argtypes = [c_int]
    lib.fst_set_debug.restype = None
    lib.fst_device_pci_bus.argtypes = [c_int, c_char_p, c_int]
    lib.fst_device_numa_node.argtypes = [c_int]
    lib.fst_pin_numa.argtypes = [c_int]
    lib.fst_host_alloc.argtypes = [c_uint64]
    lib.fst_host_alloc.restype = c_uint64
    lib.fst_host_free.argtypes = [c_uint64]
    lib.fst_host_free.restype = None
    lib.fst_read_host.argtypes = [c_uint64, c_uint64, c_void_p]
    lib.fst_io_alignment.restype = c_int
    lib.fst_get_metrics.argtypes = [POINTER(Metrics)]
    lib.fst_reader_create.argtypes = [POINTER(ReaderConfig), POINTER(c_uint64)]
    lib.fst_reader_submit.argtypes = [
        c_uint64, c_char_p, c_uint64, c_uint64, c_uint64, c_uint64, c_uint64, POINTER(c_int64),
    ]
    lib.fst_reader_wait.argtypes = [c_uint64, c_int64, c_int64, POINTER(c_uint64)]
    lib.fst_reader_destroy.argtypes = [c_uint64]
    lib.fst_reader_order_after.argtypes = [c_uint64, c_uint64]
    lib.fst_device_alloc.argtypes = [c_uint64]
    lib.fst_device_alloc.restype = c_uint64
    lib.fst_device_free.argtypes = [c_uint64]
    lib.fst_device_free.restype = None
    lib.fst_memcpy_h2d_async.argtypes = [c_uint64, c_uint64, c_uint64]
    lib.fst_reader_inject_fault.argtypes = [c_uint64, c_int64, c_int, c_int64]
    lib.fst_gather.argtypes = [
        POINTER(Copy2D), c_uint64, c_uint64, c_uint64, c_uint64, c_uint64, c_uint64,
    ]
    lib.fst_gather_static.argtypes = lib.fst_gather.argtypes
    lib.fst_gather_limited.argtypes = lib.fst_gather.argtypes + [ctypes.c_uint32]
    lib.fst_gather_host.argtypes = [POINTER(Copy2D), c_uint64, c_int]
    lib.fst_realign.argtypes = [c_uint64, c_uint64, c_uint64, c_uint64]
    lib.fst_release_workspaces.restype = c_int
    lib.fst_gds_supported.argtypes = [c_int]
    lib.fst_convert.argtypes = [POINTER(ConvertOp), c_uint64, c_uint64]
    lib.fst_arena_create.argtypes = [c_uint64, POINTER(c_uint64)]
    lib.fst_arena_export.argtypes = [c_uint64, c_void_p, c_uint64]
    lib.fst_arena_open_peer.argtypes = [c_void_p, c_uint64, POINTER(c_uint64)]
    lib.fst_arena_close_peer.argtypes = [c_uint64]
    lib.fst_arena_destroy.argtypes = [c_uint64]
    if lib.fst_abi_version() != ABI_VERSION:
        raise ImportError(
            f"{LIB_PATH} has ABI version {lib.fst_abi_version()}, this package needs {ABI_VERSION}; rebuild it"
        )
    return lib


lib = _load()


def last_error() -> str:
    return lib.fst_last_error().decode("utf-8", "replace")


def check(status: int, what: str) -> None:
    """Raise :class:`NativeError` (a ``RuntimeError``) for a negative status."""
    if status < 0:
        text = last_error() or f"status {status}"
        if status == EGDS and "gds" not in text:
            text = "gds: " + text
        raise NativeError(status, f"{what}: {text}")


def cuda_device_count() -> int:
    return int(lib.fst_cuda_device_count())


def get_metrics() -> Metrics:
    m = Metrics()
    check(lib.fst_get_metrics(byref(m)), "fst_get_metrics")
    return m


class PackedOps:
    """An op table packed once for repeated launches: a contiguous ``(n, 6)`` uint64 array
    (one ``fst_copy2d_t`` per row, filled without a Python loop per field) and the pointer the
    C entry points take."""

    def __init__(self, ops: Sequence[Tuple[int, int, int, int, int, int]]):
        import numpy as np

        self.array = np.ascontiguousarray(np.array(ops, dtype=np.uint64).reshape(-1, 6))
        self.count = int(self.array.shape[0])
        self.pointer = self.array.ctypes.data_as(POINTER(Copy2D))


def pack_ops(ops: Sequence[Tuple[int, int, int, int, int, int]]) -> PackedOps:
    return PackedOps(ops)


def make_ops(ops: Sequence[Tuple[int, int, int, int, int, int]]):
    """Pack (src, dst, rows, row_bytes, src_pitch, dst_pitch) tuples; returns the pointer the C
    entry points take (it keeps its array alive)."""
    packed = PackedOps(ops)
    pointer = packed.pointer
    pointer._fst_keepalive = packed
    return pointer


def gather(ops: Sequence[Tuple[int, int, int, int, int, int]], stream: int,
           src_span: Tuple[int, int] = (0, 0), dst_span: Tuple[int, int] = (0, 0)) -> None:
    """Device gather: one launch for all ops on ``stream`` (``fst_gather``)."""
    if not ops:
        return
    arr = make_ops(ops)
    check(
        lib.fst_gather(arr, len(ops), src_span[0], src_span[1], dst_span[0], dst_span[1], stream),
        "fst_gather",
    )


def gather_limited(ops: Sequence[Tuple[int, int, int, int, int, int]], stream: int, max_ctas: int,
                   src_span: Tuple[int, int] = (0, 0), dst_span: Tuple[int, int] = (0, 0)) -> None:
    """``fst_gather_limited``: the device gather on a grid of at most ``max_ctas`` CTAs."""
    if not ops:
        return
    arr = make_ops(ops)
    check(
        lib.fst_gather_limited(arr, len(ops), src_span[0], src_span[1], dst_span[0], dst_span[1], stream,
                               max_ctas),
        "fst_gather_limited",
    )


def gather_static(ops: Sequence[Tuple[int, int, int, int, int, int]], stream: int,
                  src_span: Tuple[int, int] = (0, 0), dst_span: Tuple[int, int] = (0, 0)) -> None:
    """``fst_gather_static``: the device gather with its op table in a fixed array of the
    library (at most ``GATHER_STATIC_MAX_OPS`` ops); allocates nothing.  Calls on different
    streams must not overlap."""
    if not ops:
        return
    arr = make_ops(ops)
    check(
        lib.fst_gather_static(arr, len(ops), src_span[0], src_span[1], dst_span[0], dst_span[1], stream),
        "fst_gather_static",
    )


def gather_host(ops: Sequence[Tuple[int, int, int, int, int, int]], threads: int = 8) -> None:
    """Host-memory gather (``fst_gather_host``), used only when the loader's device is cpu."""
    if not ops:
        return
    arr = make_ops(ops)
    check(lib.fst_gather_host(arr, len(ops), threads), "fst_gather_host")


def convert(ops: Sequence[Tuple[int, int, int, int, int]], stream: int) -> None:
    """``fst_convert``: (src, dst, n_elements, src_code, dst_code) tuples, one launch."""
    if not ops:
        return
    arr = (ConvertOp * len(ops))()
    for i, o in enumerate(ops):
        a = arr[i]
        a.src, a.dst, a.n_elements, a.src_dtype, a.dst_dtype = o
    check(lib.fst_convert(arr, len(ops), stream), "fst_convert")


def realign(dst: int, src: int, nbytes: int, stream: int) -> None:
    check(lib.fst_realign(dst, src, nbytes, stream), "fst_realign")
