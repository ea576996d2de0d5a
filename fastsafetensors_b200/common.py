"""safetensors header parsing, tensor frames, and instantiation of tensors over a file image.

API-compatible with upstream ``fastsafetensors/common.py`` (``SafeTensorsMetadata``,
``TensorFrame``, ``SingleGroup``, ``get_device_numa_node``).  Tensor instantiation differs: a
file image is a ``torch.uint8`` tensor and every tensor is a typed view of it, and a tensor
whose byte offset is not a multiple of its element size (upstream passes such a pointer on
unchanged, ``common.py:328-345``) is first moved to an aligned side arena by the realign path.
"""

from __future__ import annotations

import json
import logging
import os
import sys
from collections import OrderedDict
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from . import _native as nat
from . import cpp as fstcpp
from .st_types import Device, DeviceType, DType

MAX_HEADER_BYTES = 100_000_000


def init_logger(name: str) -> logging.Logger:
    return logging.getLogger(name)


def set_debug() -> None:
    logging.basicConfig(format="[%(levelname)s] %(message)s", level=logging.DEBUG, force=True)


def is_debug(logger: logging.Logger) -> bool:
    return logger.isEnabledFor(logging.DEBUG)


def is_gpu_found() -> bool:
    return fstcpp.is_cuda_found()


def get_device_numa_node(device: Optional[int]) -> Optional[int]:
    """NUMA node of a CUDA device, or None when it cannot be told (common.py:40-51)."""
    if device is None or not sys.platform.startswith("linux"):
        return None
    node = int(nat.lib.fst_device_numa_node(device))
    return node if node >= 0 else None


class SingleGroup:
    """Stand-in process group of one rank (kept for callers of upstream's API)."""

    def size(self) -> int:
        return 1

    def rank(self) -> int:
        return 0


@dataclass
class TensorFrame:
    """dtype, shape and element strides/offsets of a (possibly sliced) tensor in a file."""

    dtype: DType
    shape: List[int]
    data_offsets: List[int]
    strides: List[int]
    offsets: List[int]
    sliced: bool

    @classmethod
    def from_buffer(cls, entry: Dict[str, Any]) -> "TensorFrame":
        shape = entry["shape"]
        strides = [0] * len(shape)
        acc = 1
        for i in range(len(shape) - 1, -1, -1):
            strides[i] = acc
            acc *= shape[i]
        return cls(DType(entry["dtype"]), shape, list(entry["data_offsets"]), strides,
                   [0] * len(shape), False)

    def __repr__(self) -> str:
        return str({"dtype": self.dtype, "shape": self.shape, "data_offsets": self.data_offsets})

    def _empty(self) -> "TensorFrame":
        return TensorFrame(self.dtype, [], self.data_offsets, [], [], False)

    def __getitem__(self, _val) -> "TensorFrame":
        """Frame of ``t[_val]`` with the semantics of Python sequence indexing per dimension
        (common.py:418-471): ints keep their dimension with extent 1, an empty slice on any
        dimension yields the empty frame."""
        if isinstance(_val, (slice, int)):
            index: Tuple = (_val,)
        elif isinstance(_val, tuple):
            index = _val
        else:
            raise Exception(f"[BUG] Unsupported index type for DiskTensor: {_val}")
        if len(index) > len(self.shape):
            raise Exception(f"[BUG] tried to get too large slice {_val} from {self.shape}")
        shape: List[int] = []
        strides: List[int] = []
        offsets: List[int] = []
        for dim, item in enumerate(index):
            extent = self.shape[dim]
            if isinstance(item, int):
                if not -extent <= item < extent:
                    raise IndexError(
                        f"[BUG] tried to access index {item} at dim={dim} for shape={self.shape}"
                    )
                picked = range(item % extent, item % extent + 1)
            elif isinstance(item, slice):
                if item.step == 0:
                    raise ValueError("[BUG] slice step cannot be zero")
                picked = range(*item.indices(extent))
            else:
                raise Exception(f"[BUG] Unsupported index type for DiskTensor: {_val} at dim={dim}")
            if len(picked) == 0:
                return self._empty()
            offsets.append(self.offsets[dim] + picked.start)
            strides.append(self.strides[dim] * picked.step)
            shape.append(len(picked))
        rest = len(index)
        return TensorFrame(self.dtype, shape + self.shape[rest:], self.data_offsets,
                           strides + self.strides[rest:], offsets + self.offsets[rest:], True)


def _read_exact(fd: int, length: int, filename: str) -> bytes:
    parts = []
    left = length
    while left > 0:
        chunk = os.read(fd, left)
        if not chunk:
            raise Exception(
                f"{filename}: UnexpectedEOF, expected {length} more bytes but got {length - left}"
            )
        parts.append(chunk)
        left -= len(chunk)
    return b"".join(parts)


def _header_length_checked(n: int, buffer_len: int, where: str) -> None:
    if n > MAX_HEADER_BYTES:
        raise Exception(f"{where}: HeaderTooLarge, n={n}, buffer_len={buffer_len}")
    if n > buffer_len - 8:
        raise Exception(f"{where}: InvalidHeaderLength, n={n}, buffer_len={buffer_len}")


def _wrap_raw(addr: int, nbytes: int, on_gpu: bool, device: Device):
    """Zero-copy ``torch.uint8`` view of raw memory that no torch tensor owns."""
    import ctypes

    import torch

    if nbytes == 0:
        return torch.empty(0, dtype=torch.uint8, device=device.as_str() if on_gpu else "cpu")
    if not on_gpu:
        return torch.frombuffer((ctypes.c_ubyte * nbytes).from_address(addr), dtype=torch.uint8)

    class _Span:
        __cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (addr, False), "version": 2,
        }

    return torch.as_tensor(_Span(), device=device.as_str())


class SafeTensorsMetadata:
    """Parsed and validated header of one ``.safetensors`` file (common.py:183-243)."""

    def __init__(self, string: str, header_length: int, size_bytes: int, framework,
                 src: str = "", keep_orig_dict: bool = False):
        self.src = src
        self.framework = framework
        ser = json.loads(string, object_pairs_hook=OrderedDict)
        self.metadata = ser.pop("__metadata__", "") or ""
        self.header_length = header_length
        self.size_bytes = size_bytes
        self.aligned = header_length % framework.get_device_ptr_align() == 0
        if keep_orig_dict:
            self.ser = ser
        self.tensors: Dict[str, TensorFrame] = {}
        cursor = 0
        for name, entry in sorted(ser.items(), key=lambda kv: kv[1]["data_offsets"][0]):
            frame = TensorFrame.from_buffer(entry)
            begin, end = frame.data_offsets
            if begin != cursor or end < begin:
                raise Exception(
                    f"validate(tensor {name}): InvalidOffset s={begin}, start={cursor}, e={end}, src={src}"
                )
            count = 1
            for extent in frame.shape:
                count *= extent
            nbytes = count * frame.dtype.bits // 8
            if end - begin != nbytes:
                raise Exception(
                    f"validate(tensor {name}): TensorInvalidInfo, e-s={end - begin}, nbytes={nbytes}, src={src}"
                )
            self.tensors[name] = frame
            cursor = end
        self.data_bytes = cursor
        if cursor + header_length > size_bytes:
            raise Exception(
                f"MetadataIncompleteBuffer, src={src}, start={cursor}, header_length={header_length}, size_bytes={size_bytes}"
            )
        # bytes after the last tensor (alignment padding) are allowed

    @classmethod
    def from_buffer(cls, buf: int, buffer_len: int, filename: str, framework):
        """Parse a whole file image that sits in host memory at address ``buf``."""
        if buffer_len < 8:
            raise Exception(f"from_buffer: HeaderTooSmall, filename={filename}, buffer_len={buffer_len}")
        n = int.from_bytes(fstcpp.read_buffer(buf, 8), byteorder="little", signed=False)
        _header_length_checked(n, buffer_len, f"from_buffer: filename={filename}")
        return cls(fstcpp.read_buffer(buf + 8, n).decode("utf-8"), n + 8, buffer_len, framework)

    @classmethod
    def from_fd(cls, fd: int, filename: str, framework, keep_orig_dict: bool = False):
        buffer_len = os.fstat(fd).st_size
        if buffer_len < 8:
            raise Exception(f"{filename}: HeaderTooSmall, buffer_len={buffer_len}")
        n = int.from_bytes(_read_exact(fd, 8, filename), byteorder="little", signed=False)
        _header_length_checked(n, buffer_len, filename)
        text = _read_exact(fd, n, filename).decode("utf-8")
        return cls(text, n + 8, buffer_len, framework, filename, keep_orig_dict=keep_orig_dict)

    @classmethod
    def from_file(cls, filename: str, framework):
        fd = os.open(filename, os.O_RDONLY, 0o644)
        try:
            return cls.from_fd(fd, filename, framework=framework)
        finally:
            os.close(fd)

    def __repr__(self) -> str:
        return str({"__metadata__": self.metadata, "tensors": self.tensors})

    # -------------------------------------------------------------------------------------
    def get_tensors(self, gbuf, device: Device, copy_start_offset: int,
                    dtype: DType = DType.AUTO) -> Dict[str, Any]:
        """Typed views of every tensor over the file image ``gbuf``.

        The byte of the file at offset ``o`` sits at ``gbuf[o - copy_start_offset]``
        (common.py:319-353).  Tensors whose address is not a multiple of their element size
        are gathered into one aligned side arena first (one kernel launch for all of them on a
        device image), so every view is legal and results stay byte-identical to the file.
        ``dtype`` other than AUTO narrows every tensor in place, as upstream does
        (common.py:355-375).
        """
        import torch

        from .frameworks._torch import TorchTensor, dtype_convert

        on_gpu = device.type != DeviceType.CPU
        image = getattr(gbuf, "owner", None)
        base = gbuf.get_base_address()
        if image is None:
            image = _wrap_raw(base, gbuf.get_length(), on_gpu, device)
        elif image.data_ptr() != base:
            image = image[base - image.data_ptr():]

        spans: Dict[str, Tuple[int, int, int]] = {}  # name -> (offset in image, nbytes, itemsize)
        misaligned: List[str] = []
        for name, frame in self.tensors.items():
            off = self.header_length + frame.data_offsets[0] - copy_start_offset
            nbytes = frame.data_offsets[1] - frame.data_offsets[0]
            itemsize = max(1, frame.dtype.bits // 8)
            gbuf.check_range(off, nbytes)
            spans[name] = (off, nbytes, itemsize)
            if nbytes and (base + off) % itemsize:
                misaligned.append(name)

        arena = None
        arena_off: Dict[str, int] = {}
        if misaligned:
            total = 0
            for name in misaligned:
                arena_off[name] = total
                total += (spans[name][1] + 15) // 16 * 16
            arena = torch.empty(total, dtype=torch.uint8, device=image.device)
            ops = [
                (base + spans[n][0], arena.data_ptr() + arena_off[n], 1, spans[n][1], 0, 0)
                for n in misaligned
            ]
            if on_gpu:
                stream = int(torch.cuda.current_stream(image.device).cuda_stream)
                nat.gather(ops, stream, (base, gbuf.get_length()), (arena.data_ptr(), total))
            else:
                nat.gather_host(ops, threads=4)

        out: Dict[str, Any] = {}
        for name, frame in self.tensors.items():
            off, nbytes, _ = spans[name]
            raw = arena[arena_off[name]: arena_off[name] + nbytes] if name in arena_off \
                else image[off: off + nbytes]
            native_shape = self.framework.get_native_shape(frame.dtype, frame.shape)
            t = raw.view(dtype_convert[frame.dtype]).reshape(native_shape)
            if dtype != DType.AUTO and dtype != frame.dtype:
                if dtype.bits > frame.dtype.bits:
                    raise Exception(
                        f"Online type conversion to larger sizes is not supported ({frame.dtype} -> {dtype})"
                    )
                converted = t.to(dtype=dtype_convert[dtype])
                count = converted.numel()
                t = raw[: count * dtype.bits // 8].view(dtype_convert[dtype]).reshape(frame.shape)
                t.copy_(converted)
                frame.dtype = dtype
            out[name] = TorchTensor(device, frame.dtype, t)
        return out


def resolve_cudart_lib_name() -> str:
    """Upstream resolves which CUDA runtime to ``dlopen``; here the runtime is linked into the
    native library, so there is nothing to resolve."""
    return ""
