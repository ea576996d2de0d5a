"""CPU restatement (numpy) of upstream fastsafetensors' load path.  TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA path: tests, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` leg of ``bench.py`` may import it; the product (``fastsafetensors_b200``) never
does.  It restates, with plain numpy slicing on host bytes, what upstream computes on the path
file -> buffer -> tensors -> tensor-parallel shards; every function names the upstream lines it
follows.  Upstream's algorithm for this path is first-party (Python in ``fastsafetensors/`` plus
``fastsafetensors/cpp/ext.cpp``); nothing comes from an absent third-party dependency.

Pinning.  ``tests/test_oracle_golden.py`` checks this module against
``tests/golden/reference_outputs.json``, which ``tests/golden/make_golden.py`` produced by
running upstream itself (built from its sources into ``oracle/_ref``) on the tiny synthetic
checkpoints: single rank, and 2/4/8 gloo ranks for shards, column groups, broadcasts and pushes.
"""

from __future__ import annotations

import hashlib
import json
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

MAX_HEADER = 100_000_000

# bits per element of each safetensors dtype (upstream: frameworks/_torch.py:277-283 via
# torch itemsize; F4 packs two values per byte)
BITS = {
    "BOOL": 8, "I8": 8, "U8": 8, "F8_E5M2": 8, "F8_E4M3": 8, "F8_E8M0": 8, "I16": 16, "U16": 16,
    "F16": 16, "BF16": 16, "I32": 32, "U32": 32, "F32": 32, "I64": 64, "U64": 64, "F64": 64,
    "F4": 4,
}


class HeaderError(Exception):
    pass


def parse_header(blob: bytes, file_size: Optional[int] = None) -> Tuple[int, Dict[str, dict], dict]:
    """``(header_length, tensors, metadata)`` of a safetensors file image or prefix.

    Follows ``SafeTensorsMetadata.from_fd`` and ``__init__`` (common.py:270-304, 184-243):
    8-byte little-endian length n, n <= 100 000 000, n <= size - 8, JSON body; entries sorted
    by ``data_offsets[0]`` must tile the data section from 0 without holes, each entry's byte
    length must equal numel * itemsize, the last end must not pass the end of the file
    (trailing bytes are allowed).  ``tensors`` keeps that sorted order.
    """
    size = len(blob) if file_size is None else file_size
    if size < 8:
        raise HeaderError("HeaderTooSmall")
    n = int.from_bytes(blob[:8], "little")
    if n > MAX_HEADER:
        raise HeaderError("HeaderTooLarge")
    if n > size - 8:
        raise HeaderError("InvalidHeaderLength")
    doc = json.loads(blob[8:8 + n].decode("utf-8"))
    metadata = doc.pop("__metadata__", {}) or {}
    tensors: Dict[str, dict] = {}
    start = 0
    for name, e in sorted(doc.items(), key=lambda kv: kv[1]["data_offsets"][0]):
        s, t = e["data_offsets"]
        if s != start or t < s:
            raise HeaderError(f"InvalidOffset {name}")
        numel = 1
        for d in e["shape"]:
            numel *= d
        if t - s != numel * BITS[e["dtype"]] // 8:
            raise HeaderError(f"TensorInvalidInfo {name}")
        tensors[name] = e
        start = t
    if start + 8 + n > size:
        raise HeaderError("MetadataIncompleteBuffer")
    return 8 + n, tensors, metadata


def _as_bytes_matrix(raw: np.ndarray, shape: Sequence[int], bits: int) -> np.ndarray:
    """Tensor bytes as an array of shape ``shape[:-1] + [last_dim_bytes]`` (uint8), so that
    numpy slicing on any dimension moves whole elements; sub-byte dtypes share bytes on the last
    dimension only (upstream: ``get_native_shape``, _torch.py:331-350)."""
    if len(shape) == 0:
        return raw.reshape(-1)
    last_bytes = shape[-1] * bits // 8
    if shape[-1] * bits % 8:
        raise ValueError("last dimension must be divisible by the packing ratio")
    return raw.reshape(list(shape[:-1]) + [last_bytes])


def tensor_raw(file_blob: bytes, header_length: int, entry: dict) -> np.ndarray:
    """Bytes of one tensor: file[header + off0 : header + off1] (common.py:328-333 with the
    no-GDS copier's ``copy_start_offset == header_length``, copier/nogds.py:76-78)."""
    s, t = entry["data_offsets"]
    return np.frombuffer(file_blob, dtype=np.uint8, count=t - s, offset=header_length + s)


def block_bounds(extent: int, world: int, rank: int) -> Tuple[int, int]:
    """``slice(rank*B, (rank+1)*B)`` with ``B = ceil(extent/world)``, clamped as Python slicing
    clamps (tensor_factory.py:146-155)."""
    b = (extent + world - 1) // world
    return min(rank * b, extent), min((rank + 1) * b, extent)


def shard(raw: np.ndarray, shape: Sequence[int], dtype: str, dim: int, rank: int,
          world: int) -> Tuple[np.ndarray, List[int]]:
    """Bytes and shape of ``t[rank_slices[rank]].contiguous()`` (tensor_factory.py:145-175).
    ``dim == -1`` returns the whole tensor (the broadcast branch, :128-143)."""
    if dim == -1 or world == 1:
        return raw.copy(), list(shape)
    bits = BITS[dtype]
    lo, hi = block_bounds(shape[dim], world, rank)
    m = _as_bytes_matrix(raw, shape, bits)
    if dim == len(shape) - 1:
        if (lo * bits) % 8 or (hi * bits) % 8:
            raise ValueError("packed sub-byte slice bounds must align to storage units")
        lo_b, hi_b = lo * bits // 8, hi * bits // 8
    else:
        lo_b, hi_b = lo, hi
    index = [slice(None)] * dim + [slice(lo_b, hi_b)]
    out = np.ascontiguousarray(m[tuple(index)])
    new_shape = list(shape)
    new_shape[dim] = hi - lo
    return out.reshape(-1), new_shape


def multi_cols(raws: Sequence[np.ndarray], shapes: Sequence[Sequence[int]], dtype: str, dim: int,
               rank: int, world: int) -> Tuple[np.ndarray, List[int]]:
    """Per-rank concatenation on ``dim`` of each tensor's shard (tensor_factory.py:197-246,
    ``torch.cat`` of the slices)."""
    bits = BITS[dtype]
    parts = []
    extent = 0
    for raw, shape in zip(raws, shapes):
        piece, new_shape = shard(raw, shape, dtype, dim, rank, world) if world > 1 else (raw, list(shape))
        parts.append(_as_bytes_matrix(piece, new_shape, bits))
        extent += new_shape[dim]
    out = np.concatenate(parts, axis=dim)
    res_shape = list(shapes[0])
    res_shape[dim] = extent
    return np.ascontiguousarray(out).reshape(-1), res_shape


def realign_image(image: np.ndarray, header_length: int, align: int = 16) -> Tuple[np.ndarray, int]:
    """What the GDS copier's fix-up does to a 4 KiB-window image when ``header_length % 16``
    is not 0: shift everything down by that many bytes, piecewise through a temporary
    (copier/gds.py:138-159, ext.cpp:606-645).  Returns the shifted image and the shift."""
    mis = header_length % align
    if mis == 0:
        return image.copy(), 0
    out = image.copy()
    piece = 1 << 20
    count = 0
    n = image.size
    while count + mis < n:
        l = min(piece, n - mis - count)
        tmp = out[mis + count: mis + count + l].copy()
        out[count: count + l] = tmp
        count += l
    return out, mis


def frame_getitem(shape: Sequence[int], index) -> Tuple[List[int], List[int], List[int]]:
    """``(shape, strides, offsets)`` of ``TensorFrame.__getitem__`` (common.py:418-471)."""
    strides = []
    for i in range(len(shape)):
        s = 1
        for j in range(i + 1, len(shape)):
            s *= shape[j]
        strides.append(s)
    val = (index,) if isinstance(index, (slice, int)) else tuple(index)
    o_shape: List[int] = []
    o_strides: List[int] = []
    o_offsets: List[int] = []
    for dim, v in enumerate(val):
        if isinstance(v, int):
            start = v
            if start >= shape[dim] or start < -shape[dim]:
                raise IndexError
            if start < 0:
                start += shape[dim]
            step, length = 1, 1
        else:
            if v.step == 0:
                raise ValueError
            start, stop, step = v.indices(shape[dim])
            length = stop - start
            if length == 0 or (length < 0 and step > 0) or (length > 0 and step < 0):
                return [], [], []
            length = abs(length)
        o_offsets.append(start)
        o_strides.append(strides[dim] * step)
        o_shape.append((length + abs(step) - 1) // abs(step))
    for r in range(len(val), len(shape)):
        o_offsets.append(0)
        o_strides.append(strides[r])
        o_shape.append(shape[r])
    return o_shape, o_strides, o_offsets


def digest(raw: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(raw).tobytes()).hexdigest()


class FileOracle:
    """All tensors of one file, as upstream's loader would hand them out."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            self.blob = f.read()
        self.header_length, self.tensors, self.metadata = parse_header(self.blob)

    def raw(self, name: str) -> np.ndarray:
        return tensor_raw(self.blob, self.header_length, self.tensors[name])

    def get_tensor(self, name: str) -> Tuple[np.ndarray, List[int]]:
        e = self.tensors[name]
        return self.raw(name).copy(), list(e["shape"])

    def get_sharded(self, name: str, dim: int, rank: int, world: int) -> Tuple[np.ndarray, List[int]]:
        e = self.tensors[name]
        return shard(self.raw(name), e["shape"], e["dtype"], dim, rank, world)

    def get_multi_cols(self, names: Sequence[str], dim: int, rank: int, world: int):
        es = [self.tensors[n] for n in names]
        return multi_cols([self.raw(n) for n in names], [e["shape"] for e in es], es[0]["dtype"],
                          dim, rank, world)
