"""Shard geometry: tensor-parallel slices expressed as strided 2-D byte copies.

Upstream expresses a shard as a Python slice applied to a torch tensor followed by
``.contiguous()`` or ``torch.cat`` (``fastsafetensors/tensor_factory.py:145-175`` and
``:197-246``).  Here the same shard is a ``(src, dst, rows, row_bytes, src_pitch, dst_pitch)``
tuple for the gather kernel (``fst_copy2d_t`` in ``include/fst_b200.h``): a row-major tensor
of shape ``s`` cut on dimension ``d`` to ``[lo, hi)`` is ``prod(s[:d])`` rows of
``(hi-lo) * prod(s[d+1:]) * itemsize`` bytes, ``s[d] * prod(s[d+1:]) * itemsize`` bytes apart.
All arithmetic is integer and framework-free.
"""

from __future__ import annotations

from typing import List, Sequence, Tuple

Op = Tuple[int, int, int, int, int, int]  # src, dst, rows, row_bytes, src_pitch, dst_pitch


def block_size(extent: int, world_size: int) -> int:
    """Rows (or columns) per rank: ``ceil(extent / world_size)`` (tensor_factory.py:147)."""
    return (extent + world_size - 1) // world_size


def shard_bounds(extent: int, world_size: int, rank: int) -> Tuple[int, int]:
    """``[lo, hi)`` of ``rank`` on a dimension of length ``extent``, clamped as a Python slice
    ``[rank*B : (rank+1)*B]`` clamps (tensor_factory.py:153-155)."""
    b = block_size(extent, world_size)
    return min(rank * b, extent), min((rank + 1) * b, extent)


def check_even_split(name: str, extent: int, world_size: int) -> None:
    """Upstream hands unequal chunks to ``scatter``, which raises; refuse them up front."""
    if extent % world_size != 0:
        raise ValueError(
            f"cannot shard tensor {name}: dimension of length {extent} is not divisible by "
            f"world size {world_size} (scatter needs equal chunks)"
        )


def _prod(xs: Sequence[int]) -> int:
    p = 1
    for x in xs:
        p *= x
    return p


def _bytes(n_elements: int, bits: int, what: str) -> int:
    total = n_elements * bits
    if total % 8:
        raise ValueError(
            f"Malformed input: {what}: packed sub-byte slice bounds must align to storage units."
        )
    return total // 8


def slice_geometry(shape: Sequence[int], bits: int, dim: int, lo: int, hi: int) -> Tuple[int, int, int, int]:
    """``(rows, row_bytes, src_pitch, first_byte)`` of ``t[..., lo:hi, ...]`` on ``dim``."""
    if not 0 <= dim < len(shape):
        raise IndexError(f"dimension {dim} out of range for shape {list(shape)}")
    inner = _prod(shape[dim + 1:])
    rows = _prod(shape[:dim])
    row_bytes = _bytes((hi - lo) * inner, bits, f"slice [{lo}:{hi}] of shape {list(shape)} on dim {dim}")
    src_pitch = _bytes(shape[dim] * inner, bits, f"shape {list(shape)}")
    first = _bytes(lo * inner, bits, f"slice start {lo} of shape {list(shape)} on dim {dim}")
    return rows, row_bytes, src_pitch, first


def shard_op(src_addr: int, dst_addr: int, shape: Sequence[int], bits: int, dim: int,
             lo: int, hi: int, dst_pitch: int = 0) -> Op:
    """Copy ``t[..., lo:hi, ...]`` to ``dst_addr``; rows land ``dst_pitch`` bytes apart
    (default: packed, i.e. ``row_bytes``)."""
    rows, row_bytes, src_pitch, first = slice_geometry(shape, bits, dim, lo, hi)
    return (src_addr + first, dst_addr, rows, row_bytes, src_pitch, dst_pitch or row_bytes)


def scatter_ops(src_addr: int, dst_addr: int, shape: Sequence[int], bits: int, dim: int,
                world_size: int) -> Tuple[List[Op], int]:
    """Ops that pack the ``world_size`` shards of one tensor back to back at ``dst_addr``
    (rank r's shard at ``dst_addr + r * shard_bytes``).  Returns ``(ops, shard_bytes)``."""
    ops: List[Op] = []
    b = block_size(shape[dim], world_size)
    rows, row_bytes, _, _ = slice_geometry(shape, bits, dim, 0, b)
    shard_bytes = rows * row_bytes
    for r in range(world_size):
        lo, hi = shard_bounds(shape[dim], world_size, r)
        if hi > lo:
            ops.append(shard_op(src_addr, dst_addr + r * shard_bytes, shape, bits, dim, lo, hi))
    return ops, shard_bytes


def multi_col_ops(src_addrs: Sequence[int], dst_addr: int, shapes: Sequence[Sequence[int]],
                  bits: int, dim: int, world_size: int) -> Tuple[List[Op], int, List[int]]:
    """Ops that build, for every rank, the concatenation on ``dim`` of that rank's shard of each
    tensor (tensor_factory.py:197-246), the W results packed back to back at ``dst_addr``.
    Returns ``(ops, bytes_per_rank, result_shape)``."""
    first = list(shapes[0])
    per_rank_extent = 0
    row_bytes: List[int] = []
    for shape in shapes:
        if len(shape) != len(first):
            raise Exception(f"rank mismatch: {list(shape)} vs. {first} (dim={dim})")
        for d2, (a, b2) in enumerate(zip(shape, first)):
            if d2 != dim and a != b2:
                raise Exception(f"dim {d2} mismatch: {list(shape)} vs. {first} (dim={dim})")
        b = block_size(shape[dim], world_size)
        per_rank_extent += b
        row_bytes.append(slice_geometry(shape, bits, dim, 0, b)[1])
    rows = _prod(first[:dim])
    dst_pitch = sum(row_bytes)
    bytes_per_rank = rows * dst_pitch
    ops: List[Op] = []
    for r in range(world_size):
        col = 0
        for src, shape, rb in zip(src_addrs, shapes, row_bytes):
            lo, hi = shard_bounds(shape[dim], world_size, r)
            if hi > lo:
                ops.append(shard_op(src, dst_addr + r * bytes_per_rank + col, shape, bits, dim,
                                    lo, hi, dst_pitch=dst_pitch))
            col += rb
    result_shape = list(first)
    result_shape[dim] = per_rank_extent
    return ops, bytes_per_rank, result_shape
