"""Parity of the CUDA path with the oracle and with upstream's recorded outputs.  Needs a GPU.

Everything goes through the C ABI (fst_gather, fst_realign, fst_reader_*) or through the loader
API built on it.  Integer/byte work: every comparison is bit-exact."""

import os

import numpy as np
import pytest
import torch

import fastsafetensors_b200 as fst
from fastsafetensors_b200 import _native as nat
from fastsafetensors_b200 import cpp, shard_plan
from oracle import st_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CANARY = 0xA5


def stream():
    return int(torch.cuda.current_stream().cuda_stream)


def dev_bytes(arr: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(arr).to(DEV)


def run_ops_on_device(src_np, src_off, dst_size, dst_off, ops_rel):
    """ops_rel: (src_rel, dst_rel, rows, row_bytes, sp, dp) relative to src_off/dst_off."""
    src = dev_bytes(src_np)
    dst = torch.full((dst_size,), CANARY, dtype=torch.uint8, device=DEV)
    ops = [(src.data_ptr() + src_off + o[0], dst.data_ptr() + dst_off + o[1]) + tuple(o[2:]) for o in ops_rel]
    nat.gather(ops, stream(), (src.data_ptr(), src.numel()), (dst.data_ptr(), dst.numel()))
    torch.cuda.synchronize()
    return dst.cpu().numpy()


def expected_ops(src_np, src_off, dst_size, dst_off, ops_rel):
    want = np.full(dst_size, CANARY, dtype=np.uint8)
    for (s, d, rows, rb, sp, dp) in ops_rel:
        for r in range(rows):
            want[dst_off + d + r * dp: dst_off + d + r * dp + rb] = \
                src_np[src_off + s + r * sp: src_off + s + r * sp + rb]
    return want


# ------------------------------------------------------------------ gather kernel
@pytest.mark.parametrize("row_bytes", [1, 3, 15, 16, 17, 31, 64, 65, 100, 257, 512, 640, 1024, 1025, 2047, 2048, 2049,
                                       4100, 70001])
@pytest.mark.parametrize("rows", [1, 3, 33])
def test_gather_every_alignment(row_bytes, rows):
    rng = np.random.default_rng(row_bytes * 100 + rows)
    for src_mis, dst_mis, pad_s, pad_d in [(0, 0, 0, 0), (1, 0, 0, 0), (0, 1, 0, 0), (5, 5, 16, 16),
                                           (7, 2, 1, 3), (15, 9, 13, 0), (3, 12, 32, 5), (8, 0, 8, 24)]:
        sp, dp = row_bytes + pad_s, row_bytes + pad_d
        src_np = rng.integers(0, 256, 64 + rows * sp + 64, dtype=np.uint8)
        dst_size = 64 + rows * dp + 64
        ops = [(0, 0, rows, row_bytes, sp, dp)]
        got = run_ops_on_device(src_np, 32 + src_mis, dst_size, 32 + dst_mis, ops)
        want = expected_ops(src_np, 32 + src_mis, dst_size, 32 + dst_mis, ops)
        assert np.array_equal(got, want), (src_mis, dst_mis, pad_s, pad_d)


@pytest.mark.parametrize("rows", [31, 32, 33, 1000])
@pytest.mark.parametrize("row_bytes", [8, 48, 200, 256, 1000])
def test_gather_short_rows_share_a_warp(rows, row_bytes):
    """Rows of at most 1 KiB are copied several to a warp (groups of 1..16 lanes per row); the
    last sub of an op is ragged when the row count is not a multiple of the rows per sub.  Two
    such ops and a long-row op in one launch."""
    rng = np.random.default_rng(rows * 7 + row_bytes)
    sp, dp = row_bytes * 8 + 3, row_bytes + 5
    long_rb = 5000
    src_np = rng.integers(0, 256, 2 * rows * sp + 3 * long_rb + 256, dtype=np.uint8)
    a_dst, b_dst = 0, rows * dp + 11
    c_src, c_dst = 2 * rows * sp + 7, 2 * rows * dp + 40
    ops = [(1, a_dst, rows, row_bytes, sp, dp),
           (rows * sp + 2, b_dst, rows, row_bytes, sp, row_bytes + 16),
           (c_src, c_dst + rows * 16, 3, long_rb, long_rb, long_rb + 1)]
    dst_size = c_dst + rows * 16 + 3 * (long_rb + 1) + 64
    got = run_ops_on_device(src_np, 0, dst_size, 0, ops)
    assert np.array_equal(got, expected_ops(src_np, 0, dst_size, 0, ops))


def _random_ops(rng, n_ops, max_rows, max_row_bytes):
    ops, s_cur, d_cur = [], 0, 0
    for _ in range(n_ops):
        rows = int(rng.integers(1, max_rows + 1))
        rb = int(rng.integers(1, max_row_bytes + 1))
        sp = rb + int(rng.integers(0, 40))
        dp = rb + int(rng.integers(0, 40))
        s_cur += int(rng.integers(0, 17))
        d_cur += int(rng.integers(0, 17))
        ops.append((s_cur, d_cur, rows, rb, sp, dp))
        s_cur += rows * sp
        d_cur += rows * dp
    return ops, s_cur + 64, d_cur + 64


@pytest.mark.parametrize("n_ops", [2, 48, 49, 500, 20000])
def test_gather_many_ops_inline_and_table_paths(n_ops):
    """<= 48 ops travel in kernel parameters, more go through the device op table; 20000 ops
    need two table chunks."""
    rng = np.random.default_rng(n_ops)
    ops, s_size, d_size = _random_ops(rng, n_ops, 4, 3000 if n_ops <= 500 else 200)
    src_np = rng.integers(0, 256, s_size, dtype=np.uint8)
    got = run_ops_on_device(src_np, 0, d_size, 0, ops)
    assert np.array_equal(got, expected_ops(src_np, 0, d_size, 0, ops))


@pytest.mark.parametrize("max_ctas", [1, 7, 148])
def test_gather_on_a_bounded_grid(max_ctas):
    """fst_gather_limited: a few CTAs stride over all the work (inline and table paths)."""
    for n_ops in (5, 300):
        rng = np.random.default_rng(max_ctas * 1000 + n_ops)
        ops, s_size, d_size = _random_ops(rng, n_ops, 6, 5000)
        src_np = rng.integers(0, 256, s_size, dtype=np.uint8)
        src = dev_bytes(src_np)
        dst = torch.full((d_size,), CANARY, dtype=torch.uint8, device=DEV)
        abs_ops = [(src.data_ptr() + o[0], dst.data_ptr() + o[1]) + tuple(o[2:]) for o in ops]
        nat.gather_limited(abs_ops, stream(), max_ctas, (src.data_ptr(), src.numel()), (dst.data_ptr(), dst.numel()))
        torch.cuda.synchronize()
        assert np.array_equal(dst.cpu().numpy(), expected_ops(src_np, 0, d_size, 0, ops)), n_ops


def test_gather_refuses_out_of_range_ops():
    src = torch.zeros(4096, dtype=torch.uint8, device=DEV)
    dst = torch.zeros(4096, dtype=torch.uint8, device=DEV)
    s, d = src.data_ptr(), dst.data_ptr()
    with pytest.raises(nat.NativeError) as e:
        nat.gather([(s + 4000, d, 1, 200, 0, 0)], stream(), (s, 4096), (d, 4096))
    assert e.value.code == nat.ERANGE
    with pytest.raises(nat.NativeError) as e:
        nat.gather([(s, d + 100, 4, 1000, 1000, 1000)], stream(), (s, 4096), (d, 4096))
    assert e.value.code == nat.ERANGE
    with pytest.raises(nat.NativeError) as e:
        nat.gather([(s, d, 4, 100, 50, 100)], stream())
    assert e.value.code == nat.EINVAL
    torch.cuda.synchronize()
    assert int(dst.sum()) == 0


# ------------------------------------------------------------------ realign kernel
@pytest.mark.parametrize("nbytes", [1, 15, 16, 17, 255, 4096 + 3, (1 << 20) + 7, (8 << 20) + 1])
def test_realign_every_shift(nbytes):
    rng = np.random.default_rng(nbytes)
    data = rng.integers(0, 256, nbytes + 96, dtype=np.uint8)
    src = dev_bytes(data)
    for s_mis in range(16):
        for d_mis in (0, 1, 7, 15):
            dst = torch.full((nbytes + 96,), CANARY, dtype=torch.uint8, device=DEV)
            nat.realign(dst.data_ptr() + 32 + d_mis, src.data_ptr() + 16 + s_mis, nbytes, stream())
            got = dst.cpu().numpy()
            want = np.full(nbytes + 96, CANARY, dtype=np.uint8)
            want[32 + d_mis: 32 + d_mis + nbytes] = data[16 + s_mis: 16 + s_mis + nbytes]
            assert np.array_equal(got, want), (s_mis, d_mis)


def test_realign_matches_upstream_memmove_semantics():
    """Upstream shifts a 4 KiB-window image down by header_length % 16 through a temporary
    (copier/gds.py:138-159); the oracle restates it; the kernel does it out of place."""
    rng = np.random.default_rng(3)
    image = rng.integers(0, 256, (3 << 20) + 4096, dtype=np.uint8)
    for header_length in (9, 4096 + 13, 1234567):
        want, mis = st_oracle.realign_image(image, header_length)
        src = dev_bytes(image)
        dst = torch.zeros_like(src)
        nat.realign(dst.data_ptr(), src.data_ptr() + mis, image.size - mis, stream())
        got = dst.cpu().numpy()
        assert np.array_equal(got[: image.size - mis], want[: image.size - mis])


def test_realign_refuses_overlap():
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device=DEV)
    with pytest.raises(nat.NativeError) as e:
        nat.realign(buf.data_ptr(), buf.data_ptr() + 3, 1000, stream())
    assert e.value.code == nat.EINVAL


def test_legacy_memmove_shifts_in_place():
    """gds_device_buffer.memmove through a temporary, as upstream's test does (:289-303)."""
    data = np.arange(100000, dtype=np.uint32).view(np.uint8)
    img = dev_bytes(data.copy())
    tmp = torch.empty(1 << 20, dtype=torch.uint8, device=DEV)
    g = cpp.gds_device_buffer(img.data_ptr(), img.numel(), True)
    t = cpp.gds_device_buffer(tmp.data_ptr(), tmp.numel(), True)
    assert g.memmove(0, 13, t, data.size - 13) == 0
    assert np.array_equal(img.cpu().numpy()[: data.size - 13], data[13:])


# ------------------------------------------------------------------ shard geometry on device
@pytest.mark.parametrize("shape,dtype,dim,world", [
    ((64, 48), "BF16", 0, 8), ((64, 48), "BF16", 1, 8), ((4, 6, 8), "F32", 1, 3), ((16, 24, 10), "F16", 2, 2),
    ((8,), "I64", 0, 8), ((6, 10), "U8", 1, 5), ((6, 20), "F4", 1, 5), ((5, 7, 3, 4), "F64", 2, 3),
    ((1024, 1536), "BF16", 1, 8), ((3, 1000), "F16", 1, 4),
])
def test_scatter_pack_matches_oracle(shape, dtype, dim, world):
    bits = st_oracle.BITS[dtype]
    n = int(np.prod(shape)) * bits // 8
    raw = np.random.default_rng(n + dim).integers(0, 256, n, dtype=np.uint8)
    src = dev_bytes(raw)
    ops, shard_bytes = shard_plan.scatter_ops(src.data_ptr(), 0, shape, bits, dim, world)
    packed = torch.zeros(shard_bytes * world, dtype=torch.uint8, device=DEV)
    nat.gather([(o[0], o[1] + packed.data_ptr()) + o[2:] for o in ops], stream(),
               (src.data_ptr(), n), (packed.data_ptr(), packed.numel()))
    got = packed.cpu().numpy()
    for r in range(world):
        want, _ = st_oracle.shard(raw, shape, dtype, dim, r, world)
        assert np.array_equal(got[r * shard_bytes:(r + 1) * shard_bytes], want), r


def test_multi_col_pack_matches_oracle():
    shapes = [(96, 64), (96, 16), (96, 16)]
    raws = [np.random.default_rng(i).integers(0, 256, int(np.prod(s)) * 2, dtype=np.uint8) for i, s in enumerate(shapes)]
    srcs = [dev_bytes(r) for r in raws]
    for dim, shp in ((1, shapes), (0, [(s[1], s[0]) for s in shapes])):
        for world in (1, 2, 8):
            ops, per_rank, shape = shard_plan.multi_col_ops([s.data_ptr() for s in srcs], 0, shp, 16, dim, world)
            packed = torch.zeros(per_rank * world, dtype=torch.uint8, device=DEV)
            nat.gather([(o[0], o[1] + packed.data_ptr()) + o[2:] for o in ops], stream())
            got = packed.cpu().numpy()
            for r in range(world):
                want, want_shape = st_oracle.multi_cols(raws, shp, "BF16", dim, r, world)
                assert shape == want_shape
                assert np.array_equal(got[r * per_rank:(r + 1) * per_rank], want)
