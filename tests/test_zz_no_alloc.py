"""fst_gather_static: the gather entry point for callers that must not allocate.

Some processes cannot call the CUDA allocator when the loader runs: an inference server that has
already given all free HBM to its KV-cache pool (a cudaMalloc would fail), or one that bans
cudaMalloc/cudaFree after start-up because both stall every stream of the device.  For them the
library offers the same gather with its op table in a fixed device array that ships inside the
library image.  This test drives it through the C ABI, twice in a row (the array is shared and
keeps the previous call's table), and requires its output to be byte-identical both to a plain
numpy restatement of the copies (canary bytes around them included) and to the ordinary entry
point's.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""

import numpy as np
import pytest
import torch

from fastsafetensors_b200 import _native as nat

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _random_ops(rng, n_ops, max_row_bytes):
    ops, s_cur, d_cur = [], 0, 0
    for _ in range(n_ops):
        rows = int(rng.integers(1, 5))
        rb = int(rng.integers(1, max_row_bytes + 1))
        sp, dp = rb + int(rng.integers(0, 40)), rb + int(rng.integers(0, 40))
        s_cur += int(rng.integers(0, 17))
        d_cur += int(rng.integers(0, 17))
        ops.append((s_cur, d_cur, rows, rb, sp, dp))
        s_cur += rows * sp
        d_cur += rows * dp
    return ops, s_cur + 64, d_cur + 64


def _expected(ops_rel, src_np, dst_size):
    """What the copies must leave behind, computed on the host: row r of an op goes from
    src[s + r * sp ..+rb) to dst[d + r * dp ..+rb); every other byte keeps the 0xA5 fill."""
    want = np.full(dst_size, 0xA5, dtype=np.uint8)
    for (s, d, rows, rb, sp, dp) in ops_rel:
        for r in range(rows):
            want[d + r * dp: d + r * dp + rb] = src_np[s + r * sp: s + r * sp + rb]
    return want


def _run(entry, ops_rel, src, dst_size):
    dst = torch.full((dst_size,), 0xA5, dtype=torch.uint8, device=DEV)
    ops = [(src.data_ptr() + o[0], dst.data_ptr() + o[1]) + tuple(o[2:]) for o in ops_rel]
    entry(ops, int(torch.cuda.current_stream().cuda_stream),
          (src.data_ptr(), src.numel()), (dst.data_ptr(), dst.numel()))
    torch.cuda.synchronize()
    return dst.cpu().numpy()


def test_static_table_gather_matches_the_allocating_entry_point_twice():
    rng = np.random.default_rng(2024)
    # first call: a large table; second call: a smaller, different one, so entries left over
    # from the first call sit behind the ones in use
    for n_ops, max_row in ((3000, 1500), (70, 9000)):
        ops_rel, s_size, d_size = _random_ops(rng, n_ops, max_row)
        src_np = rng.integers(0, 256, s_size, dtype=np.uint8)
        src = torch.from_numpy(src_np).to(DEV)
        want = _expected(ops_rel, src_np, d_size)
        got = _run(nat.gather_static, ops_rel, src, d_size)
        assert np.array_equal(got, want), n_ops            # bit-exact, canaries included
        assert np.array_equal(_run(nat.gather, ops_rel, src, d_size), want), n_ops
        assert (want != 0xA5).any()


def test_static_table_gather_refuses_oversized_and_bad_requests():
    src = torch.zeros(1 << 16, dtype=torch.uint8, device=DEV)
    dst = torch.zeros(1 << 16, dtype=torch.uint8, device=DEV)
    s, d = src.data_ptr(), dst.data_ptr()
    too_many = [(s + i, d + i, 1, 1, 0, 0) for i in range(nat.GATHER_STATIC_MAX_OPS + 1)]
    with pytest.raises(nat.NativeError) as e:
        nat.gather_static(too_many, 0)
    assert e.value.code == nat.ELIMIT and "split" in str(e.value)
    with pytest.raises(nat.NativeError) as e:
        nat.gather_static([(s, d + (1 << 16) - 8, 1, 64, 0, 0)], 0, (s, 1 << 16), (d, 1 << 16))
    assert e.value.code == nat.ERANGE
    nat.gather_static(too_many[:-1], int(torch.cuda.current_stream().cuda_stream))   # exactly the maximum is fine
    torch.cuda.synchronize()
