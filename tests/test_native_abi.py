"""The C-ABI library without a GPU: it loads, exports what include/fst_b200.h declares, and
its host-side entry points behave (reader into host memory, host gather, fault injection)."""

import ctypes
import errno
import os
import re

import numpy as np
import pytest

from fastsafetensors_b200 import _native as nat
from fastsafetensors_b200 import cpp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "fst_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fst_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(nat.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in fst_b200.h but not exported"
    assert sorted(nat.EXPORTS) == names
    assert lib.fst_abi_version() == nat.ABI_VERSION


def test_device_entry_points_refuse_without_cuda():
    if nat.cuda_device_count() > 0:
        pytest.skip("a CUDA device is present")
    with pytest.raises(nat.NativeError) as e:
        nat.realign(4096, 8192, 16, 0)
    assert e.value.code == nat.ENOCUDA
    with pytest.raises(nat.NativeError) as e:
        nat.gather([(4096, 8192, 1, 16, 0, 0)], 0)
    assert e.value.code == nat.ENOCUDA
    with pytest.raises(nat.NativeError) as e:
        cpp.Reader(0, 2, 1 << 20)
    assert e.value.code == nat.ENOCUDA


def test_small_queries():
    assert cpp.get_alignment_size() == 4096
    addr = cpp.cpu_malloc(10000)
    assert addr and addr % 4096 == 0
    ctypes.memmove(addr, b"hello world", 11)
    assert cpp.read_buffer(addr, 11) == b"hello world"
    cpp.cpu_free(addr)
    assert cpp.set_numa_node(-1) == 0
    assert isinstance(cpp.is_cuda_found(), bool)


def _host_buf(n):
    arr = np.zeros(n + 64, dtype=np.uint8)
    return arr, arr.ctypes.data


@pytest.mark.parametrize("rows,row_bytes,src_pitch,dst_pitch,src_off,dst_off", [
    (1, 1000, 0, 0, 0, 0), (7, 13, 29, 13, 3, 5), (64, 256, 1024, 256, 0, 0),
    (5, 3 << 20, (3 << 20) + 17, 3 << 20, 1, 2), (3, 1, 2, 1, 0, 0),
])
def test_gather_host_matches_numpy(rows, row_bytes, src_pitch, dst_pitch, src_off, dst_off):
    rng = np.random.default_rng(rows * 31 + row_bytes)
    sp, dp = (src_pitch or row_bytes), (dst_pitch or row_bytes)
    src = rng.integers(0, 256, src_off + rows * sp + 64, dtype=np.uint8)
    dst = np.full(dst_off + rows * dp + 64, 0xAB, dtype=np.uint8)
    nat.gather_host([(src.ctypes.data + src_off, dst.ctypes.data + dst_off, rows, row_bytes, sp, dp)], 4)
    want = np.full_like(dst, 0xAB)
    for r in range(rows):
        want[dst_off + r * dp: dst_off + r * dp + row_bytes] = src[src_off + r * sp: src_off + r * sp + row_bytes]
    assert np.array_equal(dst, want)


def test_gather_host_rejects_bad_ops():
    a = np.zeros(64, dtype=np.uint8)
    with pytest.raises(nat.NativeError) as e:
        nat.gather_host([(a.ctypes.data, a.ctypes.data + 32, 2, 16, 8, 16)])
    assert e.value.code == nat.EINVAL
    with pytest.raises(nat.NativeError):
        nat.gather_host([(0, a.ctypes.data, 1, 16, 0, 0)])


@pytest.fixture()
def blob_file(tmp_path):
    rng = np.random.default_rng(7)
    data = rng.integers(0, 256, 5 * (1 << 20) + 12345, dtype=np.uint8)
    p = tmp_path / "blob.bin"
    p.write_bytes(data.tobytes())
    return str(p), data


@pytest.mark.parametrize("io_mode", [nat.IO_AUTO, nat.IO_DIRECT, nat.IO_BUFFERED])
@pytest.mark.parametrize("offset,length", [(0, 4096), (1, 4095), (4097, 3 << 20), (777, 5 * (1 << 20) + 12345 - 777)])
def test_reader_to_host_memory(blob_file, io_mode, offset, length, leak_check):
    path, data = blob_file
    reader = cpp.Reader(-1, 4, 256 * 1024, 2, io_mode=io_mode)
    dst = np.full(length + 100, 0xCD, dtype=np.uint8)
    buf = cpp.gds_device_buffer(dst.ctypes.data, dst.size, False)
    rid = reader.submit(path, offset, length, buf, 50)
    assert reader.wait(rid) == length
    assert np.array_equal(dst[50:50 + length], data[offset:offset + length])
    assert (dst[:50] == 0xCD).all() and (dst[50 + length:] == 0xCD).all()  # canaries
    reader.close()


def test_reader_bounds_and_errors(blob_file, leak_check):
    path, data = blob_file
    reader = cpp.Reader(-1, 2, 1 << 20)
    dst = np.zeros(1000, dtype=np.uint8)
    buf = cpp.gds_device_buffer(dst.ctypes.data, dst.size, False)
    with pytest.raises(nat.NativeError) as e:
        reader.submit(path, 0, 2000, buf, 0)            # beyond the destination
    assert e.value.code == nat.ERANGE
    with pytest.raises(nat.NativeError) as e:
        reader.submit(path, data.size - 10, 100, buf, 0)  # beyond the end of the file
    assert e.value.code == nat.EIO
    with pytest.raises(nat.NativeError) as e:
        reader.submit(path + ".missing", 0, 10, buf, 0)
    assert e.value.code == nat.EIO
    with pytest.raises(nat.NativeError) as e:
        reader.wait(12345)
    assert e.value.code == nat.EINVAL
    reader.close()


def test_reader_fault_injection_reports_after_draining(blob_file, leak_check):
    """A failing pread (EIO) in the middle of a request: wait() returns an error only after
    every window was drained, and the reader stays usable."""
    path, data = blob_file
    reader = cpp.Reader(-1, 2, 256 * 1024, 2, io_mode=nat.IO_BUFFERED)
    try:
        dst = np.zeros(4 << 20, dtype=np.uint8)
        buf = cpp.gds_device_buffer(dst.ctypes.data, dst.size, False)
        reader.inject_fault(3, errno.EIO)
        rid = reader.submit(path, 0, 4 << 20, buf, 0)
        with pytest.raises(nat.NativeError) as e:
            reader.wait(rid)
        assert e.value.code == nat.EIO
        rid = reader.submit(path, 0, 1 << 20, buf, 0)      # the next request works
        assert reader.wait(rid) == 1 << 20
        assert np.array_equal(dst[:1 << 20], data[:1 << 20])
    finally:
        reader.close()


def test_reader_resumes_after_a_short_pread(blob_file, leak_check):
    """pread may return fewer bytes than asked without being at end of file; the worker must
    keep reading (upstream treats any short count as failure, ext.cpp:688-693)."""
    path, data = blob_file
    reader = cpp.Reader(-1, 2, 256 * 1024, 2, io_mode=nat.IO_BUFFERED)
    try:
        dst = np.zeros(2 << 20, dtype=np.uint8)
        buf = cpp.gds_device_buffer(dst.ctypes.data, dst.size, False)
        reader.inject_fault(2, 0, 100)
        rid = reader.submit(path, 5, 2 << 20, buf, 0)
        assert reader.wait(rid) == 2 << 20
        assert np.array_equal(dst, data[5:5 + (2 << 20)])
    finally:
        reader.close()


def test_reader_reports_truncated_file(tmp_path, leak_check):
    """The file shrinks between submit and read: the request fails with EIO, nothing hangs."""
    p = tmp_path / "shrinks.bin"
    p.write_bytes(b"x" * (3 << 20))
    reader = cpp.Reader(-1, 1, 256 * 1024, 1, io_mode=nat.IO_BUFFERED)
    try:
        dst = np.zeros(3 << 20, dtype=np.uint8)
        buf = cpp.gds_device_buffer(dst.ctypes.data, dst.size, False)
        reader.inject_fault(1, errno.EINTR)   # first read is retried, gives time for nothing
        fd = os.open(str(p), os.O_RDWR)
        os.ftruncate(fd, 1 << 20)
        os.close(fd)
        with pytest.raises(nat.NativeError) as e:
            reader.wait(reader.submit(str(p), 0, 3 << 20, buf, 0))
        assert e.value.code == nat.EIO
    finally:
        reader.close()


def test_metrics_count_reads(blob_file, leak_check):
    path, _ = blob_file
    before = cpp.get_cpp_metrics()
    reader = cpp.Reader(-1, 2, 1 << 20, 2, io_mode=nat.IO_DIRECT)
    dst = np.zeros(1 << 20, dtype=np.uint8)
    rid = reader.submit(path, 4096, 1 << 20, cpp.gds_device_buffer(dst.ctypes.data, dst.size, False), 0)
    reader.wait(rid)
    during = cpp.get_cpp_metrics()
    # each worker allocates its own two slots the first time it has a window to read
    assert during.bounce_buffer_bytes in (2 * (1 << 20), 2 * 2 * (1 << 20))
    assert during.bytes_read - before.bytes_read >= 1 << 20
    reader.close()
    assert cpp.get_cpp_metrics().bounce_buffer_bytes == 0


def test_legacy_nogds_reader_interface(blob_file, leak_check):
    """Upstream's nogds_file_reader call sequence (tests/unit/test_fastsafetensors.py:306-338)."""
    path, data = blob_file
    reader = cpp.nogds_file_reader(False, 1024, 4, False, 0)
    addr = cpp.cpu_malloc(4 << 20)
    buf = cpp.gds_device_buffer(addr, 4 << 20, False)
    fd = os.open(path, os.O_RDONLY)
    reqs = [reader.submit_read(fd, buf, i << 20, 1 << 20, i << 20) for i in range(4)]
    assert all(r > 0 for r in reqs)
    for i, r in enumerate(reqs):
        assert reader.wait_read(r) == addr + (i << 20)
    os.close(fd)
    assert cpp.read_buffer(addr, 4 << 20) == data[:4 << 20].tobytes()
    with pytest.raises(IndexError):
        reader.submit_read(0, buf, 0, 1 << 20, (4 << 20) - 10)
    cpp.cpu_free(addr)
    del reader


def test_legacy_device_helpers_without_a_device():
    """gpu_malloc / gpu_free / memcpy_h2d_async of upstream's module API (cpp.pyi:62-63,
    ext.cpp:959-971): without a CUDA device they report failure the way upstream's do."""
    if nat.cuda_device_count() > 0:
        pytest.skip("a CUDA device is present")
    assert cpp.gpu_malloc(4096) == 0
    cpp.gpu_free(0)
    host = cpp.cpu_malloc(4096)
    assert cpp.memcpy_h2d_async(4096, host, 16) == -1
    cpp.cpu_free(host)


def test_wait_can_be_repeated_after_a_timeout(tmp_path):
    """A wait that runs out of time leaves the request registered: the same id can be waited
    for again and still reports the request's own outcome."""
    data = np.random.default_rng(5).integers(0, 256, 6 << 20, dtype=np.uint8)
    p = tmp_path / "blob.bin"
    p.write_bytes(data.tobytes())
    dst = np.zeros(data.size, dtype=np.uint8)
    buf = cpp.gds_device_buffer(dst.ctypes.data, dst.size, False)
    reader = cpp.Reader(-1, 1, 4096, 2, io_mode=nat.IO_DIRECT)   # 1536 small windows, one worker
    try:
        rid = reader.submit(str(p), 0, data.size, buf, 0)
        timed_out = 0
        for _ in range(200000):
            try:
                done = reader.wait(rid, 0)
                break
            except nat.NativeError as e:
                assert e.code == nat.ETIMEOUT
                timed_out += 1
        else:
            pytest.fail("the request never completed")
        assert done == data.size and np.array_equal(dst, data)
        with pytest.raises(nat.NativeError) as e:      # only now is the id forgotten
            reader.wait(rid, 0)
        assert e.value.code == nat.EINVAL
    finally:
        reader.close()
