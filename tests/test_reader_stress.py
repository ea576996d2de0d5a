"""Concurrency of the native reader on host memory: many requests in flight on one reader,
submitted from several Python threads, and several readers at once (the producer-thread pattern
of the pipelined loader)."""

import threading

import numpy as np
import pytest

from fastsafetensors_b200 import _native as nat
from fastsafetensors_b200 import cpp


@pytest.fixture(scope="module")
def files(tmp_path_factory):
    d = tmp_path_factory.mktemp("stress")
    out = []
    for i in range(4):
        data = np.random.default_rng(i).integers(0, 256, (3 << 20) + 1000 * i + 17, dtype=np.uint8)
        p = d / f"f{i}.bin"
        p.write_bytes(data.tobytes())
        out.append((str(p), data))
    return out


@pytest.mark.parametrize("io_mode", [nat.IO_DIRECT, nat.IO_BUFFERED])
def test_many_requests_from_many_threads_on_one_reader(files, io_mode, leak_check):
    reader = cpp.Reader(-1, 4, 128 * 1024, 2, io_mode=io_mode)
    errors = []

    def work(tid):
        try:
            rng = np.random.default_rng(100 + tid)
            for _ in range(25):
                path, data = files[int(rng.integers(0, len(files)))]
                off = int(rng.integers(0, data.size - 1))
                n = int(rng.integers(1, min(data.size - off, 700_000) + 1))
                pad = int(rng.integers(0, 64))
                dst = np.full(n + pad + 32, 0xEE, dtype=np.uint8)
                buf = cpp.gds_device_buffer(dst.ctypes.data, dst.size, False)
                rid = reader.submit(path, off, n, buf, pad)
                assert reader.wait(rid, 60000) == n
                assert np.array_equal(dst[pad:pad + n], data[off:off + n])
                assert (dst[:pad] == 0xEE).all() and (dst[pad + n:] == 0xEE).all()
        except BaseException as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=work, args=(t,)) for t in range(6)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    reader.close()
    assert not errors, errors[0]


def test_overlapping_requests_complete_in_any_wait_order(files, leak_check):
    reader = cpp.Reader(-1, 3, 64 * 1024, 2, io_mode=nat.IO_BUFFERED)
    pending = []
    for i in range(40):
        path, data = files[i % len(files)]
        off, n = 1000 * i + 3, 200_000 + 777 * i
        dst = np.zeros(n, dtype=np.uint8)
        rid = reader.submit(path, off, n, cpp.gds_device_buffer(dst.ctypes.data, n, False), 0)
        pending.append((rid, dst, data[off:off + n]))
    for rid, dst, want in reversed(pending):
        assert reader.wait(rid) == want.size
        assert np.array_equal(dst, want)
    reader.close()


def test_several_readers_side_by_side(files, leak_check):
    errors = []

    def work(i):
        try:
            path, data = files[i]
            reader = cpp.Reader(-1, 2, 256 * 1024, 2, io_mode=nat.IO_AUTO)
            dst = np.zeros(data.size, dtype=np.uint8)
            buf = cpp.gds_device_buffer(dst.ctypes.data, dst.size, False)
            for _ in range(3):
                dst[:] = 0
                assert reader.wait(reader.submit(path, 0, data.size, buf, 0)) == data.size
                assert np.array_equal(dst, data)
            reader.close()
        except BaseException as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(len(files))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[0]
