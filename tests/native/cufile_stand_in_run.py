"""Runs the reader's cuFile code path through the host-side double in ``fake_cufile.cpp``.

Started by ``tests/test_gpu_cufile.py`` as a child process with ``FST_B200_CUFILE_LIB`` naming the
built double (the library is resolved once per process, so the variable has to be there before
the first cuFile use).  NVIDIA's libcufile is never loaded here.  Prints one JSON object.

    python tests/native/cufile_stand_in_run.py <libfake_cufile.so> <work dir>
"""

import ctypes
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def main() -> None:
    fake_path, work = sys.argv[1], sys.argv[2]
    assert os.environ.get("FST_B200_CUFILE_LIB") == fake_path
    import numpy as np
    import torch

    import fastsafetensors_b200 as fst
    from fastsafetensors_b200 import _native as nat
    from fastsafetensors_b200 import cpp
    from fastsafetensors_b200.frameworks import get_framework_op
    from tests.golden import cases
    from tests.helpers import record

    dev = "cuda:0"
    out = {"reader": [], "errors": []}
    rng = np.random.default_rng(11)
    data = rng.integers(0, 256, 37 * (1 << 20) + 4321, dtype=np.uint8)
    blob = os.path.join(work, "blob.bin")
    with open(blob, "wb") as f:
        f.write(data.tobytes())

    # 1. reader, four offsets: congruent (plain vector copy out of staging) and odd (funnel shift)
    for offset in (0, 4096, 8 + 1, 123456 + 8):
        length = data.size - offset
        reader = cpp.Reader(0, 4, 1 << 20, 2, io_mode=nat.IO_CUFILE, copy_streams=2)
        try:
            dst = torch.full((length + 512,), 0x5A, dtype=torch.uint8, device=dev)
            buf = cpp.gds_device_buffer(dst.data_ptr(), dst.numel(), True)
            rid = reader.submit(blob, offset, length, buf, 256)
            done = reader.wait(rid, 120000)
            staged = cpp.get_cpp_metrics().staging_device_bytes
            got = dst.cpu().numpy()
            out["reader"].append({
                "offset": offset, "done": int(done), "length": int(length),
                "bytes_equal": bool(np.array_equal(got[256:256 + length], data[offset:])),
                "canaries": bool((got[:256] == 0x5A).all() and (got[256 + length:] == 0x5A).all()),
                "staging_while_open": int(staged)})
        finally:
            reader.close()
        out["reader"][-1]["staging_after_close"] = int(cpp.get_cpp_metrics().staging_device_bytes)

    # 2. a failing cuFileRead is reported as a "gds" error and the reader survives it
    fake = ctypes.CDLL(fake_path)
    fake.fake_cufile_fail_read.argtypes = [ctypes.c_int64]
    reader = cpp.Reader(0, 2, 1 << 20, 2, io_mode=nat.IO_CUFILE)
    try:
        dst = torch.zeros(8 << 20, dtype=torch.uint8, device=dev)
        buf = cpp.gds_device_buffer(dst.data_ptr(), dst.numel(), True)
        reader.wait(reader.submit(blob, 0, 1 << 20, buf, 0))     # the reader is up
        fake.fake_cufile_fail_read(3)
        try:
            reader.wait(reader.submit(blob, 0, 8 << 20, buf, 0))
            out["errors"].append({"raised": False})
        except nat.NativeError as e:
            out["errors"].append({"raised": True, "code": e.code, "text": str(e)})
        ok = reader.wait(reader.submit(blob, 3, 1 << 20, buf, 0)) == 1 << 20
        out["reader_survives"] = bool(ok and np.array_equal(dst[: 1 << 20].cpu().numpy(), data[3: 3 + (1 << 20)]))
    finally:
        reader.close()

    # 3. the loader with io_mode="cufile" on the odd-header checkpoint, as upstream's GDS copier
    case = [c for c in cases.CASES if c["id"] == "llama2_13b_w1_gds"][0]
    paths = cases.materialize(case, os.path.join(work, "ckpt"))
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), dev, nogds=False, io_mode="cufile", max_threads=4,
                                       slot_kb=256)
    loader.add_filenames({0: paths})
    fb = loader.copy_files_to_device()
    out["loader"] = {name: record(fb.get_tensor(name)) for name, _ in cases.plan(case)}
    fb.close()
    loader.close()

    counts = (ctypes.c_int64 * 10)()
    fake.fake_cufile_counts(counts)
    names = ("driver_open", "driver_close", "buf_register", "buf_deregister", "handle_register",
             "handle_deregister", "reads", "read_bytes", "reads_into_registered", "handles_live")
    out["fake"] = dict(zip(names, [int(c) for c in counts]))
    m = cpp.get_cpp_metrics()
    out["leaks"] = {"bounce_buffer_bytes": int(m.bounce_buffer_bytes),
                    "staging_device_bytes": int(m.staging_device_bytes),
                    "mem_used": int(get_framework_op("pytorch").get_mem_used())}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
