"""The cuFile ("gds") window source of the native reader.

Two things are checked on a GPU, neither of which calls into NVIDIA's libcufile:

* the whole cuFile code path (driver reference, register-once staging ring, per-request file
  handles, aligned windows into staging slots, realign kernel to the destination, loader on top)
  runs through a host-side double of the seven cuFile entry points, in a child process
  (``tests/native/fake_cufile.cpp``; upstream tests its GDS path the same way, through a table of
  fakes: ``tests/unit/test_fastsafetensors.py:361-376``);
* on a machine without the nvidia-fs module a cuFile request is refused at once with the "gds"
  error that callers retry on, before the cuFile driver is opened.
"""

import json
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"


def build_fake(out_dir: str) -> str:
    cuda = os.environ.get("CUDA_HOME") or "/usr/local/cuda"
    gxx = shutil.which("g++")
    if gxx is None or not os.path.exists(os.path.join(cuda, "include", "cufile.h")):
        pytest.skip("g++ or the CUDA headers are missing: the cuFile double cannot be built")
    so = os.path.join(out_dir, "libfake_cufile.so")
    subprocess.run([gxx, "-shared", "-fPIC", "-O1", "-std=c++17", "-fvisibility=hidden",
                    os.path.join(ROOT, "tests", "native", "fake_cufile.cpp"),
                    "-I", os.path.join(cuda, "include"), "-L", os.path.join(cuda, "lib64"),
                    "-Wl,-rpath," + os.path.join(cuda, "lib64"), "-lcudart", "-o", so], check=True)
    return so


@pytest.mark.gpu
def test_cufile_path_through_the_host_side_double(tmp_path, golden):
    so = build_fake(str(tmp_path))
    env = dict(os.environ, FST_B200_CUFILE_LIB=so)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "native", "cufile_stand_in_run.py"),
                           so, str(tmp_path)], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-3000:]
    out = json.loads([l for l in proc.stdout.splitlines() if l.startswith("{")][-1])
    assert [r["offset"] for r in out["reader"]] == [0, 4096, 9, 123464]
    for r in out["reader"]:
        assert r["done"] == r["length"] and r["bytes_equal"] and r["canaries"], r
        assert r["staging_while_open"] > 0 and r["staging_after_close"] == 0, r
    (err,) = out["errors"]
    assert err["raised"] and "gds" in err["text"]
    assert out["reader_survives"]
    assert out["loader"] == golden["cases"]["llama2_13b_w1_gds"][0]
    fake = out["fake"]
    # six readers (four offsets, the fault case, the loader's): one driver reference and ONE
    # registration of the staging ring each; every file handle deregistered; every read landed
    # in a registered ring
    assert fake["driver_open"] == fake["driver_close"] == 6
    assert fake["buf_register"] == fake["buf_deregister"] == 6
    assert fake["handle_register"] == fake["handle_deregister"] and fake["handles_live"] == 0
    assert fake["reads"] > 100 and fake["reads_into_registered"] == fake["reads"]
    assert out["leaks"] == {"bounce_buffer_bytes": 0, "staging_device_bytes": 0, "mem_used": 0}


@pytest.mark.gpu
def test_cufile_is_refused_with_a_gds_error_where_nvidia_fs_is_missing(tmp_path, leak_check):
    """What a caller such as vLLM relies on: ``nogds=False`` on a machine that cannot do
    GPUDirect Storage raises a ``RuntimeError`` naming "gds" (it then retries with
    ``nogds=True``) -- at once, without entering the cuFile driver."""
    import time

    import numpy as np
    import torch

    import fastsafetensors_b200 as fst
    from fastsafetensors_b200 import _native as nat
    from fastsafetensors_b200 import cpp
    from tests import synth

    if cpp.is_gds_supported(0):
        pytest.skip("nvidia-fs is loaded here: cuFile is allowed to run")
    assert not os.environ.get("FST_B200_CUFILE_LIB")
    blob = tmp_path / "blob.bin"
    blob.write_bytes(np.arange(1 << 20, dtype=np.uint8).tobytes())
    reader = cpp.Reader(0, 2, 1 << 20, 2, io_mode=nat.IO_CUFILE)
    dst = torch.zeros(1 << 20, dtype=torch.uint8, device=DEV)
    t0 = time.perf_counter()
    with pytest.raises(nat.NativeError) as e:
        reader.submit(str(blob), 0, 1 << 20, cpp.gds_device_buffer(dst.data_ptr(), dst.numel(), True), 0)
    assert time.perf_counter() - t0 < 5.0
    assert e.value.code == nat.EGDS and "gds" in str(e.value) and "nvidia-fs" in str(e.value)
    reader.close()
    # the same through the loader API
    spec = synth.config("llama3-8b", "tiny")
    paths = synth.write_checkpoint(spec, str(tmp_path / "ckpt"), fsync=False)
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), DEV, nogds=False, io_mode="cufile")
    loader.add_filenames({0: paths})
    with pytest.raises(RuntimeError, match="gds"):
        loader.copy_files_to_device()
    loader.close()
    # ... and the retry a caller then makes works
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), DEV, nogds=True)
    loader.add_filenames({0: paths})
    fb = loader.copy_files_to_device()
    assert len(fb.key_to_rank_lidx) == len(spec.tensors)
    fb.close()
    loader.close()


def test_cufile_mode_needs_a_device_destination(tmp_path):
    """CPU: a host reader asked for cuFile reads answers with the "gds" error, not a hang."""
    from fastsafetensors_b200 import _native as nat
    from fastsafetensors_b200 import cpp

    blob = tmp_path / "blob.bin"
    blob.write_bytes(b"\1" * 8192)
    reader = cpp.Reader(-1, 1, 4096, 2, io_mode=nat.IO_CUFILE)
    host = cpp.cpu_malloc(8192)
    try:
        with pytest.raises(nat.NativeError) as e:
            reader.submit(str(blob), 0, 8192, cpp.gds_device_buffer(host, 8192, False), 0)
        assert e.value.code == nat.EGDS and "gds" in str(e.value)
    finally:
        reader.close()
        cpp.cpu_free(host)


def test_the_double_builds_and_exports_what_the_reader_resolves(tmp_path):
    """CPU: the double compiles and carries the seven entry points plus the marker symbol."""
    import ctypes

    so = build_fake(str(tmp_path))
    lib = ctypes.CDLL(so)
    for name in ("cuFileDriverOpen", "cuFileDriverClose", "cuFileHandleRegister", "cuFileHandleDeregister",
                 "cuFileBufRegister", "cuFileBufDeregister", "cuFileRead", "fst_cufile_stand_in"):
        assert hasattr(lib, name), name
