"""Race and memory checking of the library's host side (worker pools, rings, request
bookkeeping, host gather) without a GPU: the library sources are built once with
ThreadSanitizer and once with AddressSanitizer, linked to ``tests/native/host_stress.cpp``
(several readers driven from several threads, injected read errors, ragged requests) and run.
A sanitizer report or a failed expectation fails the test.  compute-sanitizer plays no part:
nothing here runs on a device."""

import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "fastsafetensors_b200", "csrc")
SOURCES = ["fst_kernels.cu", "fst_reader.cu", "fst_host.cu", "fst_peer.cu"]

SANITIZERS = {
    "thread": (["-fsanitize=thread"], {"TSAN_OPTIONS": "halt_on_error=0:exitcode=66"}, "ThreadSanitizer"),
    "address": (["-fsanitize=address", "-fno-omit-frame-pointer"],
                {"ASAN_OPTIONS": "protect_shadow_gap=0:detect_leaks=1:exitcode=67"}, "AddressSanitizer"),
}


def _tool(name):
    return shutil.which(name) or (f"/usr/local/cuda/bin/{name}" if os.path.exists(f"/usr/local/cuda/bin/{name}") else None)


@pytest.mark.parametrize("kind", sorted(SANITIZERS))
def test_host_side_under_sanitizer(kind, tmp_path):
    nvcc, gxx = _tool("nvcc"), _tool("g++")
    if not nvcc or not gxx:
        pytest.skip("needs nvcc and g++")
    flags, env_extra, banner = SANITIZERS[kind]
    lib = tmp_path / f"libfst_{kind}.so"
    build = subprocess.run(
        [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O1", "-g", "-std=c++17", "-shared",
         "-Xcompiler", ",".join(["-fPIC", "-pthread"] + flags), "-I", os.path.join(ROOT, "include"), "-I", CSRC,
         "-DFST_BUILDING_LIBRARY"] + [os.path.join(CSRC, s) for s in SOURCES] + ["-o", str(lib)],
        capture_output=True, text=True)
    if build.returncode != 0 and "cannot find" in build.stderr and "san" in build.stderr:
        pytest.skip(f"lib{kind[0]}san is not installed")
    assert build.returncode == 0, build.stderr[-3000:]
    exe = tmp_path / f"host_stress_{kind}"
    link = subprocess.run(
        [gxx, "-std=c++17", "-O1", "-g", "-pthread"] + flags +
        ["-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "native", "host_stress.cpp"),
         "-L", str(tmp_path), f"-lfst_{kind}", f"-Wl,-rpath,{tmp_path}", "-o", str(exe)],
        capture_output=True, text=True)
    assert link.returncode == 0, link.stderr[-3000:]
    env = dict(os.environ, **env_extra)
    run = subprocess.run([str(exe), str(tmp_path)], capture_output=True, text=True, timeout=300, env=env)
    assert banner not in run.stderr, run.stderr[:6000]
    assert run.returncode == 0, (run.returncode, run.stdout[-1000:], run.stderr[-3000:])
    assert "host stress ok" in run.stdout
