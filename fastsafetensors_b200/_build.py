"""Builds ``libfst_b200.so`` in-tree with nvcc for sm_100a.

``python fastsafetensors_b200/_build.py`` (or ``build_native()``) compiles the sources in
``csrc/`` into ``fastsafetensors_b200/libfst_b200.so``.  The build is skipped when the library
is newer than every source and header.  nvcc cross-compiles without a GPU, so this also runs on
a machine that has none.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from typing import List, Optional

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC_DIR = os.path.join(PKG_DIR, "csrc")
INCLUDE_DIR = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_PATH = os.path.join(PKG_DIR, "libfst_b200.so")
SOURCES = ["fst_kernels.cu", "fst_reader.cu", "fst_host.cu", "fst_peer.cu"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def _inputs() -> List[str]:
    files = [os.path.join(CSRC_DIR, s) for s in SOURCES]
    files += [os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith(".h")]
    files += [os.path.join(INCLUDE_DIR, f) for f in os.listdir(INCLUDE_DIR) if f.endswith(".h")]
    return files


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(f) > built for f in _inputs())


def build_native(force: bool = False, verbose: bool = False, extra: Optional[List[str]] = None) -> str:
    """Compile the library if needed and return its path."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [
        _nvcc(),
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-O3", "-std=c++17", "-lineinfo",
        "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden,-pthread",
        "-I", INCLUDE_DIR, "-I", CSRC_DIR,
        "-DFST_BUILDING_LIBRARY",
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += extra or []
    cmd += [os.path.join(CSRC_DIR, s) for s in SOURCES]
    tmp = LIB_PATH + ".tmp"
    cmd += ["-o", tmp]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if verbose:
        sys.stderr.write(proc.stdout + proc.stderr)
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build_native(force="--force" in sys.argv, verbose="-v" in sys.argv))
