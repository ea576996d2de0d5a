"""Shared fixtures.  GPU tests carry the ``gpu`` marker; everything else runs without a GPU."""

import json
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The native library must exist before the package can be imported.  Building is part of the
# test set-up (nvcc cross-compiles without a GPU); using a stale or missing library is not.
import importlib.util  # noqa: E402

_spec = importlib.util.spec_from_file_location(
    "fst_b200_build", os.path.join(ROOT, "fastsafetensors_b200", "_build.py"))
_build = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_build)  # loaded by path: importing the package needs the library
_build.build_native()

GOLDEN_PATH = os.path.join(ROOT, "tests", "golden", "reference_outputs.json")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    with open(GOLDEN_PATH) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def case_files(tmp_path_factory):
    """``case_files(case) -> paths``: the case's checkpoint, written once per session."""
    from tests.golden import cases

    made = {}

    def get(case):
        key = case["config"]
        if key not in made:
            made[key] = cases.materialize(case, str(tmp_path_factory.mktemp(key.replace("/", "_"))))
        return made[key]

    return get


@pytest.fixture()
def leak_check():
    """After the test: no file image accounted as live, no pinned ring left allocated (the
    accounting upstream's tests assert after every test)."""
    yield
    from fastsafetensors_b200 import cpp
    from fastsafetensors_b200.frameworks import get_framework_op

    assert get_framework_op("pytorch").get_mem_used() == 0
    assert cpp.get_cpp_metrics().bounce_buffer_bytes == 0


def has_cuda() -> bool:
    import torch

    return torch.cuda.is_available()
