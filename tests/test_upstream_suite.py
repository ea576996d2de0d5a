"""Upstream's own unit tests, unmodified, run against this package.

Needs the upstream source tree (``FST_UPSTREAM_TREE``, else ``reference_path`` of BASELINE.json);
skipped where there is none.  The test files are copied to a scratch directory and run in child
processes in which ``fastsafetensors_b200.compat.install()`` has aliased upstream's module names
to this package.  Modules this build leaves out on purpose (the unified-memory copier, the DLPack
capsule bridge, the 3FS loader) are stubbed so that the test modules import, and the tests that
exercise them are deselected by name; everything else has to pass.
"""

import json
import os
import re
import shutil
import subprocess
import sys

import pytest

from tests.helpers import free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SITECUSTOMIZE = '''
import sys, types
sys.path.insert(0, {root!r})
from fastsafetensors_b200 import compat
compat.install()


def _stub(name, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    sys.modules[name] = m
    parent, _, leaf = name.rpartition(".")
    setattr(sys.modules[parent], leaf, m)


def _no(*a, **k):
    raise NotImplementedError("out of scope in this build")


class _OutOfScope:
    def __init__(self, *a, **k):
        _no()


_stub("fastsafetensors.copier.unified", UnifiedMemCopier=_OutOfScope,
      is_unified_memory_system=lambda *a, **k: False)
_stub("fastsafetensors.threefs_loader", ThreeFSLoader=_OutOfScope)
_stub("fastsafetensors.dlpack", from_cuda_buffer=_no)
'''

# out of scope here: unified-memory copier and its selection, DLPack bridge, 3FS loader
OUT_OF_SCOPE = "not Unified and not unified and not dlpack and not 3fs and not ThreeFS and not 3FS " \
               "and not test_env_var_config"


def _upstream_tree():
    tree = os.environ.get("FST_UPSTREAM_TREE")
    if not tree:
        try:
            tree = json.load(open(os.path.join(ROOT, "BASELINE.json"))).get("reference_path")
        except (OSError, ValueError):
            tree = None
    if tree and os.path.exists(os.path.join(tree, "tests", "unit", "test_fastsafetensors.py")):
        return tree
    return None


@pytest.fixture(scope="module")
def scratch(tmp_path_factory):
    tree = _upstream_tree()
    if tree is None:
        pytest.skip("no upstream source tree on this machine")
    top = tmp_path_factory.mktemp("upstream")
    unit = top / "tests" / "unit"
    unit.mkdir(parents=True)
    for name in os.listdir(os.path.join(tree, "tests", "unit")):
        if name.endswith(".py"):
            shutil.copy(os.path.join(tree, "tests", "unit", name), unit / name)
    (top / "sitecustomize.py").write_text(SITECUSTOMIZE.format(root=ROOT))
    env = {k: v for k, v in os.environ.items() if not k.startswith("TORCHELASTIC_")}
    env.update(PYTHONPATH=str(top), TEST_FASTSAFETENSORS_FRAMEWORK="pytorch", CUDA_VISIBLE_DEVICES="")
    return str(unit), env


def _counts(text: str) -> dict:
    tail = [l for l in text.splitlines() if re.search(r"\d+ (passed|failed|error)", l)][-1]
    return {k: int(n) for n, k in re.findall(r"(\d+) (passed|failed|errors?|deselected|skipped)", tail)}


@pytest.mark.parametrize("module,select,passed,deselected", [
    ("test_fastsafetensors.py", OUT_OF_SCOPE, 38, 9), ("test_config.py", "", 39, 0),
    ("test_auto_loader.py", OUT_OF_SCOPE, 23, 14)])
def test_upstream_unit_tests_pass_against_this_package(scratch, module, select, passed, deselected):
    unit, env = scratch
    proc = subprocess.run([sys.executable, "-m", "pytest", module, "-q", "-p", "no:cacheprovider"]
                          + (["-k", select] if select else []),
                          cwd=unit, env=env, capture_output=True, text=True, timeout=900)
    got = _counts(proc.stdout)
    assert proc.returncode == 0 and "failed" not in got and "errors" not in got, proc.stdout[-3000:]
    assert got.get("passed") == passed and got.get("deselected", 0) == deselected, got


def test_upstream_multi_rank_tests_pass_against_this_package(scratch):
    """tests/unit/test_multi.py the way upstream's Makefile runs it: under torchrun, here with two
    gloo ranks on the host (shuffle, F4 last-dimension sharding, F8_E8M0 collectives)."""
    unit, env = scratch
    proc = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
                           "test_multi.py", "-q", "-p", "no:cacheprovider", "test_multi.py"],
                          cwd=unit, env=env, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, (proc.stdout + proc.stderr)[-3000:]
    assert len(re.findall(r"\b3 passed", proc.stdout)) == 2, proc.stdout[-2000:]
