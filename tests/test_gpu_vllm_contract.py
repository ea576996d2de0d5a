"""vLLM's own ``fastsafetensors_weights_iterator`` driving this loader (aliased under upstream's
module name): the call sequence a ``--load-format fastsafetensors`` start-up makes.  Runs in a
child process because the alias must be installed before vLLM is imported."""

import json
import os
import subprocess
import sys

import pytest
import torch

from oracle import st_oracle
from tests.golden import cases
from tests.helpers import digest_bytes

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import json, sys, hashlib
sys.path.insert(0, sys.argv[1])
import fastsafetensors_b200.compat as compat
compat.install()
import torch
try:
    from vllm.model_executor.model_loader import weight_utils
except Exception as e:
    print(json.dumps({"skip": f"{type(e).__name__}: {e}"})); sys.exit(0)
assert weight_utils.SafeTensorsFileLoader.__module__.startswith("fastsafetensors_b200"), \
    weight_utils.SafeTensorsFileLoader.__module__
out = {}
for name, t in weight_utils.fastsafetensors_weights_iterator(sys.argv[2:], False):
    assert t.is_cuda
    raw = t.detach().contiguous().reshape(-1).view(torch.uint8).cpu().numpy().tobytes()
    out[name] = [list(t.shape), hashlib.sha256(raw).hexdigest()[:16]]
print(json.dumps({"tensors": out}))
"""


def test_vllm_iterator_yields_every_tensor_byte_identical(case_files):
    case = [c for c in cases.CASES if c["id"] == "llama3_8b_w8"][0]
    paths = sorted(case_files(case))
    proc = subprocess.run([sys.executable, "-c", CHILD, ROOT] + paths, capture_output=True, text=True,
                          timeout=600)
    lines = [l for l in proc.stdout.splitlines() if l.startswith("{")]
    assert proc.returncode == 0 and lines, proc.stderr[-2000:]
    res = json.loads(lines[-1])
    if "skip" in res:
        pytest.skip("vLLM is not importable here: " + res["skip"])
    want = {}
    for p in paths:
        fo = st_oracle.FileOracle(p)
        for n, e in fo.tensors.items():
            want[n] = [list(e["shape"]), digest_bytes(fo.raw(n))]
    assert res["tensors"] == want
