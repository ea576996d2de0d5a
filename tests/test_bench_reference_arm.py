"""The reference arm of bench.py on a tiny checkpoint: upstream itself (built into oracle/_ref)
on device "cpu" with gloo ranks; one JSON line on stdout with the keys the bench contract names."""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref", "fastsafetensors", "__init__.py")


@pytest.mark.skipif(not os.path.exists(REF), reason="oracle/_ref is not built (oracle/build_ref.sh)")
def test_reference_arm_prints_one_contract_line(tmp_path):
    env = {k: v for k, v in os.environ.items() if not k.startswith("TORCHELASTIC_")}
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--scale", "tiny",
         "--config", "llama2-13b", "--dir", str(tmp_path), "--steps", "1"],
        capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, proc.stdout
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "GB/s" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["gpu_launches"] == 0
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0, "page_cache": "dropped before every step"}
    cb = d["cpu_baseline"]
    assert cb["kind"] == "reference" and cb["value"] == d["value"] and cb["cores"] == os.cpu_count()
    # both of upstream's settings were tried and one of them was used
    assert "defaults" in cb["sample"] and "tuned" in cb["sample"]
    assert "tensor-parallel 4-way" in d["config"]["workload"]
