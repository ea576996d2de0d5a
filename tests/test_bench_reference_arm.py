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
    # run bench.py as __main__ and then report which of this repository's modules got imported
    code = ("import runpy, sys; sys.argv = ['bench.py', '--impl', 'reference', '--scale', 'tiny', '--config', "
            f"'llama2-13b', '--dir', {str(tmp_path)!r}, '--steps', '1']; "
            f"runpy.run_path({os.path.join(ROOT, 'bench.py')!r}, run_name='__main__'); "
            "sys.stderr.write('PRODUCT_MODULES=' + ','.join(sorted(m for m in sys.modules "
            "if m.startswith('fastsafetensors_b200'))) + '\\n')")
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, env=env,
                          cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, proc.stdout
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "GB/s" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["gpu_launches"] == 0 and d["steps"] == 1 and d["warmup"] == 3
    # value: upstream's shuffle phase from resident images; e2e: cold files -> shards
    assert "resident" in d["notes"]["value_phase"] and d["notes"]["whole_checkpoint_per_step"] is True
    assert d["e2e"]["value"] > 0 and d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["e2e"]["page_cache"] == "dropped before every step"
    cb = d["cpu_baseline"]
    assert cb["kind"] == "reference" and cb["value"] == d["value"] and cb["cores"] == os.cpu_count()
    # both of upstream's settings were tried and one of them was used
    assert set(cb["settings"]["tried_gbs"]) == {"defaults", "tuned"} and cb["settings"]["used"] in ("defaults", "tuned")
    assert "tensor-parallel 4-way" in d["config"]["workload"] and d["config"]["tp"] == 4
    # the arm must not import the product (and with it the native library)
    assert "PRODUCT_MODULES=\n" in proc.stderr, proc.stderr[-500:]


def test_both_arms_describe_the_same_workload():
    """The ``config`` object is computed from the checkpoint alone, so both arms print the same."""
    sys.path.insert(0, ROOT)
    import argparse

    import bench

    args = argparse.Namespace(config=None, scale="tiny", layers=0, files=0, dir="/tmp/x", steps=20, e2e_steps=0)
    one, eight = bench.Workload(args, 1), bench.Workload(args, 8)
    assert one.spec.name == "llama2-13b" and one.tp == 4 and one.n_files == 3
    assert eight.spec.name == "llama3-70b" and eight.tp == 8
    args.files = 8
    sub = bench.Workload(args, 8)
    assert sub.n_files == 8 and len(sub.paths) == 8 and "first 8 of its 30 files" in sub.label
    assert sub.data_bytes == sum(t.nbytes for t in sub.tensors) < eight.data_bytes
    assert set(sub.plan) == {t.name for t in sub.tensors}
    assert 2 <= sub.e2e_steps(args) <= 20


def test_bench_parity_expectation_agrees_with_the_oracle():
    """The bench's in-run parity check regenerates tensor bytes and slices them with plain numpy;
    here that slicing is held against the oracle's restatement of upstream's shard rule, and the
    checker is shown to notice a wrong byte."""
    sys.path.insert(0, ROOT)
    import argparse

    import numpy as np
    import torch

    import bench
    from oracle import st_oracle
    from tests import synth

    args = argparse.Namespace(config="llama3-8b", scale="tiny", layers=0, files=0, dir="/tmp/x", steps=5, e2e_steps=0)
    wl = bench.Workload(args, 8)
    seen = set()
    results = {}
    for pos in bench.parity_sample(wl):
        t = wl.tensors[pos]
        action = wl.plan[t.name]
        raw = synth.expected_bytes(wl.spec, wl.indices[pos])
        for dst in range(wl.tp):
            got = bench.expected_shard(t, raw, action, dst, wl.tp)
            dim = action[1] if action[0] == "shard" else -1
            want, _ = st_oracle.shard(raw, list(t.shape), t.dtype, dim, dst, wl.tp)
            assert np.array_equal(got, want), (t.name, dst)
            results[(t.name, dst)] = torch.from_numpy(np.array(got))
        seen.add(action[0] + (str(action[1]) if action[0] == "shard" else ""))
    assert seen == {"shard0", "shard1", "replicate"}
    ok = bench.check_parity(wl, lambda n, d: results.get((n, d)), range(wl.tp))
    assert ok["ok"] and ok["checked"] == len(results) and ok["kinds"] == ["replicate", "shard0", "shard1"]
    name, dst = next(iter(results))
    results[(name, dst)] = results[(name, dst)].clone()
    results[(name, dst)][0] ^= 1
    bad = bench.check_parity(wl, lambda n, d: results.get((n, d)), range(wl.tp))
    assert not bad["ok"] and name in bad["mismatches"][0]


def test_workload_is_cut_to_what_the_disk_holds(tmp_path, monkeypatch):
    """A checkpoint that does not fit the free disk space: other checkpoints of the benchmark
    directory go first, then files are dropped from the end, never below one per rank."""
    sys.path.insert(0, ROOT)
    import argparse
    import collections
    import shutil

    import bench

    top = tmp_path / "bench"
    (top / "some-older-checkpoint").mkdir(parents=True)
    (top / "some-older-checkpoint" / "x.safetensors").write_bytes(b"0" * 10)
    args = argparse.Namespace(config="llama3-70b", scale="tiny", layers=0, files=0, dir=str(top), steps=5,
                              e2e_steps=0)
    whole = bench.Workload(args, 8)
    assert whole.n_files == 30 and whole.disk_note == ""
    assert (top / "some-older-checkpoint").exists()
    per_file = max(sum(whole.spec.tensors[i].nbytes for i in g) for g in whole.groups) + (1 << 20)
    usage = collections.namedtuple("usage", "total used free")
    room = 12                                                   # files that still fit
    monkeypatch.setattr(shutil, "disk_usage", lambda p: usage(1 << 40, 0, (2 << 30) + room * per_file))
    cut = bench.Workload(args, 8)
    assert 8 <= cut.n_files < 30 and "cut to" in cut.disk_note and "removed some-older-checkpoint" in cut.disk_note
    assert not (top / "some-older-checkpoint").exists()
    assert len(cut.paths) == cut.n_files and f"first {cut.n_files} of its 30 files" in cut.label
    monkeypatch.setattr(shutil, "disk_usage", lambda p: usage(1 << 40, 0, 1 << 30))
    assert bench.Workload(args, 8).n_files == 8                  # one file per rank is the floor
    # a file count decided elsewhere (rank 0) is taken as it is
    assert bench.Workload(args, 8, n_files=11).n_files == 11


def test_recorded_traffic_ratio_belongs_to_the_current_kernel():
    """The DRAM-traffic ratio the bench reports comes from a profiler capture; it is only
    presented as such while the gather kernel's device code is the code that was captured."""
    sys.path.insert(0, ROOT)
    import bench

    rec = bench.recorded_traffic(2.0e9)
    assert rec["traffic_source"].startswith("profiler capture"), rec
    assert 0.9 < rec["traffic_ratio"] <= 1.05 and rec["traffic"] == int(rec["traffic_ratio"] * 2.0e9)
