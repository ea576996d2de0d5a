"""Multi-rank path on CPU: gloo ranks, device "cpu", checked against upstream's recorded
per-rank outputs (shards, broadcasts, column groups, pushes) for the same requests."""

import json
import os
import sys
from collections import OrderedDict

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.golden import cases
from tests.helpers import free_port, rendezvous

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, case, paths, port, out_dir, batched=False, backend="gloo", transport="nccl"):
    sys.path.insert(0, ROOT)
    import fastsafetensors_b200 as fst
    from fastsafetensors_b200 import cpp
    from tests.helpers import record

    rdzv = rendezvous(out_dir, port)
    if backend == "nccl":
        torch.cuda.set_device(rank)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", init_method=rdzv, rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
        device = f"cuda:{rank}"
    else:
        dist.init_process_group("gloo", init_method=rdzv, rank=rank, world_size=world)
        device = "cpu"
    loader = fst.SafeTensorsFileLoader(dist.group.WORLD, device, nogds=True, max_threads=2, slot_kb=64)
    loader.add_filenames(cases.owners(paths, world))
    # the batched run also defers the waits: files are waited for chunk by chunk inside exchange
    fb = loader.copy_files_to_device(wait=not batched)
    out = {}
    for step in case["steps"]:
        if step[0] == "plan" and batched:
            # the whole plan in one batched exchange (tiny batches force several rounds)
            plan = OrderedDict((n, (a[0], a[1] % world) if a[0] == "push" else a) for n, a in cases.plan(case))
            got = fb.exchange(plan, max_batch_bytes=1 << 20, transport=transport)
            for name, action in plan.items():
                if action[0] == "push" and action[1] != rank:
                    assert name not in got
                    out[name] = None
                else:
                    out[name] = record(got[name])
        elif step[0] == "plan":
            for name, action in cases.plan(case):
                if action[0] == "shard":
                    out[name] = record(fb.get_sharded(name, action[1]))
                elif action[0] == "replicate":
                    out[name] = record(fb.get_tensor(name))
                else:
                    t = fb.push_tensor(name, action[1] % world)
                    out[name] = record(t) if t is not None else None
        elif step[0] == "multi_cols":
            out[step[1]] = record(fb.get_multi_cols(step[2], step[3]))
        elif step[0] == "as_dict":
            for name, t in fb.as_dict(OrderedDict(step[1])).items():
                out["as_dict:" + name] = record(t)
    # every file was requested in full by the "plan" step: its image must be gone already
    if list(case["steps"]) == [("plan",)] and not case.get("skip"):
        assert all(f.gbuf is None for fs in fb.rank_loaders.values() for f in fs)
    fb.close()
    loader.close()
    assert loader.framework.get_mem_used() == 0
    assert cpp.get_cpp_metrics().bounce_buffer_bytes == 0
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(out, f)
    dist.destroy_process_group()


MULTI = [c for c in cases.CASES if c["world"] > 1 and c["id"] in
         ("llama3_8b_w2_cols", "llama2_13b_w4", "mixtral_w8", "crafted_w2")]


@pytest.mark.parametrize("batched", [False, True], ids=["per_tensor", "batched"])
@pytest.mark.parametrize("case", MULTI, ids=[c["id"] for c in MULTI])
def test_gloo_ranks_match_upstream(case, batched, golden, case_files, tmp_path):
    if batched and case["steps"][0][0] != "plan":
        pytest.skip("as_dict in the per-tensor run already goes through the batched exchange")
    paths = case_files(case)
    world = case["world"]
    port = free_port()
    mp.spawn(_rank_main, args=(world, case, paths, port, str(tmp_path), batched), nprocs=world, join=True)
    for rank in range(world):
        got = json.load(open(tmp_path / f"rank{rank}.json"))
        assert got == golden["cases"][case["id"]][rank], f"rank {rank}"


# ------------------------------------------------------------------ packed / 8-bit float dtypes
PACKED = [
    # name, dtype, shape (safetensors element counts), dim
    ("f4_rows", "F4", (8, 16), 0), ("f4_cols", "F4", (4, 32), 1), ("e8m0", "F8_E8M0", (6, 10), 1),
    ("e5m2", "F8_E5M2", (6, 8), 0), ("e4m3", "F8_E4M3", (4, 12), 1),
]


def _write_packed(path):
    import numpy as np

    from tests import synth
    from oracle import st_oracle

    rng = np.random.default_rng(77)
    entries, blobs, off = {}, [], 0
    for name, dtype, shape, _ in PACKED:
        n = int(np.prod(shape)) * st_oracle.BITS[dtype] // 8
        entries[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [off, off + n]}
        blobs.append(rng.integers(0, 120, n, dtype=np.uint8).tobytes())
        off += n
    with open(path, "wb") as f:
        f.write(synth.header_bytes(entries, odd=False))
        f.write(b"".join(blobs))


def _packed_rank(rank, world, path, port, out_dir):
    sys.path.insert(0, ROOT)
    import fastsafetensors_b200 as fst
    from tests.helpers import digest_tensor

    rdzv = rendezvous(out_dir, port)
    dist.init_process_group("gloo", init_method=rdzv, rank=rank, world_size=world)
    loader = fst.SafeTensorsFileLoader(dist.group.WORLD, "cpu", nogds=True, max_threads=2)
    loader.add_filenames({1: [path]})          # owned by rank 1
    fb = loader.copy_files_to_device()
    out = {}
    for name, _, _, dim in PACKED:
        t = fb.get_sharded(name, dim)
        out[name] = [list(t.shape), str(t.dtype), digest_tensor(t)]
    fb.close()
    loader.close()
    loader = fst.SafeTensorsFileLoader(dist.group.WORLD, "cpu", nogds=True, max_threads=2)
    loader.add_filenames({1: [path]})
    fb = loader.copy_files_to_device()
    got = fb.exchange(OrderedDict((name, ("shard", dim)) for name, _, _, dim in PACKED))
    for name, t in got.items():
        assert out[name][2] == digest_tensor(t), name      # batched path agrees
    fb.close()
    loader.close()
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(out, f)
    dist.destroy_process_group()


def test_packed_and_8bit_float_dtypes_shard_as_bytes(tmp_path):
    """F4 (two values per byte), F8_E8M0, F8_E5M2, F8_E4M3: shards must be the oracle's byte
    slices; F4 shapes shrink on the last dimension in torch's packed dtype (upstream
    _torch.py:331-350).  Upstream itself cannot scatter E5M2/E4M3 over gloo; bytes can."""
    from oracle import st_oracle
    from tests.helpers import digest_bytes

    path = str(tmp_path / "packed.safetensors")
    _write_packed(path)
    world = 2
    mp.spawn(_packed_rank, args=(world, path, free_port(), str(tmp_path)), nprocs=world, join=True)
    fo = st_oracle.FileOracle(path)
    for rank in range(world):
        got = json.load(open(tmp_path / f"rank{rank}.json"))
        for name, dtype, shape, dim in PACKED:
            raw, new_shape = fo.get_sharded(name, dim, rank, world)
            if dtype == "F4":
                new_shape = new_shape[:-1] + [new_shape[-1] // 2]
            assert got[name][0] == new_shape, name
            assert got[name][2] == digest_bytes(raw), (name, rank)


# ------------------------------------------------------------------ "every key" access pattern
def _all_keys_rank(rank, world, paths, port, out_dir, backend="gloo"):
    sys.path.insert(0, ROOT)
    import fastsafetensors_b200 as fst
    from fastsafetensors_b200 import cpp
    from tests.helpers import digest_tensor

    rdzv = rendezvous(out_dir, port)
    if backend == "nccl":
        torch.cuda.set_device(rank)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", init_method=rdzv, rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
        device = f"cuda:{rank}"
    else:
        dist.init_process_group("gloo", init_method=rdzv, rank=rank, world_size=world)
        device = "cpu"
    calls = {"n": 0}
    real = dist.broadcast

    def counting(*a, **k):
        calls["n"] += 1
        return real(*a, **k)

    dist.broadcast = counting
    loader = fst.SafeTensorsFileLoader(dist.group.WORLD, device, nogds=True, max_threads=2, slot_kb=64)
    loader.add_filenames({i: [p] for i, p in enumerate(paths)})
    fb = loader.copy_files_to_device()
    out = {}
    for k in list(fb.key_to_rank_lidx.keys()):         # what vLLM's iterator does
        out[k] = digest_tensor(fb.get_tensor(k))
    n_keys = len(out)
    fb.close()
    loader.close()
    assert loader.framework.get_mem_used() == 0
    # far fewer collectives than tensors: per file a few tensor broadcasts, then one for the image
    assert calls["n"] < n_keys // 2, (calls["n"], n_keys)
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(out, f)
    dist.destroy_process_group()


def test_asking_for_every_key_switches_to_one_broadcast_per_file(case_files, tmp_path):
    from oracle import st_oracle
    from tests.helpers import digest_bytes

    case = [c for c in cases.CASES if c["id"] == "llama3_8b_w2_cols"][0]
    paths = sorted(case_files(case))[:2]
    mp.spawn(_all_keys_rank, args=(2, paths, free_port(), str(tmp_path)), nprocs=2, join=True)
    want = {}
    for p in paths:
        fo = st_oracle.FileOracle(p)
        for n in fo.tensors:
            want[n] = digest_bytes(fo.raw(n))
    for rank in range(2):
        assert json.load(open(tmp_path / f"rank{rank}.json")) == want
