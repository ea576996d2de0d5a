"""Edge cases of the format: tensors without elements, a file without tensors, ``__metadata__``,
trailing bytes.  Checked against the ``safetensors`` package (what upstream's own tests compare
with) and against the oracle; the same cases run on a device under the ``gpu`` marker."""

import struct
from collections import OrderedDict

import numpy as np
import pytest
import torch
from safetensors.torch import load_file, save_file

import fastsafetensors_b200 as fst
from oracle import st_oracle
from tests.helpers import free_port, rendezvous


def _empty_mix(path: str) -> dict:
    tensors = {
        "e0": torch.zeros(0, dtype=torch.float16),
        "e2": torch.zeros((0, 4)),
        "mid0": torch.zeros((2, 0, 3), dtype=torch.bfloat16),
        "x": torch.arange(12, dtype=torch.float32).reshape(3, 4),
        "tail0": torch.zeros((4, 0), dtype=torch.int64),
    }
    save_file(tensors, path, metadata={"format": "pt", "origin": "edge"})
    return load_file(path)


def _check_empty_mix(device: str, tmp_path) -> None:
    path = str(tmp_path / "mix.safetensors")
    want = _empty_mix(path)
    with fst.fastsafe_open([path], device=device, nogds=True) as f:
        assert sorted(f.keys()) == sorted(want)
        assert f.metadata()[path] == {"format": "pt", "origin": "edge"}
        for name, w in want.items():
            t = f.get_tensor(name)
            assert t.shape == w.shape and t.dtype == w.dtype and t.device.type == device.split(":")[0]
            assert torch.equal(t.cpu(), w), name
    # the shards of all ranks of a 2-way group, packed by one rank: empty stays empty
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), device, nogds=True)
    loader.add_filenames({0: [path]})
    fb = loader.copy_files_to_device()
    plan = OrderedDict([("e2", ("shard", 1)), ("mid0", ("shard", 1)), ("x", ("shard", 1)),
                        ("tail0", ("shard", 0)), ("e0", ("replicate",))])
    got = fb.shard_locally(plan, 2)
    fo = st_oracle.FileOracle(path)
    for rank in range(2):
        for name, action in plan.items():
            dim = action[1] if action[0] == "shard" else -1
            raw, shape = fo.get_sharded(name, dim, rank, 2)
            t = got[rank][name].get_raw()
            assert list(t.shape) == list(shape), (name, rank)
            assert np.array_equal(t.cpu().reshape(-1).view(torch.uint8).numpy(), raw), (name, rank)
    fb.close()
    loader.close()


def _check_header_only(device: str, tmp_path) -> None:
    path = str(tmp_path / "none.safetensors")
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", 2) + b"{}")
    with fst.fastsafe_open([path], device=device, nogds=True) as f:
        assert list(f.keys()) == []
    # beside a normal file: keys of the other file are served as usual
    other = str(tmp_path / "some.safetensors")
    save_file({"w": torch.arange(6, dtype=torch.int32)}, other)
    with fst.fastsafe_open([path, other], device=device, nogds=True) as f:
        assert list(f.keys()) == ["w"]
        assert torch.equal(f.get_tensor("w").cpu(), torch.arange(6, dtype=torch.int32))


def _check_trailing_bytes(device: str, tmp_path) -> None:
    """Bytes after the last tensor are legal (upstream common.py:278-291) and are not copied into
    any tensor."""
    path = str(tmp_path / "trail.safetensors")
    save_file({"a": torch.arange(5, dtype=torch.int16), "b": torch.ones(3, dtype=torch.uint8)}, path)
    with open(path, "ab") as fh:
        fh.write(b"\xee" * 37)
    with fst.fastsafe_open([path], device=device, nogds=True) as f:
        assert torch.equal(f.get_tensor("a").cpu(), torch.arange(5, dtype=torch.int16))
        assert torch.equal(f.get_tensor("b").cpu(), torch.ones(3, dtype=torch.uint8))


CHECKS = [_check_empty_mix, _check_header_only, _check_trailing_bytes]


@pytest.mark.parametrize("check", CHECKS, ids=lambda c: c.__name__[7:])
def test_on_cpu(check, tmp_path):
    check("cpu", tmp_path)


@pytest.mark.gpu
@pytest.mark.parametrize("check", CHECKS, ids=lambda c: c.__name__[7:])
def test_on_device(check, tmp_path):
    check("cuda:0", tmp_path)


# ------------------------------------------------------------------ two ranks, tensors without elements
def _two_rank_main(rank, world, path, port, out_dir, backend):
    import json
    import os

    import torch.distributed as dist

    rdzv = rendezvous(out_dir, port)
    if backend == "nccl":
        torch.cuda.set_device(rank)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", init_method=rdzv, rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
        device = f"cuda:{rank}"
    else:
        dist.init_process_group("gloo", init_method=rdzv, rank=rank, world_size=world)
        device = "cpu"
    fo = st_oracle.FileOracle(path)
    plan = OrderedDict([("e2", ("shard", 1)), ("mid0", ("shard", 1)), ("x", ("shard", 1)),
                        ("tail0", ("shard", 0)), ("e0", ("replicate",)), ("x2", ("push", 1))])
    report = {}
    for mode in ("exchange", "per_tensor"):
        loader = fst.SafeTensorsFileLoader(dist.group.WORLD, device, nogds=True)
        loader.add_filenames({1: [path]})          # rank 1 owns the file
        fb = loader.copy_files_to_device()
        if mode == "exchange":
            got = {n: t.get_raw() for n, t in fb.exchange(plan).items()}
        else:
            got = {}
            for name, action in plan.items():
                if action[0] == "shard":
                    got[name] = fb.get_sharded(name, action[1])
                elif action[0] == "replicate":
                    got[name] = fb.get_tensor(name)
                else:
                    t = fb.push_tensor(name, action[1])
                    if t is not None:
                        got[name] = t
        for name, action in plan.items():
            if action[0] == "push" and action[1] != rank:
                assert name not in got
                continue
            dim = action[1] if action[0] == "shard" else -1
            raw, shape = fo.get_sharded(name, dim, rank, world)
            t = got[name]
            ok = list(t.shape) == list(shape) and np.array_equal(
                t.cpu().contiguous().reshape(-1).view(torch.uint8).numpy(), raw)
            report[f"{mode}:{name}"] = bool(ok)
        fb.close()
        loader.close()
    with open(os.path.join(out_dir, f"r{rank}.json"), "w") as f:
        json.dump(report, f)
    dist.destroy_process_group()


def _run_two_ranks(tmp_path, backend, port):
    import json

    import torch.multiprocessing as mp

    path = str(tmp_path / "mix2.safetensors")
    save_file({"e0": torch.zeros(0, dtype=torch.float16), "e2": torch.zeros((0, 4)),
               "mid0": torch.zeros((2, 0, 3), dtype=torch.bfloat16),
               "x": torch.arange(12, dtype=torch.float32).reshape(3, 4),
               "x2": torch.arange(7, dtype=torch.int16),
               "tail0": torch.zeros((4, 0), dtype=torch.int64)}, path)
    mp.spawn(_two_rank_main, args=(2, path, port, str(tmp_path), backend), nprocs=2, join=True)
    for rank in range(2):
        report = json.load(open(tmp_path / f"r{rank}.json"))
        assert report and all(report.values()), (rank, report)


def test_two_gloo_ranks_with_empty_tensors(tmp_path):
    _run_two_ranks(tmp_path, "gloo", free_port())


@pytest.mark.gpu
def test_two_nccl_ranks_with_empty_tensors(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run_two_ranks(tmp_path, "nccl", free_port())
