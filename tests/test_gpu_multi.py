"""Multi-GPU path: one process per GPU over NCCL, checked against upstream's recorded per-rank
outputs.  Cases run when the box has at least as many GPUs as the case has ranks."""

import json

import pytest
import torch
import torch.multiprocessing as mp

from tests.golden import cases
from tests.test_multi_cpu import _all_keys_rank, _rank_main
from tests.helpers import free_port

pytestmark = pytest.mark.gpu
MULTI = [c for c in cases.CASES if c["world"] > 1]


@pytest.mark.parametrize("batched", [False, "nccl", "peer"], ids=["per_tensor", "batched_nccl", "batched_peer"])
@pytest.mark.parametrize("case", MULTI, ids=[c["id"] for c in MULTI])
def test_nccl_ranks_match_upstream(case, batched, golden, case_files, tmp_path):
    world = case["world"]
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    if batched and case["steps"][0][0] != "plan":
        pytest.skip("as_dict in the per-tensor run already goes through the batched exchange")
    paths = case_files(case)
    port = free_port()
    mp.spawn(_rank_main, args=(world, case, paths, port, str(tmp_path), bool(batched), "nccl", batched or "nccl"),
             nprocs=world, join=True)
    for rank in range(world):
        got = json.load(open(tmp_path / f"rank{rank}.json"))
        assert got == golden["cases"][case["id"]][rank], f"rank {rank}"


def test_every_key_access_over_nccl(case_files, tmp_path):
    """The vLLM access pattern (get_tensor of every key) on two GPUs: results byte-identical to
    the files, served by one image broadcast per file after the first few tensors."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from oracle import st_oracle
    from tests.helpers import digest_bytes

    case = [c for c in cases.CASES if c["id"] == "llama3_8b_w2_cols"][0]
    paths = sorted(case_files(case))[:2]
    mp.spawn(_all_keys_rank, args=(2, paths, free_port(), str(tmp_path), "nccl"), nprocs=2, join=True)
    want = {}
    for p in paths:
        fo = st_oracle.FileOracle(p)
        for n in fo.tensors:
            want[n] = digest_bytes(fo.raw(n))
    for rank in range(2):
        assert json.load(open(tmp_path / f"rank{rank}.json")) == want


@pytest.mark.parametrize("queue_size", [0, 2])
def test_pipeline_over_nccl_every_rank_gets_every_tensor(queue_size, case_files, tmp_path):
    """ParallelLoader on two GPUs: batches of two files, each image broadcast once, producer and
    consumer on different threads; every rank ends up with every tensor of every file."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from tests.test_parallel_loader import CASE, _expected
    from tests.test_parallel_loader import _rank_main as pipeline_rank

    paths = sorted(case_files(CASE))[:7]          # odd count: the last batch has one file only
    want = {k: list(v) for k, v in _expected(paths).items()}
    mp.spawn(pipeline_rank, args=(2, paths, free_port(), str(tmp_path), queue_size, "nccl"), nprocs=2, join=True)
    for rank in range(2):
        assert json.load(open(tmp_path / f"rank{rank}.json")) == want, rank
