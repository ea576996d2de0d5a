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


# ------------------------------------------------------------------ W ranks emulated on one GPU
class _OneGpuArena:
    """Stands in for ``PeerArena`` when all ranks live in one process: every rank's arena is a
    slice of one device buffer, so a "peer" address is an ordinary address of the same GPU."""

    def __init__(self, pool: torch.Tensor, rank: int, world: int, nbytes: int):
        self.nbytes = nbytes
        self.peer_base = [pool.data_ptr() + r * nbytes for r in range(world)]
        self.address = self.peer_base[rank]
        self._mine = pool[rank * nbytes:(rank + 1) * nbytes]

    def view(self, nbytes: int):
        return self._mine[:nbytes]


class _RankOf:
    """Group stub: rank and size only (no collective is issued in the emulation)."""

    real_pg = None

    def __init__(self, rank, world):
        self._rank, self._world = rank, world

    def rank(self):
        return self._rank

    def size(self):
        return self._world


PLAN_CASES = [c for c in MULTI if c["steps"][0][0] == "plan"]


@pytest.mark.parametrize("order", ["region", "interleave"])
@pytest.mark.parametrize("split", [0, 8], ids=["one_launch", "own_region_beside"])
@pytest.mark.parametrize("case", PLAN_CASES, ids=[c["id"] for c in PLAN_CASES])
def test_peer_exchange_arithmetic_for_every_world_size_on_one_gpu(case, split, order, golden, case_files,
                                                                   monkeypatch):
    """The peer exchange of W ranks run by ONE process on ONE GPU: each emulated rank owns the
    files i mod W, builds its own chunk layouts and destination addresses exactly as a real rank
    does (``PeerShardExchange._prepare``), and its gather launches store into the other ranks'
    arenas -- here slices of one buffer.  Every rank must end up with what upstream delivered to
    it.  This covers the address arithmetic of 4- and 8-rank groups on a box with one GPU; the
    transport itself (IPC mappings, NVLink) is what the multi-process tests above cover."""
    import fastsafetensors_b200 as fst
    from collections import OrderedDict
    from fastsafetensors_b200.batch import PeerShardExchange
    from tests.helpers import record

    monkeypatch.setenv("FST_B200_PEER_REMOTE_CTAS", str(split))
    monkeypatch.setenv("FST_B200_PEER_ORDER", order)
    world = case["world"]
    paths = sorted(case_files(case))
    plan = OrderedDict((n, (a[0], a[1] % world) if a[0] == "push" else a) for n, a in cases.plan(case))
    loaders, buffers, exchanges = [], [], []
    for rank in range(world):
        loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), "cuda:0", nogds=True, max_threads=2, slot_kb=64)
        loader.pg = _RankOf(rank, world)
        loader.add_filenames(cases.owners(paths, world))
        fb = loader.copy_files_to_device(wait=False)
        loaders.append(loader)
        buffers.append(fb)
    # first pass only sizes the arenas (every rank computes the same need)
    probe = PeerShardExchange(buffers[0], plan, world, 0, chunk_bytes=1 << 16,
                              arena=_OneGpuArena(torch.zeros(world, dtype=torch.uint8, device="cuda:0"), 0, world, 1))
    need = (probe.recv_need + 255) // 256 * 256
    pool = torch.full((world * need,), 0xEE, dtype=torch.uint8, device="cuda:0")
    for rank in range(world):
        ex = PeerShardExchange(buffers[rank], plan, world, rank, chunk_bytes=1 << 16,
                               arena=_OneGpuArena(pool, rank, world, need))
        assert ex.recv_need == probe.recv_need
        exchanges.append(ex)
    for ex in exchanges:
        ex.run()
    torch.cuda.synchronize()
    for rank, ex in enumerate(exchanges):
        got = ex.results()
        want = golden["cases"][case["id"]][rank]
        for name, action in plan.items():
            if action[0] == "push" and action[1] != rank:
                assert name not in got and want[name] is None
            else:
                assert record(got[name]) == want[name], (rank, name)
    del exchanges, got, ex, probe
    for fb, loader in zip(buffers, loaders):
        fb.close()
        loader.close()
