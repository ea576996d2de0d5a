"""PipelineParallel / ParallelLoader: the producer-consumer iterator (upstream
parallel_loader.py:126-505) on CPU, one rank and two gloo ranks, against the oracle."""

import json
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import fastsafetensors_b200 as fst
from fastsafetensors_b200 import cpp
from fastsafetensors_b200.frameworks import get_framework_op
from oracle import st_oracle
from tests.golden import cases
from tests.helpers import digest_bytes, digest_tensor
from tests.helpers import free_port, rendezvous

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CASE = [c for c in cases.CASES if c["id"] == "llama3_70b_w8"][0]   # 30 small files


def _expected(paths):
    want = {}
    for p in paths:
        fo = st_oracle.FileOracle(p)
        for n, e in fo.tensors.items():
            want[n] = (list(e["shape"]), digest_bytes(fo.raw(n)))
    return want


@pytest.mark.parametrize("producer_thread", [False, True], ids=["native_read_ahead", "producer_thread"])
@pytest.mark.parametrize("queue_size", [-1, 0, 2])
def test_single_rank_yields_every_tensor_once(queue_size, producer_thread, case_files, leak_check):
    paths = sorted(case_files(CASE))
    want = _expected(paths)
    it = fst.ParallelLoader(None, paths, queue_size=queue_size, use_tqdm_on_load=False, device="cpu",
                            nogds=True, max_threads=2, slot_kb=64, producer_thread=producer_thread)
    got = {}
    for key, t in it.iterate_weights():
        assert key not in got
        got[key] = (list(t.shape), digest_tensor(t))
    it.close()
    assert got == want


def test_order_follows_files_then_keys(case_files, leak_check):
    paths = sorted(case_files(CASE))[:3]
    it = fst.ParallelLoader(None, paths, use_tqdm_on_load=False, device="cpu", nogds=True)
    keys = [k for k, _ in it.iterate_weights()]
    it.close()
    want = []
    for p in paths:   # one rank: one file per batch, keys in data-offset order
        want += list(st_oracle.FileOracle(p).tensors)
    assert keys == want


@pytest.mark.parametrize("producer_thread", [False, True], ids=["native_read_ahead", "producer_thread"])
def test_producer_error_reaches_the_consumer(producer_thread, case_files, tmp_path, leak_check):
    paths = sorted(case_files(CASE))[:2] + [str(tmp_path / "missing.safetensors")]
    it = fst.ParallelLoader(None, paths, use_tqdm_on_load=False, device="cpu", nogds=True, queue_size=2,
                            producer_thread=producer_thread)
    seen = set()
    with pytest.raises(Exception):
        for key, _ in it.iterate_weights():
            seen.add(key)
    it.close()
    # the failure is delivered in order: every tensor of the two good files came first
    want = set()
    for p in paths[:2]:
        want |= set(st_oracle.FileOracle(p).tensors)
    assert seen == want


def test_read_ahead_depth_follows_queue_size(case_files, leak_check):
    """How many batches have their reads queued beyond the one being consumed: none for -1, one
    for 0, queue_size + 1 for N > 0 (the images upstream's queue and producer hold)."""
    paths = sorted(case_files(CASE))[:8]
    for queue_size, ahead in ((-1, 0), (0, 1), (2, 3)):
        it = fst.ParallelLoader(None, paths, queue_size=queue_size, use_tqdm_on_load=False, device="cpu",
                                nogds=True, max_threads=2, slot_kb=64)
        real = it.loader.copy_files_to_device
        submitted = []

        def spy(*a, _real=real, **kw):
            assert kw.get("wait") is False
            submitted.append(1)
            return _real(*a, **kw)

        it.loader.copy_files_to_device = spy
        gen = it.iterate_weights()
        next(gen)                                  # the first tensor of the first batch
        assert len(submitted) == 1 + ahead, queue_size
        gen.close()
        it.close()


@pytest.mark.parametrize("producer_thread", [False, True], ids=["native_read_ahead", "producer_thread"])
def test_consumer_may_stop_early(producer_thread, case_files, leak_check):
    paths = sorted(case_files(CASE))
    it = fst.ParallelLoader(None, paths, queue_size=2, use_tqdm_on_load=False, device="cpu", nogds=True,
                            producer_thread=producer_thread)
    gen = it.iterate_weights()
    next(gen)
    gen.close()            # runs the generator's cleanup: producer stops, queued batches are freed
    it.close()


def test_only_one_producer_is_supported(case_files):
    with pytest.raises(ValueError):
        fst.ParallelLoader(None, case_files(CASE), max_concurrent_producers=2, device="cpu", nogds=True)


def _rank_main(rank, world, paths, port, out_dir, queue_size, backend="gloo"):
    sys.path.insert(0, ROOT)
    rdzv = rendezvous(out_dir, port)
    device = "cpu"
    if backend == "nccl":
        torch.cuda.set_device(rank)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        device = f"cuda:{rank}"
        dist.init_process_group("nccl", init_method=rdzv, rank=rank, world_size=world, device_id=torch.device(device))
    else:
        dist.init_process_group("gloo", init_method=rdzv, rank=rank, world_size=world)
    it = fst.ParallelLoader(dist.group.WORLD, paths, queue_size=queue_size, use_tqdm_on_load=False,
                            device=device, nogds=True, max_threads=2, slot_kb=64)
    got = {}
    for key, t in it.iterate_weights():
        got[key] = (list(t.shape), digest_tensor(t))
    it.close()
    assert get_framework_op("pytorch").get_mem_used() == 0
    assert cpp.get_cpp_metrics().bounce_buffer_bytes == 0
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(got, f)
    dist.destroy_process_group()


@pytest.mark.parametrize("queue_size", [0, 1])
def test_two_ranks_every_rank_gets_every_tensor(queue_size, case_files, tmp_path):
    paths = sorted(case_files(CASE))[:7]          # odd count: the last batch has one file only
    want = {k: list(v) for k, v in _expected(paths).items()}
    mp.spawn(_rank_main, args=(2, paths, free_port(), str(tmp_path), queue_size), nprocs=2, join=True)
    for rank in range(2):
        got = json.load(open(tmp_path / f"rank{rank}.json"))
        assert got == want, rank


def test_auto_loader_reads_its_configuration(case_files, tmp_path, monkeypatch, leak_check):
    """AutoLoader: settings come from $FASTSAFETENSORS_CONFIG (upstream docs/configuration.md)."""
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps({
        "loader": "base", "base": {"copier_type": "nogds", "max_threads": 2, "debug_log": True},
        "parallel": {"use_pipeline": True, "queue_size": 1, "use_tqdm_on_load": False, "bogus": 1},
        "debug": {"set_numa": False}, "unknown": 3,
    }))
    monkeypatch.setenv("FASTSAFETENSORS_CONFIG", str(cfg))
    paths = sorted(case_files(CASE))[:4]
    it = fst.AutoLoader(None, paths, device="cpu")
    assert it.config.queue_size == 1 and it.config.use_pipeline and it.config.set_numa is False
    assert it.config.get_extension_config("base") == {"copier_type": "nogds", "max_threads": 2}
    got = {k: (list(t.shape), digest_tensor(t)) for k, t in it.iterate_weights()}
    it.close()
    assert got == _expected(paths)
    monkeypatch.setenv("FASTSAFETENSORS_CONFIG", str(tmp_path / "nope.json"))
    with pytest.raises(FileNotFoundError):
        fst.load_config()
    monkeypatch.delenv("FASTSAFETENSORS_CONFIG")
    assert fst.load_config().create_parallel_kwargs() == {"queue_size": -1}
    with pytest.raises(ValueError):
        fst.LoaderConfig(max_concurrent_producers=2)


def test_no_group_means_batches_of_one_file():
    """``pg=None`` is a single process whatever the loader object is (upstream
    parallel_loader.py:150-159 sizes its batches from the ``pg`` argument)."""
    from unittest.mock import MagicMock

    from fastsafetensors_b200.parallel_loader import PipelineParallel

    pipeline = PipelineParallel(None, MagicMock(), ["a.safetensors", "b.safetensors"])
    assert pipeline.weight_files_batches == [["a.safetensors"], ["b.safetensors"]]
    assert pipeline.need_clone is True
