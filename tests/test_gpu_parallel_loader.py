"""PipelineParallel / ParallelLoader on a CUDA device (upstream parallel_loader.py:284-308,
364-412), in both arrangements: the native reader as producer (reads of the batches ahead queued
without waiting, files waited for at first use), and upstream's producer thread (``add_filenames``
/ ``copy_files_to_device`` / ``reset`` for batch k+1 on one thread while another takes tensors of
batch k and closes it -- native submit and wait from one thread, tensor instantiation and image
release from another)."""

import threading

import pytest
import torch

import fastsafetensors_b200 as fst
from oracle import st_oracle
from tests.golden import cases
from tests.helpers import digest_bytes, digest_tensor

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
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
def test_pipeline_on_cuda_yields_every_tensor_once(queue_size, producer_thread, case_files, leak_check):
    paths = sorted(case_files(CASE))
    want = _expected(paths)
    it = fst.ParallelLoader(None, paths, queue_size=queue_size, use_tqdm_on_load=False, device=DEV,
                            nogds=True, max_threads=4, slot_kb=64, producer_thread=producer_thread)
    got, consumer = {}, threading.get_ident()
    producers = set()
    real_copy = it.loader.copy_files_to_device

    def spy(*a, **kw):
        producers.add(threading.get_ident())
        return real_copy(*a, **kw)

    it.loader.copy_files_to_device = spy
    keep = []
    for key, t in it.iterate_weights():
        assert key not in got and t.is_cuda
        keep.append(t)                       # clones: they outlive their batch's image
        got[key] = (list(t.shape), digest_tensor(t))
    it.close()
    assert got == want
    if producer_thread:
        assert producers and consumer not in producers      # the copies ran on the producer thread
    else:
        assert producers == {consumer}                      # queued from the consumer, read natively
    # tensors kept past the end of their batch still hold their own bytes
    torch.cuda.synchronize()
    for (key, (_, d)), t in zip(got.items(), keep):
        assert digest_tensor(t) == d, key


def test_pipeline_on_cuda_consumer_may_stop_early(case_files, leak_check):
    paths = sorted(case_files(CASE))
    it = fst.ParallelLoader(None, paths, queue_size=2, use_tqdm_on_load=False, device=DEV, nogds=True,
                            max_threads=2, slot_kb=64)
    gen = it.iterate_weights()
    key, t = next(gen)
    assert t.is_cuda
    gen.close()
    it.close()
