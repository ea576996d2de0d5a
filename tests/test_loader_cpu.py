"""Host logic and the loader's CPU mode (device "cpu"), checked against upstream's recorded
outputs and against the oracle.  No GPU needed."""

import itertools
import json
import os
import struct
from collections import OrderedDict

import numpy as np
import pytest
import torch

import fastsafetensors_b200 as fst
from fastsafetensors_b200 import _native as nat
from fastsafetensors_b200 import shard_plan
from fastsafetensors_b200.frameworks import get_framework_op
from fastsafetensors_b200.st_types import DType
from oracle import st_oracle
from tests.golden import cases
from tests.helpers import digest_bytes, record, tensor_bytes

FW = get_framework_op("pytorch")


# ------------------------------------------------------------------ TensorFrame
def _frame(shape):
    return fst.TensorFrame.from_buffer({"dtype": "F16", "shape": list(shape), "data_offsets": [0, 0]})


def test_tensor_frame_matches_upstream_vectors(golden):
    for rec in golden["frames"]:
        shape, expr = rec[0], rec[1]
        index = eval(expr, {"slice": slice})
        if len(rec) == 3:
            with pytest.raises({"IndexError": IndexError, "ValueError": ValueError}[rec[2]]):
                _frame(shape)[index]
        else:
            got = _frame(shape)[index]
            assert [got.shape, got.strides, got.offsets] == rec[2:], expr


def test_tensor_frame_matches_python_sequences():
    """Exhaustive 1-d check against list slicing (upstream test_fastsafetensors.py:799-849)."""
    n = 7
    ref = list(range(n))
    vals = [None] + list(range(-n - 2, n + 3))
    for start, stop, step in itertools.product(vals, vals, [None, 1, 2, 3, -1, -2, -3]):
        got = _frame((n, 2))[slice(start, stop, step)]
        want = ref[slice(start, stop, step)]
        if not want:
            assert got.shape == []
            continue
        assert got.shape == [len(want), 2]
        assert got.offsets[0] == want[0]
        assert got.strides[0] == 2 * (step or 1)
    with pytest.raises(ValueError):
        _frame((n,))[slice(0, 3, 0)]
    with pytest.raises(Exception):
        _frame((n,))[slice(None), slice(None)]


# ------------------------------------------------------------------ header validation
def _blob(doc, extra=b""):
    body = json.dumps(doc).encode()
    return struct.pack("<Q", len(body)) + body + extra


@pytest.mark.parametrize("blob,word", [
    (b"\0" * 7, "HeaderTooSmall"),
    (struct.pack("<Q", 100_000_001) + b"{}" * 8, "HeaderTooLarge"),
    (struct.pack("<Q", 500) + b"{}", "InvalidHeaderLength"),
    (_blob({"a": {"dtype": "F16", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 3), "MetadataIncompleteBuffer"),
    (_blob({"a": {"dtype": "F16", "shape": [2], "data_offsets": [1, 5]}}, b"\0" * 8), "InvalidOffset"),
    (_blob({"a": {"dtype": "F16", "shape": [3], "data_offsets": [0, 4]}}, b"\0" * 8), "TensorInvalidInfo"),
])
def test_header_errors(tmp_path, blob, word):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(blob)
    with pytest.raises(Exception, match=word):
        fst.SafeTensorsMetadata.from_file(str(p), FW)
    arr = np.frombuffer(blob, dtype=np.uint8).copy()
    with pytest.raises(Exception, match=word):
        fst.SafeTensorsMetadata.from_buffer(arr.ctypes.data, arr.size, "mem", FW)


def test_header_matches_oracle(case_files):
    for case in cases.CASES[:4]:
        for path in case_files(case):
            meta = fst.SafeTensorsMetadata.from_file(path, FW)
            hl, tensors, md = st_oracle.parse_header(open(path, "rb").read())
            assert meta.header_length == hl
            assert list(meta.tensors) == list(tensors)
            assert meta.metadata == md
            for n, e in tensors.items():
                f = meta.tensors[n]
                assert (f.dtype.value, f.shape, f.data_offsets) == (e["dtype"], e["shape"], e["data_offsets"])


# ------------------------------------------------------------------ shard geometry
@pytest.mark.parametrize("shape,dtype,dim,world", [
    ((16, 12), "F16", 0, 4), ((16, 12), "F16", 1, 4), ((4, 6, 8), "F32", 1, 3), ((4, 6, 8), "F32", 2, 8),
    ((2, 4, 6), "BF16", 2, 2), ((8,), "I64", 0, 8), ((6, 10), "U8", 1, 5), ((6, 10), "F4", 1, 5),
    ((5, 7, 3, 4), "F64", 2, 3),
])
def test_scatter_ops_match_oracle(shape, dtype, dim, world):
    bits = st_oracle.BITS[dtype]
    n = int(np.prod(shape)) * bits // 8
    src = np.random.default_rng(n).integers(0, 256, n, dtype=np.uint8)
    ops, shard_bytes = shard_plan.scatter_ops(src.ctypes.data, 0, shape, bits, dim, world)
    packed = np.zeros(shard_bytes * world, dtype=np.uint8)
    nat.gather_host([(o[0], o[1] + packed.ctypes.data) + o[2:] for o in ops], 2)
    for r in range(world):
        want, _ = st_oracle.shard(src, shape, dtype, dim, r, world)
        assert np.array_equal(packed[r * shard_bytes:(r + 1) * shard_bytes], want), r


def test_multi_col_ops_match_oracle():
    shapes = [(6, 8), (6, 4), (6, 12)]
    raws = [np.random.default_rng(i).integers(0, 256, int(np.prod(s)) * 2, dtype=np.uint8) for i, s in enumerate(shapes)]
    for world in (1, 2, 4):
        ops, per_rank, shape = shard_plan.multi_col_ops([r.ctypes.data for r in raws], 0, shapes, 16, 1, world)
        packed = np.zeros(per_rank * world, dtype=np.uint8)
        nat.gather_host([(o[0], o[1] + packed.ctypes.data) + o[2:] for o in ops], 1)
        for r in range(world):
            want, want_shape = st_oracle.multi_cols(raws, shapes, "F16", 1, r, world)
            assert shape == want_shape
            assert np.array_equal(packed[r * per_rank:(r + 1) * per_rank], want)


def test_uneven_split_is_refused():
    with pytest.raises(ValueError):
        shard_plan.check_even_split("t", 10, 4)
    with pytest.raises(ValueError):  # F4 columns must split on byte boundaries
        shard_plan.scatter_ops(4096, 0, (2, 6), 4, 1, 2)


# ------------------------------------------------------------------ loader, one rank, device cpu
SINGLE = [c for c in cases.CASES if c["world"] == 1]


@pytest.mark.parametrize("case", SINGLE, ids=[c["id"] for c in SINGLE])
@pytest.mark.parametrize("io_mode", ["auto", "direct"])
def test_loader_cpu_single_rank_matches_upstream(case, io_mode, golden, case_files, leak_check):
    paths = case_files(case)
    want = golden["cases"][case["id"]][0]
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), "cpu", nogds=case.get("nogds", True),
                                       io_mode=io_mode, max_threads=4, slot_kb=64)
    loader.add_filenames({0: paths})
    fb = loader.copy_files_to_device()
    got = {}
    for step in case["steps"]:
        if step[0] == "plan":
            for name, action in cases.plan(case):
                if action[0] == "shard":
                    got[name] = record(fb.get_sharded(name, action[1]))
                elif action[0] == "replicate":
                    got[name] = record(fb.get_tensor(name))
                else:
                    got[name] = record(fb.push_tensor(name, 0))
        elif step[0] == "multi_cols":
            got[step[1]] = record(fb.get_multi_cols(step[2], step[3]))
    assert got == want
    assert list(fb.key_to_rank_lidx) == loader.get_keys() or set(fb.key_to_rank_lidx) == set(loader.get_keys())
    fb.close()
    loader.close()


def test_fastsafe_open_forms_and_metadata(case_files, leak_check):
    case = cases.CASES[0]
    path = case_files(case)[0]
    fo = st_oracle.FileOracle(path)
    for arg in (path, [path], {0: [path]}):
        with fst.fastsafe_open(arg, framework="pt", device="cpu", nogds=True) as f:
            assert f.metadata()[path] == fo.metadata
            assert sorted(f.keys()) == sorted(fo.tensors)
            for k in list(f.keys())[:5]:
                assert digest_bytes(tensor_bytes(f.get_tensor(k))) == digest_bytes(fo.raw(k))


def test_duplicate_keys_across_files_are_refused(tmp_path, case_files):
    import shutil

    path = case_files(cases.CASES[0])[0]
    twin = str(tmp_path / "twin.safetensors")
    shutil.copy(path, twin)
    loader = fst.SafeTensorsFileLoader(None, "cpu", nogds=True)
    loader.add_filenames({0: [path, twin]})
    with pytest.raises(Exception, match="must be unique"):
        loader.copy_files_to_device()
    loader.close()
    assert FW.get_mem_used() == 0


def test_narrowing_dtype_conversion(tmp_path, leak_check):
    from safetensors.torch import save_file

    t = {"w": torch.randn(8, 16), "v": torch.randn(5)}
    p = str(tmp_path / "f32.safetensors")
    save_file(t, p)
    loader = fst.SafeTensorsFileLoader(None, "cpu", nogds=True)
    loader.add_filenames({0: [p]})
    fb = loader.copy_files_to_device(dtype=DType.BF16)
    for k in t:
        got = fb.get_tensor(k)
        assert got.dtype == torch.bfloat16
        assert torch.equal(got, t[k].to(torch.bfloat16))
    fb.close()
    loader.close()
    loader = fst.SafeTensorsFileLoader(None, "cpu", nogds=True)
    loader.add_filenames({0: [p]})
    with pytest.raises(Exception, match="larger sizes"):
        loader.copy_files_to_device(dtype=DType.F64)
    loader.close()


def test_auto_free_after_last_tensor(case_files, leak_check):
    """Upstream regression (test_fastsafetensors.py:852-894): with auto_mem_delete each file is
    freed when, and only when, all of its own tensors were requested."""
    case = [c for c in cases.CASES if c["id"] == "crafted_w1"][0]
    paths = case_files(case)
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), "cpu", nogds=True)
    loader.add_filenames({0: paths})
    fb = loader.copy_files_to_device()
    fb.auto_mem_delete = True
    names0 = [n for (f, n, *_rest) in cases.CRAFTED if f == 0]
    names1 = [n for (f, n, *_rest) in cases.CRAFTED if f == 1]
    for n in names0[:-1]:
        fb.get_tensor(n)
    assert fb.rank_loaders[0][0].gbuf is not None
    fb.get_multi_cols([names0[-1]], dim=0)
    assert fb.rank_loaders[0][0].gbuf is None and fb.rank_loaders[0][1].gbuf is not None
    fb.as_dict(OrderedDict((n, -1) for n in names1[:2]))
    assert fb.rank_loaders[0][1].gbuf is not None
    fb.close()
    loader.close()


def test_missing_key_and_missing_file():
    loader = fst.SafeTensorsFileLoader(None, "cpu", nogds=True)
    with pytest.raises(Exception):
        loader.add_filenames({0: ["/nonexistent/file.safetensors"]})
    loader.close()


MULTI_PLAN = [c for c in cases.CASES if c["world"] > 1 and c["steps"][0][0] == "plan"]


@pytest.mark.parametrize("case", MULTI_PLAN, ids=[c["id"] for c in MULTI_PLAN])
def test_shard_locally_produces_every_ranks_tensors(case, golden, case_files, leak_check):
    """One process owning all files produces what each of W ranks received from upstream."""
    paths = case_files(case)
    world = case["world"]
    plan = OrderedDict((n, (a[0], a[1] % world) if a[0] == "push" else a) for n, a in cases.plan(case))
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), "cpu", nogds=True, max_threads=4, slot_kb=64)
    loader.add_filenames({0: paths})
    fb = loader.copy_files_to_device()
    per_rank = fb.shard_locally(plan, world)
    assert len(per_rank) == world
    for rank, tensors in enumerate(per_rank):
        want = {k: v for k, v in golden["cases"][case["id"]][rank].items() if v is not None}
        assert {k: record(v) for k, v in tensors.items()} == want
    fb.close()
    loader.close()


def test_deferred_wait_overlaps_reads_with_packing(golden, case_files, leak_check):
    """copy_files_to_device(wait=False): the reads are queued, each file is waited for by the
    first access to one of its tensors; shard_locally works through the files in order."""
    case = [c for c in cases.CASES if c["id"] == "llama3_70b_w8"][0]       # 30 files
    paths = case_files(case)
    world = case["world"]
    plan = OrderedDict(cases.plan(case))
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), "cpu", nogds=True, max_threads=2, slot_kb=64)
    loader.add_filenames({0: paths})
    fb = loader.copy_files_to_device(wait=False)
    factories = fb.rank_loaders[0]
    assert all(f.pending for f in factories)
    per_rank = fb.shard_locally(plan, world)
    assert not any(f.pending for f in factories)
    for rank, tensors in enumerate(per_rank):
        want = {k: v for k, v in golden["cases"][case["id"]][rank].items() if v is not None}
        assert {k: record(v) for k, v in tensors.items()} == want
    fb.close()
    # per-tensor access completes just the file it touches; close() drains what is still pending
    loader.reset()
    loader.add_filenames({0: paths})
    fb = loader.copy_files_to_device(wait=False)
    name = next(iter(fb.rank_loaders[0][3].metadata.tensors))
    fo = st_oracle.FileOracle(fb.rank_loaders[0][3].metadata.src)
    assert digest_bytes(tensor_bytes(fb.get_tensor(name))) == digest_bytes(fo.raw(name))
    assert not fb.rank_loaders[0][3].pending and fb.rank_loaders[0][4].pending
    fb.close()
    loader.close()


def test_deferred_wait_reports_a_failed_read_at_first_access(case_files, leak_check):
    import errno

    case = [c for c in cases.CASES if c["id"] == "llama3_8b_w8"][0]
    paths = case_files(case)
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), "cpu", nogds=True, max_threads=1, slot_kb=4)
    loader.add_filenames({0: paths})
    loader.copier_constructor.reader.inject_fault(3, errno.EIO)
    fb = loader.copy_files_to_device(wait=False)           # nothing is raised here
    with pytest.raises(Exception, match="failed"):
        for name in fb.key_to_rank_lidx:
            fb.get_tensor(name)
    fb.close()
    loader.close()


def test_fix_alignment_pads_the_header_only(case_files, tmp_path, leak_check):
    from fastsafetensors_b200.fix_alignment import aligned_copy

    case = [c for c in cases.CASES if c["id"] == "llama2_13b_w4"][0]     # odd header lengths
    src = sorted(case_files(case))[0]
    dst = str(tmp_path / "aligned.safetensors")
    assert aligned_copy(src, dst) is True
    a, b = st_oracle.FileOracle(src), st_oracle.FileOracle(dst)
    assert a.header_length % 16 != 0 and b.header_length % 16 == 0
    assert a.metadata == b.metadata and list(a.tensors) == list(b.tensors)
    for n in a.tensors:
        assert a.tensors[n] == b.tensors[n] and np.array_equal(a.raw(n), b.raw(n))
    assert aligned_copy(dst, str(tmp_path / "again.safetensors")) is False
    with fst.fastsafe_open(dst, device="cpu", nogds=True) as f:
        k = f.keys()[0]
        assert digest_bytes(tensor_bytes(f.get_tensor(k))) == digest_bytes(a.raw(k))
