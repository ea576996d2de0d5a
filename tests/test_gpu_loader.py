"""File -> HBM through the native reader and the loader API, on a GPU, checked against the file
bytes, the oracle and upstream's recorded outputs."""

import errno
import os
from collections import OrderedDict

import numpy as np
import pytest
import torch

import fastsafetensors_b200 as fst
from fastsafetensors_b200 import _native as nat
from fastsafetensors_b200 import cpp, shard_plan
from fastsafetensors_b200.batch import BatchLayout
from oracle import st_oracle
from tests.golden import cases
from tests.helpers import digest_bytes, record, tensor_bytes

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def blob_file(tmp_path_factory):
    rng = np.random.default_rng(11)
    data = rng.integers(0, 256, 37 * (1 << 20) + 4321, dtype=np.uint8)
    p = tmp_path_factory.mktemp("blob") / "blob.bin"
    p.write_bytes(data.tobytes())
    return str(p), data


@pytest.mark.parametrize("io_mode", [nat.IO_DIRECT, nat.IO_BUFFERED, nat.IO_AUTO])
@pytest.mark.parametrize("offset", [0, 4096, 8 + 1, 8 + 4567, 123456 + 8])
@pytest.mark.parametrize("plain_dma_only", [False, True])
def test_reader_to_hbm(blob_file, io_mode, offset, plain_dma_only, leak_check):
    """Even offsets take the plain DMA, odd ones the staging ring + realign kernel (or, with
    plain_dma_only, a DMA to an unaligned address).  Slots of 1 MiB force many windows."""
    path, data = blob_file
    length = data.size - offset
    before = cpp.get_cpp_metrics()
    reader = cpp.Reader(0, 4, 1 << 20, 2, io_mode=io_mode, copy_streams=2, plain_dma_only=plain_dma_only)
    try:
        dst = torch.full((length + 512,), 0x5A, dtype=torch.uint8, device=DEV)
        buf = cpp.gds_device_buffer(dst.data_ptr(), dst.numel(), True)
        rid = reader.submit(path, offset, length, buf, 256)
        assert reader.wait(rid, 60000) == length
        got = dst.cpu().numpy()
        assert np.array_equal(got[256:256 + length], data[offset:])
        assert (got[:256] == 0x5A).all() and (got[256 + length:] == 0x5A).all()
        after = cpp.get_cpp_metrics()
        assert after.bytes_h2d - before.bytes_h2d == length
        realigned = after.bytes_realigned - before.bytes_realigned
        if offset % 16 == 0 or plain_dma_only:
            assert realigned == 0
        else:
            assert realigned == length
            assert after.staging_device_bytes > 0
    finally:
        reader.close()
    assert cpp.get_cpp_metrics().staging_device_bytes == 0


def test_reader_failure_is_reported_and_reader_survives(blob_file, leak_check):
    path, data = blob_file
    reader = cpp.Reader(0, 2, 1 << 20, 2, io_mode=nat.IO_BUFFERED)
    try:
        dst = torch.zeros(8 << 20, dtype=torch.uint8, device=DEV)
        buf = cpp.gds_device_buffer(dst.data_ptr(), dst.numel(), True)
        reader.inject_fault(4, errno.EIO)
        with pytest.raises(nat.NativeError) as e:
            reader.wait(reader.submit(path, 0, 8 << 20, buf, 0))
        assert e.value.code == nat.EIO
        assert reader.wait(reader.submit(path, 3, 1 << 20, buf, 0)) == 1 << 20
        assert np.array_equal(dst[: 1 << 20].cpu().numpy(), data[3: 3 + (1 << 20)])
    finally:
        reader.close()


# ------------------------------------------------------------------ loader on cuda, one rank
SINGLE = [c for c in cases.CASES if c["world"] == 1]


@pytest.mark.parametrize("case", SINGLE, ids=[c["id"] for c in SINGLE])
def test_loader_cuda_single_rank_matches_upstream(case, golden, case_files, leak_check):
    paths = case_files(case)
    want = golden["cases"][case["id"]][0]
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), torch.device(DEV), nogds=case.get("nogds", True),
                                       max_threads=4, slot_kb=64)
    loader.add_filenames({0: paths})
    fb = loader.copy_files_to_device()
    got = {}
    for step in case["steps"]:
        if step[0] == "plan":
            for name, action in cases.plan(case):
                if action[0] == "shard":
                    t = fb.get_sharded(name, action[1])
                elif action[0] == "replicate":
                    t = fb.get_tensor(name)
                else:
                    t = fb.push_tensor(name, 0)
                assert t.is_cuda
                got[name] = record(t)
        elif step[0] == "multi_cols":
            got[step[1]] = record(fb.get_multi_cols(step[2], step[3]))
    assert got == want
    fb.close()
    loader.close()


def test_odd_header_goes_through_the_realign_kernel(case_files, leak_check):
    """llama2-13b twin: header length is odd, so host and device addresses are never congruent
    modulo 16 and every window is shifted by the kernel; tensors stay byte-identical."""
    case = [c for c in cases.CASES if c["id"] == "llama2_13b_w4"][0]
    paths = case_files(case)
    before = cpp.get_cpp_metrics()
    with fst.fastsafe_open(paths, device=DEV, nogds=True) as f:
        mid = cpp.get_cpp_metrics()
        total = sum(os.path.getsize(p) - st_oracle.FileOracle(p).header_length for p in paths)
        assert mid.bytes_realigned - before.bytes_realigned == total
        for p in paths:
            fo = st_oracle.FileOracle(p)
            assert fo.header_length % 2 == 1
            for name in fo.tensors:
                t = f.get_tensor(name)
                assert t.data_ptr() % 2 == 0
                assert digest_bytes(tensor_bytes(t)) == digest_bytes(fo.raw(name)), name


# ------------------------------------------------------------------ owner-side packing for W ranks
MULTI = [c for c in cases.CASES if c["world"] > 1 and c["steps"][0][0] == "plan"]


@pytest.mark.parametrize("case", MULTI, ids=[c["id"] for c in MULTI])
def test_owner_packing_for_all_ranks_matches_upstream(case, golden, case_files, leak_check):
    """One GPU plays every owner in turn: for each file it builds the batch layout of the whole
    plan, fills all W outgoing regions with the gather kernel, and each region must hold exactly
    what upstream delivered to that rank (the transport that follows only moves the regions)."""
    paths = sorted(case_files(case))
    world = case["world"]
    plan = OrderedDict((n, (a[0], a[1] % world) if a[0] == "push" else a) for n, a in cases.plan(case))
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), DEV, nogds=True, max_threads=4, slot_kb=256)
    loader.add_filenames({0: paths})
    fb = loader.copy_files_to_device()
    layout = BatchLayout(world)
    frames, src_addr = {}, {}
    for name, action in plan.items():
        _, lidx = fb.key_to_rank_lidx[name]
        factory = fb.rank_loaders[0][lidx]
        frames[name] = factory.metadata.tensors[name]
        src_addr[name] = factory.tensors[name].data_ptr()
        layout.add(name, frames[name], lidx % world, action)
    stream = int(torch.cuda.current_stream().cuda_stream)
    for owner in range(world):
        sizes = layout.region_bytes[owner]
        buf = torch.zeros(max(1, sum(sizes)), dtype=torch.uint8, device=DEV)
        region = [buf.data_ptr() + sum(sizes[:d]) for d in range(world)]
        mine = {n: f for n, f in frames.items() if layout.where[n][0] == owner}
        nat.gather(layout.fill_ops(owner, mine, src_addr, region), stream, (0, 0), (buf.data_ptr(), buf.numel()))
        host = buf.cpu().numpy()
        for dst in range(world):
            base = sum(sizes[:dst])
            for slot in layout.slots[owner][dst]:
                rec = golden["cases"][case["id"]][dst][slot.name]
                assert rec is not None and rec[0] == slot.shape, slot.name
                assert digest_bytes(host[base + slot.offset: base + slot.offset + slot.nbytes]) == rec[2], \
                    (slot.name, owner, dst)
    fb.close()
    loader.close()


@pytest.mark.parametrize("case", MULTI, ids=[c["id"] for c in MULTI])
def test_shard_locally_with_deferred_reads_matches_upstream(case, golden, case_files, leak_check):
    """The end-to-end call sequence of the benchmark on one GPU: reads queued without waiting,
    ``shard_locally`` working through the files in read order, one gather launch per file; every
    destination's tensors must be what upstream delivered to that rank."""
    if case["steps"][0][0] != "plan":
        pytest.skip("case has no whole-checkpoint plan")
    paths = sorted(case_files(case))
    world = case["world"]
    plan = OrderedDict((n, (a[0], a[1] % world) if a[0] == "push" else a) for n, a in cases.plan(case))
    before = cpp.get_cpp_metrics()
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), DEV, nogds=True, max_threads=4, slot_kb=64)
    loader.add_filenames({0: paths})
    fb = loader.copy_files_to_device(wait=False)
    assert all(f.pending for f in fb.rank_loaders[0])
    per_rank = fb.shard_locally(plan, world)
    assert not any(f.pending for f in fb.rank_loaders[0])
    launches = cpp.get_cpp_metrics().kernel_launches - before.kernel_launches
    for rank, tensors in enumerate(per_rank):
        want = {k: v for k, v in golden["cases"][case["id"]][rank].items() if v is not None}
        assert {k: record(v) for k, v in tensors.items()} == want, rank
    assert launches >= len(paths)          # at least one gather launch per file
    del per_rank, tensors
    fb.close()
    loader.close()


@pytest.mark.parametrize("shape,dim,world", [
    ((4096, 14336), 1, 8),     # Llama-3-8B down_proj
    ((14336, 4096), 0, 8),     # Llama-3-8B gate/up
    ((8192, 28672), 1, 8),     # Llama-3-70B down_proj, 7 KiB segments at 56 KiB pitch
    ((8192, 8192), 1, 8),      # Llama-3-70B o_proj, 2 KiB segments
    ((128256, 8192), 0, 8),    # Llama-3-70B embed_tokens / lm_head, 2.1 GB
    ((5120, 13824), 1, 4),     # Llama-2-13B down_proj (fp16)
    ((4096, 14336), 1, 1),     # Mixtral w2 pushed whole
])
def test_full_size_tensors_by_properties(shape, dim, world):
    """Tensors at the benchmark configurations' real sizes (too big for the golden file): the
    pack must equal ``torch.chunk`` of the same tensor bit for bit, preserve the checksum of
    checksums, and agree with the oracle on a sample of rows."""
    bits = 16
    g = torch.Generator(device=DEV).manual_seed(5)
    t = torch.randint(0, 1 << 15, shape, dtype=torch.int16, device=DEV, generator=g)
    n = t.numel() * 2
    ops, shard_bytes = shard_plan.scatter_ops(t.data_ptr(), 0, shape, bits, dim, world)
    packed = torch.empty(n, dtype=torch.uint8, device=DEV)
    nat.gather([(o[0], o[1] + packed.data_ptr()) + o[2:] for o in ops],
               int(torch.cuda.current_stream().cuda_stream), (t.data_ptr(), n), (packed.data_ptr(), n))
    assert int(packed.view(torch.int64).sum()) == int(t.view(torch.int64).sum())  # checksum of checksums
    want = torch.cat([c.contiguous().reshape(-1) for c in t.chunk(world, dim=dim)])
    assert torch.equal(packed.view(torch.int16), want)
    if dim == 1:
        raw = t[:64].cpu().numpy().view(np.uint8).reshape(-1)
        got0 = packed[: shard_bytes].view(torch.int16).reshape(shape[0], -1)[:64].cpu().numpy().view(np.uint8).reshape(-1)
        want0, _ = st_oracle.shard(raw, (64, shape[1]), "BF16", 1, 0, world)
        assert np.array_equal(got0, want0)


# ------------------------------------------------------------------ load-time narrowing
def test_convert_kernel_matches_torch_bit_for_bit():
    """fst_convert against torch.Tensor.to on the same device, including ties, denormals,
    infinities and values that overflow the target."""
    g = torch.Generator(device=DEV).manual_seed(9)
    n = (1 << 20) + 37
    base = torch.randn(n, device=DEV, generator=g) * 3.0
    special = torch.tensor([0.0, -0.0, 1.0, 65504.0, 65520.0, 1e-8, -1e-8, 3.3895e38, float("inf"),
                            -float("inf"), 1.00390625, 1.001953125, 2.0 ** -24, 2.0 ** -25, 1e30],
                           device=DEV)
    src32 = torch.cat([base, special, base * 1e-6, base * 1e6])
    stream = int(torch.cuda.current_stream().cuda_stream)
    cases_ = [(src32, "F32", torch.float16, "F16"), (src32, "F32", torch.bfloat16, "BF16"),
              (src32.double() * 1.0000001, "F64", torch.float32, "F32"),
              (src32.double(), "F64", torch.bfloat16, "BF16"), (src32.double(), "F64", torch.float16, "F16"),
              (src32.half(), "F16", torch.bfloat16, "BF16"), (src32.bfloat16(), "BF16", torch.float16, "F16")]
    for src, s_name, dst_t, d_name in cases_:
        for shift in (0, 1):          # shift 1 element: the unaligned (element-wise) path
            s = src[shift:]
            want = s.to(dst_t)
            got = torch.empty(s.numel() + 8, dtype=dst_t, device=DEV)[shift: shift + s.numel()]
            nat.convert([(s.data_ptr(), got.data_ptr(), s.numel(), nat.DT_CODES[s_name], nat.DT_CODES[d_name])], stream)
            torch.cuda.synchronize()
            a = got.view(torch.int16 if dst_t != torch.float32 else torch.int32)
            b = want.view(a.dtype)
            assert torch.equal(a, b), (s_name, d_name, shift)
    with pytest.raises(nat.NativeError):
        nat.convert([(src32.data_ptr(), src32.data_ptr() + 4, 10, 1, 3)], stream)       # overlap
    with pytest.raises(nat.NativeError):
        nat.convert([(src32.data_ptr(), base.data_ptr(), 10, 2, 1)], stream)            # widening


def test_loader_narrowing_on_cuda_matches_torch(tmp_path, leak_check):
    from safetensors.torch import save_file

    from fastsafetensors_b200.st_types import DType

    torch.manual_seed(1)
    t = {"w": torch.randn(300, 257), "v": torch.randn(5), "h": torch.randn(64, 64).half(),
         "b": torch.randn(33, 3).bfloat16(), "i": torch.randint(-100, 100, (7, 9), dtype=torch.int32)}
    p = str(tmp_path / "mixed.safetensors")
    save_file(t, p)
    loader = fst.SafeTensorsFileLoader(None, DEV, nogds=True)
    loader.add_filenames({0: [p]})
    fb = loader.copy_files_to_device(dtype=DType.BF16)
    for k, ref in t.items():
        got = fb.get_tensor(k)
        assert got.dtype == torch.bfloat16 and got.is_cuda
        assert torch.equal(got.cpu().view(torch.int16), ref.to(DEV).to(torch.bfloat16).cpu().view(torch.int16)), k
    fb.close()
    loader.close()
    loader = fst.SafeTensorsFileLoader(None, DEV, nogds=True)
    loader.add_filenames({0: [p]})
    with pytest.raises(Exception, match="larger sizes"):
        loader.copy_files_to_device(dtype=DType.F64)
    loader.close()


# ------------------------------------------------------------------ cuFile window source
# NVIDIA's libcufile itself: only where GPUDirect Storage proper can work (the nvidia-fs module is
# loaded) AND the run asks for it.  Elsewhere the library refuses cuFile before opening its driver
# (tests/test_gpu_cufile.py checks that, and runs the code path through a host-side double).
def _real_cufile_allowed() -> bool:
    return os.environ.get("FST_TEST_CUFILE") == "1" and bool(cpp.is_gds_supported(0))


needs_cufile = pytest.mark.skipif(not _real_cufile_allowed(),
                                  reason="needs the nvidia-fs module and FST_TEST_CUFILE=1")


@needs_cufile
@pytest.mark.parametrize("offset", [0, 4096, 8 + 1, 123456 + 8])
def test_reader_cufile_mode(blob_file, offset, leak_check):
    """io_mode cufile: cuFileRead lands windows in the registered device staging ring, the
    realign kernel places them.  Where cuFile cannot be used at all the reader must say so with
    an error that names "gds" (callers fall back on that), and the test is skipped."""
    path, data = blob_file
    length = data.size - offset
    if not cpp.is_cufile_found():
        pytest.skip("libcufile.so is not installed")
    reader = cpp.Reader(0, 4, 1 << 20, 2, io_mode=nat.IO_CUFILE, copy_streams=2)
    try:
        dst = torch.full((length + 512,), 0x5A, dtype=torch.uint8, device=DEV)
        buf = cpp.gds_device_buffer(dst.data_ptr(), dst.numel(), True)
        try:
            rid = reader.submit(path, offset, length, buf, 256)
        except nat.NativeError as e:
            assert e.code == nat.EGDS and "gds" in str(e)
            pytest.skip(f"cuFile is not usable on this machine: {e}")
        assert reader.wait(rid, 120000) == length
        got = dst.cpu().numpy()
        assert np.array_equal(got[256:256 + length], data[offset:])
        assert (got[:256] == 0x5A).all() and (got[256 + length:] == 0x5A).all()
    finally:
        reader.close()
    assert cpp.get_cpp_metrics().staging_device_bytes == 0


@needs_cufile
def test_loader_with_cufile_matches_upstream(golden, case_files, leak_check):
    case = [c for c in cases.CASES if c["id"] == "llama2_13b_w1_gds"][0]   # odd headers
    paths = case_files(case)
    if not cpp.is_cufile_found():
        pytest.skip("libcufile.so is not installed")
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), DEV, nogds=False, io_mode="cufile", max_threads=4,
                                       slot_kb=256)
    loader.add_filenames({0: paths})
    try:
        fb = loader.copy_files_to_device()
    except RuntimeError as e:
        assert "gds" in str(e)
        loader.close()
        pytest.skip(f"cuFile is not usable on this machine: {e}")
    got = {name: record(fb.get_tensor(name)) for name, _ in cases.plan(case)}
    assert got == golden["cases"][case["id"]][0]
    fb.close()
    loader.close()


# ------------------------------------------------------------------ stream order of image reuse
def test_reader_waits_for_pending_readers_of_reused_memory(tmp_path, leak_check):
    """An image freed while a gather that reads it is still queued goes back to torch's allocator
    and is handed to the next file image at once.  The reader fills that image from its own copy
    streams, so it has to queue behind the caller's stream first (fst_reader_order_after);
    otherwise its DMA overwrites bytes the pending gather has yet to read."""
    from tests import synth

    n = 192 << 20
    specs = []
    for k, seed in enumerate((21, 22)):
        spec = synth.CheckpointSpec(f"reuse{k}", [synth.TensorSpec(f"w{k}", "U8", (n,), ("replicate",))], 1, seed)
        specs.append((spec, synth.write_checkpoint(spec, str(tmp_path / f"c{k}"), fsync=False)[0]))
    want = [synth.expected_bytes(s, 0) for s, _ in specs]
    assert not np.array_equal(want[0], want[1])
    torch.cuda.empty_cache()
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), DEV, nogds=True, max_threads=8)
    loader.add_filenames({0: [specs[0][1]]})
    fb = loader.copy_files_to_device()
    t = fb.get_tensor("w0")
    first_ptr = t.data_ptr()
    out = torch.empty(n, dtype=torch.uint8, device=DEV)
    # keep the stream busy for a while (large matmuls), then the gather that reads image 0
    a = torch.randn(8192, 8192, device=DEV, dtype=torch.bfloat16)
    for _ in range(150):
        a = (a @ a).clamp_(-1, 1)
    nat.gather([(t.data_ptr(), out.data_ptr(), 1, n, 0, 0)], int(torch.cuda.current_stream().cuda_stream),
               (t.data_ptr(), n), (out.data_ptr(), n))
    del t
    fb.close()                        # image 0 goes back to the allocator with the gather pending
    loader.reset()
    loader.add_filenames({0: [specs[1][1]]})
    fb = loader.copy_files_to_device()    # same size: the allocator hands out the same block
    t1 = fb.get_tensor("w1")
    reused = t1.data_ptr() == first_ptr
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), want[0]), "the pending gather read bytes of the next file"
    assert np.array_equal(t1.cpu().numpy(), want[1])
    del t1
    fb.close()
    loader.close()
    if not reused:
        pytest.skip("the allocator did not hand out the same block: the hazard was not exercised")


def test_legacy_device_helpers():
    """gpu_malloc / gpu_free / memcpy_h2d_async of upstream's module API."""
    addr = cpp.gpu_malloc(1 << 20)
    assert addr
    host = cpp.cpu_malloc(1 << 20)
    src = (np.arange(1 << 20) % 251).astype(np.uint8)
    import ctypes

    ctypes.memmove(host, src.ctypes.data, src.size)
    assert cpp.memcpy_h2d_async(addr, host, src.size) == 0
    torch.cuda.synchronize()

    class _Span:
        __cuda_array_interface__ = {"shape": (src.size,), "typestr": "|u1", "data": (addr, False), "version": 2}

    got = torch.as_tensor(_Span(), device=DEV).cpu().numpy()
    assert np.array_equal(got, src)
    cpp.gpu_free(addr)
    cpp.cpu_free(host)


def test_gather_refuses_wrapping_address_arithmetic():
    src = torch.zeros(4096, dtype=torch.uint8, device=DEV)
    dst = torch.zeros(4096, dtype=torch.uint8, device=DEV)
    s, d = src.data_ptr(), dst.data_ptr()
    huge = (1 << 64) - 4096
    for op in ((s, d, 3, 16, huge, 16), (s, d, 2, 16, 16, huge), (s, d, (1 << 63), 16, 16, 16)):
        for entry in (nat.gather, nat.gather_static):
            with pytest.raises(nat.NativeError) as e:
                entry([op], 0, (s, 4096), (d, 4096))
            assert e.value.code == nat.ERANGE, op
