"""Benchmark of the safetensors -> HBM load path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload: the Llama-3-8B-shaped bf16 checkpoint (4 files, 16.06 GB of tensor data, synthetic
values), loaded tensor-parallel.  With one GPU the single rank owns every file and packs the
shards of all 8 tensor-parallel ranks (what the owner of a file does before the exchange); with N
GPUs the files are owned round-robin, tensor parallelism is N-way and the shards are exchanged
over NCCL.  One JSON line is printed by rank 0:

* ``value``    GB/s of tensor data sharded per second with the file images already resident in
               HBM (gather kernel + exchange), timed with CUDA events, max over ranks;
* ``e2e``      the same checkpoint from files on disk to shards in HBM through the public loader
               API, page cache dropped before every step (cold reads), wall clock between device
               synchronisations; ``e2e_warm`` is the same with the files in the page cache;
* ``roofline`` the gather kernel against the measured HBM copy bandwidth;
* ``cpu_baseline`` upstream fastsafetensors (CPU, gloo ranks) on a bounded sample.

``--impl reference`` runs upstream's own CPU path (built into ``oracle/_ref``) on the same files.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from collections import OrderedDict

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GB = 1e9
WORKLOAD = "llama3-8b"
L2_BYTES = 126 * (1 << 20)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=("b200", "reference", "reference-cuda"))
    ap.add_argument("--config", default=WORKLOAD)
    ap.add_argument("--scale", default="full", choices=("full", "tiny"))
    ap.add_argument("--dir", default=os.environ.get("FST_BENCH_DIR", "/tmp/fst_bench"))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--warm-only", action="store_true", help="skip the cold end-to-end phase and the storage roofline")
    ap.add_argument("--threads", type=int, default=int(os.environ.get("FST_BENCH_THREADS", 16)),
                    help="reader threads (max_threads of the loader)")
    ap.add_argument("--transport", default=os.environ.get("FST_B200_TRANSPORT", "auto"),
                    choices=("auto", "nccl", "peer"),
                    help="N > 1: all_to_all over NCCL, gather-kernel stores into peer arenas, or the "
                         "library's own choice (peer for two ranks, else NCCL)")
    ap.add_argument("--ref-settings", default="best", choices=("best", "defaults", "tuned"),
                    help="--impl reference: upstream's library defaults, the rule of its perf tool, or "
                         "whichever of the two is faster in one untimed step each")
    ap.add_argument("--ref-budget", type=float, default=150.0,
                    help="--impl reference: seconds the cold phase may take before it is cut to fewer files")
    ap.add_argument("--layers", type=int, default=0,
                    help="keep only the first L transformer layers (small case for profiler captures)")
    ap.add_argument("--other-kernels-only", action="store_true",
                    help="only the stand-alone timing of the realign and convert kernels (for profiler captures)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="only the device-resident phase (for profiler captures)")
    return ap.parse_args()


def dist_env():
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)),
            int(os.environ.get("WORLD_SIZE", 1)))


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [x for x in sm if x > 0.5 * max(mx or [1])] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------
# workload
# ------------------------------------------------------------------------------------------
def plan_for(spec, tp: int) -> "OrderedDict[str, tuple]":
    return OrderedDict((t.name, (t.action[0], t.action[1] % tp) if t.action[0] == "push" else t.action)
                       for t in spec.tensors)


def read_into_page_cache(paths) -> None:
    """Buffered sequential read of every file, so that a following phase finds them cached."""
    for p in paths:
        with open(p, "rb", buffering=0) as f:
            while f.read(64 << 20):
                pass


def load_spec(args):
    """The checkpoint spec of the run; ``--layers L`` cuts it to the first L layers."""
    import re

    from tests import synth

    spec = synth.config(args.config, args.scale)
    if args.layers > 0:
        def keep(name: str) -> bool:
            m = re.search(r"(?:layers|h)\.(\d+)\.", name)
            return m is None or int(m.group(1)) < args.layers
        spec.tensors = [t for t in spec.tensors if keep(t.name)]
        spec.name = f"{spec.name}-first{args.layers}layers"
    return spec


def prepare_files(spec, directory: str, rank: int, barrier) -> list:
    from tests import synth

    out = os.path.join(directory, f"{spec.name}")
    if rank == 0:
        t0 = time.time()
        paths = synth.write_checkpoint(spec, out, fsync=True)
        sys.stderr.write(f"[bench] checkpoint {spec.name}: {len(paths)} files, "
                         f"{spec.data_bytes / GB:.2f} GB in {out} ({time.time() - t0:.1f} s)\n")
    barrier()
    groups = synth.partition(spec)
    return sorted(os.path.join(out, synth.file_name(spec, k, len(groups))) for k in range(len(groups)))


# ------------------------------------------------------------------------------------------
# this repository's arm
# ------------------------------------------------------------------------------------------
def b200_arm(args) -> dict:
    import torch
    import torch.distributed as dist

    import fastsafetensors_b200 as fst
    from fastsafetensors_b200 import _native as nat
    from fastsafetensors_b200 import cpp
    from tests import synth
    from fastsafetensors_b200.batch import PeerArenaUnavailable, PeerShardExchange, ShardExchange
    from fastsafetensors_b200.file_buffer import resolve_transport

    rank, local_rank, world = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the b200 arm has no CPU substitute")
    torch.cuda.set_device(local_rank)
    device = f"cuda:{local_rank}"
    pg = None
    if world > 1:
        import datetime

        dist.init_process_group("nccl", device_id=torch.device(device),
                                timeout=datetime.timedelta(seconds=180))
        pg = dist.group.WORLD

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.other_kernels_only:
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        peak = float(json.load(open(peaks_path))["hbm_gbs"]) if os.path.exists(peaks_path) else 6650.0
        return {"other_kernels": other_kernels(device, peak)} if rank == 0 else {}
    spec = load_spec(args)
    tp = spec.tp if world == 1 else world
    plan = plan_for(spec, tp)
    paths = prepare_files(spec, args.dir, rank, barrier)
    owners = synth.owners(paths, world)
    data_bytes = spec.data_bytes

    def open_loader():
        return fst.SafeTensorsFileLoader(pg if pg is not None else fst.SingleGroup(), torch.device(device),
                                         nogds=True, max_threads=args.threads)

    # "auto" is the library's rule: the fused peer exchange where it measured faster (two ranks),
    # the NCCL all-to-all otherwise, and NCCL on all ranks together if peer mapping is refused
    may_fall_back = False
    if world > 1:
        want = resolve_transport(args.transport, world, fst.Device.from_str(device))
        may_fall_back = want == "auto"
        args.transport = "nccl" if want == "nccl" else "peer"

    def make_exchange(fb) -> ShardExchange:
        if world > 1 and args.transport == "peer":
            try:
                return PeerShardExchange(fb, plan, tp, rank)
            except PeerArenaUnavailable as e:     # every rank gets it at the same call
                if not may_fall_back:
                    raise
                note(f"peer arenas unavailable ({e}); NCCL all-to-all instead")
                args.transport = "nccl"
        return ShardExchange(fb, plan, tp, rank if world > 1 else 0, local=(world == 1))

    def note(msg: str) -> None:
        if rank == 0:
            sys.stderr.write(f"[bench] {time.strftime('%H:%M:%S')} {msg}\n")
            sys.stderr.flush()

    # ---------------------------------------------------------------- device-resident phase
    note("device-resident phase: loading images")
    loader = open_loader()
    loader.add_filenames(owners)
    fb = loader.copy_files_to_device()
    ex = make_exchange(fb)
    stream = torch.cuda.current_stream()
    # clocks are sampled every 200 ms from here to the end of the timed region; the warm-up runs
    # for at least 1.5 s so that the short timed region is bracketed by samples taken under load
    sampler = ClockSampler(local_rank) if rank == 0 else None
    # every rank must run the same number of steps (each step ends in a collective when N > 1):
    # time the first warm-up steps, then agree on how many more fill the 1.5 s
    t_w = time.perf_counter()
    for _ in range(max(3, args.warmup)):
        ex.run()
    torch.cuda.synchronize()
    per_step = (time.perf_counter() - t_w) / max(3, args.warmup)
    extra = 0 if args.kernel_only else int(max_over_ranks(min(2000.0, 1.5 / max(per_step, 1e-6))))
    for i in range(extra):
        ex.run()
        if i % 8 == 7:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    barrier()
    m0 = cpp.get_cpp_metrics()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kernel_events = []
    torch.cuda.synchronize()
    barrier()
    start.record(stream)
    for _ in range(args.steps):
        ex.run(timing=kernel_events)     # an event pair around every gather launch
    stop.record(stream)
    torch.cuda.synchronize()
    barrier()
    m1 = cpp.get_cpp_metrics()
    resident_ms = max_over_ranks(start.elapsed_time(stop)) / args.steps
    kernel_ms_total = sum(a.elapsed_time(b) for a, b in kernel_events)
    n_launch = len(kernel_events)
    launches_timed = m1.kernel_launches - m0.kernel_launches
    payload_per_step = ex.payload_bytes                      # bytes this rank's kernel moves
    kernel_ms = kernel_ms_total / max(1, n_launch)           # average launch duration
    alg_bytes_per_launch = 2.0 * payload_per_step * args.steps / max(1, n_launch)
    achieved = alg_bytes_per_launch / (kernel_ms * 1e-3) / GB if kernel_ms > 0 else 0.0
    clocks = sampler.stop() if sampler else None
    egress = sum(ex.layout.region_bytes[rank][d] for d in range(tp) if d != rank) if world > 1 else 0
    # a light checksum of the result so the step has a device->host read
    check = int(ex.recv[:: max(1, ex.recv.numel() // 4096)].to(torch.int64).sum().item())
    if isinstance(ex, PeerShardExchange):
        ex.finish()
    del ex
    fb.close()
    loader.close()
    torch.cuda.empty_cache()

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"

    result = {
        "metric": "safetensors->HBM tensor-parallel load throughput",
        "value": round(data_bytes / (resident_ms * 1e-3) / GB, 2),
        "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": round(resident_ms, 4),
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "u8",
        "data": "synthetic",
        "config": {
            "workload": f"{spec.name} ({args.scale}): {len(spec.tensors)} tensors, {len(paths)} files, "
                        f"{data_bytes} data bytes, tensor-parallel {tp}-way"
                        + (" packed by one rank for all destinations" if world == 1 else
                           " files owned round-robin, " + ("NCCL all-to-all" if args.transport == "nccl"
                                                            else "gather kernel stores into peer arenas (NVLink)")),
            "value_phase": "file images resident in HBM -> gather kernel (+ exchange)",
            "l2": f"inputs ({payload_per_step} B per rank and step) larger than L2 ({L2_BYTES} B), no flush",
            "tp": tp,
        },
        "gpu_launches": int(launches_timed),
        "roofline": {
            "bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
            "frac": round(achieved / peak, 4),
            # dram read+write bytes of one launch: the ncu capture of a small case of this kernel
            # gave 0.993 x its algorithmic bytes (no re-reads); traffic grows in proportion
            "traffic": int(0.993 * alg_bytes_per_launch) if world == 1 else None,
            "traffic_source": "ncu small case x units processed (profiles/fst_gather_kernel_llama3-8b.md)"
                              if world == 1 else None,
            "peak_source": peak_src,
            "kernel": "fst_gather_kernel", "launches": n_launch,
            "avg_launch_ms": round(kernel_ms, 4),
            "algorithmic_bytes_per_launch": int(alg_bytes_per_launch),
        },
        "clocks": clocks,
        "result_checksum": check,
    }
    if world > 1:
        # every byte a rank sends crosses NVLink once; with the step time this is the per-GPU
        # egress rate the exchange sustains (measured peer-copy reference: 770 GB/s per direction)
        result["nvlink"] = {"transport": args.transport, "egress_bytes_per_rank_and_step": int(egress),
                            "egress_gbs_per_gpu": round(egress / (resident_ms * 1e-3) / GB, 1),
                            "reference_peer_copy_gbs": 770.0,
                            "note": "step time includes the gather kernel and the exchange"}
        if args.transport == "peer":
            # fused pack + transfer: the step cannot be faster than the slower of moving this
            # rank's payload through HBM and pushing its remote part through NVLink
            target_ms = max(2.0 * payload_per_step / (peak * GB), egress / (770.0 * GB)) * 1e3
            result["nvlink"]["fused_kernel"] = {"target_ms": round(target_ms, 4),
                                                "achieved_ms": round(kernel_ms, 4),
                                                "frac": round(target_ms / kernel_ms, 4) if kernel_ms else None}

    # ---------------------------------------------------------------- end to end (public API)
    def e2e_step():
        torch.cuda.synchronize()
        barrier()
        t0 = time.perf_counter()
        ld = open_loader()
        ld.add_filenames(owners)
        t1 = time.perf_counter()
        buf = ld.copy_files_to_device()
        t2 = time.perf_counter()
        if world == 1:
            got = buf.shard_locally(plan, tp)
            probe = next(iter(got[-1].values())).get_raw()
        else:
            got = buf.exchange(plan, transport=args.transport)
            probe = next(iter(got.values())).get_raw()
        head = probe.reshape(-1)[:1024].cpu()      # device -> host read of the result
        torch.cuda.synchronize()
        barrier()
        t3 = time.perf_counter()
        del got, probe
        buf.close()
        ld.close()
        return max_over_ranks(t3 - t0), int(head.numel() * head.element_size()), (t1 - t0, t2 - t1, t3 - t2)

    def e2e_phase(cold: bool, steps: int, warmup: int):
        times, d2h, parts = [], 0, []
        r0 = cpp.get_cpp_metrics().read_ns
        for i in range(warmup + steps):
            if cold:
                if rank == 0:
                    synth.drop_page_cache(paths)
                barrier()
            if i == warmup:
                r0 = cpp.get_cpp_metrics().read_ns
            dt, d2h, part = e2e_step()
            if i >= warmup:
                times.append(dt)
                parts.append(part)
            torch.cuda.empty_cache()
        mean = sum(times) / len(times)
        read_s = (cpp.get_cpp_metrics().read_ns - r0) / 1e9 / len(times)
        return {"value": round(data_bytes / mean / GB, 3), "unit": "GB/s",
                "h2d_bytes_per_step": int(data_bytes), "d2h_bytes_per_step": d2h,
                "s_per_step": round(mean, 4), "steps": steps, "warmup": warmup,
                "page_cache": "dropped before every step" if cold else "warm",
                "rank0_phases_s": {"open_and_headers": round(sum(p[0] for p in parts) / len(parts), 4),
                                   "copy_files_to_device": round(sum(p[1] for p in parts) / len(parts), 4),
                                   "shard_and_sync": round(sum(p[2] for p in parts) / len(parts), 4),
                                   "pread_thread_seconds": round(read_s, 3)}}

    note(f"device-resident phase done: {resident_ms:.3f} ms per step")
    if rank == 0:
        result["other_kernels"] = other_kernels(device, peak)
    if not args.no_e2e and not args.kernel_only:
        note("end-to-end phase, cold")
        mA = cpp.get_cpp_metrics()
        if not args.warm_only:
            result["e2e"] = e2e_phase(True, args.steps, min(3, max(1, args.warmup)))
            mB = cpp.get_cpp_metrics()
            result["e2e"]["io"] = {"direct_requests": mB.direct_io_requests - mA.direct_io_requests,
                                   "buffered_requests": mB.buffered_io_requests - mA.buffered_io_requests}
        note("end-to-end phase, warm")
        if rank == 0:
            read_into_page_cache(paths)
        barrier()
        mC = cpp.get_cpp_metrics()
        result["e2e_warm"] = e2e_phase(False, min(args.steps, 3), 3)
        mD = cpp.get_cpp_metrics()
        result["e2e_warm"]["io"] = {"direct_requests": mD.direct_io_requests - mC.direct_io_requests,
                                    "buffered_requests": mD.buffered_io_requests - mC.buffered_io_requests}
        if not args.warm_only:
            note("storage read roofline")
            result["storage_read"] = storage_roofline(paths, owners[rank], rank, barrier, max_over_ranks)
        if not args.warm_only and result["storage_read"]["cold_direct_gbs"]:
            result["e2e"]["frac_of_storage_read"] = round(
                result["e2e"]["value"] / result["storage_read"]["cold_direct_gbs"], 3)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0 and not args.no_cpu_baseline and not args.kernel_only:
        note("cpu baseline (upstream on the host cores)")
        result["cpu_baseline"] = cpu_baseline(spec, paths, tp)
        if world == 1:
            result["reference_cuda_nogds"] = reference_cuda_subprocess(args)
    return result if rank == 0 else {}


def other_kernels(device: str, peak: float) -> dict:
    """The path's other two kernels, timed alone with CUDA events on 1 GiB inputs (larger than
    L2): fst_realign with the source 9 bytes off a 16-byte boundary (an odd header), and
    fst_convert F32 -> BF16.  Algorithmic bytes: 2 x payload, and 4 + 2 bytes per element."""
    import torch

    from fastsafetensors_b200 import _native as nat

    n = 1 << 30
    stream = torch.cuda.current_stream()
    out = {}

    def timed(launch, alg_bytes):
        for _ in range(3):
            launch()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        a.record(stream)
        for _ in range(reps):
            launch()
        b.record(stream)
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / reps
        gbs = alg_bytes / (ms * 1e-3) / GB
        return {"avg_launch_ms": round(ms, 4), "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s",
                "frac": round(gbs / peak, 4), "algorithmic_bytes_per_launch": int(alg_bytes)}

    src = torch.empty(n + 64, dtype=torch.uint8, device=device)
    dst = torch.empty(n + 64, dtype=torch.uint8, device=device)
    out["fst_realign_kernel"] = timed(
        lambda: nat.realign(dst.data_ptr(), src.data_ptr() + 9, n, stream.cuda_stream), 2.0 * n)
    f32 = src[: n].view(torch.float32)
    bf16 = dst[: n // 2].view(torch.bfloat16)
    ops = [(f32.data_ptr(), bf16.data_ptr(), f32.numel(), nat.DT_CODES["F32"], nat.DT_CODES["BF16"])]
    out["fst_convert_kernel"] = timed(lambda: nat.convert(ops, stream.cuda_stream), 1.5 * n)
    # column split with short segments: a [524288, 2048]-byte matrix (1 GiB) split 8 ways on its
    # inner dimension, i.e. 256-byte row segments (what an 8-bit or 4-bit checkpoint gives)
    rows, width, seg = n // 2048, 2048, 256
    cols = [(src.data_ptr() + r * seg, dst.data_ptr() + r * rows * seg, rows, seg, width, seg) for r in range(8)]
    out["fst_gather_kernel_256B_segments"] = timed(
        lambda: nat.gather(cols, stream.cuda_stream, (src.data_ptr(), n), (dst.data_ptr(), n)), 2.0 * n)
    # the same split with every source 3 bytes off (funnel-shift path), and one flat misaligned copy
    off = [(c[0] + 3,) + c[1:] for c in cols]
    out["fst_gather_kernel_256B_segments_shifted"] = timed(
        lambda: nat.gather(off, stream.cuda_stream, (src.data_ptr(), n + 64), (dst.data_ptr(), n)), 2.0 * n)
    flat = [(src.data_ptr() + 5, dst.data_ptr(), 1, n, 0, 0)]
    out["fst_gather_kernel_flat_shifted"] = timed(
        lambda: nat.gather(flat, stream.cuda_stream, (src.data_ptr(), n + 64), (dst.data_ptr(), n)), 2.0 * n)
    del src, dst
    torch.cuda.empty_cache()
    return out


def storage_roofline(paths, my_paths, rank, barrier, max_over_ranks) -> dict:
    """Cold O_DIRECT read bandwidth of the same files with the same thread count, into host
    memory (the role fio plays where it is installed): the ceiling for a cold end-to-end load."""
    from fastsafetensors_b200 import _native as nat
    from fastsafetensors_b200 import cpp
    from tests import synth
    import numpy as np

    if rank == 0:
        synth.drop_page_cache(paths)
    barrier()
    total = sum(os.path.getsize(p) for p in paths)
    scratch = np.empty(max([os.path.getsize(p) for p in my_paths] or [1]), dtype=np.uint8)
    buf = cpp.gds_device_buffer(scratch.ctypes.data, scratch.size, False)
    reader = cpp.Reader(-1, 16, 4 << 20, 2, io_mode=nat.IO_DIRECT)
    barrier()
    t0 = time.perf_counter()
    for p in my_paths:
        n = os.path.getsize(p) // 4096 * 4096
        reader.wait(reader.submit(p, 0, n, buf, 0))
    barrier()
    dt = max_over_ranks(time.perf_counter() - t0)
    reader.close()
    return {"cold_direct_gbs": round(total / dt / GB, 3), "threads_per_rank": 16, "block": "4 MiB",
            "tool": "native reader, O_DIRECT, host destination (fio is not installed)"}


# ------------------------------------------------------------------------------------------
# upstream's CPU path (the checker's build in oracle/_ref), timed on the host cores
# ------------------------------------------------------------------------------------------
REF_DIR = os.path.join(ROOT, "oracle", "_ref")


def _numa_nodes() -> int:
    import glob

    return max(1, len(glob.glob("/sys/devices/system/node/node[0-9]*")))


def _reference_settings(kind: str, paths, world: int):
    """Keyword arguments for upstream's loader and for its ``copy_files_to_device``.

    ``defaults``: what a caller that passes nothing gets (vLLM does): 16 threads, a 16 MiB bounce
    buffer and a 16 GiB block, i.e. ONE read request, hence one thread, per file.
    ``tuned``: the rule of upstream's own benchmark tool (perf/fastsafetensors_perf/perf.py,
    get_auto_config): threads = physical cores, bounce = their L2 capacity, block = checkpoint
    bytes / ranks / threads rounded up to the bounce size, so that every thread has a block."""
    if kind == "defaults":
        return {}, {}
    from fastsafetensors_b200 import tune

    topo = tune.HostTopology.probe(None)
    threads = max(1, topo.physical_cores or os.cpu_count() or 1)
    bbuf_kb = topo.l2_kb or 16 * 1024
    block = max(1, sum(os.path.getsize(p) for p in paths) // world // threads)
    unit = bbuf_kb * 1024
    if block % unit:
        block += unit - block % unit
    return {"max_threads": threads, "bbuf_size_kb": bbuf_kb}, {"max_copy_block_size": block}


def _reference_rank(rank: int, world: int, paths, plan_items, phases, port: int, out_path: str,
                    settings: str = "defaults") -> None:
    """One gloo rank running UPSTREAM's loader on device "cpu": files owned round-robin, every
    tensor requested by the plan (get_sharded / get_tensor / push_tensor).  ``settings``:
    ``defaults``, ``tuned`` or ``best`` (one untimed step with each, the faster one is timed)."""
    sys.path.insert(0, REF_DIR)
    import torch
    import torch.distributed as dist

    import fastsafetensors as ref
    from tests import synth

    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))
    pg = None
    if world > 1:
        # an explicit tcp:// rendezvous of our own: drop what a launcher (torchrun) left in the
        # environment, or every rank would wait as a client of the launcher's store
        for key in [k for k in os.environ if k.startswith("TORCHELASTIC_")]:
            os.environ.pop(key)
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank,
                                world_size=world)
        pg = dist.group.WORLD

    def barrier():
        if world > 1:
            dist.barrier()

    def agreed(value):
        """Rank 0's value on every rank."""
        box = [value]
        if world > 1:
            dist.broadcast_object_list(box, src=0)
        return box[0]

    def one_step(kind: str, n_files: int, cold: bool):
        use = sorted(paths)[:n_files]
        loader_kw, copy_kw = _reference_settings(kind, use, world)
        if cold and rank == 0:
            synth.drop_page_cache(use)
        barrier()
        t0 = time.perf_counter()
        loader = ref.SafeTensorsFileLoader(pg if pg is not None else ref.SingleGroup(), "cpu", nogds=True,
                                           **loader_kw)
        loader.add_filenames(synth.owners(use, world))
        fb = loader.copy_files_to_device(**copy_kw)
        present = set(fb.key_to_rank_lidx)
        keep = []
        for name, action in plan_items:
            if name not in present:
                continue
            if action[0] == "shard":
                keep.append(fb.get_sharded(name, action[1]))
            elif action[0] == "replicate":
                keep.append(fb.get_tensor(name))
            else:
                keep.append(fb.push_tensor(name, action[1]))
        barrier()
        dt = time.perf_counter() - t0
        nbytes = sum(m.size_bytes - m.header_length for m, _ in loader.meta.values())
        del keep
        fb.close()
        loader.close()
        return dt, nbytes

    results = {}
    chosen = None if settings == "best" else settings
    tried = {}
    for label, cold, steps, warmup, budget_s in phases:
        n_files = len(paths)
        last_dt = None
        if chosen is None:
            # one untimed step with each setting over the whole checkpoint; they double as warm-up
            trial = {}
            for kind in ("defaults", "tuned"):
                trial[kind] = one_step(kind, n_files, cold)
                tried[kind] = round(trial[kind][1] / trial[kind][0] / GB, 3)
            chosen = agreed(max(tried, key=tried.get))
            last_dt = trial[chosen][0]
            if steps == 0:      # the trial of the faster setting is the sample
                results[label] = {"seconds": [trial[chosen][0]], "bytes": [trial[chosen][1]], "files": n_files}
                continue
        else:
            for _ in range(warmup):
                last_dt, _ = one_step(chosen, n_files, cold)
        # bounded sample: if the timed steps would not fit the phase's budget, go on with the
        # first files only (rank 0 decides, everyone follows)
        if last_dt is not None and last_dt * steps > budget_s:
            n_files = max(1, int(len(paths) * budget_s / (last_dt * steps)))
        n_files = agreed(n_files)
        samples = [one_step(chosen, n_files, cold) for _ in range(steps)]
        results[label] = {"seconds": [s_[0] for s_ in samples], "bytes": [s_[1] for s_ in samples],
                          "files": n_files}
    results["settings"] = {"used": chosen, "tried_gbs": tried,
                           "kwargs": [dict(d) for d in _reference_settings(chosen, sorted(paths), world)]}
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(results, f)
    if world > 1:
        dist.destroy_process_group()


def run_reference(spec, paths, tp: int, phases, timeout_s: float = 900.0, settings: str = "defaults") -> dict:
    import tempfile

    import torch.multiprocessing as mp

    if not os.path.exists(os.path.join(REF_DIR, "fastsafetensors", "__init__.py")):
        raise FileNotFoundError("oracle/_ref is missing (build it with oracle/build_ref.sh)")
    plan_items = list(plan_for(spec, tp).items())
    with tempfile.TemporaryDirectory() as tmp:
        out_path = os.path.join(tmp, "times.json")
        import socket

        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sock:   # a port that is free now
            sock.bind(("127.0.0.1", 0))
            port = sock.getsockname()[1]
        if tp == 1:
            _reference_rank(0, 1, paths, plan_items, phases, port, out_path, settings)
        else:
            ctx = mp.start_processes(_reference_rank, args=(tp, paths, plan_items, phases, port, out_path, settings),
                                     nprocs=tp, join=False, start_method="spawn")
            deadline = time.time() + timeout_s
            while not ctx.join(timeout=5):
                if time.time() > deadline:
                    for p in ctx.processes:
                        p.kill()
                    raise TimeoutError(f"upstream CPU run exceeded {timeout_s} s")
        return json.load(open(out_path))


def cpu_baseline(spec, paths, tp: int) -> dict:
    """Upstream on the host cores, one cold and one warm pass over the same checkpoint."""
    t, failure = None, None
    for settings, phases in (("best", [("cold", True, 0, 0, 1e9), ("warm", False, 1, 0, 1e9)]),
                             ("defaults", [("cold", True, 1, 0, 1e9), ("warm", False, 1, 0, 1e9)])):
        try:
            t = run_reference(spec, paths, tp, phases, timeout_s=300.0, settings=settings)
            break
        except Exception as e:  # noqa: BLE001
            failure = f"failed: {type(e).__name__}: {e}"
    if t is None:
        return {"value": None, "unit": "GB/s", "cores": os.cpu_count(), "kind": "reference", "sample": failure}
    cold, warm = t["cold"]["seconds"][0], t["warm"]["seconds"][0]
    return {"value": round(spec.data_bytes / cold / GB, 3), "unit": "GB/s", "cores": os.cpu_count(),
            "kind": "reference",
            "sample": f"upstream fastsafetensors 0.3.2, device cpu, nogds, {tp} gloo ranks, whole "
                      f"{spec.name} checkpoint once with the page cache dropped ({cold:.2f} s) and "
                      f"once warm ({warm:.2f} s); the faster of library defaults (one request per "
                      f"file) and the rule of upstream's perf tool (a block per thread), cold GB/s: "
                      f"{t['settings']['tried_gbs']}, used: {t['settings']['used']} {t['settings']['kwargs']}",
            "warm_value": round(spec.data_bytes / warm / GB, 3), "settings": t["settings"],
            "numa_nodes": _numa_nodes()}


def reference_cuda_subprocess(args) -> dict:
    """Run ``--impl reference-cuda`` in a child process (its own CUDA context and allocator)."""
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference-cuda", "--config", args.config,
           "--scale", args.scale, "--dir", args.dir, "--layers", str(args.layers)]
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
        line = [l for l in proc.stdout.splitlines() if l.startswith("{")]
        return json.loads(line[-1]) if line else {"unavailable": (proc.stderr or "no output")[-300:]}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"}


def reference_arm(args) -> dict:
    from tests import synth

    rank, _, world = dist_env()
    if rank != 0:
        return {}
    spec = load_spec(args)
    tp = spec.tp if world == 1 else world
    paths = prepare_files(spec, args.dir, 0, lambda: None)
    phases = [("cold", True, args.steps, 1, args.ref_budget), ("warm", False, min(args.steps, 3), 1, 40.0)]
    try:
        t = run_reference(spec, paths, tp, phases, timeout_s=600.0, settings=args.ref_settings)
    except Exception as e:  # noqa: BLE001
        if args.ref_settings == "defaults":
            raise
        sys.stderr.write(f"[bench] reference arm with settings {args.ref_settings!r} failed "
                         f"({type(e).__name__}: {e}); running upstream's defaults\n")
        t = run_reference(spec, paths, tp, phases, timeout_s=600.0, settings="defaults")

    def rate(ph):
        return sum(ph["bytes"]) / sum(ph["seconds"]) / GB

    cold = sum(t["cold"]["seconds"]) / len(t["cold"]["seconds"])
    v = round(rate(t["cold"]), 3)
    sample = (f"upstream fastsafetensors 0.3.2 (oracle/_ref), device cpu, nogds, {tp} gloo ranks on "
              f"{os.cpu_count()} cores, {t['cold']['files']} of {len(paths)} files of the {spec.name} "
              f"checkpoint per step, page cache dropped before every step; settings "
              f"{t['settings']['used']} {t['settings']['kwargs']} (cold GB/s of one untimed step each: "
              f"{t['settings']['tried_gbs']})")
    return {
        "impl": "reference",
        "metric": "safetensors->HBM tensor-parallel load throughput",
        "value": v, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": 1,
        "ms_per_step": round(cold * 1e3, 2), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": f"{spec.name} ({args.scale}): {len(spec.tensors)} tensors, {len(paths)} files, "
                               f"{spec.data_bytes} data bytes, tensor-parallel {tp}-way, host memory", "tp": tp},
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": os.cpu_count(), "kind": "reference",
                         "sample": sample, "numa_nodes": _numa_nodes(), "settings": t["settings"]},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "page_cache": "dropped before every step"},
        "e2e_warm": {"value": round(rate(t["warm"]), 3), "unit": "GB/s", "files": t["warm"]["files"]},
        "gpu_launches": 0,
    }


def reference_cuda_arm(args) -> dict:
    """Upstream's own CUDA path (nogds: buffered pread + synchronous cudaMemcpy per chunk) on
    one GPU: files -> HBM, every tensor instantiated.  One rank cannot shard, so this times the
    load only; it is reported beside the b200 arm, not as the reference arm."""
    sys.path.insert(0, REF_DIR)
    import torch

    import fastsafetensors as ref
    from tests import synth

    spec = load_spec(args)
    paths = prepare_files(spec, args.dir, 0, lambda: None)
    out = {}
    for label, cold in (("cold", True), ("warm", False)):
        if cold:
            synth.drop_page_cache(paths)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        loader = ref.SafeTensorsFileLoader(ref.SingleGroup(), "cuda:0", nogds=True)
        loader.add_filenames({0: paths})
        fb = loader.copy_files_to_device()
        keep = [fb.get_tensor(k) for k in fb.key_to_rank_lidx]
        torch.cuda.synchronize()
        out[label] = round(spec.data_bytes / (time.perf_counter() - t0) / GB, 3)
        del keep
        fb.close()
        loader.close()
    return {"impl": "reference-cuda", "unit": "GB/s", "cold": out["cold"], "warm": out["warm"],
            "what": "upstream fastsafetensors 0.3.2, device cuda:0, nogds, one rank, library defaults; "
                    "files -> HBM and get_tensor of every key (no sharding with one rank)"}


def main() -> None:
    args = parse_args()
    # stdout carries the one JSON line and nothing else: libraries that print to file
    # descriptor 1 (NCCL's version banner, for one) are sent to stderr for the whole run
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference-cuda":
        out = reference_cuda_arm(args)
    else:
        out = reference_arm(args) if args.impl == "reference" else b200_arm(args)
    sys.stdout.flush()
    if out:
        os.write(json_fd, (json.dumps(out) + "\n").encode())
    os.close(json_fd)


if __name__ == "__main__":
    main()
